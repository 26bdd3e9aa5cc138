/*
 * C ABI of the CUDA (sm_100a) FAISS-search backend: exact Flat and IVFFlat
 * top-k search for L2 and inner product.
 *
 * In the reference this path is C++: a `faiss::Index` subclass handed out by
 * `duckdb::GpuBackend::CpuToGpu` (src/include/gpu_backend.hpp:12-33,
 * src/gpu_backend_metal.mm:42-60).  The C++ classes in gpu_backend_cuda.hpp are
 * thin wrappers over the functions below; every function here names the
 * reference member it stands behind.
 *
 * Conventions: plain C, no exceptions; 0 = success, -1 = error with the reason
 * kept per thread (ann_cuda_last_error).  Metric codes are FAISS's:
 * 0 = METRIC_INNER_PRODUCT (larger is better, raw dot returned),
 * 1 = METRIC_L2 (SQUARED distance, smaller is better).  Results are sorted best
 * first; missing slots hold label -1 and distance +inf (L2) / -inf (IP)
 * (faiss-metal/src/MetalIndexFlat.mm:303-309, 363-367).  Labels are int64
 * (faiss::idx_t).  search() is safe to call from many threads at once on one
 * index (src/faiss_index.cpp:729-737 does so); add/reset/train are not.
 */
#ifndef ANN_CUDA_H
#define ANN_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* exported even when the library is built with hidden visibility */
#endif

#define ANN_CUDA_METRIC_INNER_PRODUCT 0
#define ANN_CUDA_METRIC_L2 1

typedef struct ann_cuda_index ann_cuda_index;

/* Reason of the calling thread's last -1 ("" if none). */
const char *ann_cuda_last_error(void);

/* GpuBackend::IsAvailable (src/include/gpu_backend.hpp:17,
 * src/gpu_backend_metal.mm:26-28): 1 if device 0..n-1 exist and are sm_100. */
int ann_cuda_available(void);
int ann_cuda_device_count(void);

/* GpuBackend::DeviceInfo (gpu_backend.hpp:20, gpu_backend_metal.mm:30-36):
 * writes e.g. "CUDA GPU (NVIDIA B200, sm_100, 148 SMs, 8 devices)". */
int ann_cuda_device_info(char *buf, size_t buflen);

/* ---- Flat --------------------------------------------------------------------
 * MetalIndexFlat(resources, d, metric) (faiss-metal/include/faiss-metal/MetalIndexFlat.h:47-59). */
int ann_cuda_flat_create(int device, int d, int metric, ann_cuda_index **out);

/* Storage precision of a flat index: StorageType of faiss-metal/include/faiss-metal/MetalIndexFlat.h:38-43
 * (Float32 = 0, Float16 = 1, BFloat16 = 2) and its extended constructor (:60).  With F16 / BF16 the rows are
 * rounded to that type (nearest even, faiss-metal/src/MetalIndexFlat.mm:211-236) when they are added and
 * only the rounded rows are kept: 2 bytes per element instead of 8 (the fp32 store keeps two TF32 planes).
 * Queries stay fp32.  Distances and neighbours are those of the ROUNDED rows, to the same 1e-4 as for the
 * fp32 store (the reference checks its fp16 index against the unrounded CPU index with 5e-2 and a top-1
 * match, faiss-metal/tests/test_metal_flat.mm:259-261); reconstruct returns the rounded row widened to
 * fp32 (:262-268).  fp16 elements beyond +-65504 become infinite, as in the reference.
 * Searched on the tensor cores with 16-bit operands (tcgen05.mma kind::f16) and the same banded candidate
 * lists, band check and exact re-ranking as the fp32 store; k above 224 and stores of fewer than ~256 rows
 * go to the exact scan.  Not available for IVFFlat, the sharded index or the allocation-free entry point. */
#define ANN_CUDA_STORAGE_F32 0
#define ANN_CUDA_STORAGE_F16 1
#define ANN_CUDA_STORAGE_BF16 2
int ann_cuda_flat_create_storage(int device, int d, int metric, int storage, ann_cuda_index **out);
/* MetalIndexFlat::getStorageType (MetalIndexFlat.h:90): one of ANN_CUDA_STORAGE_*, -1 for a null handle. */
int ann_cuda_index_storage(const ann_cuda_index *index);

/* ---- IVFFlat -----------------------------------------------------------------
 * MetalIndexIVFFlat(resources, d, nlist, metric) (faiss-metal/include/faiss-metal/MetalIndexIVFFlat.h:25-33). */
int ann_cuda_ivfflat_create(int device, int d, int64_t nlist, int metric, ann_cuda_index **out);

/* Installs trained centroids (nlist x d, host) and marks the index trained: the
 * centroid copy of index_cpu_to_metal_ivf (faiss-metal/src/MetalIndexIVFFlat.mm:291-296). */
int ann_cuda_ivfflat_set_centroids(ann_cuda_index *index, const float *centroids);

/* MetalIndexIVFFlat::train (MetalIndexIVFFlat.mm:86-100): k-means on n host rows. */
int ann_cuda_ivfflat_train(ann_cuda_index *index, int64_t n, const float *x);

/* Appends one inverted list's content as stored by the CPU index: ids and
 * rows of list `list_no` (MetalIndexIVFFlat.mm:299-311).  Host pointers. */
int ann_cuda_ivfflat_add_list(ann_cuda_index *index, int64_t list_no, int64_t n, const int64_t *ids,
                              const float *rows);

/* Reads list `list_no` back: size, then ids/rows (either may be NULL)
 * (index_metal_to_cpu_ivf, MetalIndexIVFFlat.mm:336-354). */
int64_t ann_cuda_ivfflat_list_size(const ann_cuda_index *index, int64_t list_no);
int ann_cuda_ivfflat_get_list(const ann_cuda_index *index, int64_t list_no, int64_t *ids, float *rows);
int ann_cuda_ivfflat_get_centroids(const ann_cuda_index *index, float *centroids);

/* The coarse quantiser alone: the `nprobe` nearest centroids of each of n host queries
 * under the index metric, nearest first, as list numbers (-1 past nlist) - the
 * coarse_search step of MetalIndexIVFFlat::search (MetalIndexIVFFlat.mm:60-66, 155). */
int ann_cuda_ivfflat_coarse(const ann_cuda_index *index, int64_t n, const float *x, int64_t nprobe, int64_t *lists);

/* Multi-GPU IVFFlat without a replicated coarse quantiser: every GPU ranks the centroids for ITS share of the
 * queries (ann_cuda_ivfflat_coarse_device: n x nprobe list numbers, int32, best first, nprobe = the index's),
 * the probe lists are exchanged (a few hundred KB), and every GPU scans the lists it stores for ALL queries
 * with the probes given (faiss::IndexIVF::search_preassigned with `assign`; -1 = no list).  Both are
 * stream-ordered like ann_cuda_index_search_device; ann_cuda_index_search_status collects a failed wait.
 * No counterpart in the reference (it has no multi-GPU path). */
int ann_cuda_ivfflat_coarse_device(const ann_cuda_index *index, int64_t n, const float *x_device, int32_t *lists_device,
                                   void *stream);
int ann_cuda_ivfflat_search_preassigned_device(const ann_cuda_index *index, int64_t n, const float *x_device,
                                               const int32_t *assign_device, int64_t k, float *distances_device,
                                               int64_t *labels_device, int64_t label_offset, void *stream);

/* setNprobe / getNprobe (MetalIndexIVFFlat.mm:267-279): clamped to [1, nlist]. */
int ann_cuda_ivfflat_set_nprobe(ann_cuda_index *index, int64_t nprobe);
int64_t ann_cuda_ivfflat_get_nprobe(const ann_cuda_index *index);
int64_t ann_cuda_ivfflat_nlist(const ann_cuda_index *index);

/* Sharding of the inverted lists across GPUs: this index keeps only lists with
 * list_no % shard_count == shard_rank; rows added to other lists are dropped
 * (they live on another GPU).  The coarse quantiser stays complete on every
 * shard.  No counterpart in the reference (single device).  Call before add. */
int ann_cuda_ivfflat_set_shard(ann_cuda_index *index, int shard_rank, int shard_count);

/* ---- common faiss::Index surface ------------------------------------------------ */

/* faiss::Index::add (MetalIndexFlat.mm:173-292; MetalIndexIVFFlat.mm:102-120).
 * Flat: appends rows, label = position.  IVFFlat: assigns each row to its
 * nearest centroid on the GPU; label = running ntotal. */
int ann_cuda_index_add(ann_cuda_index *index, int64_t n, const float *x);

/* Same with x in the index's device memory space (no host copy). */
int ann_cuda_index_add_device(ann_cuda_index *index, int64_t n, const float *x_device);

/* Pre-sizes the storage for `n_total` rows so add never reallocates. */
int ann_cuda_index_reserve(ann_cuda_index *index, int64_t n_total);

/* faiss::Index::search (MetalIndexFlat.mm:294-369; MetalIndexIVFFlat.mm:122-256).
 * x: n x d (host), distances/labels: n x k (host).  Synchronous. */
int ann_cuda_index_search(const ann_cuda_index *index, int64_t n, const float *x, int64_t k, float *distances,
                          int64_t *labels);

/* Same with DEVICE pointers; work is enqueued on `stream` (cudaStream_t, NULL =
 * default stream) and not synchronised.  label_offset is added to every valid
 * label (row-sharded indexes pass the shard's first row).  Should a pass of the flat
 * search find more near ties inside its error band than it kept candidates for, the
 * next more exact pass is already enqueued behind it and runs by itself (decided on
 * the device): when the stream reaches the end of the call the results are complete.
 * No counterpart in the reference (its index takes host pointers only). */
int ann_cuda_index_search_device(const ann_cuda_index *index, int64_t n, const float *x_device, int64_t k,
                                 float *distances_device, int64_t *labels_device, int64_t label_offset,
                                 void *stream);

/* Waits for `stream` and reports on the ann_cuda_index_search_device calls made on it
 * since the last such report: 0 = fine; -1 = a kernel gave up on one of its bounded
 * waits (a device in trouble), the results of those calls are not valid.  The role
 * of the command buffer's status check, MetalIndexFlat.mm:348-351. */
int ann_cuda_index_search_status(const ann_cuda_index *index, void *stream);

/* MetalIndexFlat::searchAsync and its MetalSearchToken (MetalIndexFlat.h:15-36,
 * MetalIndexFlat.mm:371-443): the search is enqueued and the call returns; `x` may be reused
 * at once, `distances` / `labels` (host) are written by ann_cuda_search_token_wait.  Each token
 * holds its own stream and staging buffers until it is waited on or freed, so several searches
 * can be in flight on one index.  _ready: 1 when the device work has finished, 0 while it
 * runs, -1 on a null token.  _wait: blocks, copies the results out, returns 0 or -1; a second
 * wait returns the first one's result.  _free may be called without a wait (the results are
 * then dropped).  Works for Flat and IVFFlat indexes. */
typedef struct ann_cuda_search_token ann_cuda_search_token;
int ann_cuda_index_search_async(const ann_cuda_index *index, int64_t n, const float *x, int64_t k, float *distances,
                                int64_t *labels, ann_cuda_search_token **token);
int ann_cuda_search_token_ready(const ann_cuda_search_token *token);
int ann_cuda_search_token_wait(ann_cuda_search_token *token);
void ann_cuda_search_token_free(ann_cuda_search_token *token);

/* faiss::Index::reset / reconstruct (MetalIndexFlat.mm:445-478). reconstruct is
 * bit-exact; for IVFFlat `key` is the label given at add time. */
int ann_cuda_index_reset(ann_cuda_index *index);
int ann_cuda_index_reconstruct(const ann_cuda_index *index, int64_t key, float *recons);

/* Flat only: copies rows [first, first+n) to host (getVectorsData / get_xb,
 * MetalIndexFlat.mm:480-487, used by index_metal_to_cpu :517-535). */
int ann_cuda_flat_get_rows(const ann_cuda_index *index, int64_t first, int64_t n, float *rows);

int64_t ann_cuda_index_ntotal(const ann_cuda_index *index);
int ann_cuda_index_d(const ann_cuda_index *index);
int ann_cuda_index_metric(const ann_cuda_index *index);
int ann_cuda_index_is_trained(const ann_cuda_index *index);
int ann_cuda_index_is_ivf(const ann_cuda_index *index);
int ann_cuda_index_device(const ann_cuda_index *index);
void ann_cuda_index_free(ann_cuda_index *index);

/* Flat search that allocates nothing.  It has no counterpart in the reference.
 * For hosts that must not allocate device memory while searching - a worker bound
 * to a fixed memory budget, a caller recording its searches into a CUDA graph, a
 * thread that cannot afford the device-wide stalls cudaMalloc / cudaFree may cause:
 * the regular entry points grow a scratch pool on first use and whenever a call is
 * larger than the ones before.  Same arguments and results as
 * ann_cuda_index_search_device, Flat indexes only, with the limits n <= 128
 * queries, k <= 16, dimension <= 1024; anything larger returns -1 with the limit
 * in ann_cuda_last_error().  All scratch lives in one fixed device array of about
 * 6 MB that every GPU loading the library holds until the process exits.  The first
 * call on a device looks up that array's address (no allocation); make that first
 * call before starting any stream capture.  Every call shares the array: calls
 * whose GPU work may overlap (other streams, other host threads) race on it and
 * must be serialised by the caller. */
int ann_cuda_flat_search_small_static(const ann_cuda_index *index, int64_t n, const float *x_device, int64_t k,
                                      float *distances_device, int64_t *labels_device, int64_t label_offset,
                                      void *stream);
/* Waits for `stream` and reports on the allocation-free searches run on `device` since
 * the last report: 0 = fine; 1 = some query had more near ties around its k-th place
 * than the 16 candidates this entry point keeps can settle (its result may differ from
 * the regular search inside that tie; repeat it with a regular entry point);
 * -1 = a kernel gave up on a bounded wait, results are not valid.  Allocates nothing.
 * No counterpart in the reference. */
int ann_cuda_flat_search_small_static_status(int device, void *stream);

/* ---- one index over several GPUs, in one process ------------------------------------
 * No counterpart in the reference (single device).  This is the object CpuToGpu hands out
 * when more than one device is configured, so that the one process that owns the index
 * (src/faiss_index.cpp:108-149) searches all GPUs through the ordinary search() call.
 * Flat (nlist = 0): rows in contiguous ranges, one per shard, labels = global positions.
 * IVFFlat (nlist > 0): inverted list l on shard l % shards, coarse quantiser on every shard.
 * search: every shard (own host thread, own stream) searches its part for all queries;
 * the per-shard top-k lists are copied into the first device's memory and merged there
 * (ann_cuda_merge_topk_device).  A device may be named more than once (several shards
 * on one GPU).  Calls on one sharded index are serialised internally. */
typedef struct ann_cuda_sharded_index ann_cuda_sharded_index;
int ann_cuda_sharded_create(const int *devices, int ndev, int d, int metric, int64_t nlist,
                            ann_cuda_sharded_index **out);
void ann_cuda_sharded_free(ann_cuda_sharded_index *index);
int ann_cuda_sharded_shard_count(const ann_cuda_sharded_index *index);
/* The shard itself (borrowed), e.g. to fill it from device memory with ann_cuda_index_add_device
 * or to read an inverted list back from its owner.  Flat shards must be filled in order: the
 * label offset of a shard is the number of rows in the shards before it. */
ann_cuda_index *ann_cuda_sharded_shard(const ann_cuda_sharded_index *index, int shard);
int64_t ann_cuda_sharded_ntotal(const ann_cuda_sharded_index *index);
/* faiss::Index::add.  Flat: the first add is cut into equal contiguous ranges, later adds go
 * behind the last shard's rows.  IVFFlat: every shard assigns the rows and keeps its lists'. */
int ann_cuda_sharded_add(ann_cuda_sharded_index *index, int64_t n, const float *x);
int ann_cuda_sharded_train(ann_cuda_sharded_index *index, int64_t n, const float *x);
int ann_cuda_sharded_set_centroids(ann_cuda_sharded_index *index, const float *centroids);
int ann_cuda_sharded_add_list(ann_cuda_sharded_index *index, int64_t list_no, int64_t n, const int64_t *ids,
                              const float *rows);
int ann_cuda_sharded_set_nprobe(ann_cuda_sharded_index *index, int64_t nprobe);
/* faiss::Index::search / reset / reconstruct with host pointers, as ann_cuda_index_search. */
int ann_cuda_sharded_search(const ann_cuda_sharded_index *index, int64_t n, const float *x, int64_t k,
                            float *distances, int64_t *labels);
int ann_cuda_sharded_reset(ann_cuda_sharded_index *index);
int ann_cuda_sharded_reconstruct(const ann_cuda_sharded_index *index, int64_t key, float *recons);
int ann_cuda_sharded_get_rows(const ann_cuda_sharded_index *index, int64_t first, int64_t n, float *rows);

/* ---- multi-GPU merge -------------------------------------------------------------
 * Final k-select over per-shard results.  parts_*: (nparts x nq x k) in DEVICE
 * memory, each (part, query) run sorted best first as search_device writes it;
 * out_*: (nq x k) device.  Enqueued on `stream`.  No counterpart in the
 * reference (single device); it is the last step of the sharded search. */
int ann_cuda_merge_topk_device(int device, const float *parts_distances, const int64_t *parts_labels, int nparts,
                               int64_t nq, int64_t k, int metric, float *out_distances, int64_t *out_labels,
                               void *stream);

/* Which flat-search kernel the library runs: "tcgen05" (tensor cores, the
 * product path) or "simt" (exact-fp32 cross-check kernel).  Selected by the
 * environment variable ANN_CUDA_FLAT_KERNEL; default tcgen05. */
const char *ann_cuda_flat_kernel_name(void);
/* Overrides that choice for the whole process; used by the tests to cross-check one
 * kernel against the other.  "tcgen05": tensor-core kernel; flat stores of two
 * million rows or more are searched with one-MMA screening (256 candidates chosen by
 * q_hi.x_hi keys under a proven error slack), smaller ones with the three-MMA split
 * product (k + 32 candidates); either way the candidates are re-ranked in exact fp32.
 * "tcgen05-screened" / "tcgen05-split": screening always / never.  "simt": the
 * exact-fp32 scan only.  Each tensor-core pass checks, for every query, that its last
 * candidate lies outside the error band above the k-th (about 0.2 % of |q||x|max for
 * screening, 0.03 % for the split product at d = 768); otherwise the query block is
 * searched again one tier up (screened -> split -> exact scan), by every entry point. */
int ann_cuda_set_flat_kernel(const char *name);

/* How many times a pass of the flat search found more rows inside its error band than
 * it kept candidates for, so that the query block was searched again one tier up
 * (screened -> split product -> exact fp32 scan).  Process-wide, since load; passes
 * repeated on the device are counted when their stream is next waited for
 * (ann_cuda_index_search_status, ann_cuda_search_token_wait). */
uint64_t ann_cuda_screen_fallbacks(void);

/* Every wait inside the tensor-core kernel is bounded; a wait that runs out makes the
 * search fail with an error instead of hanging.  Sets that bound (default 2000 ms;
 * ms <= 0 restores it).  Process-wide. */
void ann_cuda_set_wait_limit_ms(int ms);
/* Test support: with after_k_blocks >= 0 the loader of every CTA stops after that many
 * blocks of the dimension, the kernel's waits run out and the search FAILS with the
 * give-up error (it never returns partial results as success); -1 = off (default).
 * Lets a test exercise the give-up path without a fault. */
void ann_cuda_test_withhold_loads(int after_k_blocks);

/* Measurement hook.  With timing on, every search records CUDA events around
 * its flat-search kernel on the stream the kernel is launched on;
 * ann_cuda_index_last_flat_kernel_ms waits for the latest such kernel of `index`
 * and returns its duration in milliseconds (-1 if none was timed). */
void ann_cuda_set_kernel_timing(int on);
float ann_cuda_index_last_flat_kernel_ms(const ann_cuda_index *index);

/* Number of kernel launches this library has issued from the calling process
 * since load (all threads).  For the benchmark's launch accounting. */
uint64_t ann_cuda_launch_count(void);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* ANN_CUDA_H */
