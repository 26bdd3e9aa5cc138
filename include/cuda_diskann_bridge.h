/*
 * C ABI of the DiskANN batch-distance bridge, CUDA (sm_100a) implementation.
 *
 * The first three symbols keep the names, argument order, units and return
 * codes of the reference's bridge header (src/include/metal_diskann_bridge.h:8-23)
 * so that the Rust side (rust_lib/src/metal_ffi.rs:10-30) and the C++ caller
 * (src/ann_search.cpp:723-732) link against this library unchanged.
 *
 * Conventions, all entry points:
 *   - plain C, no exceptions, never aborts; 0 = success, -1 = error.  On -1
 *     the reference's callers fall back to their CPU loop
 *     (rust_lib/src/disk_provider.rs:436-453, src/ann_search.cpp:727-731); the
 *     reason is kept per thread and returned by diskann_cuda_last_error().
 *   - metric 0 = L2 (SQUARED distance), any other value = inner product,
 *     returned NEGATED (src/metal_diskann_bridge.mm:167,
 *     faiss-metal/shaders/diskann_distance.metal:148,192).
 *   - callable from any number of host threads at once.
 */
#ifndef ANN_CUDA_DISKANN_BRIDGE_H
#define ANN_CUDA_DISKANN_BRIDGE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* exported even when the library is built with hidden visibility */
#endif

/* Replaces diskann_metal_available (src/include/metal_diskann_bridge.h:8,
 * src/metal_diskann_bridge.mm:145-153).  1 if a CUDA device of compute
 * capability 10.x is usable, else 0.  Initialises lazily; cheap afterwards. */
int diskann_metal_available(void);

/* Replaces diskann_metal_batch_distances (metal_diskann_bridge.h:14,
 * src/metal_diskann_bridge.mm:155-253).  One query (dim floats) against n
 * gathered rows (n*dim contiguous floats); writes n distances.  All pointers
 * are HOST memory owned by the caller; the call is synchronous. */
int diskann_metal_batch_distances(const float *query, const float *candidates, int n, int dim, int metric,
                                  float *out_distances);

/* Replaces diskann_metal_multi_batch_distances (metal_diskann_bridge.h:22,
 * src/metal_diskann_bridge.mm:255-323).  Row i is scored against
 * queries[query_map[i]]; query_map values must be < nq.  HOST pointers. */
int diskann_metal_multi_batch_distances(const float *queries, const float *candidates,
                                        const unsigned int *query_map, int total_n, int nq, int dim, int metric,
                                        float *out_distances);

/* ---- additive entry points: device-resident tables, rows named by id -------
 * The reference gathers neighbour rows on the host before every call
 * (rust_lib/src/disk_provider.rs:420-424, 592-600; rust_lib/src/provider.rs:385-400).
 * These keep the vector table in GPU memory and take the row ids instead, so
 * the distance pass reads rows from HBM rather than over PCIe. */

typedef struct diskann_cuda_table diskann_cuda_table;

/* Last error message of the calling thread ("" if none). */
const char *diskann_cuda_last_error(void);

/* Copies num x dim fp32 rows (host) to the device `device`.  The fp32 table of
 * the in-memory provider / the .diskann vector section
 * (rust_lib/src/provider.rs:159-160, rust_lib/src/file_format.rs:3-18). */
int diskann_cuda_register_table(int device, const float *host_rows, size_t num, int dim,
                                diskann_cuda_table **out);

/* Same, rows already in device memory (adopted by reference: the caller keeps
 * ownership and must keep them alive until unregister). */
int diskann_cuda_register_table_device(int device, const float *device_rows, size_t num, int dim,
                                       diskann_cuda_table **out);

/* SQ8 table: u8 codes (num x dim) plus per-dimension min and scale, as
 * produced by quantize_sq8 (rust_lib/src/provider.rs:161-210).  Host pointers. */
int diskann_cuda_register_sq8(int device, const uint8_t *codes, const float *mins, const float *scale, size_t num,
                              int dim, diskann_cuda_table **out);

/* Same with the codes already in device memory (adopted by reference);
 * mins/scale are host pointers and are copied. */
int diskann_cuda_register_sq8_device(int device, const uint8_t *device_codes, const float *mins,
                                     const float *scale, size_t num, int dim, diskann_cuda_table **out);

int diskann_cuda_unregister(diskann_cuda_table *table);

/* out[i] = distance(queries[query_map[i]], row ids[i]); query_map may be NULL
 * when nq == 1.  For an SQ8 table the row is dequantised as
 * (code/255)*scale+min (rust_lib/src/provider.rs:138-147) and scored against the
 * fp32 query (asymmetric distance).  HOST pointers; synchronous.  ids >= num
 * or query_map >= nq give -1 and leave out_distances unspecified. */
int diskann_cuda_batch_distances_by_id(const diskann_cuda_table *table, const float *queries, int nq,
                                       const uint32_t *ids, const uint32_t *query_map, int total_n, int metric,
                                       float *out_distances);

/* Same with DEVICE pointers, enqueued on `stream` (a cudaStream_t; NULL = the
 * default stream) without synchronising.  Ids and map are range-checked on the
 * device: a bad entry writes NaN to its slot and the call still returns 0. */
int diskann_cuda_batch_distances_by_id_device(const diskann_cuda_table *table, const float *queries, int nq,
                                              const uint32_t *ids, const uint32_t *query_map, int total_n,
                                              int metric, float *out_distances, void *stream);

/* One batch of the call below: DEVICE pointers, same meaning as the arguments of
 * diskann_cuda_batch_distances_by_id_device. */
typedef struct diskann_cuda_batch {
    const float *queries;        /* nq x dim */
    const uint32_t *ids;         /* total_n row ids */
    const uint32_t *query_map;   /* total_n query numbers, NULL when nq == 1 */
    float *out_distances;        /* total_n results */
    int nq;
    int total_n;
} diskann_cuda_batch;

/* Several independent batches against one table in ONE launch (the batches of
 * concurrent searches, or the lock-step batches of several query groups,
 * rust_lib/src/disk_provider.rs:546-610).  A single batch of ~100 rows per query is
 * shorter than a few kernel-launch latencies; submitted together the batches fill
 * the GPU back to back and the kernel runs at its streaming rate.  `batches` is a
 * HOST array of `nbatches` descriptors holding device pointers; it is copied
 * during the call and may be reused on return.  Enqueued on `stream` without
 * synchronising; results and error behaviour per batch as for the single call.
 * No counterpart in the reference. */
int diskann_cuda_batch_distances_by_id_device_multi(const diskann_cuda_table *table, const diskann_cuda_batch *batches,
                                                    int nbatches, int metric, void *stream);

/* ---- serialized indexes -------------------------------------------------------------------
 * The reference stores a DiskANN index as the ".diskann" v2 image
 * (rust_lib/src/file_format.rs:3-18: 32-byte header "DANN", version 2, num_vectors,
 * dimension, max_degree, num_entry_points, metric u8 (0 = L2, 1 = IP), 3 pad bytes,
 * build_complexity; entry point ids; the fp32 vector segment; the u32 adjacency
 * segment; all little-endian), optionally followed by the SQ8 trailer
 * (rust_lib/src/index_manager.rs:513-533, read back at :629-668: "SQ8\0", dim u32,
 * qlen u64, min[dim] f32, scale[dim] f32, qlen code bytes).  The calls below take
 * such an image and put its vector segment (and its codes) on the device as tables
 * for the by-id entry points, so a persisted index can be searched without the
 * host gathering rows.  The graph (adjacency) stays with the caller. */
typedef struct diskann_cuda_index_info {
    uint32_t num_vectors, dimension, max_degree, num_entry_points, build_complexity;
    uint32_t metric;            /* 0 = L2, 1 = inner product */
    uint64_t entry_points_offset, vectors_offset, adjacency_offset;  /* byte offsets in the image */
    uint64_t standard_size;     /* bytes of the image up to the end of the adjacency segment */
    int has_sq8;                /* 1 when a well-formed SQ8 trailer follows */
    uint64_t sq8_min_offset, sq8_scale_offset, sq8_codes_offset, sq8_codes_size;
} diskann_cuda_index_info;

/* Validates the image and fills `info`.  Pure host code (no GPU needed).  -1 for a bad
 * magic / version, a truncated segment, a trailer whose dimension or length does not
 * match the header. */
int diskann_cuda_parse_index(const void *image, size_t len, diskann_cuda_index_info *info);

/* Parses and registers: `*vectors` gets the fp32 table; `*sq8` (may be NULL if the
 * caller does not want it) gets the SQ8 table, or NULL when the image has no trailer. */
int diskann_cuda_load_index(int device, const void *image, size_t len, diskann_cuda_index_info *info,
                            diskann_cuda_table **vectors, diskann_cuda_table **sq8);

/* Same, reading the image from a file. */
int diskann_cuda_load_index_file(int device, const char *path, diskann_cuda_index_info *info,
                                 diskann_cuda_table **vectors, diskann_cuda_table **sq8);

/* ---- the search loop that feeds the by-id entry points ------------------------------------
 * DiskProvider::search_batch (rust_lib/src/disk_provider.rs:470-652; the in-memory provider
 * has the same loop, rust_lib/src/provider.rs:333-427) over an image whose vectors were loaded
 * into GPU memory: every iteration each active query pops its best candidate and the unvisited
 * neighbours of all of them are scored by ONE by-id batch-distance call.  The reference's loop
 * gathers the neighbour rows on the host instead (:592-600); its Rust form cannot be compiled
 * here, so this C++ restatement is the caller the by-id path is tested and measured with.
 * The graph (adjacency, entry points) is copied out of the image and stays on the host. */
typedef struct diskann_cuda_searcher diskann_cuda_searcher;
const char *diskann_cuda_searcher_last_error(void);
/* use_sq8 != 0: score against the SQ8 codes of the image's trailer (asymmetric distance). */
int diskann_cuda_searcher_open(int device, const void *image, size_t len, int use_sq8, diskann_cuda_searcher **out);
void diskann_cuda_searcher_close(diskann_cuda_searcher *searcher);
int diskann_cuda_searcher_info(const diskann_cuda_searcher *searcher, diskann_cuda_index_info *info);
/* queries: nq x dim (host).  out_ids / out_distances: nq x k; out_counts[q] = results of query q
 * (min(k, rows reached)), best first; distances as the batch-distance ABI returns them (squared L2,
 * negated dot).  l_search is raised to k as in the reference (:486). */
int diskann_cuda_searcher_search_batch(diskann_cuda_searcher *searcher, const float *queries, int nq, int k, int l_search,
                                       uint64_t *out_ids, float *out_distances, int *out_counts);
/* Iterations, (query, row) pairs scored and batch-distance calls of the last search. */
int diskann_cuda_searcher_stats(const diskann_cuda_searcher *searcher, uint64_t *iterations, uint64_t *pairs_scored,
                                uint64_t *distance_calls);
/* With tracing on, a search records the id batch of every distance call; _trace returns the number
 * of batches and, when the arrays are given, copies ids / query_map (all batches back to back) and
 * offsets (batches + 1 entries).  The batches a real search produces, for workload generation. */
void diskann_cuda_searcher_set_trace(diskann_cuda_searcher *searcher, int on);
int64_t diskann_cuda_searcher_trace(const diskann_cuda_searcher *searcher, uint32_t *ids, uint32_t *query_map,
                                    uint64_t *offsets, int64_t max_pairs, int64_t max_batches);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* ANN_CUDA_DISKANN_BRIDGE_H */
