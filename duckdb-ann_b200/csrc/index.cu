// Index objects behind the C ABI of include/ann_cuda.h: device-resident Flat and
// IVFFlat indexes and their search drivers.
//
// Data layout in HBM (one GPU):
//   Flat      hi, lo : ntotal x dp fp32 each (TF32 split of every row, dp = d padded
//             to 32 floats), norms : ntotal fp32.  hi + lo is the original row, bit
//             for bit, so reconstruct() needs no third copy.
//   IVFFlat   centroids as a split store (nlist x dp) for the coarse quantiser;
//             vectors as hi / lo : ntotal x dp fp32 each, grouped by list (CSR:
//             list_off[nlist+1]), norms and ids (int64) : ntotal.  The reference keeps the lists in host vectors and
//             gathers them per query (faiss-metal/src/MetalIndexIVFFlat.mm:32-37,158-194);
//             here they never leave the device.
// Searches draw their scratch from a per-index pool of workspaces, one per
// concurrent caller, so `search` can run from many host threads at once
// (the reference's Metal index shares scratch without a lock,
// faiss-metal/src/MetalIndexFlat.mm:104-140).
#include "ann_cuda.h"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <memory>
#include <numeric>

#include "common.cuh"
#include "kernels.h"

using namespace anncuda;

namespace {

enum class FlatKernel { TC, SIMT };

std::atomic<int> g_flat_kernel{-1};  // -1 = not chosen yet
// one-MMA screening of the flat search: -1 = by store size, 0 = never, 1 = always (tests);
// ANN_CUDA_FLAT_SCREEN sets the initial value
std::atomic<uint64_t> g_screen_fallbacks{0};
std::atomic<int> g_flat_screen{[] {
    const char *e = getenv("ANN_CUDA_FLAT_SCREEN");
    return e ? (atoi(e) != 0 ? 1 : 0) : -1;
}()};
std::atomic<int> g_time_kernels{0};

FlatKernel flat_kernel_choice() {
    int v = g_flat_kernel.load(std::memory_order_relaxed);
    if (v < 0) {
        const char *e = getenv("ANN_CUDA_FLAT_KERNEL");
        v = (e && strcmp(e, "simt") == 0) ? 1 : 0;
        g_flat_kernel.store(v, std::memory_order_relaxed);
    }
    return v == 1 ? FlatKernel::SIMT : FlatKernel::TC;
}

// Split (hi/lo) row store that grows by doubling, at least 1024 rows at a time
// (the growth rule of faiss-metal/src/MetalIndexFlat.mm:255-270).
// A reduced-precision store (elem = kElemF16 / kElemBF16, the StorageType of
// faiss-metal/include/faiss-metal/MetalIndexFlat.h:38-43) keeps ONE plane of dp 16-bit elements per
// row behind `hi` (the rows rounded to that type; nothing else is kept of them) and no `lo`.
struct SplitStore {
    float *hi = nullptr, *lo = nullptr, *norms = nullptr;
    int64_t n = 0, cap = 0;
    int dp = 0;
    int elem = kElemF32;
    size_t row_bytes() const { return (size_t)dp * (elem == kElemF32 ? sizeof(float) : sizeof(uint16_t)); }
    // plane pointers `r` rows in (a row of a 16-bit store is half as long as the pointer type says)
    float *hi_at(int64_t r) const { return hi ? reinterpret_cast<float *>(reinterpret_cast<char *>(hi) + (size_t)r * row_bytes()) : nullptr; }
    float *lo_at(int64_t r) const { return lo ? reinterpret_cast<float *>(reinterpret_cast<char *>(lo) + (size_t)r * row_bytes()) : nullptr; }
    // L2 stores: a reference point near the data (mean of the first rows added).  norms hold
    // |x - mu|^2 and queries are searched as q - mu: distances are the same, the dot products
    // the tensor cores form are smaller, and so is their absolute error.  Fixed while n > 0.
    bool l2 = false;
    float *mu = nullptr;
    unsigned *max_norm2 = nullptr;  // device word: bits of the largest |x|^2 in the store

    int reserve(int64_t want) {
        if (want <= cap) return 0;
        float *nh = nullptr, *nl = nullptr, *nn = nullptr;
        const size_t row = row_bytes();
        const bool two = elem == kElemF32;
        if (cudaMalloc(&nh, (size_t)want * row) != cudaSuccess || (two && cudaMalloc(&nl, (size_t)want * row) != cudaSuccess) ||
            cudaMalloc(&nn, (size_t)want * sizeof(float)) != cudaSuccess) {
            cudaGetLastError();
            if (nh) cudaFree(nh);
            if (nl) cudaFree(nl);
            if (nn) cudaFree(nn);
            return set_error("out of device memory reserving %lld rows of %d floats (x2 for the TF32 split)",
                             (long long)want, dp);
        }
        if (n > 0) {
            ANN_CUDA_TRY(cudaMemcpy(nh, hi, (size_t)n * row, cudaMemcpyDeviceToDevice));
            if (two) ANN_CUDA_TRY(cudaMemcpy(nl, lo, (size_t)n * row, cudaMemcpyDeviceToDevice));
            ANN_CUDA_TRY(cudaMemcpy(nn, norms, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice));
        }
        release_buffers();
        hi = nh; lo = nl; norms = nn; cap = want;
        return 0;
    }
    int grow_for(int64_t extra) {
        if (n + extra <= cap) return 0;
        int64_t want = std::max<int64_t>(cap * 2, 1024);
        while (want < n + extra) want *= 2;
        return reserve(want);
    }
    // x: device rows (cnt x d)
    int append_device(const float *x, int64_t cnt, int d, cudaStream_t stream) {
        if (cnt <= 0) return 0;
        if (grow_for(cnt)) return -1;
        if (l2 && n == 0) {
            if (!mu) ANN_CUDA_TRY(cudaMalloc(&mu, (size_t)dp * sizeof(float)));
            if (launch_column_mean(x, std::min<int64_t>(cnt, 16384), d, mu, stream)) return -1;
        }
        if (!max_norm2) ANN_CUDA_TRY(cudaMalloc(&max_norm2, sizeof(unsigned)));
        if (n == 0) ANN_CUDA_TRY(cudaMemsetAsync(max_norm2, 0, sizeof(unsigned), stream));
        if (elem != kElemF32) {
            if (launch_split_rows_h16(x, cnt, d, dp, hi_at(n), nullptr, norms + n, stream,
                                      l2 ? mu : nullptr, false, max_norm2, elem, nullptr))
                return -1;
        } else if (launch_split_rows(x, cnt, d, dp, hi + n * dp, lo + n * dp, norms + n, stream, l2 ? mu : nullptr, false,
                                     max_norm2)) {
            return -1;
        }
        n += cnt;
        return 0;
    }
    const float *center() const { return l2 ? mu : nullptr; }
    void release_buffers() {
        if (hi) cudaFree(hi);
        if (lo) cudaFree(lo);
        if (norms) cudaFree(norms);
        hi = lo = norms = nullptr;
        cap = 0;
    }
    void release_all() {
        release_buffers();
        if (mu) cudaFree(mu);
        mu = nullptr;
        if (max_norm2) cudaFree(max_norm2);
        max_norm2 = nullptr;
    }
};

constexpr int kStatusWords = 8;
constexpr int kTiers = 4;
constexpr int kStatusWait = 0, kStatusTier0 = 1, kStatusFallbacks = kStatusTier0 + kTiers;
static_assert(kStatusFallbacks < kStatusWords, "status words");

struct Workspace {
    cudaStream_t own_stream = nullptr;
    cudaStream_t bound = nullptr;  // stream whose work may still use these buffers
    GrowBuf x, qhi, qlo, qn, part_key, part_idx, sel_key, sel_idx, status, out_d, out_i;
    GrowBuf item_q, item_rb, item_re, item_slot, scratch, probes_key, probes, qtau, sched, gq, items, qconst, part_cnt;
    // Flat tier chain: one word per query of the block, set by the band check of the latest tensor-core tier
    // for the queries it could not prove complete; the exact tier then repairs those queries only.
    GrowBuf over_q;
    GrowBuf bad_q;  // 16-bit stores: queries that overflow the type (set when the queries are split)
    GrowBuf complete_to;  // per query: key below which the merged candidates of several replace-max lists are complete
    // Exact tier, threshold scan of the flagged queries: the compacted list of them, each one's place in it, the
    // fill of its candidate buffer, the buffers, and the queries left for the item scan
    GrowBuf flag_aux, flag_rank, flag_counts, cand_key, cand_idx, left_q;
    bool over_q_valid = false;  // a tensor-core tier of the current block search has (been enqueued to) set them
    // Status words (device: `status`, pinned host copy: `status_host`), kStatusWords ints:
    //   [0]      first give-up code of a bounded wait inside a kernel; sticky for one API call
    //   [1 + t]  tier t of the flat search (see kTierScreen ...) found more rows inside its error band
    //            than it kept candidates for: kScreenOverflow; per query block
    //   [5]      how often a tier flagged such an overflow during the API call
    int *status_host = nullptr;  // pinned
    int fallbacks_seen = 0;      // part of status_host[4] already added to the process-wide counter
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;  // bracket the flat kernel when timing is on
    bool timed = false;
    void release() {
        if (ev0) cudaEventDestroy(ev0);
        if (ev1) cudaEventDestroy(ev1);
        for (GrowBuf *b : {&x, &qhi, &qlo, &qn, &part_key, &part_idx, &sel_key, &sel_idx, &status, &out_d, &out_i,
                           &item_q, &item_rb, &item_re, &item_slot, &scratch, &probes_key, &probes, &qtau, &sched, &gq, &items,
                           &qconst, &part_cnt, &over_q, &bad_q, &complete_to, &flag_aux, &flag_rank, &flag_counts, &cand_key,
                           &cand_idx, &left_q})
            b->release();
        if (status_host) cudaFreeHost(status_host);
        if (own_stream) cudaStreamDestroy(own_stream);
    }
};

}  // namespace

struct ann_cuda_index {
    int device = 0;
    int d = 0, dp = 0;
    int metric = ANN_CUDA_METRIC_L2;
    bool ivf = false;
    bool trained = true;
    int64_t ntotal = 0;

    SplitStore store;  // Flat: the database.  IVFFlat: the centroids.

    // IVFFlat
    int64_t nlist = 0, nprobe = 1;
    int shard_rank = 0, shard_count = 1;
    // Inverted-list rows, grouped by list: ONE plane of plain fp32 values (rows x dp) behind vhi.  The list
    // scan splits each row tile into its TF32 hi / lo parts in shared memory (GroupedWork::derive_lo), so a
    // row costs 4 bytes per element in memory and from DRAM, not 8.  vlo stays null.
    float *vhi = nullptr, *vlo = nullptr;
    float *vnorm = nullptr;                // rows: squared norms
    float *vrnorm = nullptr;               // rows: |x - centroid of its list|^2 (L2; rebuilt with the CSR form)
    int64_t vrnorm_cap = 0;
    int64_t *ids = nullptr;   // rows
    int64_t rows = 0, rows_cap = 0;
    std::vector<int32_t> row_list;  // list of every stored row, physical order (host)
    bool rows_sorted = true;        // physical order is already grouped by list
    bool coarse_exact = true;       // probe lists are re-ranked in exact fp32 (see ivf_update_coarse_policy)
    mutable bool csr_dirty = true;
    mutable int64_t *list_off = nullptr;  // device, nlist + 1
    mutable std::vector<int64_t> list_off_host;
    mutable std::mutex build_mu;

    mutable std::mutex ws_mu;
    mutable std::vector<Workspace *> ws_free;
    mutable Workspace *last_timed_ws = nullptr;

    Workspace *acquire_ws(cudaStream_t user_stream, bool internal) const {
        {
            std::lock_guard<std::mutex> lock(ws_mu);
            for (size_t i = 0; i < ws_free.size(); i++) {
                Workspace *w = ws_free[i];
                if (internal ? (w->bound == w->own_stream) : (w->bound == user_stream && w->bound != w->own_stream)) {
                    ws_free.erase(ws_free.begin() + i);
                    return w;
                }
            }
        }
        Workspace *w = new Workspace();
        if (cudaStreamCreateWithFlags(&w->own_stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaMallocHost(&w->status_host, kStatusWords * sizeof(int)) != cudaSuccess) {
            cudaGetLastError();
            w->release();
            delete w;
            set_error("could not create a search workspace");
            return nullptr;
        }
        memset(w->status_host, 0, kStatusWords * sizeof(int));
        w->bound = internal ? w->own_stream : user_stream;
        return w;
    }
    void release_ws(Workspace *w) const {
        std::lock_guard<std::mutex> lock(ws_mu);
        ws_free.push_back(w);
    }
};

namespace {

struct WsLease {
    const ann_cuda_index *idx;
    Workspace *ws;
    WsLease(const ann_cuda_index *i, cudaStream_t s, bool internal) : idx(i), ws(i->acquire_ws(s, internal)) {}
    ~WsLease() {
        if (ws) idx->release_ws(ws);
    }
};

constexpr int64_t kQueryBlock = 16384;  // queries per pass, bounds the scratch size
constexpr int64_t kScreenMinRows = 2000000;  // flat stores this large are searched with one-MMA screening

// ---- k-means helper kernels (index build, not the search path) -------------------------------
__global__ void kmeans_accumulate_kernel(const float *__restrict__ x, int64_t n, int d, const int32_t *__restrict__ assign,
                                         double *__restrict__ sums, int *__restrict__ counts) {
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n;
         r += (int64_t)gridDim.x * (blockDim.x >> 5)) {
        const int c = assign[r];
        if (c < 0) continue;
        if (lane == 0) atomicAdd(&counts[c], 1);
        // double sums: the order of the atomic adds then cannot change the rounded centroid, so
        // training gives the same lists on every run
        for (int j = lane; j < d; j += 32) atomicAdd(&sums[(int64_t)c * d + j], (double)x[r * (int64_t)d + j]);
    }
}
// k-means++-style seeding, one step: every point updates its squared distance to the
// nearest centre chosen so far (the newest is centre[step - 1]) and competes for being the
// next centre with score D^2 / E^(1/4), E ~ Exp(1) drawn from a hash of (seed, step, point).
// With E^1 the arg-max would be an exact draw with probability ~ D^2 (k-means++); the
// fourth root tempers the noise to a factor of about three, so a group of points that has no
// centre yet (D^2 orders of magnitude larger) always wins over groups that have one, and the
// last few uncovered groups are not left to a hub centroid.
__device__ __forceinline__ uint32_t hash32(uint32_t a) {
    a ^= a >> 16; a *= 0x7feb352du; a ^= a >> 15; a *= 0x846ca68bu; a ^= a >> 16;
    return a;
}
__global__ void kmeanspp_step_kernel(const float *__restrict__ x, int64_t n, int d, const float *__restrict__ newest,
                                     float *__restrict__ dmin, uint32_t seed, int step,
                                     unsigned long long *__restrict__ best) {
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n;
         r += (int64_t)gridDim.x * (blockDim.x >> 5)) {
        float acc = 0.f;
        for (int j = lane; j < d; j += 32) {
            const float t = x[r * (int64_t)d + j] - newest[j];
            acc = fmaf(t, t, acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            const float dm = step == 1 ? acc : fminf(dmin[r], acc);
            dmin[r] = dm;
            const uint32_t h = hash32(hash32((uint32_t)r ^ seed) + (uint32_t)step * 0x9E3779B9u);
            const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
            const float score = dm / sqrtf(sqrtf(-__logf(u)));
            if (score > 0.f)
                atomicMax(best, ((unsigned long long)__float_as_uint(score) << 32) | (unsigned long long)(uint32_t)r);
        }
    }
}
__global__ void kmeanspp_take_kernel(const float *__restrict__ x, int d, float *__restrict__ dst,
                                     unsigned long long *__restrict__ best) {
    const int64_t r = (int64_t)(*best & 0xffffffffull);
    for (int j = threadIdx.x; j < d; j += blockDim.x) dst[j] = x[r * (int64_t)d + j];
    __syncthreads();
    if (threadIdx.x == 0) *best = 0ull;
}
__global__ void kmeans_update_kernel(float *__restrict__ cent, const double *__restrict__ sums,
                                     const int *__restrict__ counts, int64_t nlist, int d) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nlist * d) return;
    const int c = (int)(t / d);
    if (counts[c] > 0) cent[t] = (float)(sums[t] / (double)counts[c]);  // an empty cluster keeps its centroid
}
__global__ void gather_rows_kernel(const float *__restrict__ shi, const float *__restrict__ slo,
                                   const float *__restrict__ snorm, const int64_t *__restrict__ src_ids,
                                   const int64_t *__restrict__ perm, int64_t n, int dp, float *__restrict__ dhi,
                                   float *__restrict__ dlo, float *__restrict__ dnorm, int64_t *__restrict__ dst_ids) {
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n;
         r += (int64_t)gridDim.x * (blockDim.x >> 5)) {
        const int64_t s = perm[r];
        for (int c = lane; c < dp; c += 32) {
            dhi[r * (int64_t)dp + c] = shi[s * (int64_t)dp + c];
            if (slo) dlo[r * (int64_t)dp + c] = slo[s * (int64_t)dp + c];
        }
        if (lane == 0) {
            dst_ids[r] = src_ids[s];
            dnorm[r] = snorm[s];
        }
    }
}
__global__ void find_id_kernel(const int64_t *__restrict__ ids, int64_t n, int64_t key, long long *found) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n && ids[t] == key) atomicMin(found, (long long)t);
}

// ---- status words -----------------------------------------------------------------------------------
int ws_status_ready(Workspace &ws) {
    if (ws.status.ensure(kStatusWords * sizeof(int))) return -1;
    return 0;
}
// All status words to zero, in stream order.
int ws_clear_status(Workspace &ws, cudaStream_t stream) {
    if (ws_status_ready(ws)) return -1;
    ANN_CUDA_TRY(cudaMemsetAsync(ws.status.ptr, 0, kStatusWords * sizeof(int), stream));
    return 0;
}
int ws_publish_status(Workspace &ws, cudaStream_t stream) {
    ANN_CUDA_TRY(cudaMemcpyAsync(ws.status_host, ws.status.ptr, kStatusWords * sizeof(int), cudaMemcpyDeviceToHost, stream));
    return 0;
}
// Adds the overflows the device counted since the last look to the process-wide counter.  Only
// meaningful after the stream has been synchronised.
void ws_absorb_fallbacks(Workspace &ws) {
    const int seen = ws.status_host[kStatusFallbacks];
    if (seen > ws.fallbacks_seen) g_screen_fallbacks.fetch_add((uint64_t)(seen - ws.fallbacks_seen), std::memory_order_relaxed);
    ws.fallbacks_seen = seen;
}

// ---- top-k over a split store (flat database, or IVF centroids) ---------------------------------
struct TopkOpts {
    int k_rank = 0;      // > 0: banded lists - the kernel keeps the (at most k) candidates that the error slack
                         // of its keys cannot rule out of the best k_rank (see ScreenInput)
    bool one_mma = false;  // with k_rank: one-MMA keys (screened search); else the split product
    int check_rank = 0;  // > 0: band check - is the last of the k candidates beyond the slack above the
                         // check_rank-th?  If not, status word kStatusTier0 + tier becomes kScreenOverflow
    int tier = 0;
    bool exact = false;  // exact-fp32 scan instead of the tensor cores
    const int *gate = nullptr;  // device word: run only if it holds kScreenOverflow (a fallback pass)
    // a pass of a tier chain (flat_tier_search): the queries were split by the first pass, the band check runs
    // inside the re-ranking kernel that follows, and the caller publishes the status words once at the end
    bool chained = false;
    // exact tier: repair only the queries whose word in ws.over_q is set (the others keep their results)
    bool flagged_only = false;
    // with flagged_only: what the tier before left for every query of the block (prev_k per query, user-facing
    // distances and labels) - its k-th distance bounds the true one
    const float *prev_d = nullptr;
    const int64_t *prev_i = nullptr;
    int prev_k = 0;
    // replace-max lists (k beyond the append lists): the merge may hand on more candidates than one list is
    // long - up to this many - with the bound below which they are complete in ws.complete_to; *wide_used
    // receives the number of candidates per query that came out (k if the selection has no such lists)
    int wide_out = 0;
    int *wide_used = nullptr;
};
// x_dev: nq x d queries on the device.  Leaves (nq x k) keys and int32 rows, best
// first, in ws.sel_key / ws.sel_idx.  The status words must have been cleared by the caller.
int split_store_topk(const ann_cuda_index &ix, const SplitStore &st, Workspace &ws, const float *x_dev, int64_t nq,
                     int k, cudaStream_t stream, const TopkOpts &o = TopkOpts()) {
    const int dp = st.dp, d = ix.d;
    const size_t k_buf = (size_t)std::max(k, o.wide_out);
    // the kernel loads the query planes in whole tiles (one more when it pairs up an odd number of tiles)
    const size_t nq_rows = ((size_t)(nq + 127) / 128 + 1) * 128;
    if (ws.qhi.ensure(nq_rows * dp * 4) || ws.qlo.ensure(nq_rows * dp * 4) || ws.qn.ensure((size_t)nq * 4) ||
        ws.sel_key.ensure((size_t)nq * k_buf * 4) || ws.sel_idx.ensure((size_t)nq * k_buf * 4) || ws_status_ready(ws))
        return -1;
    if (o.wide_used) *o.wide_used = k;
    int *status = ws.status.as<int>();
    if (!o.exact && flat_kernel_choice() == FlatKernel::TC) {
        // the split of the queries is the same in every tier: a gated fallback pass finds it in place
        // (16-bit store: the two 16-bit parts of q - mu; a query element that overflows the type flags both
        // tensor-core tiers, which sends the block to the exact scan)
        if (st.elem != kElemF32 && (!o.chained || o.k_rank <= 0))
            return set_error("internal: a 16-bit store is searched with banded lists through the tier chain only");
        if (!(o.chained && o.gate) &&
            (st.elem != kElemF32
                 ? launch_split_rows_h16(x_dev, nq, d, dp, ws.qhi.ptr, ws.qlo.ptr, ws.qn.as<float>(), stream, st.center(), true,
                                         nullptr, st.elem, status + kStatusTier0, ws.bad_q.as<int32_t>())
                 : launch_split_rows(x_dev, nq, d, dp, ws.qhi.as<float>(), ws.qlo.as<float>(), ws.qn.as<float>(), stream,
                                     st.center(), true)))
            return -1;
        // (the static schedule and the pair mode serve the one-MMA tiers and, for 16-bit stores, the two-part tier)
        const FlatPlan plan = o.k_rank > 0 && (o.one_mma || st.elem != kElemF32)
                                  ? make_flat_plan_screened(nq, st.n, k, sm_count(ix.device))
                                  : make_flat_plan(nq, st.n, k, sm_count(ix.device));
        const ScreenInput screen{o.k_rank, ws.qn.as<float>(), st.max_norm2, d, o.one_mma, st.elem};
        const size_t qtau_bytes = (size_t)plan.nq_tiles * 128 * 4, sched_bytes = plan.sched_ints * 4;
        if (ws.part_key.ensure(plan.part_entries * 4) || ws.part_idx.ensure(plan.part_entries * 4) ||
            ws.qtau.ensure(qtau_bytes) || ws.sched.ensure(sched_bytes))
            return -1;
        // Thresholds "none yet", scheduler memory zero.  Append selection: a list is the first part_cnt
        // entries of its row's buffer, unsorted - every list empty means every count zero.  Other
        // selections: index -1 in the k slots the merge reads.  One kernel, gated like the pass.
        const bool append = plan.lists_sorted;
        const size_t cnt_words = (size_t)plan.nq_tiles * plan.lists_per_qt * 128;
        if (append && ws.part_cnt.ensure(cnt_words * 4)) return -1;
        if (launch_flat_scratch_init(ws.qtau.as<uint32_t>(), qtau_bytes / 4, ws.sched.as<int>(), plan.sched_ints,
                                     append ? ws.part_cnt.as<int32_t>() : nullptr, cnt_words,
                                     append ? nullptr : ws.part_idx.as<int32_t>(), plan.part_entries / plan.list_stride,
                                     plan.list_stride, k, stream, o.gate, o.chained ? ws.over_q.as<int32_t>() : nullptr, (size_t)nq))
            return -1;
        const bool timing = !o.gate && g_time_kernels.load(std::memory_order_relaxed) != 0;
        if (timing) {
            if (!ws.ev0) {
                ANN_CUDA_TRY(cudaEventCreate(&ws.ev0));
                ANN_CUDA_TRY(cudaEventCreate(&ws.ev1));
            }
            ANN_CUDA_TRY(cudaEventRecord(ws.ev0, stream));
        }
        if (st.elem != kElemF32
                ? launch_flat_tc_h16(plan, st.hi, nullptr, st.norms, st.n, ws.qhi.as<float>(), ws.qlo.as<float>(), nq, dp, k,
                                     ix.metric, ws.part_key.as<float>(), ws.part_idx.as<int32_t>(), ws.qtau.as<uint32_t>(),
                                     ws.sched.as<int>(), status + kStatusWait, ix.device, stream, nullptr, &screen, o.gate,
                                     append ? ws.part_cnt.as<int32_t>() : nullptr)
                : launch_flat_tc(plan, st.hi, st.lo, st.norms, st.n, ws.qhi.as<float>(), ws.qlo.as<float>(), nq, dp, k,
                                 ix.metric, ws.part_key.as<float>(), ws.part_idx.as<int32_t>(), ws.qtau.as<uint32_t>(),
                                 ws.sched.as<int>(), status + kStatusWait, ix.device, stream, nullptr,
                                 o.k_rank > 0 ? &screen : nullptr, o.gate, append ? ws.part_cnt.as<int32_t>() : nullptr))
            return -1;
        if (timing) {
            ANN_CUDA_TRY(cudaEventRecord(ws.ev1, stream));
            ws.timed = true;
            ix.last_timed_ws = &ws;
        }
        // per query: the lists of its query tile, filtered by the query's final threshold, sorted once
        // (lists in shared memory, k <= 16: whole lists of k slots, no fill counts; the per-query threshold word
        // holds the smallest "largest key of a full list", above which nothing can be among the k best)
        const bool small_lists = !append && k <= kSmemListMax;
        if ((append || small_lists)
                ? launch_merge_filtered(ws.part_key.as<float>(), ws.part_idx.as<int32_t>(),
                                           append ? ws.part_cnt.as<int32_t>() : nullptr, nullptr,
                                           nullptr, ws.qtau.as<uint32_t>(), plan.lists_per_qt, nq, k, plan.list_stride,
                                           ws.sel_key.as<float>(), ws.sel_idx.as<int32_t>(), stream,
                                           ws.sched.as<int>() + plan.nq_tiles, o.gate)
                   : [&] {
                         // several replace-max lists per query: their union holds more than one list's length
                         int k_out = 0;
                         float *complete_to = nullptr;
                         if (o.wide_out > k && o.wide_used && plan.lists_per_qt > 1 && plan.lists_per_qt <= 32 &&
                             !ws.complete_to.ensure((size_t)nq * 4)) {
                             k_out = (int)std::min<int64_t>(o.wide_out, (int64_t)plan.lists_per_qt * k);
                             complete_to = ws.complete_to.as<float>();
                             *o.wide_used = k_out;
                         }
                         return launch_merge_parts(ws.part_key.as<float>(), ws.part_idx.as<int32_t>(), 0,
                                                   ws.sched.as<int>() + plan.nq_tiles, nullptr, plan.lists_per_qt, nq, k,
                                                   plan.list_stride, ws.sel_key.as<float>(), ws.sel_idx.as<int32_t>(), ix.device,
                                                   stream, false, nullptr, o.gate, nullptr, k_out, complete_to);
                     }())
            return -1;
        // (a list that holds every row of the store has left nothing out)
        if (!o.chained && o.check_rank > 0 && k < st.n &&
            launch_screen_check(ws.sel_key.as<float>(), nq, k, o.check_rank, ws.qn.as<float>(), st.max_norm2, d, ix.metric,
                                o.k_rank > 0 && o.one_mma, status + kStatusTier0 + o.tier, status + kStatusFallbacks, stream,
                                o.gate))
            return -1;
        return o.chained ? 0 : ws_publish_status(ws, stream);
    }
    // exact-fp32 scan: items = (query, database chunk), laid out on the device
    // (all queries: enough items to fill the device; flagged queries only: nobody knows here how many there are,
    // so every query is cut into as many chunks as the merge takes and the scratch allows - one hard query
    // among thousands is then still scanned by dozens of warps)
    const int64_t fill = (int64_t)sm_count(ix.device) * 32 / std::max<int64_t>(nq, 1) + 1;
    const int64_t wide = std::max<int64_t>(fill, (int64_t)(16 << 20) / std::max<int64_t>(nq * k, 1));
    int chunks = (int)std::max<int64_t>(1, std::min<int64_t>({(int64_t)kMergeCandidates / k, (st.n + 255) / 256,
                                                             o.flagged_only ? wide : fill}));
    const int32_t *only_q = o.flagged_only ? ws.over_q.as<int32_t>() : nullptr;
    const int64_t per = (st.n + chunks - 1) / chunks;
    chunks = (int)((st.n + per - 1) / per);
    const int64_t n_items = nq * chunks;
    if (ws.item_q.ensure(n_items * 4) || ws.item_rb.ensure(n_items * 8) || ws.item_re.ensure(n_items * 8) ||
        ws.part_key.ensure((size_t)n_items * k * 4) || ws.part_idx.ensure((size_t)n_items * k * 4))
        return -1;
    // Flagged queries first get one pass over the store that keeps the rows at or below the k-th distance
    // the tier before found (work cut by rows: a single hard query is scanned by the whole device); the item
    // scan below then runs for the queries that pass could not settle - normally none.
    bool items_laid_out = false;
    if (o.flagged_only && o.prev_d && o.prev_i && st.max_norm2 && st.n <= (int64_t)0x7fffffff &&
        scan_flagged_group(dp) > 0) {
        const int lists = std::max(2, kFlaggedCandidates / k);
        const int cap = lists * k;
        const int r_max = (int)std::max<int64_t>(1, std::min<int64_t>(nq, kFlaggedEntries / cap));
        if (cap <= kMergeCandidates) {
            if (ws.flag_aux.ensure((size_t)(nq + 1) * 4) || ws.flag_rank.ensure((size_t)nq * 4) ||
                ws.flag_counts.ensure((size_t)r_max * 4) || ws.left_q.ensure((size_t)nq * 4) ||
                ws.cand_key.ensure((size_t)r_max * cap * 4) || ws.cand_idx.ensure((size_t)r_max * cap * 4))
                return -1;
            if (launch_scan_flagged(st.hi, st.lo, dp, d, st.n, x_dev, d, only_q, nq, ws.flag_aux.as<int>(),
                                    ws.flag_rank.as<int32_t>(), ws.flag_counts.as<int>(), r_max, cap, o.prev_k,
                                    (int)std::min<int64_t>(o.prev_k, st.n) - 1, o.prev_d, o.prev_i, st.max_norm2, ix.metric,
                                    ws.cand_key.as<float>(), ws.cand_idx.as<int32_t>(), ix.device, stream, o.gate, st.elem) ||
                launch_select_flagged(ws.cand_key.as<float>(), ws.cand_idx.as<int32_t>(), ws.flag_counts.as<int>(),
                                      ws.flag_rank.as<int32_t>(), only_q, r_max, cap, nq, k, ws.sel_key.as<float>(),
                                      ws.sel_idx.as<int32_t>(), ws.left_q.as<int32_t>(), ws.item_q.as<int32_t>(),
                                      ws.item_rb.as<int64_t>(), ws.item_re.as<int64_t>(), chunks, per, st.n, stream, o.gate))
                return -1;
            only_q = ws.left_q.as<int32_t>();
            items_laid_out = true;  // (by the kernel that decided which queries are left)
        }
    }
    if (!items_laid_out && launch_fill_chunk_items(ws.item_q.as<int32_t>(), ws.item_rb.as<int64_t>(), ws.item_re.as<int64_t>(),
                                                   nq, chunks, per, st.n, stream, only_q))
        return -1;
    if (launch_scan_items(st.hi, st.lo, dp, d, x_dev, d, ws.item_q.as<int32_t>(), ws.item_rb.as<int64_t>(),
                          ws.item_re.as<int64_t>(), n_items, k, ix.metric, ws.part_key.as<float>(),
                          ws.part_idx.as<int32_t>(), nullptr, ix.device, stream, o.gate, st.elem))
        return -1;
    if (launch_merge_parts(ws.part_key.as<float>(), ws.part_idx.as<int32_t>(), 1, nullptr, nullptr, chunks, nq, k, k,
                           ws.sel_key.as<float>(), ws.sel_idx.as<int32_t>(), ix.device, stream, false, nullptr, o.gate, only_q))
        return -1;
    return o.chained ? 0 : ws_publish_status(ws, stream);
}

// Allocates the four row arrays of an IVF store for `cap` rows (all or nothing).
int ivf_alloc_rows(int64_t cap, int dp, float **hi, float **lo, float **norm, int64_t **ids) {
    *hi = *lo = *norm = nullptr;
    *ids = nullptr;
    if (cudaMalloc(hi, (size_t)cap * dp * 4) != cudaSuccess || cudaMalloc(norm, (size_t)cap * 4) != cudaSuccess ||
        cudaMalloc(ids, (size_t)cap * 8) != cudaSuccess) {
        cudaGetLastError();
        for (void *p : {(void *)*hi, (void *)*norm, (void *)*ids})
            if (p) cudaFree(p);
        *hi = *norm = nullptr;
        *ids = nullptr;
        return set_error("out of device memory for %lld inverted-list rows of %d floats", (long long)cap, dp);
    }
    return 0;
}
void ivf_free_rows(ann_cuda_index &ix) {
    for (void *p : {(void *)ix.vhi, (void *)ix.vlo, (void *)ix.vnorm, (void *)ix.ids})
        if (p) cudaFree(p);
    ix.vhi = ix.vlo = ix.vnorm = nullptr;
    ix.ids = nullptr;
    if (ix.vrnorm) cudaFree(ix.vrnorm);
    ix.vrnorm = nullptr;
    ix.vrnorm_cap = 0;
}

// ---- IVF: (re)build the CSR form after adds ------------------------------------------------------
int ivf_finalize_lists(const ann_cuda_index &cix) {
    std::lock_guard<std::mutex> lock(cix.build_mu);
    if (!cix.csr_dirty) return 0;
    ann_cuda_index &ix = const_cast<ann_cuda_index &>(cix);
    const int64_t n = ix.rows;
    std::vector<int64_t> off((size_t)ix.nlist + 1, 0);
    for (int64_t i = 0; i < n; i++) off[(size_t)ix.row_list[i] + 1]++;
    for (int64_t l = 0; l < ix.nlist; l++) off[l + 1] += off[l];
    if (!ix.rows_sorted && n > 0) {
        // stable counting sort by list: rows keep their add order inside a list
        std::vector<int64_t> cursor(off.begin(), off.end() - 1), perm((size_t)n);
        for (int64_t i = 0; i < n; i++) perm[(size_t)cursor[ix.row_list[i]]++] = i;
        float *nh = nullptr, *nl = nullptr, *nn = nullptr;
        int64_t *ni = nullptr, *dperm = nullptr;
        const int64_t cap = std::max<int64_t>(n, 1);
        if (ivf_alloc_rows(cap, ix.dp, &nh, &nl, &nn, &ni)) return -1;
        if (cudaMalloc(&dperm, (size_t)n * 8) != cudaSuccess) {
            cudaGetLastError();
            for (void *p : {(void *)nh, (void *)nn, (void *)ni}) cudaFree(p);
            return set_error("out of device memory regrouping the inverted lists");
        }
        ANN_CUDA_TRY(cudaMemcpy(dperm, perm.data(), (size_t)n * 8, cudaMemcpyHostToDevice));
        gather_rows_kernel<<<(unsigned)std::min<int64_t>((n + 7) / 8, (int64_t)sm_count(ix.device) * 32), 256>>>(
            ix.vhi, ix.vlo, ix.vnorm, ix.ids, dperm, n, ix.dp, nh, nl, nn, ni);
        count_launch();
        ANN_CUDA_TRY(cudaGetLastError());
        ANN_CUDA_TRY(cudaDeviceSynchronize());
        cudaFree(dperm);
        ivf_free_rows(ix);
        ix.vhi = nh;
        ix.vlo = nl;
        ix.vnorm = nn;
        ix.ids = ni;
        ix.rows_cap = cap;
        std::vector<int32_t> sorted_list((size_t)n);
        for (int64_t i = 0; i < n; i++) sorted_list[i] = ix.row_list[perm[i]];
        ix.row_list.swap(sorted_list);
        ix.rows_sorted = true;
    }
    if (!ix.list_off) ANN_CUDA_TRY(cudaMalloc(&ix.list_off, (size_t)(ix.nlist + 1) * 8));
    ANN_CUDA_TRY(cudaMemcpy(ix.list_off, off.data(), (size_t)(ix.nlist + 1) * 8, cudaMemcpyHostToDevice));
    ix.list_off_host.swap(off);
    if (ix.metric != 0 && n > 0) {
        // L2: the list scan works with query residuals against the list centroid and needs
        // |x - c|^2 of every row in place of |x|^2
        if (ix.vrnorm_cap < n) {
            if (ix.vrnorm) cudaFree(ix.vrnorm);
            ix.vrnorm = nullptr;
            ix.vrnorm_cap = 0;
            ANN_CUDA_TRY(cudaMalloc(&ix.vrnorm, (size_t)ix.rows_cap * 4));
            ix.vrnorm_cap = ix.rows_cap;
        }
        if (launch_residual_norms(ix.vhi, ix.vlo, n, ix.d, ix.dp, ix.list_off, (int)ix.nlist, ix.store.hi, ix.store.lo,
                                  ix.vrnorm, nullptr))
            return -1;
        ANN_CUDA_TRY(cudaDeviceSynchronize());
    }
    ix.csr_dirty = false;
    return 0;
}

int ivf_grow_rows(ann_cuda_index &ix, int64_t extra) {
    if (ix.rows + extra <= ix.rows_cap) return 0;
    int64_t want = std::max<int64_t>(ix.rows_cap * 2, 1024);
    while (want < ix.rows + extra) want *= 2;
    float *nh = nullptr, *nl = nullptr, *nn = nullptr;
    int64_t *ni = nullptr;
    if (ivf_alloc_rows(want, ix.dp, &nh, &nl, &nn, &ni)) return -1;
    if (ix.rows > 0) {
        ANN_CUDA_TRY(cudaMemcpy(nh, ix.vhi, (size_t)ix.rows * ix.dp * 4, cudaMemcpyDeviceToDevice));
        ANN_CUDA_TRY(cudaMemcpy(nn, ix.vnorm, (size_t)ix.rows * 4, cudaMemcpyDeviceToDevice));
        ANN_CUDA_TRY(cudaMemcpy(ni, ix.ids, (size_t)ix.rows * 8, cudaMemcpyDeviceToDevice));
    }
    ivf_free_rows(ix);
    ix.vhi = nh;
    ix.vlo = nl;
    ix.vnorm = nn;
    ix.ids = ni;
    ix.rows_cap = want;
    return 0;
}

bool ivf_owns(const ann_cuda_index &ix, int64_t list_no) { return list_no % ix.shard_count == ix.shard_rank; }

// ---- coarse quantiser -----------------------------------------------------------------------------
// The nprobe nearest centroids of every query, best first, as int32 list numbers in `probes`
// (device, nq x nprobe).  The tensor-core pass selects a few more candidates than asked for and
// they are re-ranked by their exact fp32 distance: centroids of neighbouring cells can differ by
// less than the split-TF32 error of the first pass, and a wrong probe list loses whole lists.
constexpr int kCoarseMargin = 8;
constexpr int kSelectMargin = 8;
int coarse_probes(const ann_cuda_index &ix, Workspace &ws, const float *x_dev, int64_t nq, int nprobe,
                  int32_t *probes, cudaStream_t stream, bool exact) {
    if (!exact) {
        if (split_store_topk(ix, ix.store, ws, x_dev, nq, nprobe, stream)) return -1;
        ANN_CUDA_TRY(cudaMemcpyAsync(probes, ws.sel_idx.ptr, (size_t)nq * nprobe * 4, cudaMemcpyDeviceToDevice, stream));
        return 0;
    }
    const int k_c = (int)std::min<int64_t>(ix.nlist, (int64_t)nprobe + kCoarseMargin);
    if (split_store_topk(ix, ix.store, ws, x_dev, nq, k_c, stream)) return -1;
    return launch_refine_finalize(ix.store.hi, ix.store.lo, ix.dp, ix.d, x_dev, ix.d, ws.sel_idx.as<int32_t>(), nq, k_c,
                                  nprobe, ix.metric, nullptr, 0, nullptr, nullptr, ix.device, stream, nullptr, nullptr,
                                  nullptr, probes);
}

// Decides whether the tensor-core ranking of the centroids may pick the probe lists by itself.
// Its keys are off by up to ~2^-20 |q - mu| |c| (mu = the centroid store's reference point); that
// is harmless when it is far below the spacing of the centroids, and wrong lists otherwise
// (several centroids inside one tight cluster far from the origin).  The spacing is taken as
// the smallest exact distance between two centroids, |q - mu| as twice the largest |c - mu|.
int ivf_update_coarse_policy(ann_cuda_index &ix) {
    ix.coarse_exact = true;
    if (ix.metric == 0 || ix.nlist < 2 || ix.store.n != ix.nlist) {
        ix.coarse_exact = ix.metric != 0 && ix.nlist >= 2;  // inner product: no cancellation to guard against
        return 0;
    }
    const int64_t nl = ix.nlist;
    float *rows = nullptr;
    ANN_CUDA_TRY(cudaMalloc(&rows, (size_t)nl * ix.d * 4));
    int rc = 0;
    std::vector<float> d2((size_t)nl * 2), norms((size_t)nl), mu((size_t)ix.dp, 0.f);
    {
        WsLease lease(&ix, nullptr, true);
        if (!lease.ws) {
            cudaFree(rows);
            return -1;
        }
        Workspace &ws = *lease.ws;
        cudaStream_t s = ws.own_stream;
        rc = launch_join_rows(ix.store.hi, ix.store.lo, nl, ix.d, ix.dp, rows, s);
        for (int64_t q0 = 0; q0 < nl && rc == 0; q0 += kQueryBlock) {
            const int64_t nb = std::min(kQueryBlock, nl - q0);
            if (ws.out_d.ensure((size_t)nb * 2 * 4) || ws.out_i.ensure((size_t)nb * 2 * 8)) rc = -1;
            if (rc == 0) rc = ws_clear_status(ws, s);
            if (rc == 0) rc = split_store_topk(ix, ix.store, ws, rows + q0 * ix.d, nb, 2, s);
            if (rc == 0)
                rc = launch_refine_finalize(ix.store.hi, ix.store.lo, ix.dp, ix.d, rows + q0 * ix.d, ix.d,
                                            ws.sel_idx.as<int32_t>(), nb, 2, 2, ix.metric, nullptr, 0, ws.out_d.as<float>(),
                                            ws.out_i.as<int64_t>(), ix.device, s);
            if (rc == 0 && cudaMemcpyAsync(d2.data() + q0 * 2, ws.out_d.ptr, (size_t)nb * 2 * 4, cudaMemcpyDeviceToHost, s) !=
                               cudaSuccess)
                rc = set_error("copy failed");
            if (rc == 0 && cudaStreamSynchronize(s) != cudaSuccess) rc = set_error("device error ranking the centroids");
        }
    }
    if (rc == 0 && (cudaMemcpy(norms.data(), ix.store.norms, (size_t)nl * 4, cudaMemcpyDeviceToHost) != cudaSuccess ||
                    (ix.store.center() &&
                     cudaMemcpy(mu.data(), ix.store.center(), (size_t)ix.dp * 4, cudaMemcpyDeviceToHost) != cudaSuccess)))
        rc = set_error("copy failed");
    cudaFree(rows);
    if (rc) return -1;
    double gap = INFINITY, r2 = 0, mu2 = 0;
    for (int64_t i = 0; i < nl; i++) {
        gap = std::min<double>(gap, std::max(d2[i * 2 + 1], 0.f));
        r2 = std::max<double>(r2, norms[i]);
    }
    for (int j = 0; j < ix.d; j++) mu2 += (double)mu[j] * mu[j];
    const double r = std::sqrt(r2), cmax = r + std::sqrt(mu2);
    const double err = std::ldexp(1.0, -20) * 2.0 * r * cmax;
    ix.coarse_exact = !(err <= 2.5e-5 * gap);
    return 0;
}

// Nearest centroid of n device rows -> host vector.
int ivf_assign_device(const ann_cuda_index &ix, const float *x_dev, int64_t n, std::vector<int32_t> &assign,
                      bool exact) {
    assign.resize((size_t)n);
    WsLease lease(&ix, nullptr, true);
    if (!lease.ws) return -1;
    Workspace &ws = *lease.ws;
    cudaStream_t s = ws.own_stream;
    for (int64_t q0 = 0; q0 < n; q0 += kQueryBlock) {
        const int64_t nb = std::min(kQueryBlock, n - q0);
        if (ws.probes.ensure((size_t)nb * 4) || ws_clear_status(ws, s)) return -1;
        if (coarse_probes(ix, ws, x_dev + q0 * ix.d, nb, 1, ws.probes.as<int32_t>(), s, exact)) return -1;
        ANN_CUDA_TRY(cudaMemcpyAsync(assign.data() + q0, ws.probes.ptr, (size_t)nb * 4, cudaMemcpyDeviceToHost, s));
        ANN_CUDA_TRY(cudaStreamSynchronize(s));
        if (ws.status_host[kStatusWait])
            return set_error("flat kernel gave up on a wait (code %d)", ws.status_host[kStatusWait]);
    }
    return 0;
}

// Appends rows (device, n x d) with known lists and labels.
int ivf_append(ann_cuda_index &ix, const float *x_dev, int64_t n, const int32_t *lists, const int64_t *labels) {
    std::vector<int64_t> dst((size_t)n), kept_ids;
    int64_t kept = 0;
    for (int64_t i = 0; i < n; i++) {
        if (lists[i] >= 0 && lists[i] < ix.nlist && ivf_owns(ix, lists[i])) {
            dst[i] = ix.rows + kept++;
        } else {
            dst[i] = -1;
        }
    }
    if (kept == 0) return 0;
    if (ivf_grow_rows(ix, kept)) return -1;
    kept_ids.reserve((size_t)kept);
    for (int64_t i = 0; i < n; i++)
        if (dst[i] >= 0) kept_ids.push_back(labels[i]);
    int64_t *ddst = nullptr;
    ANN_CUDA_TRY(cudaMalloc(&ddst, (size_t)n * 8));
    cudaError_t e = cudaMemcpy(ddst, dst.data(), (size_t)n * 8, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(ix.ids + ix.rows, kept_ids.data(), (size_t)kept * 8, cudaMemcpyHostToDevice);
    int rc = 0;
    if (e == cudaSuccess) rc = launch_scatter_rows(x_dev, n, ix.d, ix.dp, ddst, ix.vhi, ix.vlo, ix.vnorm, nullptr);
    if (e == cudaSuccess && rc == 0) e = cudaDeviceSynchronize();
    cudaFree(ddst);
    if (e != cudaSuccess) return set_error("appending rows failed: %s", cudaGetErrorString(e));
    if (rc) return -1;
    // the host-side list of every stored row grows only now that the rows are in place: a failed
    // append leaves row_list as long as ix.rows
    for (int64_t i = 0; i < n; i++) {
        if (dst[i] < 0) continue;
        if (!ix.row_list.empty() && lists[i] < ix.row_list.back()) ix.rows_sorted = false;
        ix.row_list.push_back(lists[i]);
    }
    ix.rows += kept;
    ix.csr_dirty = true;
    return 0;
}

int ensure_device(const ann_cuda_index *ix, DeviceGuard &g) {
    if (!g.ok) return set_error("cudaSetDevice(%d) failed", ix->device);
    return 0;
}

// ---- flat search: tiers ---------------------------------------------------------------------------
// A flat search runs in up to four tiers, each exact within its own proof:
//   0  screened    one-MMA keys; lists of up to kScreenMaxList candidates pruned by the k-th key plus
//                  the one-MMA error slack (stores of kScreenMinRows rows and more, k <= kScreenMaxK);
//   1  split       three-MMA keys.  k <= 12: the 16 best in shared memory.  k <= kScreenMaxK: the same
//                  banded lists of up to kScreenMaxList candidates, under the much smaller slack of the
//                  split product.  Larger k: the k + kSplitSpare best;
//   2  split-wide  (only after a 16-list of tier 1) banded lists of tier 1's second form;
//   3  exact       direct-form fp32 scan (scan_items_kernel), no tensor cores.
// Tiers 0-2 end with the band check of key_slack: if the last candidate of some query is still
// within the slack above the k-th, rows that belong among the exact k best may be missing and the
// tier's overflow word is set; the block is then searched again one tier up.  All tiers re-rank
// their candidates by the exact fp32 distance, so the answer never depends on the tier.
enum { kTierScreen = 0, kTierSplit = 1, kTierSplitWide = 2, kTierExact = 3 };
static_assert(kTierExact == kTiers - 1, "tier count");

// Banded lists are append buffers: they need a store of more rows than the shared-memory lists hold
// (a smaller store fits a list whole and needs no band at all).
bool banded_lists_fit(const ann_cuda_index &ix, int k_sel) {
    return k_sel <= kScreenMaxK && ix.store.max_norm2 &&
           std::min<int64_t>(kScreenMaxList, ix.store.n) > std::max(k_sel, kSmemListMax);
}

int flat_first_tier(const ann_cuda_index &ix, int k_sel) {
    if (flat_kernel_choice() != FlatKernel::TC) return kTierExact;
    // 16-bit store: one 16-bit part of the query per product, then two, then the exact scan - always
    // with banded lists (stores too small for them, and k beyond them, are scanned exactly)
    // (bf16 rounds a query element to 8 bits: the band of a single part is eight times as wide as fp16's and
    // holds more rows than a list keeps once k is more than a few dozen - measured at 20M x 768, k = 100:
    // every block went on to the two-part product - so larger k starts there)
    if (ix.store.elem != kElemF32) {
        if (!banded_lists_fit(ix, k_sel)) return kTierExact;
        return (ix.store.elem == kElemBF16 && k_sel > 32) ? kTierSplit : kTierScreen;
    }
    // (ANN_CUDA_FLAT_SCREEN=0 turns screening off, =1 applies it to stores of any size)
    const int screen_env = g_flat_screen.load(std::memory_order_relaxed);
    // The one-MMA band holds ~0.3 k rows above the k-th on the stores measured (5M-20M unit-norm rows of 768
    // floats), and a list keeps 256 - k of them: from k ~ 200 on the screened pass only discovers that it
    // overflowed (k = 200: 180 ms against 140 ms when the split product's banded lists go first).  Forcing the
    // screened tier (tests) takes it for every k the lists can hold.
    constexpr int kScreenTierMaxK = 160;
    if (banded_lists_fit(ix, k_sel) &&
        (screen_env == 1 || (screen_env != 0 && ix.store.n >= kScreenMinRows && k_sel <= kScreenTierMaxK)))
        return kTierScreen;
    return kTierSplit;
}

// The tier after `tier` for this search (tier 2 exists only behind a 16-list).
int flat_next_tier(const ann_cuda_index &ix, int k_sel, int tier) {
    if (tier == kTierScreen) return kTierSplit;
    if (ix.store.elem != kElemF32) return kTierExact;
    if (tier == kTierSplit && k_sel <= 12 && banded_lists_fit(ix, k_sel)) return kTierSplitWide;
    return kTierExact;
}

int flat_tier_search(const ann_cuda_index &ix, Workspace &ws, int64_t nq, const float *x_dev, int64_t k, float *d_dev,
                     int64_t *i_dev, int64_t label_offset, cudaStream_t stream, int tier, const int *gate) {
    const int k_sel = (int)std::min<int64_t>(k, ix.store.n);
    const int64_t n = ix.store.n;
    TopkOpts o;
    o.tier = tier;
    o.gate = gate;
    o.chained = true;
    int k_list = k_sel, k_cand = 0;
    const bool banded = tier == kTierScreen || tier == kTierSplitWide ||
                        (tier == kTierSplit && (k_sel > 12 || ix.store.elem != kElemF32) && banded_lists_fit(ix, k_sel));
    if (ws.over_q.ensure((size_t)nq * 4) || (ix.store.elem != kElemF32 && ws.bad_q.ensure((size_t)nq * 4))) return -1;
    if (tier == kTierExact) {
        o.exact = true;
        // behind a tensor-core tier of the same block search: only the queries that tier flagged
        o.flagged_only = ws.over_q_valid;
        if (o.flagged_only) {
            o.prev_d = d_dev;
            o.prev_i = i_dev;
            o.prev_k = (int)k;
        }
    } else if (banded) {
        k_list = (int)std::min<int64_t>((int64_t)kScreenMaxList, n);
        o.k_rank = o.check_rank = k_sel;
        o.one_mma = tier == kTierScreen;
    } else {
        // Spare candidates beyond k for the band check: the rows inside the error band of the k-th key grow
        // with k and with the store (5M unit-norm rows of 768 floats: ~15 at k = 256, ~33 at k = 512, ~130 at
        // k = 2048), so a quarter of k, at least kSplitSpare, as far as the longest list allows.
        const int64_t spare = std::max<int64_t>(kSplitSpare, std::min<int64_t>(k_sel / 4, (int64_t)kMaxListK - k_sel));
        k_list = (int)std::min<int64_t>(k_sel <= 12 ? 16 : (int64_t)k_sel + spare, n);
        o.check_rank = k_list > k_sel ? k_sel : 0;
        // replace-max lists: every CTA that worked on a query tile leaves a list of ITS rows' best k_list, so the
        // merge can hand on up to 512 candidates more than one list is long (k = 2,048: the longest list holds
        // 2,112, the error band of a 5M-row store ~130 rows above the 2,048-th)
        if (k_list > kAppendMaxK) {
            o.wide_out = (int)std::min<int64_t>((int64_t)k_list + 512, n);
            o.wide_used = &k_cand;
        }
    }
    if (split_store_topk(ix, ix.store, ws, x_dev, nq, k_list, stream, o)) return -1;
    const bool widened = k_cand > k_list;  // the merge handed on more than one list's length, with ws.complete_to
    if (widened) k_list = k_cand;          // what the re-ranking below sees
    // banded lists: only what lies within the slack of the k-th ranking key needs the exact distance.  The
    // band check of the pass (is the last candidate still inside the band?) runs in the same kernel and
    // leaves its finding in this tier's overflow word, which gates the next tier.
    // (a list that holds every row of the store has left nothing out: no check)
    int *status = ws.status.as<int>();
    const bool tc = tier != kTierExact && flat_kernel_choice() == FlatKernel::TC;
    const RefineBand band{tc ? ws.sel_key.as<float>() : nullptr, k_sel, ws.qn.as<float>(), ix.store.max_norm2, ix.d, o.one_mma,
                          ix.store.elem, banded, (tc && k_list < n) ? o.check_rank : 0, status + kStatusTier0 + tier,
                          status + kStatusFallbacks, tc ? ws.over_q.as<int32_t>() : nullptr,
                          o.flagged_only ? ws.over_q.as<int32_t>() : nullptr,
                          (tc && ix.store.elem != kElemF32) ? ws.bad_q.as<int32_t>() : nullptr,
                          (tc && widened) ? ws.complete_to.as<float>() : nullptr};
    if (tc) ws.over_q_valid = true;  // (its scratch-init kernel cleared the words, this kernel sets them)
    // (a 16-bit store always hands the band over: it says how the rows are to be read)
    const bool give = (tc && (banded || band.check_rank > 0)) || ix.store.elem != kElemF32 || o.flagged_only;
    return launch_refine_finalize(ix.store.hi, ix.store.lo, ix.dp, ix.d, x_dev, ix.d, ws.sel_idx.as<int32_t>(), nq, k_list,
                                  (int)k, ix.metric, nullptr, label_offset, d_dev, i_dev, ix.device, stream, nullptr, nullptr,
                                  nullptr, nullptr, gate, give ? &band : nullptr);
}

// The whole search for one block of queries, all pointers on the device.
// Flat: tier_hint = lowest tier to start from.  gated = false runs that one tier and leaves the
// finding of its band check in the status words for the host to act on; gated = true enqueues the
// higher tiers behind it, each running only if the tier before it flagged an overflow.
// IVF: given_probes (may be null) = nq x nprobe list numbers on the device, best first, -1 = none; the
// coarse quantiser is then skipped (the probes were chosen elsewhere, e.g. by another shard's GPU).
int search_block_device(const ann_cuda_index &ix, Workspace &ws, int64_t nq, const float *x_dev, int64_t k,
                        float *d_dev, int64_t *i_dev, int64_t label_offset, cudaStream_t stream, int tier_hint,
                        bool gated, const int32_t *given_probes = nullptr) {
    if (!ix.ivf) {
        const int k_sel = (int)std::min<int64_t>(k, ix.store.n);
        int tier = flat_first_tier(ix, k_sel);
        // a search that starts at its first tier has no flagged queries yet; one that repeats from a higher
        // tier (the host's repeat after reading the band check) inherits those of the pass before it
        if (tier_hint <= tier) ws.over_q_valid = false;
        while (tier < tier_hint && tier < kTierExact) tier = flat_next_tier(ix, k_sel, tier);
        const int *gate = nullptr;
        for (;;) {
            if (flat_tier_search(ix, ws, nq, x_dev, k, d_dev, i_dev, label_offset, stream, tier, gate)) return -1;
            if (!gated || tier == kTierExact) return 0;
            gate = ws.status.as<int>() + kStatusTier0 + tier;
            tier = flat_next_tier(ix, k_sel, tier);
        }
    }
    const int nprobe = (int)std::min<int64_t>(std::max<int64_t>(ix.nprobe, 1), ix.nlist);
    // The list scan ranks by split-TF32 keys, off by up to ~2^-20 |q - c||x|: a few more
    // candidates than asked for are selected and the exact re-ranking at the end decides the
    // k-th place, so a near tie at the boundary is settled in fp32.
    if (k > kMaxK) return set_error("k is limited to %d", kMaxK);
    int k_sel = (int)k;
    if (flat_kernel_choice() == FlatKernel::TC) k_sel += kSelectMargin;
    // coarse quantiser: nprobe nearest centroids under the index metric
    const int64_t n_items = nq * nprobe;
    if (ws.probes.ensure((size_t)n_items * 4) || ws.item_slot.ensure(n_items * 4) ||
        ws.scratch.ensure((size_t)(ix.nlist + 1) * 2 * 4))
        return -1;
    if (given_probes) {
        ANN_CUDA_TRY(cudaMemcpyAsync(ws.probes.ptr, given_probes, (size_t)n_items * 4, cudaMemcpyDeviceToDevice, stream));
    } else if (coarse_probes(ix, ws, x_dev, nq, nprobe, ws.probes.as<int32_t>(), stream, ix.coarse_exact)) {
        return -1;
    }
    if (ws.qtau.ensure((size_t)nq * 4)) return -1;
    ANN_CUDA_TRY(cudaMemsetAsync(ws.qtau.ptr, 0xFF, (size_t)nq * 4, stream));
    if (flat_kernel_choice() == FlatKernel::TC) {
        // Tensor-core list scan: queries are grouped by the list they probe (padded to tiles
        // of 128), every (list, query tile) pair is one work item of the flat kernel, and each
        // list row is read once per query tile instead of once per query.
        const int64_t max_tiles = n_items / 128 + ix.nlist + 1;
        const int64_t max_rows = max_tiles * 128;
        const FlatPlan plan = make_grouped_plan(max_tiles, k_sel, sm_count(ix.device));
        if (ws.gq.ensure((size_t)max_rows * 4) || ws.items.ensure((size_t)max_tiles * 16) || ws.sched.ensure(64) ||
            ws.qhi.ensure((size_t)max_rows * ix.dp * 4) || ws.qlo.ensure((size_t)max_rows * ix.dp * 4) ||
            ws.part_key.ensure(plan.part_entries * 4) || ws.part_idx.ensure(plan.part_entries * 4) || ws_status_ready(ws))
            return -1;
        int *n_tiles = ws.sched.as<int>(), *item_counter = ws.sched.as<int>() + 1;
        ANN_CUDA_TRY(cudaMemsetAsync(ws.sched.ptr, 0, 64, stream));
        ANN_CUDA_TRY(cudaMemsetAsync(ws.gq.ptr, 0xFF, (size_t)max_rows * 4, stream));  // padding rows: no query
        // no clearing of the list memory: every list a query refers to is written in full by
        // the CTA that scans its (list, query tile) item, and empty lists are never referred to
        if (launch_group_probes(ws.probes.as<int32_t>(), nq, nprobe, ix.nlist, ix.list_off, ws.scratch.as<int>(), n_tiles,
                                ws.items.as<int4>(), ws.gq.as<int32_t>(), ws.item_slot.as<int32_t>(), stream))
            return -1;
        // L2: residual queries (see split_gathered_kernel); keys carry the per-row constant
        // only outside the scan kernel (shared thresholds, merge)
        const bool residual = ix.metric != 0;
        if (residual && ws.qconst.ensure((size_t)max_rows * 4)) return -1;
        float *qconst = residual ? ws.qconst.as<float>() : nullptr;
        if (launch_split_gathered(x_dev, ix.d, ix.dp, ws.gq.as<int32_t>(), n_tiles, max_rows, ws.qhi.as<float>(),
                                  ws.qlo.as<float>(), stream, residual ? ws.items.as<int4>() : nullptr,
                                  residual ? ix.store.hi : nullptr, residual ? ix.store.lo : nullptr, qconst))
            return -1;
        // append mode: finished rows stay unsorted with their fill count; in every mode the per-query
        // merge streams the lists of all probes and filters them by the query's final threshold
        // before it sorts (see merge_filtered_kernel), so nprobe * k is not limited
        const bool filtered = plan.lists_sorted;
        if (filtered && ws.part_cnt.ensure((size_t)max_rows * 4)) return -1;
        GroupedWork gw{ws.items.as<int4>(), n_tiles, item_counter, ws.gq.as<int32_t>(), qconst,
                       filtered ? ws.part_cnt.as<int32_t>() : nullptr, /*derive_lo=*/true};
        const bool timing = g_time_kernels.load(std::memory_order_relaxed) != 0;
        if (timing) {
            if (!ws.ev0) {
                ANN_CUDA_TRY(cudaEventCreate(&ws.ev0));
                ANN_CUDA_TRY(cudaEventCreate(&ws.ev1));
            }
            ANN_CUDA_TRY(cudaEventRecord(ws.ev0, stream));
        }
        if (launch_flat_tc(plan, ix.vhi, ix.vlo, residual ? ix.vrnorm : ix.vnorm, ix.rows, ws.qhi.as<float>(),
                           ws.qlo.as<float>(), max_rows, ix.dp,
                           k_sel, ix.metric, ws.part_key.as<float>(), ws.part_idx.as<int32_t>(), ws.qtau.as<uint32_t>(),
                           nullptr, ws.status.as<int>() + kStatusWait, ix.device, stream, &gw))
            return -1;
        if (timing) {
            ANN_CUDA_TRY(cudaEventRecord(ws.ev1, stream));
            ws.timed = true;
            ix.last_timed_ws = &ws;
        }
        if (ws_publish_status(ws, stream)) return -1;
        if (ws.sel_key.ensure((size_t)nq * k_sel * 4) || ws.sel_idx.ensure((size_t)nq * k_sel * 4)) return -1;
        if (launch_merge_filtered(ws.part_key.as<float>(), ws.part_idx.as<int32_t>(),
                                  filtered ? ws.part_cnt.as<int32_t>() : nullptr, ws.item_slot.as<int32_t>(), qconst,
                                  ws.qtau.as<uint32_t>(), nprobe, nq, k_sel, plan.list_stride, ws.sel_key.as<float>(),
                                  ws.sel_idx.as<int32_t>(), stream))
            return -1;
        // IP: the selected distances are recomputed exactly from hi + lo, as for Flat.  L2: the
        // residual form keeps the scan's own distance accurate unless the row nearly coincides
        // with the query; only those are recomputed.
        return launch_refine_finalize(ix.vhi, ix.vlo, ix.dp, ix.d, x_dev, ix.d, ws.sel_idx.as<int32_t>(), nq, k_sel, (int)k,
                                      ix.metric, ix.ids, label_offset, d_dev, i_dev, ix.device, stream,
                                      residual ? ws.sel_key.as<float>() : nullptr, ix.vrnorm, ix.vnorm);
    }
    // exact-fp32 cross-check path: one warp per (query, list)
    if (ws.item_q.ensure(n_items * 4) || ws.item_rb.ensure(n_items * 8) || ws.item_re.ensure(n_items * 8) ||
        ws.part_key.ensure((size_t)n_items * k_sel * 4) || ws.part_idx.ensure((size_t)n_items * k_sel * 4))
        return -1;
    if (launch_build_ivf_items(ws.probes.as<int32_t>(), nq, nprobe, ix.nlist, ix.list_off, ws.item_q.as<int32_t>(),
                               ws.item_rb.as<int64_t>(), ws.item_re.as<int64_t>(), ws.item_slot.as<int32_t>(),
                               ws.scratch.as<int>(), stream))
        return -1;
    if (launch_scan_items(ix.vhi, ix.vlo, ix.dp, ix.d, x_dev, ix.d, ws.item_q.as<int32_t>(), ws.item_rb.as<int64_t>(),
                          ws.item_re.as<int64_t>(), n_items, k_sel, ix.metric, ws.part_key.as<float>(),
                          ws.part_idx.as<int32_t>(), ws.qtau.as<uint32_t>(), ix.device, stream))
        return -1;
    if (ws.sel_key.ensure((size_t)nq * k_sel * 4) || ws.sel_idx.ensure((size_t)nq * k_sel * 4)) return -1;
    if (launch_merge_filtered(ws.part_key.as<float>(), ws.part_idx.as<int32_t>(), nullptr, ws.item_slot.as<int32_t>(), nullptr,
                              ws.qtau.as<uint32_t>(), nprobe, nq, k_sel, k_sel, ws.sel_key.as<float>(),
                              ws.sel_idx.as<int32_t>(), stream))
        return -1;
    return launch_finalize(ws.sel_key.as<float>(), ws.sel_idx.as<int32_t>(), nq, k_sel, (int)k, ix.metric, ix.ids,
                           label_offset, d_dev, i_dev, stream);
}

// keep_sticky: leave the wait word and the fallback counter as they are (they accumulate over the
// calls on a caller's stream until ann_cuda_index_search_status collects them).
int search_device_impl(const ann_cuda_index &ix, Workspace &ws, int64_t n, const float *x_dev, int64_t k, float *d_dev,
                       int64_t *i_dev, int64_t label_offset, cudaStream_t stream, int tier_hint, bool gated,
                       bool keep_sticky = false, const int32_t *given_probes = nullptr) {
    if (k <= 0) return set_error("k must be > 0");  // MetalIndexFlat.mm:297
    if (n <= 0) return 0;
    if (!ix.trained) return set_error("search: index must be trained first");  // MetalIndexIVFFlat.mm:125
    const int64_t stored = ix.ivf ? ix.rows : ix.store.n;
    if (ix.ntotal == 0 || stored == 0) return launch_fill_missing(d_dev, i_dev, n * k, ix.metric, stream);
    if (k > kMaxK && (ix.ivf || ix.store.n > kMaxK)) return set_error("k is limited to %d", kMaxK);
    if (ix.ivf && ivf_finalize_lists(ix)) return -1;
    const bool fresh = ws.status.ptr == nullptr;
    if (ws_status_ready(ws)) return -1;
    if (fresh || !keep_sticky) {
        if (ws_clear_status(ws, stream)) return -1;
        ws.fallbacks_seen = 0;
    }
    for (int64_t q0 = 0; q0 < n; q0 += kQueryBlock) {
        const int64_t nb = std::min(kQueryBlock, n - q0);
        // the overflow words speak of one block of queries
        if (q0 > 0 || keep_sticky)
            ANN_CUDA_TRY(cudaMemsetAsync(ws.status.as<int>() + kStatusTier0, 0, kTiers * sizeof(int), stream));
        const int64_t np = ix.ivf ? std::min<int64_t>(std::max<int64_t>(ix.nprobe, 1), ix.nlist) : 0;
        if (search_block_device(ix, ws, nb, x_dev + q0 * ix.d, k, d_dev + q0 * k, i_dev + q0 * k, label_offset, stream,
                                tier_hint, gated, given_probes ? given_probes + q0 * np : nullptr))
            return -1;
    }
    return ws_publish_status(ws, stream);
}

int upload_and(ann_cuda_index *ix, int64_t n, const float *x_host,
               int (*fn)(ann_cuda_index *, int64_t, const float *)) {
    // host rows -> device in slabs of at most 256 MB
    const int64_t slab = std::max<int64_t>(1, (256ll << 20) / ((int64_t)ix->d * 4));
    float *buf = nullptr;
    ANN_CUDA_TRY(cudaMalloc(&buf, (size_t)std::min(slab, n) * ix->d * 4));
    int rc = 0;
    for (int64_t r0 = 0; r0 < n && rc == 0; r0 += slab) {
        const int64_t nb = std::min(slab, n - r0);
        cudaError_t e = cudaMemcpy(buf, x_host + r0 * ix->d, (size_t)nb * ix->d * 4, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            rc = set_error("host to device copy failed: %s", cudaGetErrorString(e));
            break;
        }
        rc = fn(ix, nb, buf);
        if (rc == 0 && cudaDeviceSynchronize() != cudaSuccess) rc = set_error("device error during add");
    }
    cudaFree(buf);
    return rc;
}

int add_device_impl(ann_cuda_index *ix, int64_t n, const float *x_dev) {
    if (!ix->ivf) {
        if (ix->store.append_device(x_dev, n, ix->d, nullptr)) return -1;
        ANN_CUDA_TRY(cudaStreamSynchronize(nullptr));
        ix->ntotal = ix->store.n;
        return 0;
    }
    if (!ix->trained) return set_error("add: index must be trained first");  // MetalIndexIVFFlat.mm:103
    std::vector<int32_t> assign;
    if (ivf_assign_device(*ix, x_dev, n, assign, ix->coarse_exact)) return -1;
    std::vector<int64_t> labels((size_t)n);
    std::iota(labels.begin(), labels.end(), ix->ntotal);  // label = running ntotal (MetalIndexIVFFlat.mm:112)
    if (ivf_append(*ix, x_dev, n, assign.data(), labels.data())) return -1;
    ix->ntotal += n;
    return 0;
}

}  // namespace

// =================================================================================================
extern "C" {

const char *ann_cuda_last_error(void) { return last_error_ref().c_str(); }

int ann_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int ann_cuda_available(void) {
    static int cached = -1;
    if (cached >= 0) return cached;
    const int n = ann_cuda_device_count();
    int ok = n > 0;
    for (int i = 0; i < n && ok; i++) {
        cudaDeviceProp p;
        if (cudaGetDeviceProperties(&p, i) != cudaSuccess || p.major != 10) ok = 0;
    }
    cached = ok;
    return ok;
}

int ann_cuda_device_info(char *buf, size_t buflen) {
    if (!buf || buflen == 0) return set_error("null buffer");
    const int n = ann_cuda_device_count();
    if (n <= 0) {
        snprintf(buf, buflen, "CUDA: not available");
        return 0;
    }
    cudaDeviceProp p;
    ANN_CUDA_TRY(cudaGetDeviceProperties(&p, 0));
    snprintf(buf, buflen, "CUDA GPU (%s, sm_%d%d, %d SMs, %.0f GB, %d device%s)", p.name, p.major, p.minor,
             p.multiProcessorCount, (double)p.totalGlobalMem / 1e9, n, n == 1 ? "" : "s");
    return 0;
}

const char *ann_cuda_flat_kernel_name(void) { return flat_kernel_choice() == FlatKernel::TC ? "tcgen05" : "simt"; }

int ann_cuda_set_flat_kernel(const char *name) {
    if (name && strcmp(name, "tcgen05") == 0) {
        g_flat_kernel.store(0);
        g_flat_screen.store(-1);
        return 0;
    }
    if (name && strcmp(name, "tcgen05-screened") == 0) {  // one-MMA screening for stores of any size
        g_flat_kernel.store(0);
        g_flat_screen.store(1);
        return 0;
    }
    if (name && strcmp(name, "tcgen05-split") == 0) {  // three-MMA split product for every pair
        g_flat_kernel.store(0);
        g_flat_screen.store(0);
        return 0;
    }
    if (name && strcmp(name, "simt") == 0) {
        g_flat_kernel.store(1);
        return 0;
    }
    return set_error("unknown flat kernel name (tcgen05 | tcgen05-screened | tcgen05-split | simt)");
}

uint64_t ann_cuda_screen_fallbacks(void) { return g_screen_fallbacks.load(std::memory_order_relaxed); }

void ann_cuda_set_wait_limit_ms(int ms) { set_flat_wait_limit_ns(ms > 0 ? (uint64_t)ms * 1000000ull : 0); }
void ann_cuda_test_withhold_loads(int after_k_blocks) { set_flat_test_withhold_after(after_k_blocks < 0 ? -1 : after_k_blocks); }

void ann_cuda_set_kernel_timing(int on) { g_time_kernels.store(on ? 1 : 0); }

float ann_cuda_index_last_flat_kernel_ms(const ann_cuda_index *ix) {
    if (!ix || !ix->last_timed_ws || !ix->last_timed_ws->timed) return -1.f;
    DeviceGuard g(ix->device);
    float ms = -1.f;
    if (cudaEventSynchronize(ix->last_timed_ws->ev1) != cudaSuccess) return -1.f;
    if (cudaEventElapsedTime(&ms, ix->last_timed_ws->ev0, ix->last_timed_ws->ev1) != cudaSuccess) return -1.f;
    return ms;
}

uint64_t ann_cuda_launch_count(void) { return launch_count_value(); }

static int create_common(int device, int d, int metric, bool ivf, int64_t nlist, ann_cuda_index **out) {
    if (!out) return set_error("null output handle");
    *out = nullptr;
    if (d <= 0) return set_error("dimension must be > 0");
    if (metric != ANN_CUDA_METRIC_L2 && metric != ANN_CUDA_METRIC_INNER_PRODUCT)
        return set_error("unsupported metric %d (L2 and inner product only)", metric);
    if (ivf && nlist <= 0) return set_error("nlist must be > 0");
    if (device < 0 || device >= ann_cuda_device_count()) return set_error("no CUDA device %d", device);
    cudaDeviceProp p;
    ANN_CUDA_TRY(cudaGetDeviceProperties(&p, device));
    if (p.major != 10) return set_error("device %d is sm_%d%d; this library is built for sm_100a only", device, p.major, p.minor);
    ann_cuda_index *ix = new ann_cuda_index();
    ix->device = device;
    ix->d = d;
    ix->dp = pad_dim(d);
    ix->metric = metric;
    ix->ivf = ivf;
    ix->store.dp = ix->dp;
    ix->store.l2 = ix->metric != 0;
    ix->nlist = nlist;
    ix->trained = !ivf;
    *out = ix;
    return 0;
}

int ann_cuda_flat_create(int device, int d, int metric, ann_cuda_index **out) {
    return create_common(device, d, metric, false, 0, out);
}

int ann_cuda_flat_create_storage(int device, int d, int metric, int storage, ann_cuda_index **out) {
    if (storage != ANN_CUDA_STORAGE_F32 && storage != ANN_CUDA_STORAGE_F16 && storage != ANN_CUDA_STORAGE_BF16)
        return set_error("unknown storage type %d", storage);
    if (create_common(device, d, metric, false, 0, out)) return -1;
    if (storage != ANN_CUDA_STORAGE_F32) {
        // one plane of 16-bit elements, rows padded to whole 128-byte K blocks
        (*out)->store.elem = storage == ANN_CUDA_STORAGE_F16 ? kElemF16 : kElemBF16;
        (*out)->dp = (d + 63) / 64 * 64;
        (*out)->store.dp = (*out)->dp;
    }
    return 0;
}

int ann_cuda_index_storage(const ann_cuda_index *ix) {
    if (!ix) return -1;
    return ix->store.elem == kElemF16 ? ANN_CUDA_STORAGE_F16 : ix->store.elem == kElemBF16 ? ANN_CUDA_STORAGE_BF16 : ANN_CUDA_STORAGE_F32;
}

int ann_cuda_ivfflat_create(int device, int d, int64_t nlist, int metric, ann_cuda_index **out) {
    return create_common(device, d, metric, true, nlist, out);
}

void ann_cuda_index_free(ann_cuda_index *ix) {
    if (!ix) return;
    DeviceGuard g(ix->device);
    cudaDeviceSynchronize();
    ix->store.release_all();
    ivf_free_rows(*ix);
    if (ix->list_off) cudaFree(ix->list_off);
    for (Workspace *w : ix->ws_free) {
        w->release();
        delete w;
    }
    delete ix;
}

int ann_cuda_ivfflat_set_centroids(ann_cuda_index *ix, const float *centroids) {
    if (!ix || !ix->ivf || !centroids) return set_error("invalid arguments");
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    ix->store.n = 0;
    float *buf = nullptr;
    ANN_CUDA_TRY(cudaMalloc(&buf, (size_t)ix->nlist * ix->d * 4));
    cudaError_t e = cudaMemcpy(buf, centroids, (size_t)ix->nlist * ix->d * 4, cudaMemcpyHostToDevice);
    int rc = e == cudaSuccess ? ix->store.append_device(buf, ix->nlist, ix->d, nullptr) : set_error("centroid upload failed");
    cudaDeviceSynchronize();
    cudaFree(buf);
    if (rc) return -1;
    ix->trained = true;
    ix->csr_dirty = true;  // the rows' residual norms refer to the centroids
    return ivf_update_coarse_policy(*ix);
}

int ann_cuda_ivfflat_get_centroids(const ann_cuda_index *ix, float *centroids) {
    if (!ix || !ix->ivf || !centroids) return set_error("invalid arguments");
    if (!ix->trained) return set_error("index is not trained");
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    float *buf = nullptr;
    ANN_CUDA_TRY(cudaMalloc(&buf, (size_t)ix->nlist * ix->d * 4));
    int rc = launch_join_rows(ix->store.hi, ix->store.lo, ix->nlist, ix->d, ix->dp, buf, nullptr);
    cudaError_t e = cudaMemcpy(centroids, buf, (size_t)ix->nlist * ix->d * 4, cudaMemcpyDeviceToHost);
    cudaFree(buf);
    if (rc) return -1;
    if (e != cudaSuccess) return set_error("centroid download failed: %s", cudaGetErrorString(e));
    return 0;
}

int ann_cuda_ivfflat_train(ann_cuda_index *ix, int64_t n, const float *x) {
    if (!ix || !ix->ivf || !x) return set_error("invalid arguments");
    if (n < ix->nlist) return set_error("train: need at least nlist = %lld rows, got %lld", (long long)ix->nlist, (long long)n);
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    const int d = ix->d;
    const int64_t nlist = ix->nlist;
    float *dx = nullptr, *cent = nullptr;
    double *sums = nullptr;
    int *counts = nullptr;
    int32_t *dassign = nullptr;
    int rc = 0;
    auto cleanup = [&] {
        for (void *p : {(void *)dx, (void *)cent, (void *)sums, (void *)counts, (void *)dassign})
            if (p) cudaFree(p);
    };
    if (cudaMalloc(&dx, (size_t)n * d * 4) != cudaSuccess || cudaMalloc(&cent, (size_t)nlist * d * 4) != cudaSuccess ||
        cudaMalloc(&sums, (size_t)nlist * d * 8) != cudaSuccess || cudaMalloc(&counts, (size_t)nlist * 4) != cudaSuccess ||
        cudaMalloc(&dassign, (size_t)n * 4) != cudaSuccess) {
        cudaGetLastError();
        cleanup();
        return set_error("out of device memory in train");
    }
    cudaMemcpy(dx, x, (size_t)n * d * 4, cudaMemcpyHostToDevice);
    // initial centroids: k-means++ seeding (each next centre drawn with probability ~ squared
    // distance to the nearest centre so far), so that well separated groups each get a centre
    {
        float *dmin = nullptr;
        unsigned long long *best = nullptr;
        if (cudaMalloc(&dmin, (size_t)n * 4) != cudaSuccess || cudaMalloc(&best, 8) != cudaSuccess) {
            cudaGetLastError();
            if (dmin) cudaFree(dmin);
            cleanup();
            return set_error("out of device memory in train");
        }
        cudaMemset(best, 0, 8);
        cudaMemcpy(cent, dx, (size_t)d * 4, cudaMemcpyDeviceToDevice);  // first centre: the first training row
        const unsigned blocks = (unsigned)std::min<int64_t>((n + 7) / 8, 148 * 16);
        for (int64_t c = 1; c < nlist; c++) {
            kmeanspp_step_kernel<<<blocks, 256>>>(dx, n, d, cent + (c - 1) * d, dmin, 0x1234567u, (int)c, best);
            kmeanspp_take_kernel<<<1, 256>>>(dx, d, cent + c * d, best);
        }
        count_launch((int)(2 * (nlist - 1)));
        const cudaError_t e = cudaDeviceSynchronize();
        cudaFree(dmin);
        cudaFree(best);
        if (e != cudaSuccess) {
            cleanup();
            return set_error("device error in k-means++ seeding: %s", cudaGetErrorString(e));
        }
    }
    const int saved_metric = ix->metric;
    ix->metric = ANN_CUDA_METRIC_L2;  // Lloyd iterations assign by L2
    ix->trained = true;
    std::vector<int32_t> assign;
    std::vector<int> hcount((size_t)nlist);
    std::vector<float> hcent;
    uint64_t rng = 0x9E3779B97F4A7C15ull;  // fixed seed: training is deterministic
    auto next_uniform = [&rng]() {
        rng ^= rng << 13;
        rng ^= rng >> 7;
        rng ^= rng << 17;
        return (double)(rng >> 11) / 9007199254740992.0;
    };
    const int kIterations = 20;
    for (int it = 0; it < kIterations && rc == 0; it++) {
        ix->store.n = 0;
        rc = ix->store.append_device(cent, nlist, d, nullptr);
        if (rc == 0) rc = ivf_assign_device(*ix, dx, n, assign, false);  // Lloyd steps: the fast ranking will do
        if (rc) break;
        cudaMemcpy(dassign, assign.data(), (size_t)n * 4, cudaMemcpyHostToDevice);
        cudaMemset(sums, 0, (size_t)nlist * d * 8);
        cudaMemset(counts, 0, (size_t)nlist * 4);
        kmeans_accumulate_kernel<<<(unsigned)std::min<int64_t>((n + 7) / 8, 148 * 16), 256>>>(dx, n, d, dassign, sums, counts);
        kmeans_update_kernel<<<(unsigned)((nlist * d + 255) / 256), 256>>>(cent, sums, counts, nlist, d);
        count_launch(2);
        if (cudaDeviceSynchronize() != cudaSuccess) rc = set_error("device error in train");
        // Empty clusters are re-seeded by splitting large ones (the remedy k-means
        // implementations such as FAISS's use): without it, clusters that start without a
        // centroid all fall to one hub centroid and a single list swallows them.
        if (rc == 0 && it + 1 < kIterations) {
            cudaMemcpy(hcount.data(), counts, (size_t)nlist * 4, cudaMemcpyDeviceToHost);
            int64_t empty = 0;
            for (int64_t c = 0; c < nlist; c++) empty += hcount[c] == 0;
            if (empty > 0) {
                hcent.resize((size_t)nlist * d);
                cudaMemcpy(hcent.data(), cent, (size_t)nlist * d * 4, cudaMemcpyDeviceToHost);
                for (int64_t ci = 0; ci < nlist; ci++) {
                    if (hcount[ci] != 0) continue;
                    int64_t cj = 0;
                    for (int tries = 0; tries < 1 << 20; tries++) {  // pick a cluster with probability ~ its size
                        cj = (int64_t)(next_uniform() * nlist) % nlist;
                        const double p = (hcount[cj] - 1.0) / (double)(n - nlist + 1);
                        if (next_uniform() < p) break;
                    }
                    const float eps = 1.0f / 1024.0f;
                    for (int j = 0; j < d; j++) {
                        const float v = hcent[cj * d + j];
                        hcent[ci * d + j] = v * ((j & 1) ? 1 + eps : 1 - eps);
                        hcent[cj * d + j] = v * ((j & 1) ? 1 - eps : 1 + eps);
                    }
                    hcount[ci] = hcount[cj] / 2;
                    hcount[cj] -= hcount[ci];
                }
                cudaMemcpy(cent, hcent.data(), (size_t)nlist * d * 4, cudaMemcpyHostToDevice);
            }
        }
    }
    ix->metric = saved_metric;
    if (rc == 0) {
        ix->store.n = 0;
        rc = ix->store.append_device(cent, nlist, d, nullptr);
        cudaDeviceSynchronize();
    }
    cleanup();
    if (rc) {
        ix->trained = false;
        return -1;
    }
    ix->csr_dirty = true;
    return ivf_update_coarse_policy(*ix);
}

int ann_cuda_ivfflat_add_list(ann_cuda_index *ix, int64_t list_no, int64_t n, const int64_t *ids, const float *rows) {
    if (!ix || !ix->ivf || list_no < 0 || list_no >= ix->nlist || n < 0 || (n > 0 && (!ids || !rows)))
        return set_error("invalid arguments");
    if (n == 0) return 0;
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    ix->ntotal += n;
    if (!ivf_owns(*ix, list_no)) return 0;
    float *buf = nullptr;
    ANN_CUDA_TRY(cudaMalloc(&buf, (size_t)n * ix->d * 4));
    cudaError_t e = cudaMemcpy(buf, rows, (size_t)n * ix->d * 4, cudaMemcpyHostToDevice);
    int rc = 0;
    if (e != cudaSuccess) {
        rc = set_error("list upload failed: %s", cudaGetErrorString(e));
    } else {
        std::vector<int32_t> lists((size_t)n, (int32_t)list_no);
        rc = ivf_append(*ix, buf, n, lists.data(), ids);
    }
    cudaFree(buf);
    return rc;
}

int64_t ann_cuda_ivfflat_list_size(const ann_cuda_index *ix, int64_t list_no) {
    if (!ix || !ix->ivf || list_no < 0 || list_no >= ix->nlist) return -1;
    DeviceGuard g(ix->device);
    if (ivf_finalize_lists(*ix)) return -1;
    return ix->list_off_host[list_no + 1] - ix->list_off_host[list_no];
}

int ann_cuda_ivfflat_get_list(const ann_cuda_index *ix, int64_t list_no, int64_t *ids, float *rows) {
    if (!ix || !ix->ivf || list_no < 0 || list_no >= ix->nlist) return set_error("invalid arguments");
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    if (ivf_finalize_lists(*ix)) return -1;
    const int64_t b = ix->list_off_host[list_no], n = ix->list_off_host[list_no + 1] - b;
    if (n == 0) return 0;
    if (ids) ANN_CUDA_TRY(cudaMemcpy(ids, ix->ids + b, (size_t)n * 8, cudaMemcpyDeviceToHost));
    if (rows) {
        float *buf = nullptr;
        ANN_CUDA_TRY(cudaMalloc(&buf, (size_t)n * ix->d * 4));
        int rc = launch_join_rows(ix->vhi + b * ix->dp, nullptr, n, ix->d, ix->dp, buf, nullptr);
        cudaError_t e = cudaMemcpy(rows, buf, (size_t)n * ix->d * 4, cudaMemcpyDeviceToHost);
        cudaFree(buf);
        if (rc) return -1;
        if (e != cudaSuccess) return set_error("list download failed: %s", cudaGetErrorString(e));
    }
    return 0;
}

int ann_cuda_ivfflat_coarse(const ann_cuda_index *ix, int64_t n, const float *x, int64_t nprobe, int64_t *lists) {
    if (!ix || !ix->ivf || n < 0 || (n > 0 && (!x || !lists)) || nprobe <= 0) return set_error("invalid arguments");
    if (!ix->trained) return set_error("index is not trained");
    if (n == 0) return 0;
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    const int np = (int)std::min<int64_t>(nprobe, ix->nlist);
    WsLease lease(ix, nullptr, true);
    if (!lease.ws) return -1;
    Workspace &ws = *lease.ws;
    cudaStream_t s = ws.own_stream;
    std::vector<int32_t> tmp;
    for (int64_t q0 = 0; q0 < n; q0 += kQueryBlock) {
        const int64_t nb = std::min(kQueryBlock, n - q0);
        if (ws.x.ensure((size_t)nb * ix->d * 4)) return -1;
        ANN_CUDA_TRY(cudaMemcpyAsync(ws.x.ptr, x + q0 * ix->d, (size_t)nb * ix->d * 4, cudaMemcpyHostToDevice, s));
        if (ws.probes.ensure((size_t)nb * np * 4) || ws_clear_status(ws, s)) return -1;
        if (coarse_probes(*ix, ws, ws.x.as<float>(), nb, np, ws.probes.as<int32_t>(), s, ix->coarse_exact)) return -1;
        tmp.resize((size_t)nb * np);
        ANN_CUDA_TRY(cudaMemcpyAsync(tmp.data(), ws.probes.ptr, (size_t)nb * np * 4, cudaMemcpyDeviceToHost, s));
        ANN_CUDA_TRY(cudaStreamSynchronize(s));
        for (int64_t q = 0; q < nb; q++)
            for (int64_t p = 0; p < nprobe; p++) lists[(q0 + q) * nprobe + p] = p < np ? tmp[q * np + p] : -1;
    }
    return 0;
}

int ann_cuda_ivfflat_coarse_device(const ann_cuda_index *ix, int64_t n, const float *x_device, int32_t *lists_device,
                                   void *stream) {
    if (!ix || !ix->ivf || n < 0 || (n > 0 && (!x_device || !lists_device))) return set_error("invalid arguments");
    if (!ix->trained) return set_error("index is not trained");
    if (n == 0) return 0;
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    WsLease lease(ix, s, false);
    if (!lease.ws) return -1;
    Workspace &ws = *lease.ws;
    const int np = (int)std::min<int64_t>(std::max<int64_t>(ix->nprobe, 1), ix->nlist);
    // (the words of a workspace that has never searched start at zero; later ones keep what the stream's
    // earlier calls left for ann_cuda_index_search_status to collect)
    const bool fresh = ws.status.ptr == nullptr;
    if (ws_status_ready(ws) || (fresh && ws_clear_status(ws, s))) return -1;
    for (int64_t q0 = 0; q0 < n; q0 += kQueryBlock) {
        const int64_t nb = std::min(kQueryBlock, n - q0);
        if (coarse_probes(*ix, ws, x_device + q0 * ix->d, nb, np, lists_device + q0 * np, s, ix->coarse_exact)) return -1;
    }
    return ws_publish_status(ws, s);
}

int ann_cuda_ivfflat_search_preassigned_device(const ann_cuda_index *ix, int64_t n, const float *x_device,
                                               const int32_t *assign_device, int64_t k, float *distances_device,
                                               int64_t *labels_device, int64_t label_offset, void *stream) {
    if (!ix || !ix->ivf || n < 0 || (n > 0 && (!x_device || !assign_device || !distances_device || !labels_device)))
        return set_error("invalid arguments");
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    WsLease lease(ix, s, false);
    if (!lease.ws) return -1;
    return search_device_impl(*ix, *lease.ws, n, x_device, k, distances_device, labels_device, label_offset, s, 0, true, true,
                              assign_device);
}

int ann_cuda_ivfflat_set_nprobe(ann_cuda_index *ix, int64_t nprobe) {
    if (!ix || !ix->ivf) return set_error("not an IVFFlat index");
    ix->nprobe = std::max<int64_t>(1, std::min(nprobe, ix->nlist));  // MetalIndexIVFFlat.mm:275-279
    return 0;
}
int64_t ann_cuda_ivfflat_get_nprobe(const ann_cuda_index *ix) { return ix && ix->ivf ? ix->nprobe : -1; }
int64_t ann_cuda_ivfflat_nlist(const ann_cuda_index *ix) { return ix && ix->ivf ? ix->nlist : -1; }

int ann_cuda_ivfflat_set_shard(ann_cuda_index *ix, int shard_rank, int shard_count) {
    if (!ix || !ix->ivf || shard_count <= 0 || shard_rank < 0 || shard_rank >= shard_count)
        return set_error("invalid shard arguments");
    if (ix->rows > 0) return set_error("set_shard must be called before rows are added");
    ix->shard_rank = shard_rank;
    ix->shard_count = shard_count;
    return 0;
}

int ann_cuda_index_reserve(ann_cuda_index *ix, int64_t n_total) {
    if (!ix || n_total < 0) return set_error("invalid arguments");
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    if (!ix->ivf) return ix->store.reserve(n_total);
    return n_total > ix->rows ? ivf_grow_rows(*ix, n_total - ix->rows) : 0;
}

int ann_cuda_index_add_device(ann_cuda_index *ix, int64_t n, const float *x_device) {
    if (!ix || n < 0 || (n > 0 && !x_device)) return set_error("invalid arguments");
    if (n == 0) return 0;
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    return add_device_impl(ix, n, x_device);
}

int ann_cuda_index_add(ann_cuda_index *ix, int64_t n, const float *x) {
    if (!ix || n < 0 || (n > 0 && !x)) return set_error("invalid arguments");
    if (n == 0) return 0;
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    if (!ix->ivf && ix->store.grow_for(n)) return -1;
    return upload_and(ix, n, x, add_device_impl);
}

int ann_cuda_index_search_device(const ann_cuda_index *ix, int64_t n, const float *x_device, int64_t k,
                                 float *distances_device, int64_t *labels_device, int64_t label_offset, void *stream) {
    if (!ix || n < 0 || (n > 0 && (!x_device || !distances_device || !labels_device)))
        return set_error("invalid arguments");
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    WsLease lease(ix, s, false);
    if (!lease.ws) return -1;
    // Nothing is waited for here, so every fallback tier is enqueued behind the first one, gated on
    // the device by the band check of the tier before it: the results are complete when the stream
    // gets there, whatever the data.  Give-up codes of bounded waits accumulate in the workspace of
    // this stream until ann_cuda_index_search_status collects them.
    return search_device_impl(*ix, *lease.ws, n, x_device, k, distances_device, labels_device, label_offset, s, 0, true,
                              true);
}

int ann_cuda_index_search_status(const ann_cuda_index *ix, void *stream) {
    if (!ix) return set_error("null index");
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ANN_CUDA_TRY(cudaStreamSynchronize(s));
    // every idle workspace that served this stream
    std::vector<Workspace *> mine;
    {
        std::lock_guard<std::mutex> lock(ix->ws_mu);
        for (size_t i = 0; i < ix->ws_free.size();) {
            Workspace *w = ix->ws_free[i];
            if (w->bound == s && w->bound != w->own_stream) {
                mine.push_back(w);
                ix->ws_free.erase(ix->ws_free.begin() + i);
            } else {
                i++;
            }
        }
    }
    int code = 0, rc = 0;
    for (Workspace *w : mine) {
        if (!w->status.ptr) continue;  // never searched
        ws_absorb_fallbacks(*w);
        if (!code) code = w->status_host[kStatusWait];
        // start over: the wait word and the fallback counter are sticky until collected here
        if (ws_clear_status(*w, s) || ws_publish_status(*w, s)) rc = -1;
        w->fallbacks_seen = 0;
    }
    if (cudaStreamSynchronize(s) != cudaSuccess) rc = set_error("device error while collecting the search status");
    for (Workspace *w : mine) ix->release_ws(w);
    if (rc) return -1;
    if (code)
        return set_error("a search on this stream gave up on a wait inside the flat kernel (code %d): its results are not valid",
                         code);
    return 0;
}

int ann_cuda_index_search(const ann_cuda_index *ix, int64_t n, const float *x, int64_t k, float *distances,
                          int64_t *labels) {
    if (!ix || n < 0 || (n > 0 && (!x || !distances || !labels))) return set_error("invalid arguments");
    if (k <= 0) return set_error("k must be > 0");
    if (n == 0) return 0;
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    WsLease lease(ix, nullptr, true);
    if (!lease.ws) return -1;
    Workspace &ws = *lease.ws;
    cudaStream_t s = ws.own_stream;
    // query blocks keep the staging buffers bounded
    for (int64_t q0 = 0; q0 < n; q0 += kQueryBlock) {
        const int64_t nb = std::min(kQueryBlock, n - q0);
        if (ws.x.ensure((size_t)nb * ix->d * 4) || ws.out_d.ensure((size_t)nb * k * 4) || ws.out_i.ensure((size_t)nb * k * 8))
            return -1;
        ANN_CUDA_TRY(cudaMemcpyAsync(ws.x.ptr, x + q0 * ix->d, (size_t)nb * ix->d * 4, cudaMemcpyHostToDevice, s));
        // This call waits for its results anyway, so a tier whose band check flags an overflow is
        // repeated one tier up from here (no gated launches on the common path: one query per call
        // is how the extension searches, src/faiss_index.cpp:737).
        for (int tier = 0;;) {
            if (search_device_impl(*ix, ws, nb, ws.x.as<float>(), k, ws.out_d.as<float>(), ws.out_i.as<int64_t>(), 0, s, tier,
                                   false))
                return -1;
            ANN_CUDA_TRY(cudaMemcpyAsync(distances + q0 * k, ws.out_d.ptr, (size_t)nb * k * 4, cudaMemcpyDeviceToHost, s));
            ANN_CUDA_TRY(cudaMemcpyAsync(labels + q0 * k, ws.out_i.ptr, (size_t)nb * k * 8, cudaMemcpyDeviceToHost, s));
            ANN_CUDA_TRY(cudaStreamSynchronize(s));
            if (ws.status_host[kStatusWait])
                return set_error("flat kernel gave up on a wait (code %d)", ws.status_host[kStatusWait]);
            int flagged = -1;
            for (int t = kTierScreen; t <= kTierExact; t++)
                if (ws.status_host[kStatusTier0 + t] == kScreenOverflow) flagged = t;
            if (flagged < 0) break;
            if (flagged >= kTierExact) return set_error("the exact tier reported an overflow");  // it has no band check
            g_screen_fallbacks.fetch_add(1, std::memory_order_relaxed);
            tier = flagged + 1;
        }
    }
    return 0;
}

// ---- asynchronous search (MetalIndexFlat.h:15-36, MetalIndexFlat.mm:371-443) --------------------
// The token keeps one workspace (its stream and staging buffers) leased until it is waited on or
// freed, so several searches can be in flight on one index.
struct ann_cuda_search_token {
    const ann_cuda_index *ix = nullptr;
    WsLease *lease = nullptr;
    cudaEvent_t done = nullptr;
    int64_t n = 0, k = 0;
    float *distances = nullptr;
    int64_t *labels = nullptr;
    bool waited = false;
    int rc = 0;
};

int ann_cuda_index_search_async(const ann_cuda_index *ix, int64_t n, const float *x, int64_t k, float *distances,
                                int64_t *labels, ann_cuda_search_token **out) {
    if (!out) return set_error("invalid arguments");
    *out = nullptr;
    if (!ix || n < 0 || (n > 0 && (!x || !distances || !labels))) return set_error("invalid arguments");
    if (k <= 0) return set_error("k must be > 0");
    auto *t = new ann_cuda_search_token();
    t->ix = ix;
    t->n = n;
    t->k = k;
    t->distances = distances;
    t->labels = labels;
    if (n == 0) {
        t->waited = true;
        *out = t;
        return 0;
    }
    DeviceGuard g(ix->device);
    int rc = ensure_device(ix, g);
    if (!rc) {
        t->lease = new WsLease(ix, nullptr, true);
        if (!t->lease->ws) rc = -1;
    }
    if (!rc) {
        Workspace &ws = *t->lease->ws;
        cudaStream_t s = ws.own_stream;
        rc = ws.x.ensure((size_t)n * ix->d * 4) || ws.out_d.ensure((size_t)n * k * 4) || ws.out_i.ensure((size_t)n * k * 8);
        // the copy out of pageable memory is staged before the call returns: x may be reused at once
        if (!rc && cudaMemcpyAsync(ws.x.ptr, x, (size_t)n * ix->d * 4, cudaMemcpyHostToDevice, s) != cudaSuccess)
            rc = set_error("query upload failed");
        // all tiers are enqueued now, gated on the device: the wait only has to collect the results
        if (!rc) rc = search_device_impl(*ix, ws, n, ws.x.as<float>(), k, ws.out_d.as<float>(), ws.out_i.as<int64_t>(), 0, s, 0, true);
        if (!rc && (cudaEventCreateWithFlags(&t->done, cudaEventDisableTiming) != cudaSuccess ||
                    cudaEventRecord(t->done, s) != cudaSuccess))
            rc = set_error("event record failed");
    }
    if (rc) {
        ann_cuda_search_token_free(t);
        return -1;
    }
    *out = t;
    return 0;
}

int ann_cuda_search_token_ready(const ann_cuda_search_token *t) {
    if (!t) return set_error("null token");
    if (t->waited || !t->done) return 1;
    return cudaEventQuery(t->done) == cudaSuccess ? 1 : 0;
}

int ann_cuda_search_token_wait(ann_cuda_search_token *t) {
    if (!t) return set_error("null token");
    if (t->waited) return t->rc;
    t->waited = true;
    const ann_cuda_index *ix = t->ix;
    DeviceGuard g(ix->device);
    Workspace &ws = *t->lease->ws;
    cudaStream_t s = ws.own_stream;
    auto finish = [&](int rc) {
        t->rc = rc;
        delete t->lease;
        t->lease = nullptr;
        return rc;
    };
    if (cudaMemcpyAsync(t->distances, ws.out_d.ptr, (size_t)t->n * t->k * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaMemcpyAsync(t->labels, ws.out_i.ptr, (size_t)t->n * t->k * 8, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess)
        return finish(set_error("asynchronous search failed: %s", cudaGetErrorString(cudaGetLastError())));
    ws_absorb_fallbacks(ws);
    if (ws.status_host[kStatusWait]) return finish(set_error("flat kernel gave up on a wait (code %d)", ws.status_host[kStatusWait]));
    return finish(0);
}

void ann_cuda_search_token_free(ann_cuda_search_token *t) {
    if (!t) return;
    if (t->lease) {
        // never hand a workspace back while its stream still writes into it
        if (t->lease->ws) {
            DeviceGuard g(t->ix->device);
            cudaStreamSynchronize(t->lease->ws->own_stream);
        }
        delete t->lease;
    }
    if (t->done) cudaEventDestroy(t->done);
    delete t;
}

int ann_cuda_index_reset(ann_cuda_index *ix) {
    if (!ix) return set_error("null index");
    DeviceGuard g(ix->device);
    cudaDeviceSynchronize();
    ix->ntotal = 0;
    if (!ix->ivf) {
        ix->store.n = 0;
    } else {
        ix->rows = 0;
        ix->row_list.clear();
        ix->rows_sorted = true;
        ix->csr_dirty = true;
    }
    return 0;
}

int ann_cuda_index_reconstruct(const ann_cuda_index *ix, int64_t key, float *recons) {
    if (!ix || !recons) return set_error("invalid arguments");
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    if (!ix->ivf) {
        if (key < 0 || key >= ix->store.n) return set_error("reconstruct: key %lld out of range", (long long)key);
        return ann_cuda_flat_get_rows(ix, key, 1, recons);
    }
    if (ix->rows == 0) return set_error("reconstruct: key %lld not found", (long long)key);
    long long *found = nullptr, h = 0x7fffffffffffffffll;
    ANN_CUDA_TRY(cudaMalloc(&found, 8));
    cudaMemcpy(found, &h, 8, cudaMemcpyHostToDevice);
    find_id_kernel<<<(unsigned)((ix->rows + 255) / 256), 256>>>(ix->ids, ix->rows, key, found);
    count_launch();
    cudaMemcpy(&h, found, 8, cudaMemcpyDeviceToHost);
    cudaFree(found);
    if (h == 0x7fffffffffffffffll) return set_error("reconstruct: key %lld not found", (long long)key);
    float *buf = nullptr;
    ANN_CUDA_TRY(cudaMalloc(&buf, (size_t)ix->d * 4));
    int rc = launch_join_rows(ix->vhi + h * ix->dp, nullptr, 1, ix->d, ix->dp, buf, nullptr);
    cudaError_t e = cudaMemcpy(recons, buf, (size_t)ix->d * 4, cudaMemcpyDeviceToHost);
    cudaFree(buf);
    if (rc) return -1;
    if (e != cudaSuccess) return set_error("reconstruct failed: %s", cudaGetErrorString(e));
    return 0;
}

int ann_cuda_flat_get_rows(const ann_cuda_index *ix, int64_t first, int64_t n, float *rows) {
    if (!ix || ix->ivf || !rows || first < 0 || n < 0 || first + n > ix->store.n) return set_error("invalid arguments");
    if (n == 0) return 0;
    DeviceGuard g(ix->device);
    if (ensure_device(ix, g)) return -1;
    const int64_t slab = std::max<int64_t>(1, (256ll << 20) / ((int64_t)ix->d * 4));
    float *buf = nullptr;
    ANN_CUDA_TRY(cudaMalloc(&buf, (size_t)std::min(slab, n) * ix->d * 4));
    int rc = 0;
    for (int64_t r0 = 0; r0 < n && rc == 0; r0 += slab) {
        const int64_t nb = std::min(slab, n - r0);
        rc = launch_join_rows(ix->store.hi_at(first + r0), ix->store.lo_at(first + r0), nb, ix->d, ix->dp, buf, nullptr,
                              ix->store.elem);
        if (rc == 0 && cudaMemcpy(rows + r0 * ix->d, buf, (size_t)nb * ix->d * 4, cudaMemcpyDeviceToHost) != cudaSuccess)
            rc = set_error("device to host copy failed");
    }
    cudaFree(buf);
    return rc;
}

int64_t ann_cuda_index_ntotal(const ann_cuda_index *ix) { return ix ? ix->ntotal : -1; }
int ann_cuda_index_d(const ann_cuda_index *ix) { return ix ? ix->d : -1; }
int ann_cuda_index_metric(const ann_cuda_index *ix) { return ix ? ix->metric : -1; }
int ann_cuda_index_is_trained(const ann_cuda_index *ix) { return ix ? (int)ix->trained : 0; }
int ann_cuda_index_is_ivf(const ann_cuda_index *ix) { return ix ? (int)ix->ivf : 0; }
int ann_cuda_index_device(const ann_cuda_index *ix) { return ix ? ix->device : -1; }

int ann_cuda_merge_topk_device(int device, const float *parts_distances, const int64_t *parts_labels, int nparts,
                               int64_t nq, int64_t k, int metric, float *out_distances, int64_t *out_labels,
                               void *stream) {
    if (!parts_distances || !parts_labels || !out_distances || !out_labels || nparts <= 0 || nq < 0 || k <= 0)
        return set_error("invalid arguments");
    DeviceGuard g(device);
    if (!g.ok) return set_error("cudaSetDevice(%d) failed", device);
    return launch_merge_results(parts_distances, parts_labels, nparts, nq, (int)k, metric, out_distances, out_labels,
                                device, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// =================================================================================================
// Flat search without any allocation.
//
// Some hosts of this library may not allocate device memory while they search: a
// database worker that runs under a fixed memory budget and treats any allocation
// made behind its back as a leak, a caller that records its searches into a CUDA
// graph (allocation calls are not permitted between begin and end of a capture),
// or a latency-critical thread for which cudaMalloc / cudaFree - which can
// synchronise the whole device - are off limits.  The regular search entry points
// take their scratch from a growing pool, so their first call, and any call larger
// than the ones before it, allocates.
//
// ann_cuda_flat_search_small_static runs the same kernels as
// ann_cuda_index_search_device for a small query batch, with ALL scratch (the TF32
// split of the queries, the per-CTA candidate lists, the shared thresholds, the
// scheduler counters, the merged selection) carved out of one file-scope device
// array of fixed size.  The array exists once per device that loads the library
// (about 6 MB, held until the process exits) and is shared by every call: it keeps
// whatever the last call left in it, so everything that has to start from a known
// state is cleared on the stream at the start of each call, and two calls whose GPU
// work overlaps (different streams, or different host threads) would trample each
// other - callers must serialise them.
namespace {

constexpr int64_t kStaticMaxQueries = 128;  // one query tile
constexpr int kStaticMaxDim = 1024;
constexpr int kStaticMaxK = 16;             // the shared-memory selection mode
constexpr int kStaticMaxLists = 304;        // k-lists the kernel may start for the one query tile

constexpr size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }
constexpr size_t kOffQhi = 0;
constexpr size_t kOffQlo = kOffQhi + align256((size_t)kStaticMaxQueries * kStaticMaxDim * 4);
constexpr size_t kOffQn = kOffQlo + align256((size_t)kStaticMaxQueries * kStaticMaxDim * 4);
constexpr size_t kOffQtau = kOffQn + align256((size_t)kStaticMaxQueries * 4);
constexpr size_t kOffSched = kOffQtau + align256(128 * 4);
constexpr size_t kOffStatus = kOffSched + align256(2 * 4);
constexpr size_t kOffPartKey = kOffStatus + align256(4);
constexpr size_t kOffPartIdx = kOffPartKey + align256((size_t)kStaticMaxLists * 128 * kStaticMaxK * 4);
constexpr size_t kOffSelKey = kOffPartIdx + align256((size_t)kStaticMaxLists * 128 * kStaticMaxK * 4);
constexpr size_t kOffSelIdx = kOffSelKey + align256((size_t)kStaticMaxQueries * kStaticMaxK * 4);
constexpr size_t kStaticScratchBytes = kOffSelIdx + align256((size_t)kStaticMaxQueries * kStaticMaxK * 4);

// The scratch itself.  In host code this name is only a handle for the runtime, not a
// device address: the address a kernel can use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on `device` (which must be current); looked up
// once per device and cached.
int static_scratch_base(int device, unsigned char **out) {
    static std::mutex mu;
    static unsigned char *cached[64];
    if (device < 0 || device >= 64) return set_error("device index %d out of range", device);
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[device]) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            return set_error("cudaGetSymbolAddress(static scratch) failed on device %d: %s", device, cudaGetErrorString(e));
        cached[device] = static_cast<unsigned char *>(p);
    }
    *out = cached[device];
    return 0;
}

}  // namespace

extern "C" int ann_cuda_flat_search_small_static(const ann_cuda_index *ix, int64_t n, const float *x_device, int64_t k,
                                                  float *distances_device, int64_t *labels_device,
                                                  int64_t label_offset, void *stream) {
    if (!ix || n < 0 || (n > 0 && (!x_device || !distances_device || !labels_device)))
        return set_error("invalid arguments");
    if (ix->ivf) return set_error("the allocation-free search exists for Flat indexes only");
    if (k <= 0) return set_error("k must be > 0");
    if (n > kStaticMaxQueries)
        return set_error("allocation-free search: %lld queries exceed the limit of %lld per call", (long long)n,
                         (long long)kStaticMaxQueries);
    if (k > kStaticMaxK)
        return set_error("allocation-free search: k = %lld exceeds the limit of %d", (long long)k, kStaticMaxK);
    if (ix->dp > kStaticMaxDim)
        return set_error("allocation-free search: dimension %d exceeds the limit of %d", ix->d, kStaticMaxDim);
    if (n == 0) return 0;
    DeviceGuard g(ix->device);
    if (!g.ok) return set_error("cudaSetDevice(%d) failed", ix->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (ix->ntotal == 0 || ix->store.n == 0) return launch_fill_missing(distances_device, labels_device, n * k, ix->metric, s);
    unsigned char *base = nullptr;
    if (static_scratch_base(ix->device, &base)) return -1;  // first call on a device: looks the address up
    const int k_sel = (int)std::min<int64_t>(k, ix->store.n);
    // like the regular split-product search: 16 candidates for k <= 12, so that near ties at the
    // k-th place are settled by the exact re-ranking below (k = 13..16: no spare, no band check)
    if (ix->store.elem != kElemF32) return set_error("allocation-free search: fp32 storage only");
    const int k_list = k_sel <= 12 ? (int)std::min<int64_t>(16, ix->store.n) : k_sel;
    const FlatPlan plan = make_flat_plan(n, ix->store.n, k_list, sm_count(ix->device));
    if (plan.list_stride > kStaticMaxK)
        return set_error("allocation-free search: lists of %d entries exceed the limit of %d", plan.list_stride, kStaticMaxK);
    if (plan.nq_tiles != 1 || plan.lists_per_qt > kStaticMaxLists)
        return set_error("allocation-free search: this device needs %d candidate lists, the static scratch holds %d",
                         plan.lists_per_qt, kStaticMaxLists);
    float *qhi = reinterpret_cast<float *>(base + kOffQhi), *qlo = reinterpret_cast<float *>(base + kOffQlo);
    float *qn = reinterpret_cast<float *>(base + kOffQn);
    uint32_t *qtau = reinterpret_cast<uint32_t *>(base + kOffQtau);
    int *sched = reinterpret_cast<int *>(base + kOffSched), *status = reinterpret_cast<int *>(base + kOffStatus);
    float *part_key = reinterpret_cast<float *>(base + kOffPartKey);
    int32_t *part_idx = reinterpret_cast<int32_t *>(base + kOffPartIdx);
    float *sel_key = reinterpret_cast<float *>(base + kOffSelKey);
    int32_t *sel_idx = reinterpret_cast<int32_t *>(base + kOffSelIdx);
    // The array still holds the previous call's lists, thresholds and counters.  The two status
    // words (wait give-up code, band overflow) are sticky until ..._static_status reads them.
    ANN_CUDA_TRY(cudaMemsetAsync(qtau, 0xFF, 128 * 4, s));
    ANN_CUDA_TRY(cudaMemsetAsync(sched, 0, 2 * 4, s));
    ANN_CUDA_TRY(cudaMemsetAsync(part_idx, 0xFF, plan.part_entries * 4, s));
    if (launch_split_rows(x_device, n, ix->d, ix->dp, qhi, qlo, qn, s, ix->store.center(), true)) return -1;
    if (launch_flat_tc(plan, ix->store.hi, ix->store.lo, ix->store.norms, ix->store.n, qhi, qlo, n, ix->dp, k_list,
                       ix->metric, part_key, part_idx, qtau, sched, status, ix->device, s))
        return -1;
    if (launch_merge_parts(part_key, part_idx, 0, sched + plan.nq_tiles, nullptr, plan.lists_per_qt, n, k_list,
                           plan.list_stride, sel_key, sel_idx, ix->device, s))
        return -1;
    if (k_list > k_sel && k_list < ix->store.n &&
        launch_screen_check(sel_key, n, k_list, k_sel, qn, ix->store.max_norm2, ix->d, ix->metric, false, status + 1, nullptr, s))
        return -1;
    return launch_refine_finalize(ix->store.hi, ix->store.lo, ix->dp, ix->d, x_device, ix->d, sel_idx, n, k_list, (int)k,
                                  ix->metric, nullptr, label_offset, distances_device, labels_device, ix->device, s);
}

extern "C" int ann_cuda_flat_search_small_static_status(int device, void *stream) {
    DeviceGuard g(device);
    if (!g.ok) return set_error("cudaSetDevice(%d) failed", device);
    unsigned char *base = nullptr;
    if (static_scratch_base(device, &base)) return -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ANN_CUDA_TRY(cudaStreamSynchronize(s));
    int words[2] = {0, 0};
    ANN_CUDA_TRY(cudaMemcpy(words, base + kOffStatus, sizeof words, cudaMemcpyDeviceToHost));  // pageable target: no allocation
    ANN_CUDA_TRY(cudaMemset(base + kOffStatus, 0, sizeof words));
    if (words[0]) return set_error("allocation-free search: the flat kernel gave up on a wait (code %d); results are not valid", words[0]);
    if (words[1] == kScreenOverflow) return 1;
    return 0;
}
