// Second-stage k-selection: merges partial lists into sorted results.
//
// The first-stage kernels (tensor-core flat search, list scan) leave several
// unsorted k-lists per query, one per database chunk / probed list / GPU shard.
// Here one thread block per query loads all candidates into shared memory, sorts
// them with a bitonic network and writes the k best, best first.  This is the
// role of the reference's MetalSelect pass over a materialised distance row
// (faiss-metal/src/MetalSelect.mm:31-74), applied to k * parts candidates
// instead of the whole database.
#include "common.cuh"
#include "kernels.h"
#include "select.cuh"

namespace anncuda {
namespace {

constexpr int kMergeThreads = 256;
constexpr int kMaxCandidates = kMergeCandidates;
// 2 * 2^-21 |v||x| <= 0.25e-4 * dist  <=>  dist >= 0.038 |v||x|
constexpr float kRefineBelow = 0.04f;

// A gated kernel runs only behind a pass whose band check flagged an overflow (see kernels.h).
__device__ __forceinline__ bool gate_closed(const int *gate) { return gate && *gate != kScreenOverflow; }

__host__ __device__ inline int next_pow2(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

// Ascending bitonic sort of P (power of two) (key, val) pairs in shared memory.
// Ties are broken by val so the result does not depend on the input order.
__device__ void bitonic_sort(float *keys, int32_t *vals, int P) {
    for (int size = 2; size <= P; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int t = threadIdx.x; t < (P >> 1); t += blockDim.x) {
                int lo = 2 * t - (t & (stride - 1));
                int hi = lo + stride;
                bool asc = ((lo & size) == 0);
                float a = keys[lo], b = keys[hi];
                int32_t va = vals[lo], vb = vals[hi];
                bool a_after_b = (a > b) || (a == b && va > vb);
                if (a_after_b == asc) {
                    keys[lo] = b; keys[hi] = a;
                    vals[lo] = vb; vals[hi] = va;
                }
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kMergeThreads)
merge_parts_kernel(const float *__restrict__ part_key, const int32_t *__restrict__ part_idx, int layout,
                   const int *__restrict__ lists_started, const int32_t *__restrict__ slot_of, int nparts, int64_t nq,
                   int k, int list_stride, int P_max, const float *__restrict__ slot_key_offset,
                   float *__restrict__ out_key, int32_t *__restrict__ out_idx, const int *gate,
                   const int32_t *__restrict__ only_q, int k_out, float *__restrict__ complete_to) {
    extern __shared__ float smem_f[];
    // per list (up to 32 of them when complete_to is asked for): entries present, largest key
    __shared__ int list_cnt[32];
    __shared__ unsigned list_max[32];
    if (gate_closed(gate)) return;
    float *keys = smem_f;
    int32_t *vals = reinterpret_cast<int32_t *>(smem_f + P_max);
    const int64_t q = blockIdx.x;
    if (only_q && !only_q[q]) return;  // a pass that repairs the flagged queries only
    if (complete_to && threadIdx.x < 32) {
        list_cnt[threadIdx.x] = 0;
        list_max[threadIdx.x] = 0u;
    }
    if (complete_to) __syncthreads();
    int nlists = nparts;
    if (layout == 0) {
        const int started = lists_started[q >> 7];
        nlists = started < nparts ? started : nparts;
    }
    const int total = nlists * k;
    int P = 2;  // sort only as many slots as this query has candidates
    while (P < total) P <<= 1;
    if (P > P_max) P = P_max;
    for (int t = threadIdx.x; t < P; t += blockDim.x) {
        float key = kInf;
        int32_t val = 0x7fffffff;
        if (t < total) {
            const int p = t / k, j = t - p * k;
            int64_t list;
            if (layout == 0)
                list = ((q >> 7) * (int64_t)nparts + p) * 128 + (q & 127);
            else
                list = slot_of ? (int64_t)slot_of[q * nparts + p] : q * nparts + p;
            const int32_t idx = list >= 0 ? part_idx[list * list_stride + j] : -1;
            if (idx >= 0) {
                key = part_key[list * list_stride + j] + (slot_key_offset ? slot_key_offset[list] : 0.f);
                val = idx;
                if (complete_to) {
                    atomicAdd(&list_cnt[p], 1);
                    atomicMax(&list_max[p], float_to_ordered(key));
                }
            }
        }
        keys[t] = key;
        vals[t] = val;
    }
    bitonic_sort(keys, vals, P);
    // k_out entries go out (k_out >= k: the union of the lists holds more than one list's length)
    for (int j = threadIdx.x; j < k_out; j += blockDim.x) {
        const bool ok = j < P && vals[j] != 0x7fffffff;
        out_key[q * k_out + j] = ok ? keys[j] : kInf;
        out_idx[q * k_out + j] = ok ? vals[j] : -1;
    }
    // Every list holds the k best keys of ITS rows: a row that is in no list has a key at least as large as
    // the largest key of the (full) list its rows went to.  The union is therefore complete below the smallest
    // of those maxima - a list that is not full left nothing out.
    if (complete_to && threadIdx.x == 0) {
        float t_min = kInf;
        for (int p = 0; p < nlists; p++)
            if (list_cnt[p] >= k) t_min = fminf(t_min, ordered_to_float(list_max[p]));
        complete_to[q] = t_min;
    }
}

// The k best of a flagged query's candidate buffer (the rows the threshold scan appended, in no order),
// sorted best first.  left_q[q] says whether the query still needs the item scan: its buffer overflowed,
// it got no buffer, or the bound let fewer than k rows through (it was no bound at all).  The block also
// lays out the query's items for that scan (query q against rows [c * per, (c + 1) * per) for each of
// `chunks` chunks; "skip" unless the query is left).
__global__ void __launch_bounds__(kMergeThreads)
select_flagged_kernel(const float *__restrict__ cand_key, const int32_t *__restrict__ cand_idx,
                      const int *__restrict__ counts, const int32_t *__restrict__ rank_of,
                      const int32_t *__restrict__ over_q, int r_max, int cap, int k, float *__restrict__ out_key,
                      int32_t *__restrict__ out_idx, int32_t *__restrict__ left_q, int32_t *__restrict__ item_query,
                      int64_t *__restrict__ range_begin, int64_t *__restrict__ range_end, int chunks, int64_t per,
                      int64_t n, const int *gate) {
    extern __shared__ float smem_f[];
    if (gate_closed(gate)) return;
    const int64_t q = blockIdx.x;
    const bool flagged = over_q[q] != 0;
    const int r = flagged ? rank_of[q] : -1;
    const int cnt = (r >= 0 && r < r_max) ? counts[r] : -1;
    const bool left = flagged && (cnt < k || cnt > cap);
    if (threadIdx.x == 0) left_q[q] = left ? 1 : 0;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        const int64_t i = q * chunks + c;
        item_query[i] = left ? (int32_t)q : kItemSkip;
        range_begin[i] = c * per;
        range_end[i] = (c + 1) * per < n ? (c + 1) * per : n;
    }
    if (!flagged || left) return;
    int P = 2;
    while (P < cnt) P <<= 1;
    float *keys = smem_f;
    int32_t *vals = reinterpret_cast<int32_t *>(smem_f + P);
    for (int t = threadIdx.x; t < P; t += blockDim.x) {
        keys[t] = t < cnt ? cand_key[(int64_t)r * cap + t] : kInf;
        vals[t] = t < cnt ? cand_idx[(int64_t)r * cap + t] : 0x7fffffff;
    }
    bitonic_sort(keys, vals, P);
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
        out_key[q * k + j] = keys[j];
        out_idx[q * k + j] = vals[j];
    }
}

// (key, val) order used by every merge here: smaller key first, ties by smaller val
__device__ __forceinline__ bool pair_after(float a, int32_t va, float b, int32_t vb) {
    return (a > b) || (a == b && va > vb);
}

// Same result as merge_parts_kernel when every input list is already sorted best first:
// the lists are merged pairwise.  For two ascending lists A and B of K2 entries,
// min(A[i], B[K2-1-i]) is a bitonic sequence holding the K2 smallest of their union; a
// bitonic merge (log2 K2 steps, not log2^2) sorts it.  log2(lists) such rounds leave the
// answer in list 0.  For 16 lists of 128 this is ~8k compare-exchanges instead of ~68k.
__global__ void __launch_bounds__(kMergeThreads)
merge_sorted_kernel(const float *__restrict__ part_key, const int32_t *__restrict__ part_idx, int layout,
                    const int *__restrict__ lists_started, const int32_t *__restrict__ slot_of, int nparts, int64_t nq,
                    int k, int list_stride, int K2, int L2n, const float *__restrict__ slot_key_offset,
                    float *__restrict__ out_key, int32_t *__restrict__ out_idx, const int *gate) {
    extern __shared__ float smem_f[];
    if (gate_closed(gate)) return;
    float *keys = smem_f;                                              // [L2n][K2]
    int32_t *vals = reinterpret_cast<int32_t *>(smem_f + L2n * K2);
    const int64_t q = blockIdx.x;
    int nlists = nparts;
    if (layout == 0) {
        const int started = lists_started[q >> 7];
        nlists = started < nparts ? started : nparts;
    }
    int L = 1;  // lists that take part, rounded up to a power of two
    while (L < nlists) L <<= 1;
    const int kshift = 31 - __clz(K2);
    for (int t = threadIdx.x; t < L * K2; t += blockDim.x) {
        const int p = t >> kshift, j = t & (K2 - 1);
        float key = kInf;
        int32_t val = 0x7fffffff;
        if (p < nlists && j < k) {
            int64_t list;
            if (layout == 0)
                list = ((q >> 7) * (int64_t)nparts + p) * 128 + (q & 127);
            else
                list = slot_of ? (int64_t)slot_of[q * nparts + p] : q * nparts + p;
            const int32_t idx = list >= 0 ? part_idx[list * list_stride + j] : -1;
            if (idx >= 0) {
                key = part_key[list * list_stride + j] + (slot_key_offset ? slot_key_offset[list] : 0.f);
                val = idx;
            }
        }
        keys[t] = key;
        vals[t] = val;
    }
    __syncthreads();
    // `step` = distance between surviving lists; the survivor of a pair stays in the left slot
    for (int step = 1; step < L; step <<= 1) {
        const int pairs = L / (2 * step);
        for (int t = threadIdx.x; t < pairs * K2; t += blockDim.x) {
            const int p = t >> kshift, i = t & (K2 - 1);
            const int a = (2 * p * step) * K2 + i;
            const int b = ((2 * p + 1) * step) * K2 + (K2 - 1 - i);
            const float ka = keys[a], kb = keys[b];
            const int32_t va = vals[a], vb = vals[b];
            if (pair_after(ka, va, kb, vb)) {
                keys[a] = kb;
                vals[a] = vb;
            }
        }
        __syncthreads();
        for (int stride = K2 >> 1; stride > 0; stride >>= 1) {
            const int sshift = 31 - __clz(stride);
            for (int t = threadIdx.x; t < pairs * (K2 >> 1); t += blockDim.x) {
                const int p = t >> (kshift - 1), c = t & ((K2 >> 1) - 1);
                const int lo = (2 * p * step) * K2 + ((c >> sshift) << (sshift + 1)) + (c & (stride - 1));
                const int hi = lo + stride;
                const float ka = keys[lo], kb = keys[hi];
                const int32_t va = vals[lo], vb = vals[hi];
                if (pair_after(ka, va, kb, vb)) {
                    keys[lo] = kb; keys[hi] = ka;
                    vals[lo] = vb; vals[hi] = va;
                }
            }
            __syncthreads();
        }
    }
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
        const bool ok = vals[j] != 0x7fffffff;
        out_key[q * k + j] = ok ? keys[j] : kInf;
        out_idx[q * k + j] = ok ? vals[j] : -1;
    }
}

// Streaming top-k over the lists of one query's probes.  Candidates above the query's final
// threshold are dropped as they are read; the survivors collect in a shared buffer of `cap` pairs;
// when the next round of reads might not fit, the buffer is sorted, cut to its best k and its k-th
// key becomes the threshold.  Exact for any input and any number of lists; with the threshold the
// scan kernel leaves behind, the usual case is one small sort at the end.
constexpr int kFilterCap = 2048;
__global__ void __launch_bounds__(kMergeThreads)
merge_filtered_kernel(const float *__restrict__ part_key, const int32_t *__restrict__ part_idx,
                      const int32_t *__restrict__ part_cnt, const int32_t *__restrict__ slot_of,
                      const float *__restrict__ slot_key_offset, const uint32_t *__restrict__ qtau, int nparts,
                      int k, int list_stride, int cap, float *__restrict__ out_key, int32_t *__restrict__ out_idx,
                      const int *__restrict__ lists_started, const int *gate) {
    extern __shared__ float smem_f[];
    if (gate_closed(gate)) return;
    float *keys = smem_f;
    int32_t *vals = reinterpret_cast<int32_t *>(smem_f + cap);
    __shared__ int count;
    const int64_t q = blockIdx.x;
    if (threadIdx.x == 0) count = 0;
    // the scan's threshold was rounded up when it was published: a key equal to it stays in
    float tau = ordered_to_float(qtau[q]);
    if (!(tau == tau)) tau = kInf;  // nothing published
    __syncthreads();
    auto shrink = [&]() {  // sort what is there, keep the best k, tighten the threshold
        __syncthreads();
        const int c = count;
        int P = 2;
        while (P < c) P <<= 1;
        for (int t = c + threadIdx.x; t < P; t += blockDim.x) {
            keys[t] = kInf;
            vals[t] = 0x7fffffff;
        }
        bitonic_sort(keys, vals, P);
        if (c > k) {
            tau = fminf(tau, keys[k - 1]);
            __syncthreads();
            if (threadIdx.x == 0) count = k;
        }
        __syncthreads();
    };
    int nlists = nparts;
    if (lists_started) {
        const int started = lists_started[q >> 7];
        nlists = started < nparts ? started : nparts;
    }
    if (lists_started && !part_cnt) {
        // Whole lists of list_stride slots (empty ones carry index -1), many and short: one flat walk over
        // (list, slot) pairs instead of a loop over the lists (a single query of a small-k search has ~200
        // lists of 16 entries - a block-wide sort of all of them took 62 us, this takes a few).
        const int total = nlists * list_stride;
        for (int t0 = 0; t0 < total; t0 += blockDim.x) {
            __syncthreads();
            const int have = count;
            __syncthreads();
            if (have + (int)blockDim.x > cap) shrink();
            const int t = t0 + threadIdx.x;
            if (t < total) {
                const int p = t / list_stride, j = t - p * list_stride;
                const int64_t g = ((q >> 7) * (int64_t)nparts + p) * 128 + (q & 127);
                const int32_t idx = part_idx[(size_t)g * list_stride + j];
                const float key = part_key[(size_t)g * list_stride + j];
                if (idx >= 0 && key <= tau) {
                    const int pos = atomicAdd(&count, 1);
                    keys[pos] = key;
                    vals[pos] = idx;
                }
            }
        }
        nlists = 0;  // (done: the loop below has nothing left)
    }
    for (int p = 0; p < nlists; p++) {
        const int64_t g = lists_started ? ((q >> 7) * (int64_t)nparts + p) * 128 + (q & 127) : (int64_t)slot_of[q * nparts + p];
        if (g < 0) continue;  // block-uniform
        int c = part_cnt ? part_cnt[g] : list_stride;
        c = c < list_stride ? c : list_stride;
        const float off = slot_key_offset ? slot_key_offset[g] : 0.f;
        for (int j0 = 0; j0 < c; j0 += blockDim.x) {
            // Is there room for one more round of reads?  Every thread must take the same branch
            // (shrink() has barriers inside): the count is read between two barriers, after the
            // additions of the round before and before anybody adds again.
            __syncthreads();
            const int have = count;
            __syncthreads();
            if (have + (int)blockDim.x > cap) shrink();
            const int j = j0 + threadIdx.x;
            if (j < c) {
                const int32_t idx = part_idx[(size_t)g * list_stride + j];
                const float key = part_key[(size_t)g * list_stride + j] + off;
                if (idx >= 0 && key <= tau) {
                    const int pos = atomicAdd(&count, 1);
                    keys[pos] = key;
                    vals[pos] = idx;
                }
            }
        }
    }
    shrink();
    const int c = count;
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
        const bool ok = j < c && vals[j] != 0x7fffffff;
        out_key[q * k + j] = ok ? keys[j] : kInf;
        out_idx[q * k + j] = ok ? vals[j] : -1;
    }
}

// One kernel in place of three or four memsets in front of a flat_tc launch (see kernels.h).
__global__ void flat_scratch_init_kernel(uint32_t *qtau, size_t qtau_words, int *sched, size_t sched_ints, int32_t *cnt,
                                         size_t cnt_words, int32_t *idx, size_t lists, int list_stride, int k,
                                         const int *gate, int32_t *over_q, size_t nq) {
    if (gate_closed(gate)) return;
    const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x, step = (size_t)gridDim.x * blockDim.x;
    if (over_q)
        for (size_t i = t0; i < nq; i += step) over_q[i] = 0;
    for (size_t i = t0; i < qtau_words; i += step) qtau[i] = 0xffffffffu;
    for (size_t i = t0; i < sched_ints; i += step) sched[i] = 0;
    if (cnt)
        for (size_t i = t0; i < cnt_words; i += step) cnt[i] = 0;
    if (idx)
        for (size_t i = t0; i < lists * (size_t)k; i += step) idx[(i / k) * (size_t)list_stride + i % k] = -1;
}

// Band check of a tensor-core ranking.  The guarantee of the screened search (and of the split
// product with spare candidates) holds while the LAST of the k_list candidates of a query lies
// beyond the slack above its k_rank-th key.  If it is still inside that band, rows may have been
// left out: *overflow (0 so far) becomes kScreenOverflow and the search is repeated one tier up
// (split product, then the exact fp32 scan).
__global__ void screen_check_kernel(const float *__restrict__ sel_key, int64_t nq, int k_list, int k_rank,
                                    const float *__restrict__ q_norm2, const unsigned *__restrict__ x_max_norm2, int d,
                                    int l2, int screened, int *__restrict__ overflow, int *__restrict__ overflow_count,
                                    const int *gate) {
    if (gate_closed(gate)) return;
    const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= nq) return;
    const float last = sel_key[q * k_list + k_list - 1], kth = sel_key[q * k_list + k_rank - 1];
    if (last < kInf && last <= kth + key_slack(q_norm2[q], __uint_as_float(*x_max_norm2), d, l2 != 0, screened != 0)) {
        if (atomicCAS(overflow, 0, kScreenOverflow) == 0 && overflow_count) atomicAdd(overflow_count, 1);
    }
}

// Exact fp32 re-evaluation of the selected pairs, sort, and user-facing output.
__global__ void __launch_bounds__(128)
refine_finalize_kernel(const float *__restrict__ xhi, const float *__restrict__ xlo, int dp, int d,
                       const float *__restrict__ queries, int q_stride, const int32_t *__restrict__ sel_idx,
                       int k_sel, int k_out, int P, int metric, const int64_t *__restrict__ ids,
                       int64_t label_offset, const float *__restrict__ approx_key, const float *__restrict__ rnorm,
                       const float *__restrict__ xnorm, float *__restrict__ out_d, int64_t *__restrict__ out_i,
                       int32_t *__restrict__ out_row, const int *gate, const RefineBand band) {
    extern __shared__ float smem_f[];
    if (gate_closed(gate)) return;
    float *keys = smem_f;
    int32_t *vals = reinterpret_cast<int32_t *>(smem_f + P);
    const int64_t q = blockIdx.x;
    if (band.only_q && !band.only_q[q]) return;  // a pass that repairs the flagged queries only
    // candidates beyond the slack above the rank-th ranking key cannot be among the exact best
    float band_cut = kInf;
    if (band.key) {
        const float slack =
            key_slack(band.q_norm2[q], __uint_as_float(*band.x_max_norm2), band.d, metric != 0, band.one_mma, band.elem);
        if (band.cut && band.rank <= k_sel) band_cut = band.key[q * k_sel + band.rank - 1] + slack;
        // band check of the selecting pass: the last candidate still inside the band means rows may be missing
        if (threadIdx.x == 0 && band.check_rank > 0 && band.check_rank < k_sel) {
            float last = band.key[q * k_sel + k_sel - 1];
            const float kth = band.key[q * k_sel + band.check_rank - 1];
            // (candidates merged from several lists: complete only below the bound the merge found)
            if (band.complete_to) last = fminf(last, band.complete_to[q]);
            if ((last < kInf && last <= kth + slack) || (band.bad_q && band.bad_q[q])) {
                if (atomicCAS(band.overflow, 0, kScreenOverflow) == 0 && band.overflow_count) atomicAdd(band.overflow_count, 1);
                if (band.over_q) band.over_q[q] = 1;
            }
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const bool l2 = metric != 0;
    const float *qv = queries + q * (int64_t)q_stride;
    for (int j = warp; j < P; j += nwarps) {
        float key = kInf;
        int32_t val = 0x7fffffff;
        if (j < k_sel && !(band.key && band.cut && band.key[q * k_sel + j] > band_cut)) {
            const int32_t idx = sel_idx[q * k_sel + j];
            bool keep_approx = false;
            if (idx >= 0 && approx_key) {
                // The scan formed dist = |x - c|^2 - 2 v.x + const with v = q - c on split-TF32
                // tensor cores: the dot product is off by at most ~2^-21 |v| |x|, the distance by
                // twice that.  |v| <= |q - x| + |x - c| (triangle inequality), both known here.  Keep
                // the scan's value when that error is below a quarter of the 1e-4 tolerance.
                const float a = approx_key[q * k_sel + j];
                const float vmax = sqrtf(fmaxf(a, 0.f)) + sqrtf(rnorm[idx]);
                keep_approx = a >= kRefineBelow * vmax * sqrtf(xnorm[idx]);
                if (keep_approx) {
                    key = a;
                    val = idx;
                }
            }
            if (idx >= 0 && !keep_approx) {
                const float *h = xhi + (int64_t)idx * dp;
                const float *l = xlo ? xlo + (int64_t)idx * dp : nullptr;
                // (16-bit store: xhi holds dp elements of the band's type per row, widened exactly)
                const uint16_t *h16 = reinterpret_cast<const uint16_t *>(xhi) + (int64_t)idx * dp;
                float acc = 0.f;
                for (int c = lane; c < d; c += 32) {
                    float x = band.elem != kElemF32 ? h16_to_float(h16[c], band.elem)
                                                    : h[c] + (l ? l[c] : 0.f);  // exact: lo = x - hi
                    float a = qv[c];
                    if (l2) {
                        float t = a - x;
                        acc = fmaf(t, t, acc);
                    } else {
                        acc = fmaf(a, x, acc);
                    }
                }
                acc = warp_sum(acc);
                key = l2 ? acc : -acc;
                val = idx;
            }
        }
        if (lane == 0) {
            keys[j] = key;
            vals[j] = val;
        }
    }
    bitonic_sort(keys, vals, P);
    for (int j = threadIdx.x; j < k_out; j += blockDim.x) {
        const bool ok = j < k_sel && vals[j] != 0x7fffffff;
        if (out_row) {  // row numbers only (the coarse quantiser's probe lists)
            out_row[q * k_out + j] = ok ? vals[j] : -1;
            continue;
        }
        float dist = l2 ? kInf : -kInf;
        int64_t label = -1;
        if (ok) {
            dist = l2 ? keys[j] : -keys[j];
            label = ids ? ids[vals[j]] : (int64_t)vals[j] + label_offset;
        }
        out_d[q * k_out + j] = dist;
        out_i[q * k_out + j] = label;
    }
}

__global__ void finalize_kernel(const float *__restrict__ sel_key, const int32_t *__restrict__ sel_idx, int64_t nq,
                                int k_sel, int k_out, int metric, const int64_t *__restrict__ ids,
                                int64_t label_offset, float *__restrict__ out_d, int64_t *__restrict__ out_i) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nq * k_out) return;
    const int64_t q = t / k_out;
    const int j = (int)(t - q * k_out);
    const bool l2 = metric != 0;
    float dist = l2 ? kInf : -kInf;
    int64_t label = -1;
    if (j < k_sel) {
        const int32_t idx = sel_idx[q * k_sel + j];
        if (idx >= 0) {
            const float key = sel_key[q * k_sel + j];
            dist = l2 ? key : -key;
            label = ids ? ids[idx] : (int64_t)idx + label_offset;
        }
    }
    out_d[t] = dist;
    out_i[t] = label;
}

__global__ void __launch_bounds__(kMergeThreads)
merge_results_kernel(const float *__restrict__ parts_d, const int64_t *__restrict__ parts_i, int nparts, int64_t nq,
                     int k, int P, int metric, float *__restrict__ out_d, int64_t *__restrict__ out_i) {
    extern __shared__ float smem_f[];
    float *keys = smem_f;
    int32_t *vals = reinterpret_cast<int32_t *>(smem_f + P);
    const int64_t q = blockIdx.x;
    const bool l2 = metric != 0;
    const int total = nparts * k;
    for (int t = threadIdx.x; t < P; t += blockDim.x) {
        float key = kInf;
        int32_t val = 0x7fffffff;
        if (t < total) {
            const int p = t / k, j = t - p * k;
            const int64_t src = ((int64_t)p * nq + q) * k + j;
            if (parts_i[src] >= 0) {
                key = l2 ? parts_d[src] : -parts_d[src];
                val = t;
            }
        }
        keys[t] = key;
        vals[t] = val;
    }
    bitonic_sort(keys, vals, P);
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
        const bool ok = vals[j] != 0x7fffffff;
        float dist = l2 ? kInf : -kInf;
        int64_t label = -1;
        if (ok) {
            const int t = vals[j];
            const int p = t / k, jj = t - p * k;
            const int64_t src = ((int64_t)p * nq + q) * k + jj;
            dist = parts_d[src];
            label = parts_i[src];
        }
        out_d[q * k + j] = dist;
        out_i[q * k + j] = label;
    }
}

__global__ void fill_missing_kernel(float *d, int64_t *i, int64_t n, int metric) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    d[t] = metric != 0 ? kInf : -kInf;
    i[t] = -1;
}

template <class K>
int opt_in_smem(K kernel, size_t smem) {
    if (smem > 48 * 1024) ANN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    return 0;
}

}  // namespace

int launch_merge_parts(const float *part_key, const int32_t *part_idx, int layout, const int *lists_started,
                       const int32_t *slot_of, int nparts, int64_t nq, int k, int list_stride, float *out_key,
                       int32_t *out_idx, int device, cudaStream_t stream, bool lists_sorted,
                       const float *slot_key_offset, const int *gate, const int32_t *only_q, int k_out,
                       float *complete_to) {
    (void)device;
    if (only_q || complete_to || k_out > 0) lists_sorted = false;  // (the pairwise merge of sorted lists has none of these)
    if (k_out <= 0) k_out = k;
    if (k_out < k || (complete_to && nparts > 32)) return set_error("merge: invalid output length or too many lists");
    if (nq <= 0) return 0;
    const int total = nparts * k;
    if (total > kMaxCandidates) return set_error("merge: %d candidates per query exceeds %d", total, kMaxCandidates);
    if (lists_sorted) {
        const int K2 = next_pow2(k < 2 ? 2 : k), L2n = next_pow2(nparts);
        const size_t smem = (size_t)K2 * L2n * 8;
        if (smem <= 200 * 1024) {
            if (opt_in_smem(merge_sorted_kernel, smem)) return -1;
            merge_sorted_kernel<<<(unsigned)nq, kMergeThreads, smem, stream>>>(
                part_key, part_idx, layout, lists_started, slot_of, nparts, nq, k, list_stride, K2, L2n, slot_key_offset,
                out_key, out_idx, gate);
            count_launch();
            ANN_CUDA_TRY(cudaGetLastError());
            return 0;
        }
    }
    const int P = next_pow2(total < 2 ? 2 : total);
    const size_t smem = (size_t)P * 8;
    if (opt_in_smem(merge_parts_kernel, smem)) return -1;
    merge_parts_kernel<<<(unsigned)nq, kMergeThreads, smem, stream>>>(part_key, part_idx, layout, lists_started, slot_of,
                                                                      nparts, nq, k, list_stride, P, slot_key_offset, out_key,
                                                                      out_idx, gate, only_q, k_out, complete_to);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_select_flagged(const float *cand_key, const int32_t *cand_idx, const int *counts, const int32_t *rank_of,
                          const int32_t *over_q, int r_max, int cap, int64_t nq, int k, float *out_key, int32_t *out_idx,
                          int32_t *left_q, int32_t *item_query, int64_t *range_begin, int64_t *range_end, int chunks,
                          int64_t per, int64_t n, cudaStream_t stream, const int *gate) {
    if (nq <= 0) return 0;
    if (cap > kMaxCandidates || k > cap) return set_error("select: %d candidates per query exceeds %d", cap, kMaxCandidates);
    const size_t smem = (size_t)next_pow2(cap < 2 ? 2 : cap) * 8;
    if (opt_in_smem(select_flagged_kernel, smem)) return -1;
    select_flagged_kernel<<<(unsigned)nq, kMergeThreads, smem, stream>>>(cand_key, cand_idx, counts, rank_of, over_q, r_max,
                                                                         cap, k, out_key, out_idx, left_q, item_query,
                                                                         range_begin, range_end, chunks, per, n, gate);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_merge_filtered(const float *part_key, const int32_t *part_idx, const int32_t *part_cnt,
                          const int32_t *slot_of, const float *slot_key_offset, const uint32_t *qtau, int nparts,
                          int64_t nq, int k, int list_stride, float *out_key, int32_t *out_idx,
                          cudaStream_t stream, const int *lists_started, const int *gate) {
    if (nq <= 0) return 0;
    // room for the k kept entries plus one round of reads, as a power of two for the sort
    int cap = kFilterCap;
    while (cap < k + kMergeThreads) cap <<= 1;
    const size_t smem = (size_t)cap * 8;
    if (opt_in_smem(merge_filtered_kernel, smem)) return -1;
    merge_filtered_kernel<<<(unsigned)nq, kMergeThreads, smem, stream>>>(part_key, part_idx, part_cnt, slot_of,
                                                                        slot_key_offset, qtau, nparts, k, list_stride,
                                                                        cap, out_key, out_idx, lists_started, gate);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_screen_check(const float *sel_key, int64_t nq, int k_list, int k_rank, const float *q_norm2,
                        const unsigned *x_max_norm2, int d, int metric, bool screened, int *overflow,
                        int *overflow_count, cudaStream_t stream, const int *gate) {
    if (nq <= 0 || k_list <= k_rank) return 0;
    screen_check_kernel<<<(unsigned)((nq + 255) / 256), 256, 0, stream>>>(sel_key, nq, k_list, k_rank, q_norm2, x_max_norm2,
                                                                          d, metric != 0, screened ? 1 : 0, overflow,
                                                                          overflow_count, gate);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_flat_scratch_init(uint32_t *qtau, size_t qtau_words, int *sched, size_t sched_ints, int32_t *cnt,
                             size_t cnt_words, int32_t *idx, size_t lists, int list_stride, int k, cudaStream_t stream,
                             const int *gate, int32_t *over_q, size_t nq) {
    size_t most = qtau_words > sched_ints ? qtau_words : sched_ints;
    if (cnt && cnt_words > most) most = cnt_words;
    if (idx && lists * (size_t)k > most) most = lists * (size_t)k;
    if (most == 0) return 0;
    const unsigned blocks = (unsigned)std::min<size_t>((most + 255) / 256, 1184);
    flat_scratch_init_kernel<<<blocks, 256, 0, stream>>>(qtau, qtau_words, sched, sched_ints, cnt, cnt_words, idx, lists,
                                                         list_stride, k, gate, over_q, nq);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_refine_finalize(const float *xhi, const float *xlo, int dp, int d, const float *queries, int q_stride,
                           const int32_t *sel_idx, int64_t nq, int k_sel, int k_out, int metric,
                           const int64_t *ids, int64_t label_offset, float *out_d, int64_t *out_i, int device,
                           cudaStream_t stream, const float *approx_key, const float *rnorm, const float *xnorm,
                           int32_t *out_row, const int *gate, const RefineBand *band) {
    (void)device;
    if (nq <= 0) return 0;
    const int P = next_pow2(k_sel < 2 ? 2 : k_sel);
    const size_t smem = (size_t)P * 8;
    if (opt_in_smem(refine_finalize_kernel, smem)) return -1;
    refine_finalize_kernel<<<(unsigned)nq, 128, smem, stream>>>(xhi, xlo, dp, d, queries, q_stride, sel_idx, k_sel,
                                                                k_out, P, metric, ids, label_offset, approx_key, rnorm, xnorm,
                                                                out_d, out_i, out_row, gate,
                                                                band ? *band
                                                                     : RefineBand{nullptr, 0, nullptr, nullptr, 0, false, kElemF32,
                                                                                  false, 0, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr});
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_finalize(const float *sel_key, const int32_t *sel_idx, int64_t nq, int k_sel, int k_out, int metric,
                    const int64_t *ids, int64_t label_offset, float *out_d, int64_t *out_i, cudaStream_t stream) {
    const int64_t n = nq * k_out;
    if (n <= 0) return 0;
    finalize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(sel_key, sel_idx, nq, k_sel, k_out, metric, ids,
                                                                    label_offset, out_d, out_i);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_merge_results(const float *parts_d, const int64_t *parts_i, int nparts, int64_t nq, int k, int metric,
                         float *out_d, int64_t *out_i, int device, cudaStream_t stream) {
    (void)device;
    if (nq <= 0) return 0;
    const int total = nparts * k;
    if (total > kMaxCandidates) return set_error("merge: %d candidates per query exceeds %d", total, kMaxCandidates);
    const int P = next_pow2(total < 2 ? 2 : total);
    const size_t smem = (size_t)P * 8;
    if (opt_in_smem(merge_results_kernel, smem)) return -1;
    merge_results_kernel<<<(unsigned)nq, kMergeThreads, smem, stream>>>(parts_d, parts_i, nparts, nq, k, P, metric,
                                                                        out_d, out_i);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_fill_missing(float *d, int64_t *i, int64_t n, int metric, cudaStream_t stream) {
    if (n <= 0) return 0;
    fill_missing_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(d, i, n, metric);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

}  // namespace anncuda
