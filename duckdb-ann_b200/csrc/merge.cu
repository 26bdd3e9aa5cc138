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
                   int k, int list_stride, int P_max,
                   float *__restrict__ out_key, int32_t *__restrict__ out_idx) {
    extern __shared__ float smem_f[];
    float *keys = smem_f;
    int32_t *vals = reinterpret_cast<int32_t *>(smem_f + P_max);
    const int64_t q = blockIdx.x;
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
                key = part_key[list * list_stride + j];
                val = idx;
            }
        }
        keys[t] = key;
        vals[t] = val;
    }
    bitonic_sort(keys, vals, P);
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
        const bool ok = j < P && vals[j] != 0x7fffffff;
        out_key[q * k + j] = ok ? keys[j] : kInf;
        out_idx[q * k + j] = ok ? vals[j] : -1;
    }
}

// Exact fp32 re-evaluation of the selected pairs, sort, and user-facing output.
__global__ void __launch_bounds__(128)
refine_finalize_kernel(const float *__restrict__ xhi, const float *__restrict__ xlo, int dp, int d,
                       const float *__restrict__ queries, int q_stride, const int32_t *__restrict__ sel_idx,
                       int k_sel, int k_out, int P, int metric, const int64_t *__restrict__ ids,
                       int64_t label_offset, float *__restrict__ out_d, int64_t *__restrict__ out_i) {
    extern __shared__ float smem_f[];
    float *keys = smem_f;
    int32_t *vals = reinterpret_cast<int32_t *>(smem_f + P);
    const int64_t q = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const bool l2 = metric != 0;
    const float *qv = queries + q * (int64_t)q_stride;
    for (int j = warp; j < P; j += nwarps) {
        float key = kInf;
        int32_t val = 0x7fffffff;
        if (j < k_sel) {
            const int32_t idx = sel_idx[q * k_sel + j];
            if (idx >= 0) {
                const float *h = xhi + (int64_t)idx * dp;
                const float *l = xlo ? xlo + (int64_t)idx * dp : nullptr;
                float acc = 0.f;
                for (int c = lane; c < d; c += 32) {
                    float x = h[c] + (l ? l[c] : 0.f);  // exact: lo = x - hi
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
                       int32_t *out_idx, int device, cudaStream_t stream) {
    (void)device;
    if (nq <= 0) return 0;
    const int total = nparts * k;
    if (total > kMaxCandidates) return set_error("merge: %d candidates per query exceeds %d", total, kMaxCandidates);
    const int P = next_pow2(total < 2 ? 2 : total);
    const size_t smem = (size_t)P * 8;
    if (opt_in_smem(merge_parts_kernel, smem)) return -1;
    merge_parts_kernel<<<(unsigned)nq, kMergeThreads, smem, stream>>>(part_key, part_idx, layout, lists_started, slot_of,
                                                                      nparts, nq, k, list_stride, P, out_key, out_idx);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_refine_finalize(const float *xhi, const float *xlo, int dp, int d, const float *queries, int q_stride,
                           const int32_t *sel_idx, int64_t nq, int k_sel, int k_out, int metric,
                           const int64_t *ids, int64_t label_offset, float *out_d, int64_t *out_i, int device,
                           cudaStream_t stream) {
    (void)device;
    if (nq <= 0) return 0;
    const int P = next_pow2(k_sel < 2 ? 2 : k_sel);
    const size_t smem = (size_t)P * 8;
    if (opt_in_smem(refine_finalize_kernel, smem)) return -1;
    refine_finalize_kernel<<<(unsigned)nq, 128, smem, stream>>>(xhi, xlo, dp, d, queries, q_stride, sel_idx, k_sel,
                                                                k_out, P, metric, ids, label_offset, out_d, out_i);
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
