// Row preparation kernels: TF32 hi/lo split, zero padding, row norms.
//
// The row-norm part takes the role of the reference's l2_norm shaders
// (faiss-metal/shaders/l2_norm.metal:7,30; faiss-metal/src/MetalL2Norm.mm:42-68):
// out[r] = sum_j x[r][j]^2 in fp32, computed when rows are added (database) or
// at the start of a search (queries).  All of it is streaming HBM work: one warp
// per row, coalesced loads, shuffle reduction.
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace anncuda {

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }
uint64_t launch_count_value() { return g_launches.load(std::memory_order_relaxed); }

namespace {

constexpr int kWarps = 8;

__device__ __forceinline__ float to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// MODE 0: split into hi/lo; MODE 1: pad only (out = hi).
template <int MODE>
__global__ void __launch_bounds__(kWarps * 32)
prep_rows_kernel(const float *__restrict__ x, int64_t n, int d, int dp, float *__restrict__ hi,
                 float *__restrict__ lo, float *__restrict__ norms) {
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); r < n; r += (int64_t)gridDim.x * kWarps) {
        const float *src = x + r * (int64_t)d;
        float acc = 0.f;
        for (int c = lane; c < dp; c += 32) {
            float v = c < d ? src[c] : 0.f;
            acc = fmaf(v, v, acc);
            if (MODE == 0) {
                float h = to_tf32(v);
                hi[r * (int64_t)dp + c] = h;
                lo[r * (int64_t)dp + c] = v - h;
            } else {
                hi[r * (int64_t)dp + c] = v;
            }
        }
        acc = warp_sum(acc);
        if (norms && lane == 0) norms[r] = acc;
    }
}

__global__ void __launch_bounds__(kWarps * 32)
join_rows_kernel(const float *__restrict__ hi, const float *__restrict__ lo, int64_t n, int d, int dp,
                 float *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); r < n; r += (int64_t)gridDim.x * kWarps)
        for (int c = lane; c < d; c += 32)
            out[r * (int64_t)d + c] = hi[r * (int64_t)dp + c] + (lo ? lo[r * (int64_t)dp + c] : 0.f);
}

__global__ void __launch_bounds__(kWarps * 32)
scatter_rows_kernel(const float *__restrict__ x, int64_t n, int d, int dp, const int64_t *__restrict__ dst_row,
                    float *__restrict__ hi, float *__restrict__ lo, float *__restrict__ norms) {
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); r < n; r += (int64_t)gridDim.x * kWarps) {
        const int64_t dst = dst_row[r];
        if (dst < 0) continue;  // warp-uniform
        float acc = 0.f;
        for (int c = lane; c < dp; c += 32) {
            const float v = c < d ? x[r * (int64_t)d + c] : 0.f;
            const float h = to_tf32(v);
            acc = fmaf(v, v, acc);
            hi[dst * (int64_t)dp + c] = h;
            lo[dst * (int64_t)dp + c] = v - h;
        }
        acc = warp_sum(acc);
        if (lane == 0) norms[dst] = acc;
    }
}

__global__ void __launch_bounds__(kWarps * 32)
split_gathered_kernel(const float *__restrict__ x, int d, int dp, const int32_t *__restrict__ qrow_query,
                      const int *__restrict__ n_tiles, int64_t max_rows, float *__restrict__ hi,
                      float *__restrict__ lo) {
    const int lane = threadIdx.x & 31;
    int64_t rows = (int64_t)(*n_tiles) * 128;
    if (rows > max_rows) rows = max_rows;
    for (int64_t g = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); g < rows; g += (int64_t)gridDim.x * kWarps) {
        const int32_t q = qrow_query[g];
        for (int c = lane; c < dp; c += 32) {
            const float v = (q >= 0 && c < d) ? x[q * (int64_t)d + c] : 0.f;
            const float h = to_tf32(v);
            hi[g * (int64_t)dp + c] = h;
            lo[g * (int64_t)dp + c] = v - h;
        }
    }
}

unsigned grid_for(int64_t n) {
    int64_t b = (n + kWarps - 1) / kWarps;
    if (b > 148 * 64) b = 148 * 64;
    if (b < 1) b = 1;
    return (unsigned)b;
}

}  // namespace

int launch_split_rows(const float *x, int64_t n, int d, int dp, float *hi, float *lo, float *norms,
                      cudaStream_t stream) {
    if (n <= 0) return 0;
    prep_rows_kernel<0><<<grid_for(n), kWarps * 32, 0, stream>>>(x, n, d, dp, hi, lo, norms);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_pad_rows(const float *x, int64_t n, int d, int dp, float *out, float *norms, cudaStream_t stream) {
    if (n <= 0) return 0;
    prep_rows_kernel<1><<<grid_for(n), kWarps * 32, 0, stream>>>(x, n, d, dp, out, nullptr, norms);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_join_rows(const float *hi, const float *lo, int64_t n, int d, int dp, float *out, cudaStream_t stream) {
    if (n <= 0) return 0;
    join_rows_kernel<<<grid_for(n), kWarps * 32, 0, stream>>>(hi, lo, n, d, dp, out);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_split_gathered(const float *x, int d, int dp, const int32_t *qrow_query, const int *n_tiles,
                          int64_t max_rows, float *hi, float *lo, cudaStream_t stream) {
    if (max_rows <= 0) return 0;
    split_gathered_kernel<<<grid_for(max_rows), kWarps * 32, 0, stream>>>(x, d, dp, qrow_query, n_tiles, max_rows, hi, lo);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_scatter_rows(const float *x, int64_t n, int d, int dp, const int64_t *dst_row, float *hi, float *lo,
                        float *norms, cudaStream_t stream) {
    if (n <= 0) return 0;
    scatter_rows_kernel<<<grid_for(n), kWarps * 32, 0, stream>>>(x, n, d, dp, dst_row, hi, lo, norms);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

}  // namespace anncuda
