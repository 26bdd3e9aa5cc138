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

static std::atomic<uint64_t> g_wait_limit_ns{2000000000ull};
static std::atomic<int> g_withhold_after{-1};
uint64_t flat_wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }
void set_flat_wait_limit_ns(uint64_t ns) { g_wait_limit_ns.store(ns ? ns : 2000000000ull, std::memory_order_relaxed); }
int flat_test_withhold_after() { return g_withhold_after.load(std::memory_order_relaxed); }
void set_flat_test_withhold_after(int k_blocks) { g_withhold_after.store(k_blocks, std::memory_order_relaxed); }

namespace {

constexpr int kWarps = 8;

__device__ __forceinline__ float to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// MODE 0: split into hi/lo; MODE 1: pad only (out = hi).
// With `mu` (d floats) the norm is taken about mu, |x - mu|^2, and with `center_rows` the
// planes hold x - mu as well (queries); without it they hold x itself (database rows, so that
// hi + lo stays the stored row bit for bit).  Squared L2 distances do not change when the same
// vector is taken off both operands, but the dot product the tensor cores form then has the
// magnitude |q - mu||x| instead of |q||x|, and with it its absolute error.
template <int MODE>
__global__ void __launch_bounds__(kWarps * 32)
prep_rows_kernel(const float *__restrict__ x, int64_t n, int d, int dp, float *__restrict__ hi,
                 float *__restrict__ lo, float *__restrict__ norms, const float *__restrict__ mu, int center_rows,
                 unsigned *__restrict__ max_norm2_bits) {
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); r < n; r += (int64_t)gridDim.x * kWarps) {
        const float *src = x + r * (int64_t)d;
        float acc = 0.f, raw = 0.f;
        for (int c = lane; c < dp; c += 32) {
            float v = c < d ? src[c] : 0.f;
            const float w = (mu && c < d) ? v - mu[c] : v;
            acc = fmaf(w, w, acc);
            raw = fmaf(v, v, raw);
            if (center_rows) v = w;
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
        if (max_norm2_bits) {  // largest |x|^2 of the store (non-negative floats order like their bits)
            raw = warp_sum(raw);
            if (lane == 0) atomicMax(max_norm2_bits, __float_as_uint(raw));
        }
    }
}

// Rows or queries for a 16-bit store (elem = kElemF16 / kElemBF16; dp a multiple of 64 elements).
//  Database rows (center_rows = 0): h = the row rounded to the 16-bit type - from then on THAT is the stored
//    row; norms[r] = |h - mu|^2 and the store's largest |h|^2 are taken from the rounded values, so that
//    the keys formed from them belong to the rows that are kept.
//  Queries (center_rows = 1): w = q - mu is split into two 16-bit parts, h = round(w), l = round(w - h);
//    norms[r] = |w|^2 (unrounded).  A finite query element that overflows the 16-bit type (fp16: above
//    65504) makes every tensor-core key of the block meaningless: overflow[0..1] (the status words of the
//    two tensor-core tiers, may be null) are set to kScreenOverflow, which sends the block to the exact scan,
//    and bad_row[r] (may be null) says for every query whether it is such a one.
__global__ void __launch_bounds__(kWarps * 32)
prep_rows_h16_kernel(const float *__restrict__ x, int64_t n, int d, int dp, uint16_t *__restrict__ hi,
                     uint16_t *__restrict__ lo, float *__restrict__ norms, const float *__restrict__ mu, int center_rows,
                     unsigned *__restrict__ max_norm2_bits, int elem, int *__restrict__ overflow,
                     int32_t *__restrict__ bad_row) {
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); r < n; r += (int64_t)gridDim.x * kWarps) {
        const float *src = x + r * (int64_t)d;
        float acc = 0.f, raw = 0.f;
        bool bad = false;
        for (int c = lane; c < dp; c += 32) {
            const float v = c < d ? src[c] : 0.f;
            const float m = (mu && c < d) ? mu[c] : 0.f;
            if (center_rows) {
                const float w = v - m;
                const uint16_t hb = float_to_h16(w, elem);
                const float hf = h16_to_float(hb, elem);
                bad |= !isfinite(hf) && isfinite(w);
                hi[r * (int64_t)dp + c] = hb;
                if (lo) lo[r * (int64_t)dp + c] = float_to_h16(isfinite(hf) ? w - hf : 0.f, elem);
                acc = fmaf(w, w, acc);
            } else {
                const uint16_t hb = float_to_h16(v, elem);
                const float hf = h16_to_float(hb, elem);
                hi[r * (int64_t)dp + c] = hb;
                const float w = c < d ? hf - m : 0.f;
                acc = fmaf(w, w, acc);
                raw = fmaf(hf, hf, raw);
            }
        }
        acc = warp_sum(acc);
        if (norms && lane == 0) norms[r] = acc;
        if (max_norm2_bits) {
            raw = warp_sum(raw);
            if (lane == 0) atomicMax(max_norm2_bits, __float_as_uint(raw));
        }
        const bool any_bad = __any_sync(0xffffffffu, bad);
        if (bad_row && lane == 0) bad_row[r] = any_bad ? 1 : 0;  // (per row: the band checks count it as failed)
        if (overflow && any_bad && lane == 0) {
            overflow[0] = kScreenOverflow;
            overflow[1] = kScreenOverflow;
        }
    }
}

// mu[c] += (sum over this block's rows of x[r][c]) / n; mu zero on entry
__global__ void __launch_bounds__(128)
column_mean_kernel(const float *__restrict__ x, int64_t n, int d, float *__restrict__ mu) {
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c >= d) return;
    const int64_t per = (n + gridDim.y - 1) / gridDim.y;
    const int64_t r0 = blockIdx.y * per, r1 = r0 + per < n ? r0 + per : n;
    float acc = 0.f;
    for (int64_t r = r0; r < r1; r++) acc += x[r * (int64_t)d + c];
    if (r1 > r0) atomicAdd(mu + c, acc / (float)n);
}

// (elem != kElemF32: `hi` holds 16-bit elements, widened exactly)
__global__ void __launch_bounds__(kWarps * 32)
join_rows_kernel(const float *__restrict__ hi, const float *__restrict__ lo, int64_t n, int d, int dp,
                 float *__restrict__ out, int elem) {
    const int lane = threadIdx.x & 31;
    const uint16_t *h16 = reinterpret_cast<const uint16_t *>(hi);
    for (int64_t r = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); r < n; r += (int64_t)gridDim.x * kWarps)
        for (int c = lane; c < d; c += 32)
            out[r * (int64_t)d + c] = elem != kElemF32 ? h16_to_float(h16[r * (int64_t)dp + c], elem)
                                                       : hi[r * (int64_t)dp + c] + (lo ? lo[r * (int64_t)dp + c] : 0.f);
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
            acc = fmaf(v, v, acc);
            if (lo) {
                const float h = to_tf32(v);
                hi[dst * (int64_t)dp + c] = h;
                lo[dst * (int64_t)dp + c] = v - h;
            } else {  // one plane of plain rows
                hi[dst * (int64_t)dp + c] = v;
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) norms[dst] = acc;
    }
}

// Gathered query rows of the grouped list scan.  With centroids given (L2), row g becomes the
// residual v = q - c of its query against the centroid of the list its tile scans, and
// qconst[g] = |v|^2 + 2 v.c, so that for a list row x
//     |x - q|^2 = |x - c|^2 - 2 v.x + qconst[g]:
// the dot product the tensor cores form has the magnitude |v||x| instead of |q||x|, which
// takes an order of magnitude off its absolute error for clustered data.
__global__ void __launch_bounds__(kWarps * 32)
split_gathered_kernel(const float *__restrict__ x, int d, int dp, const int32_t *__restrict__ qrow_query,
                      const int *__restrict__ n_tiles, int64_t max_rows, const int4 *__restrict__ items,
                      const float *__restrict__ chi, const float *__restrict__ clo, float *__restrict__ hi,
                      float *__restrict__ lo, float *__restrict__ qconst) {
    const int lane = threadIdx.x & 31;
    int64_t rows = (int64_t)(*n_tiles) * 128;
    if (rows > max_rows) rows = max_rows;
    for (int64_t g = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); g < rows; g += (int64_t)gridDim.x * kWarps) {
        const int32_t q = qrow_query[g];
        const int64_t list = (chi && q >= 0) ? items[g >> 7].w : -1;
        float acc = 0.f;
        for (int c = lane; c < dp; c += 32) {
            float v = (q >= 0 && c < d) ? x[q * (int64_t)d + c] : 0.f;
            if (list >= 0 && c < d) {
                const float cen = chi[list * dp + c] + clo[list * dp + c];
                v -= cen;
                acc = fmaf(v, fmaf(2.f, cen, v), acc);  // v^2 + 2 v c
            }
            const float h = to_tf32(v);
            hi[g * (int64_t)dp + c] = h;
            lo[g * (int64_t)dp + c] = v - h;
        }
        if (qconst) {
            acc = warp_sum(acc);
            if (lane == 0) qconst[g] = acc;
        }
    }
}

// |x - c|^2 of every row of a list-grouped store, c = centroid of the row's list
__global__ void __launch_bounds__(kWarps * 32)
residual_norms_kernel(const float *__restrict__ xhi, const float *__restrict__ xlo, int64_t n, int d, int dp,
                      const int64_t *__restrict__ list_off, int nlist, const float *__restrict__ chi,
                      const float *__restrict__ clo, float *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); r < n; r += (int64_t)gridDim.x * kWarps) {
        int lo_l = 0, hi_l = nlist;  // list_off[lo_l] <= r < list_off[hi_l]
        while (hi_l - lo_l > 1) {
            const int mid = (lo_l + hi_l) >> 1;
            if (list_off[mid] <= r) lo_l = mid;
            else hi_l = mid;
        }
        float acc = 0.f;
        for (int c = lane; c < d; c += 32) {
            // (xlo null: xhi holds the plain rows)
            const float v = (xhi[r * (int64_t)dp + c] + (xlo ? xlo[r * (int64_t)dp + c] : 0.f)) -
                            (chi[(int64_t)lo_l * dp + c] + clo[(int64_t)lo_l * dp + c]);
            acc = fmaf(v, v, acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) out[r] = acc;
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
                      cudaStream_t stream, const float *mu, bool center_rows, unsigned *max_norm2_bits) {
    if (n <= 0) return 0;
    prep_rows_kernel<0><<<grid_for(n), kWarps * 32, 0, stream>>>(x, n, d, dp, hi, lo, norms, mu, center_rows ? 1 : 0,
                                                                 max_norm2_bits);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_column_mean(const float *x, int64_t n, int d, float *mu, cudaStream_t stream) {
    if (n <= 0) return 0;
    ANN_CUDA_TRY(cudaMemsetAsync(mu, 0, (size_t)d * sizeof(float), stream));
    dim3 grid((unsigned)((d + 127) / 128), (unsigned)(n < 64 ? n : 64));
    column_mean_kernel<<<grid, 128, 0, stream>>>(x, n, d, mu);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_pad_rows(const float *x, int64_t n, int d, int dp, float *out, float *norms, cudaStream_t stream) {
    if (n <= 0) return 0;
    prep_rows_kernel<1><<<grid_for(n), kWarps * 32, 0, stream>>>(x, n, d, dp, out, nullptr, norms, nullptr, 0, nullptr);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_split_rows_h16(const float *x, int64_t n, int d, int dp, void *hi, void *lo, float *norms, cudaStream_t stream,
                          const float *mu, bool center_rows, unsigned *max_norm2_bits, int elem, int *overflow,
                          int32_t *bad_row) {
    if (n <= 0) return 0;
    prep_rows_h16_kernel<<<grid_for(n), kWarps * 32, 0, stream>>>(x, n, d, dp, static_cast<uint16_t *>(hi),
                                                                  static_cast<uint16_t *>(lo), norms, mu, center_rows ? 1 : 0,
                                                                  max_norm2_bits, elem, overflow, bad_row);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_join_rows(const float *hi, const float *lo, int64_t n, int d, int dp, float *out, cudaStream_t stream, int elem) {
    if (n <= 0) return 0;
    join_rows_kernel<<<grid_for(n), kWarps * 32, 0, stream>>>(hi, lo, n, d, dp, out, elem);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_split_gathered(const float *x, int d, int dp, const int32_t *qrow_query, const int *n_tiles,
                          int64_t max_rows, float *hi, float *lo, cudaStream_t stream, const int4 *items,
                          const float *cent_hi, const float *cent_lo, float *qconst) {
    if (max_rows <= 0) return 0;
    split_gathered_kernel<<<grid_for(max_rows), kWarps * 32, 0, stream>>>(x, d, dp, qrow_query, n_tiles, max_rows, items,
                                                                          cent_hi, cent_lo, hi, lo, qconst);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_residual_norms(const float *xhi, const float *xlo, int64_t n, int d, int dp, const int64_t *list_off,
                          int nlist, const float *cent_hi, const float *cent_lo, float *out, cudaStream_t stream) {
    if (n <= 0) return 0;
    residual_norms_kernel<<<grid_for(n), kWarps * 32, 0, stream>>>(xhi, xlo, n, d, dp, list_off, nlist, cent_hi, cent_lo,
                                                                   out);
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
