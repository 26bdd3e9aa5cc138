// DiskANN batch-distance bridge for sm_100a: L2 / inner-product / SQ8-asymmetric
// distance of many (query, row) pairs in one launch.
//
// Replaces the reference's Metal bridge (src/metal_diskann_bridge.mm) and its
// four kernels (faiss-metal/shaders/diskann_distance.metal:15,64,111,155) behind
// the same three C symbols, and adds entry points that take row ids into a
// device-resident table.  The work is a pure stream over the candidate rows,
// so the kernels are shaped for HBM bandwidth: one warp per row, 128-bit
// loads that bypass L1 allocation for the rows, several rows in flight per
// warp, warp-shuffle reductions.  There is no CPU path in this file.
#include "cuda_diskann_bridge.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cstring>
#include <memory>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

using namespace anncuda;

// ---------------------------------------------------------------------------------------------
// Kernels
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ float4 ld_stream4(const float4 *p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint4 ld_stream4u(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float acc4(float acc, float4 q, float4 x, bool l2) {
    if (l2) {
        float a = q.x - x.x, b = q.y - x.y, c = q.z - x.z, d = q.w - x.w;
        acc = fmaf(a, a, acc);
        acc = fmaf(b, b, acc);
        acc = fmaf(c, c, acc);
        acc = fmaf(d, d, acc);
    } else {
        acc = fmaf(q.x, x.x, acc);
        acc = fmaf(q.y, x.y, acc);
        acc = fmaf(q.z, x.z, acc);
        acc = fmaf(q.w, x.w, acc);
    }
    return acc;
}

// fp32 rows.  WPR warps cooperate on one row (1 for large batches; 4 for the
// small single-query batches, where there are fewer rows than resident warps).
// ids == nullptr: row i is candidates[i*dim ...] (the reference's gathered layout,
// src/metal_diskann_bridge.mm:180-198); else row ids[i] of the table.
// qmap == nullptr: every row uses query 0.
template <int WPR, bool VEC4>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
batch_distance_f32_kernel(const float *__restrict__ table, size_t num, int dim, const float *__restrict__ queries,
                          int nq, const uint32_t *__restrict__ ids, const uint32_t *__restrict__ qmap, int total_n,
                          int metric, float *__restrict__ out, const diskann_cuda_batch *__restrict__ batches) {
    if (batches) {  // several batches in one launch: blockIdx.y picks the batch
        const diskann_cuda_batch b = batches[blockIdx.y];
        queries = b.queries;
        nq = b.nq;
        ids = b.ids;
        qmap = b.query_map;
        total_n = b.total_n;
        out = b.out_distances;
    }
    constexpr int kRowsPerBlock = kWarpsPerBlock / WPR;
    __shared__ float partial[kWarpsPerBlock];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = warp % WPR;  // which slice of the row this warp sums
    const bool l2 = (metric == 0);
    for (long long row0 = (long long)blockIdx.x * kRowsPerBlock; row0 < total_n;
         row0 += (long long)gridDim.x * kRowsPerBlock) {
        const long long i = row0 + warp / WPR;
        float acc = 0.f;
        bool valid = i < total_n;
        size_t r = 0;
        uint32_t qi = 0;
        if (valid) {
            r = ids ? (size_t)ids[i] : (size_t)i;
            qi = qmap ? qmap[i] : 0u;
            if (r >= num || qi >= (uint32_t)nq) valid = false;
        }
        if (valid) {
            const float *x = table + r * (size_t)dim;
            const float *q = queries + (size_t)qi * dim;
            if (VEC4) {
                const float4 *x4 = reinterpret_cast<const float4 *>(x);
                const float4 *q4 = reinterpret_cast<const float4 *>(q);
                const int n4 = dim >> 2;
                int c = sub * 32 + lane;
                constexpr int kStep = 32 * WPR;
                // four independent 16-byte loads in flight per lane
                for (; c + 3 * kStep < n4; c += 4 * kStep) {
                    float4 a0 = ld_stream4(x4 + c), a1 = ld_stream4(x4 + c + kStep);
                    float4 a2 = ld_stream4(x4 + c + 2 * kStep), a3 = ld_stream4(x4 + c + 3 * kStep);
                    acc = acc4(acc, __ldg(q4 + c), a0, l2);
                    acc = acc4(acc, __ldg(q4 + c + kStep), a1, l2);
                    acc = acc4(acc, __ldg(q4 + c + 2 * kStep), a2, l2);
                    acc = acc4(acc, __ldg(q4 + c + 3 * kStep), a3, l2);
                }
                for (; c < n4; c += kStep) acc = acc4(acc, __ldg(q4 + c), ld_stream4(x4 + c), l2);
            } else {
                for (int c = sub * 32 + lane; c < dim; c += 32 * WPR) {
                    float xv = __ldg(x + c), qv = __ldg(q + c);
                    if (l2) {
                        float t = qv - xv;
                        acc = fmaf(t, t, acc);
                    } else {
                        acc = fmaf(qv, xv, acc);
                    }
                }
            }
        }
        acc = warp_sum(acc);
        if (WPR > 1) {
            if (lane == 0) partial[warp] = acc;
            __syncthreads();
            if (sub == 0 && lane == 0) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < WPR; w++) s += partial[warp + w];
                acc = s;
            }
            __syncthreads();
        }
        if (sub == 0 && lane == 0 && i < total_n) {
            out[i] = valid ? (l2 ? acc : -acc) : __int_as_float(0x7fc00000);
        }
    }
}

// Several batches in one launch, fp32 rows: the rows of all batches form one sequence
// (row_off[b] = first row of batch b) that the warps of a grid sized to the GPU walk with a
// stride, one row per warp at a time; a warp keeps its place in the batch list as it advances.
template <bool VEC4>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
batch_distance_f32_multi_kernel(const float *__restrict__ table, size_t num, int dim,
                                const diskann_cuda_batch *__restrict__ batches, const int *__restrict__ row_off,
                                int nbatches, int metric) {
    const int lane = threadIdx.x & 31;
    const bool l2 = (metric == 0);
    const long long warps_total = (long long)gridDim.x * kWarpsPerBlock;
    const long long rows_all = row_off[nbatches];
    int b = 0;
    for (long long u = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); u < rows_all; u += warps_total) {
        while (u >= row_off[b + 1]) b++;  // u only grows
        const diskann_cuda_batch d = batches[b];
        const int i = (int)(u - row_off[b]);
        const size_t r = (size_t)d.ids[i];
        const uint32_t qi = d.query_map ? d.query_map[i] : 0u;
        const bool valid = r < num && qi < (uint32_t)d.nq;
        float acc = 0.f;
        if (valid) {
            const float *x = table + r * (size_t)dim;
            const float *q = d.queries + (size_t)qi * dim;
            if (VEC4) {
                const float4 *x4 = reinterpret_cast<const float4 *>(x);
                const float4 *q4 = reinterpret_cast<const float4 *>(q);
                const int n4 = dim >> 2;
                int c = lane;
                for (; c + 96 < n4; c += 128) {  // four independent 16-byte loads in flight per lane
                    float4 a0 = ld_stream4(x4 + c), a1 = ld_stream4(x4 + c + 32);
                    float4 a2 = ld_stream4(x4 + c + 64), a3 = ld_stream4(x4 + c + 96);
                    acc = acc4(acc, __ldg(q4 + c), a0, l2);
                    acc = acc4(acc, __ldg(q4 + c + 32), a1, l2);
                    acc = acc4(acc, __ldg(q4 + c + 64), a2, l2);
                    acc = acc4(acc, __ldg(q4 + c + 96), a3, l2);
                }
                for (; c < n4; c += 32) acc = acc4(acc, __ldg(q4 + c), ld_stream4(x4 + c), l2);
            } else {
                for (int c = lane; c < dim; c += 32) {
                    const float xv = __ldg(x + c), qv = __ldg(q + c);
                    if (l2) {
                        const float t = qv - xv;
                        acc = fmaf(t, t, acc);
                    } else {
                        acc = fmaf(qv, xv, acc);
                    }
                }
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) d.out_distances[i] = valid ? (l2 ? acc : -acc) : __int_as_float(0x7fc00000);
    }
}

// code/255 rounded exactly as an IEEE fp32 division: multiply by the rounded
// reciprocal, then one fused correction step.  Equal to (float)c / 255.0f for
// all 256 codes (checked exhaustively by the unit tests on the host formula).
__device__ __forceinline__ float code_over_255(float c) {
    const float inv = 1.0f / 255.0f;
    float q = __fmul_rn(c, inv);
    float r = fmaf(-q, 255.0f, c);
    return fmaf(r, inv, q);
}

// Dequantise one code exactly as the reference does, (code/255)*scale+min with
// separate roundings (rust_lib/src/provider.rs:142-143), and add to the sum.
__device__ __forceinline__ float sq8_acc(float acc, float q, uint32_t code, float s, float m, bool l2) {
    float xh = __fadd_rn(__fmul_rn(code_over_255((float)code), s), m);
    if (l2) {
        float t = q - xh;
        return fmaf(t, t, acc);
    }
    return fmaf(q, xh, acc);
}

// SQ8 rows with dim % 4 == 0 and dim <= 512.  Lane l owns the 4*WPL consecutive
// dimensions starting at 4*WPL*l of EVERY row, so its slice of scale/255 stays in
// registers for the whole kernel and its slice of (query - min) is rebuilt only
// when the query changes (rows of one query are adjacent in DiskANN's lock-step
// batches, rust_lib/src/disk_provider.rs:546-581).  A row is then WPL coalesced
// 4-byte loads per lane and nothing else: the only traffic per row is its codes.
//
// The kernel is bound by instruction issue, not by HBM, so the per-element work is
// cut to four instructions: a byte permute drops the code into the mantissa of
// 2^23 (giving the float 2^23 + code), one subtraction yields the code as a float,
// and two fused multiply-adds form (q - min) - code * (scale / 255) and its square.
// The dequantised value code * (scale / 255) + min differs from the reference's
// (code / 255) * scale + min (rust_lib/src/provider.rs:142-143) by at most an ulp
// or two of the product, orders of magnitude inside the 1e-4 distance tolerance.
// Eight rows are processed together so that eight independent sums are in flight.
constexpr int kSq8RowsPerWarp = 8;

// code byte `b` of word w as a float
template <int B>
__device__ __forceinline__ float code_as_float(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | B)) - 8388608.0f;
}

// Sums eight per-lane values over the warp with 9 shuffles instead of 40: each exchange
// halves the number of values a lane carries (the lane keeps the half its bit selects and
// adds the partner's copy of it).  Afterwards every lane holds the total of row lane >> 2.
__device__ __forceinline__ float warp_sum8(const float (&a)[8], int lane) {
    float b[4], c[2];
    const bool h4 = lane & 16, h3 = lane & 8, h2 = lane & 4;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float keep = h4 ? a[4 + i] : a[i];
        const float send = h4 ? a[i] : a[4 + i];
        b[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const float keep = h3 ? b[2 + i] : b[i];
        const float send = h3 ? b[i] : b[2 + i];
        c[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    const float keep = h2 ? c[1] : c[0];
    const float send = h2 ? c[0] : c[1];
    float v = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}

template <int WPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
batch_distance_sq8_regs_kernel(const uint8_t *__restrict__ codes, size_t num, int dim,
                               const float *__restrict__ mins, const float *__restrict__ scale,
                               const float *__restrict__ queries, int nq, const uint32_t *__restrict__ ids,
                               const uint32_t *__restrict__ qmap, int total_n, int metric,
                               float *__restrict__ out, const diskann_cuda_batch *__restrict__ batches) {
    if (batches) {
        const diskann_cuda_batch b = batches[blockIdx.y];
        queries = b.queries;
        nq = b.nq;
        ids = b.ids;
        qmap = b.query_map;
        total_n = b.total_n;
        out = b.out_distances;
    }
    const int lane = threadIdx.x & 31;
    const long long warp_global = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const long long warps_total = (long long)gridDim.x * kWarpsPerBlock;
    const bool l2 = (metric == 0);
    const int d0 = lane * 4 * WPL;   // first dimension of this lane
    const bool active = d0 < dim;    // dim is a multiple of 4 * WPL
    float s[WPL * 4];   // scale / 255 of my dimensions
    float qa[WPL * 4];  // L2: q - min;  IP: q * scale / 255
    float qmin = 0.f;   // IP: sum over my dimensions of q * min
#pragma unroll
    for (int j = 0; j < WPL * 4; j++) {
        s[j] = active ? __fdiv_rn(__ldg(scale + d0 + j), 255.0f) : 0.f;
        qa[j] = 0.f;
    }
    uint32_t cur_q = 0xffffffffu;
    auto load_query = [&](uint32_t qi) {
        cur_q = qi;
        qmin = 0.f;
#pragma unroll
        for (int j = 0; j < WPL * 4; j++) {
            const float qv = active ? __ldg(queries + (size_t)qi * dim + d0 + j) : 0.f;
            const float mv = active ? __ldg(mins + d0 + j) : 0.f;
            qa[j] = l2 ? qv - mv : qv * s[j];
            qmin = fmaf(qv, mv, qmin);
        }
    };
    // one element of one row: acc += ((q - min) - c * s)^2   or   acc += c * (q * s)
    auto step = [&](float acc, float c, int j) -> float {
        if (l2) {
            const float diff = fmaf(-c, s[j], qa[j]);
            return fmaf(diff, diff, acc);
        }
        return fmaf(c, qa[j], acc);
    };
    // contiguous run of row groups per warp: consecutive groups mostly share their query
    const long long n_groups = ((long long)total_n + kSq8RowsPerWarp - 1) / kSq8RowsPerWarp;
    const long long per_warp = (n_groups + warps_total - 1) / warps_total;
    const long long g_first = warp_global * per_warp;
    const long long g_last = g_first + per_warp < n_groups ? g_first + per_warp : n_groups;
    for (long long g = g_first; g < g_last; g++) {
        const long long base = g * kSq8RowsPerWarp;
        uint32_t w[kSq8RowsPerWarp][WPL];
        uint32_t qi[kSq8RowsPerWarp];
        bool ok[kSq8RowsPerWarp];
        bool same_query = true;
#pragma unroll
        for (int t = 0; t < kSq8RowsPerWarp; t++) {
            const long long i = base + t;
            ok[t] = false;
            qi[t] = 0;
#pragma unroll
            for (int j = 0; j < WPL; j++) w[t][j] = 0;
            if (i < total_n) {
                const size_t r = ids ? (size_t)ids[i] : (size_t)i;
                qi[t] = qmap ? qmap[i] : 0u;
                ok[t] = r < num && qi[t] < (uint32_t)nq;
                if (ok[t] && active) {
                    const uint32_t *p = reinterpret_cast<const uint32_t *>(codes + r * (size_t)dim + d0);
#pragma unroll
                    for (int j = 0; j < WPL; j++)
                        asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(w[t][j]) : "l"(p + j));
                }
                if (ok[t] && qi[t] != qi[0]) same_query = false;
                if (!ok[t]) same_query = false;
            } else {
                same_query = false;
            }
        }
        float acc[kSq8RowsPerWarp];
#pragma unroll
        for (int t = 0; t < kSq8RowsPerWarp; t++) acc[t] = 0.f;
        if (same_query) {  // warp-uniform: ids, map and bounds are the same in every lane
            if (qi[0] != cur_q) load_query(qi[0]);
#pragma unroll
            for (int j = 0; j < WPL; j++) {
#pragma unroll
                for (int t = 0; t < kSq8RowsPerWarp; t++) {
                    acc[t] = step(acc[t], code_as_float<0>(w[t][j]), j * 4 + 0);
                    acc[t] = step(acc[t], code_as_float<1>(w[t][j]), j * 4 + 1);
                    acc[t] = step(acc[t], code_as_float<2>(w[t][j]), j * 4 + 2);
                    acc[t] = step(acc[t], code_as_float<3>(w[t][j]), j * 4 + 3);
                }
            }
            if (!l2) {  // inner product: add this lane's share of q.min, the same for every row
#pragma unroll
                for (int t = 0; t < kSq8RowsPerWarp; t++) acc[t] += qmin;
            }
        } else {
#pragma unroll
            for (int t = 0; t < kSq8RowsPerWarp; t++) {
                if (base + t >= total_n || !ok[t]) continue;  // warp-uniform
                if (qi[t] != cur_q) load_query(qi[t]);
#pragma unroll
                for (int j = 0; j < WPL; j++) {
                    acc[t] = step(acc[t], code_as_float<0>(w[t][j]), j * 4 + 0);
                    acc[t] = step(acc[t], code_as_float<1>(w[t][j]), j * 4 + 1);
                    acc[t] = step(acc[t], code_as_float<2>(w[t][j]), j * 4 + 2);
                    acc[t] = step(acc[t], code_as_float<3>(w[t][j]), j * 4 + 3);
                }
                if (!l2) acc[t] += qmin;
            }
        }
        static_assert(kSq8RowsPerWarp == 8, "warp_sum8 reduces eight rows");
        const float v = warp_sum8(acc, lane);  // total of row lane >> 2
        if ((lane & 3) == 0) {
            bool good = false;
#pragma unroll
            for (int t = 0; t < kSq8RowsPerWarp; t++)
                if ((lane >> 2) == t) good = ok[t];
            const long long i = base + (lane >> 2);
            if (i < total_n) out[i] = good ? (l2 ? v : -v) : __int_as_float(0x7fc00000);
        }
    }
}

// SQ8 rows with dim % 16 == 0 and dim <= 512: integer dot products, pipelined through
// shared memory.
//
// Latency.  The register kernel above must read ids, then (dependent) the code rows, then
// compute, with room for only eight rows in flight per warp.  Here each warp runs a
// four-stage cp.async ring of eight rows per stage (ids are read 32 rows at a time, one
// block ahead; rows one to three groups ahead), so ~9 KB of codes per warp are always in
// flight while it computes on the oldest stage.
//
// Arithmetic.  With the latency hidden, converting every code to fp32 and doing two fused
// multiply-adds on it (>= 4 instructions per code) is what bounds the kernel, not HBM.  The
// distance is therefore split into the part that depends on the codes linearly and parts
// that do not depend on the query:
//     L2:  sum_d ((q_d - min_d) - s_d c_d)^2 = A - 2 sum_d w_d c_d + N_r,   w_d = (q_d - min_d) s_d
//     IP:  sum_d q_d (min_d + s_d c_d)       = sum_d q_d min_d + sum_d w_d c_d,  w_d = q_d s_d
// with s_d = scale_d / 255, A = sum_d (q_d - min_d)^2 once per query and N_r = sum_d (s_d c_d)^2
// once per row, computed when the table is registered.  sum_d w_d c_d runs on the integer
// dot-product instruction (dp4a, four codes per instruction): the weights of one query are
// put on a common power-of-two scale as 23-bit signed integers and cut into three byte limbs
// (two unsigned, the top one signed), so three dp4a per 4-code word give three exact integer
// sums, 0.75 instructions per code.  The sums are accumulated straight into the mantissa of
// 2^23 (resp. 2^23 + 2^22), which makes them floats without a conversion instruction.
//
// Accuracy.  The integer sums are exact; the weights carry 2^-23 of the largest weight of the
// query, which is what fp32 accumulation loses as well.  What the split adds is cancellation
// in A - 2 cross + N_r when a row almost coincides with the query, so a row whose distance
// comes out below 2% of A + N_r is recomputed in the direct form (q - min - s c)^2 from the
// codes still in shared memory.
constexpr int kPipeStages = 4;
constexpr int kPipeMaxDim = 512;
constexpr float kSq8ExactBelow = 0.02f;  // redo a row directly if dist < this * (A + N_r)

__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// d = c + sum of four products of the bytes of a (unsigned) and of b (unsigned / signed)
__device__ __forceinline__ uint32_t dp4a_uu(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int32_t dp4a_us(uint32_t a, uint32_t b, int32_t c) {
    int32_t d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// N_r = sum_d (s_d c_d)^2 of every row, for the kernel below
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
sq8_row_norms_kernel(const uint8_t *__restrict__ codes, size_t num, int dim, const float *__restrict__ scale,
                     float *__restrict__ norms) {
    const int lane = threadIdx.x & 31;
    const int words = dim >> 2;  // dim is a multiple of 16
    for (size_t r = (size_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); r < num;
         r += (size_t)gridDim.x * kWarpsPerBlock) {
        const uint32_t *row = reinterpret_cast<const uint32_t *>(codes + r * (size_t)dim);
        float acc = 0.f;
        for (int wi = lane; wi < words; wi += 32) {
            const uint32_t w = __ldg(row + wi);
            const float4 sv = __ldg(reinterpret_cast<const float4 *>(scale) + wi);
            const float v0 = (float)(w & 255u) * __fdiv_rn(sv.x, 255.0f);
            const float v1 = (float)((w >> 8) & 255u) * __fdiv_rn(sv.y, 255.0f);
            const float v2 = (float)((w >> 16) & 255u) * __fdiv_rn(sv.z, 255.0f);
            const float v3 = (float)(w >> 24) * __fdiv_rn(sv.w, 255.0f);
            acc = fmaf(v0, v0, acc);
            acc = fmaf(v1, v1, acc);
            acc = fmaf(v2, v2, acc);
            acc = fmaf(v3, v3, acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) norms[r] = acc;
    }
}

// WPL: 4-code words per lane (lane l owns words l, l + 32, ...); FULL: dim == 128 * WPL, so
// every lane owns WPL words and no load needs a predicate.
template <int WPL, bool L2, bool FULL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
batch_distance_sq8_dp4a_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ norms, size_t num, int dim,
                               const float *__restrict__ mins, const float *__restrict__ scale,
                               const float *__restrict__ queries, int nq, const uint32_t *__restrict__ ids,
                               const uint32_t *__restrict__ qmap, int total_n, float *__restrict__ out,
                               const diskann_cuda_batch *__restrict__ batches, const int *__restrict__ group_off,
                               int nbatches) {
    static_assert(kPipeStages == 4 && kSq8RowsPerWarp == 8, "one id block of 32 rows fills the four stages");
    extern __shared__ __align__(16) uint8_t sq8_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t kNone = 0xffffffffu;
    constexpr uint32_t kFull = 0xffffffffu;
    // A warp takes a CONTIGUOUS run of row groups, so that consecutive groups mostly share
    // their query and its registers are rebuilt once per query, not once per group.  With
    // several batches in one launch (batches != null) the groups of all batches form one
    // sequence (group_off[b] = first group of batch b) that is cut evenly over the warps of a
    // grid sized to the GPU; a run that crosses a batch boundary is worked off piece by piece.
    const int warps_total = (int)gridDim.x * kWarpsPerBlock;
    const int warp_global = (int)blockIdx.x * kWarpsPerBlock + warp;
    const int groups_all = batches ? group_off[nbatches] : (total_n + kSq8RowsPerWarp - 1) / kSq8RowsPerWarp;
    const int per_warp = (groups_all + warps_total - 1) / warps_total;
    const int run_first = warp_global * per_warp;
    if (run_first >= groups_all) return;  // whole warp; the kernel has no block-wide barrier
    const int run_end = min(groups_all, run_first + per_warp);
    // the piece being worked on (one batch): set before every call of process_piece below
    int n_my = run_end - run_first;
    int row_first = run_first * kSq8RowsPerWarp;
    int row_end = min(total_n, row_first + n_my * kSq8RowsPerWarp);

    const int stage_bytes = kSq8RowsPerWarp * dim;
    uint8_t *ring = sq8_smem + (size_t)warp * kPipeStages * stage_bytes;  // this warp's four stages
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
    const int words = dim >> 2;            // 4-code words per row
    const bool copier = lane < (dim >> 4);  // lane l copies 16-byte piece l of every row
    const uint8_t *copy_src = codes + lane * 16;
    const uint32_t copy_dst = ring_s + lane * 16;

    bool act[WPL];       // does word lane + 32 j exist?
    float sc[WPL * 4];   // scale / 255 of my dimensions
    uint32_t wl[WPL], wm[WPL], wh[WPL];  // byte limbs of my weights, four dimensions per word
    float back = 0.f;    // value of one unit of the integer weights
    float qconst = 0.f;  // L2: A = sum (q - min)^2;  IP: sum q * min
#pragma unroll
    for (int j = 0; j < WPL; j++) {
        act[j] = FULL || lane + 32 * j < words;
        float4 sv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (act[j]) sv = __ldg(reinterpret_cast<const float4 *>(scale) + lane + 32 * j);
        sc[4 * j] = __fdiv_rn(sv.x, 255.0f);
        sc[4 * j + 1] = __fdiv_rn(sv.y, 255.0f);
        sc[4 * j + 2] = __fdiv_rn(sv.z, 255.0f);
        sc[4 * j + 3] = __fdiv_rn(sv.w, 255.0f);
        wl[j] = wm[j] = wh[j] = 0u;
    }
    uint32_t cur_q = kNone;
    auto load_query = [&](uint32_t qi) {
        cur_q = qi;
        float w[WPL * 4];
        float part = 0.f, wmax = 0.f;
#pragma unroll
        for (int j = 0; j < WPL; j++) {
            float4 qv = make_float4(0.f, 0.f, 0.f, 0.f), mv = qv;
            if (act[j]) {
                qv = __ldg(reinterpret_cast<const float4 *>(queries + (size_t)qi * dim) + lane + 32 * j);
                mv = __ldg(reinterpret_cast<const float4 *>(mins) + lane + 32 * j);
            }
            const float qs[4] = {qv.x, qv.y, qv.z, qv.w}, ms[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                if (L2) {
                    const float qa = qs[e] - ms[e];
                    w[4 * j + e] = qa * sc[4 * j + e];
                    part = fmaf(qa, qa, part);
                } else {
                    w[4 * j + e] = qs[e] * sc[4 * j + e];
                    part = fmaf(qs[e], ms[e], part);
                }
                wmax = fmaxf(wmax, fabsf(w[4 * j + e]));
            }
        }
        qconst = warp_sum(part);
        wmax = warp_max(wmax);
        // common scale: the power of two above the largest weight maps to 2^22
        float inv = 0.f;
        back = 0.f;
        if (wmax > 1e-30f && wmax < 1e30f) {
            const float top = __int_as_float((__float_as_int(wmax) & 0x7f800000) + 0x00800000);
            inv = 4194304.0f / top;
            back = top / 4194304.0f;
        }
#pragma unroll
        for (int j = 0; j < WPL; j++) {
            uint32_t l = 0, m = 0, h = 0;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int v = __float2int_rn(w[4 * j + e] * inv);  // |v| <= 2^22
                l |= ((uint32_t)v & 255u) << (8 * e);
                m |= (((uint32_t)v >> 8) & 255u) << (8 * e);
                h |= (((uint32_t)v >> 16) & 255u) << (8 * e);  // signed byte: v >> 16 in [-64, 64]
            }
            wl[j] = l;
            wm[j] = m;
            wh[j] = h;
        }
    };
    // this lane's share of sum_d w_d c_d of one row, in integer weight units; `row` already
    // points at this lane's first word
    auto row_dot = [&](const uint32_t *row) -> float {
        uint32_t al = 0x4B000000u, am = 0x4B000000u;  // the float 2^23: sums land in its mantissa
        int32_t ah = 0x4B400000;                      // 2^23 + 2^22: room for a signed sum
#pragma unroll
        for (int j = 0; j < WPL; j++) {
            uint32_t w = 0;
            if (FULL || act[j]) w = row[32 * j];
            al = dp4a_uu(w, wl[j], al);
            am = dp4a_uu(w, wm[j], am);
            ah = dp4a_us(w, wh[j], ah);
        }
        const float fl = __uint_as_float(al) - 8388608.0f;
        const float fm = __uint_as_float(am) - 8388608.0f;
        const float fh = __int_as_float(ah) - 12582912.0f;
        return fmaf(fh, 65536.0f, fmaf(fm, 256.0f, fl));
    };
    // this lane's share of the L2 distance of one row in the direct form (rare path)
    auto row_exact = [&](const uint32_t *row, uint32_t qi) -> float {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < WPL; j++) {
            if (!act[j]) continue;
            const uint32_t w = row[32 * j];
            const float4 qv = __ldg(reinterpret_cast<const float4 *>(queries + (size_t)qi * dim) + lane + 32 * j);
            const float4 mv = __ldg(reinterpret_cast<const float4 *>(mins) + lane + 32 * j);
            const float qs[4] = {qv.x, qv.y, qv.z, qv.w}, ms[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float c = (float)((w >> (8 * e)) & 255u);
                const float diff = fmaf(-c, sc[4 * j + e], qs[e] - ms[e]);
                acc = fmaf(diff, diff, acc);
            }
        }
        return acc;
    };
    // distance from the reduced integer dot product `v` and the row's N_r
    auto finish = [&](float v, float nrm) -> float {
        return L2 ? fmaf(-2.0f * back, v, qconst + nrm) : -fmaf(back, v, qconst);
    };

    // Row ids, query numbers and row norms are read 32 rows (four groups, one per ring stage)
    // at a time, one block ahead of the copies that need them: lane L holds row 32 b + L of
    // the run; an unusable row (outside the run, id or query out of range) is kNone.
    auto fetch_block = [&](int blk, uint32_t &rid, uint32_t &rq, float &nrm) {
        rid = kNone;
        rq = kNone;
        nrm = 0.f;
        const int i = row_first + blk * 32 + lane;
        if (i < row_end) {
            const uint32_t r = ids ? ids[i] : (uint32_t)i;
            const uint32_t q = qmap ? qmap[i] : 0u;
            if ((size_t)r < num && q < (uint32_t)nq) {
                rid = r;
                rq = q;
                if (L2) nrm = __ldg(norms + r);
            }
        }
    };
    // starts the copies of group `sub` (0..3) of an id block into ring stage `sub`; always commits
    auto issue = [&](int sub, uint32_t rid) {
        const uint32_t dst = copy_dst + (uint32_t)(sub * stage_bytes);
#pragma unroll
        for (int t = 0; t < kSq8RowsPerWarp; t++) {
            const uint32_t r = __shfl_sync(kFull, rid, sub * 8 + t);
            if (r != kNone && copier) cp_async16(dst + (uint32_t)(t * dim), copy_src + (size_t)r * (uint32_t)dim);
        }
        cp_async_commit();
    };
    // distances of group `sub` of the current id block; `row0` is the index of its first row
    auto compute = [&](int sub, int row0, uint32_t rq, float nrm_reg) {
        const uint32_t *rows = reinterpret_cast<const uint32_t *>(ring + sub * stage_bytes) + lane;
        const uint32_t q0 = __shfl_sync(kFull, rq, sub * 8);
        const uint32_t same = __ballot_sync(kFull, rq == q0) >> (sub * 8);
        if (q0 != kNone && (same & 0xffu) == 0xffu) {
            // the usual case, eight valid rows of one query: straight-line code, eight
            // independent dot products for the scheduler to interleave
            float acc[kSq8RowsPerWarp];  // q0's registers were built before the wait
#pragma unroll
            for (int t = 0; t < kSq8RowsPerWarp; t++) acc[t] = row_dot(rows + t * words);
            const float v = warp_sum8(acc, lane);  // total of row lane >> 2
            const float nrm = __shfl_sync(kFull, nrm_reg, sub * 8 + (lane >> 2));
            float dist = finish(v, nrm);
            if (L2) {
                uint32_t redo = __ballot_sync(kFull, (lane & 3) == 0 && !(dist >= kSq8ExactBelow * (qconst + nrm)));
                while (redo) {  // warp-uniform, rare
                    const int owner = __ffs(redo) - 1;
                    redo &= redo - 1;
                    const float ex = warp_sum(row_exact(rows + (owner >> 2) * words, q0));
                    if (lane == owner) dist = ex;
                }
            }
            if ((lane & 3) == 0) out[row0 + (lane >> 2)] = dist;
        } else {
#pragma unroll 1
            for (int t = 0; t < kSq8RowsPerWarp; t++) {
                const uint32_t q = __shfl_sync(kFull, rq, sub * 8 + t);
                const float nrm = __shfl_sync(kFull, nrm_reg, sub * 8 + t);
                float dist = __int_as_float(0x7fc00000);
                if (q != kNone) {  // warp-uniform
                    if (q != cur_q) load_query(q);
                    dist = finish(warp_sum(row_dot(rows + t * words)), nrm);
                    if (L2 && !(dist >= kSq8ExactBelow * (qconst + nrm)))
                        dist = warp_sum(row_exact(rows + t * words, q));
                }
                if (lane == 0 && row0 + t < total_n) out[row0 + t] = dist;
            }
        }
    };
    auto process_piece = [&]() {
    uint32_t rid_a, rq_a, rid_b, rq_b;  // id blocks b and b + 1
    float nrm_a, nrm_b;
    fetch_block(0, rid_a, rq_a, nrm_a);
    fetch_block(1, rid_b, rq_b, nrm_b);
    issue(0, rid_a);
    issue(1, rid_a);
    issue(2, rid_a);
    // One loop body for all four stages (the stage is a run-time value): the body is large,
    // and four copies of it thrash the instruction cache for nothing.
#pragma unroll 1
    for (int n = 0; n < n_my; n++) {
        const int sub = n & 3;
        // start the copies of the group three ahead (stage (n + 3) & 3, freed by the last
        // step), then wait for this step's own group
        issue((sub + 3) & 3, sub == 0 ? rid_a : rid_b);
        {   // a new query's registers are built while this step's rows are still in flight
            const uint32_t q_next = __shfl_sync(kFull, rq_a, sub * 8);
            if (q_next != kNone && q_next != cur_q) load_query(q_next);
        }
        cp_async_wait<3>();
        __syncwarp();
        compute(sub, row_first + n * kSq8RowsPerWarp, rq_a, nrm_a);
        __syncwarp();  // everyone is done with this stage before it is refilled
        if (sub == 3) {
            rid_a = rid_b;
            rq_a = rq_b;
            nrm_a = nrm_b;
            fetch_block((n >> 2) + 2, rid_b, rq_b, nrm_b);
        }
    }
    cp_async_wait<0>();
    __syncwarp();
    };
    if (!batches) {
        process_piece();
        return;
    }
    int b = 0;  // batch holding group run_first: the last b with group_off[b] <= run_first
    {
        int hi = nbatches;
        while (hi - b > 1) {
            const int mid = (b + hi) >> 1;
            if (group_off[mid] <= run_first) b = mid;
            else hi = mid;
        }
    }
    for (int g = run_first; g < run_end; b++) {
        const int b_first = group_off[b], b_end = group_off[b + 1];
        const int piece_end = min(run_end, b_end);
        if (piece_end > g) {
            const diskann_cuda_batch d = batches[b];
            queries = d.queries;
            nq = d.nq;
            ids = d.ids;
            qmap = d.query_map;
            total_n = d.total_n;
            out = d.out_distances;
            n_my = piece_end - g;
            row_first = (g - b_first) * kSq8RowsPerWarp;
            row_end = min(total_n, row_first + n_my * kSq8RowsPerWarp);
            cur_q = kNone;  // query numbers of another batch mean other queries
            process_piece();
            g = piece_end;
        }
    }
}

// SQ8 rows, any dimension: one warp per row, byte loads.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
batch_distance_sq8_generic_kernel(const uint8_t *__restrict__ codes, size_t num, int dim,
                                  const float *__restrict__ mins, const float *__restrict__ scale,
                                  const float *__restrict__ queries, int nq, const uint32_t *__restrict__ ids,
                                  const uint32_t *__restrict__ qmap, int total_n, int metric,
                                  float *__restrict__ out, const diskann_cuda_batch *__restrict__ batches) {
    if (batches) {
        const diskann_cuda_batch b = batches[blockIdx.y];
        queries = b.queries;
        nq = b.nq;
        ids = b.ids;
        qmap = b.query_map;
        total_n = b.total_n;
        out = b.out_distances;
    }
    const int lane = threadIdx.x & 31;
    const bool l2 = (metric == 0);
    for (long long i = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); i < total_n;
         i += (long long)gridDim.x * kWarpsPerBlock) {
        size_t r = ids ? (size_t)ids[i] : (size_t)i;
        uint32_t qi = qmap ? qmap[i] : 0u;
        const bool ok = r < num && qi < (uint32_t)nq;
        float acc = 0.f;
        if (ok) {
            const uint8_t *c = codes + r * (size_t)dim;
            const float *q = queries + (size_t)qi * dim;
            for (int d = lane; d < dim; d += 32)
                acc = sq8_acc(acc, __ldg(q + d), (uint32_t)__ldg(c + d), __ldg(scale + d), __ldg(mins + d), l2);
        }
        acc = warp_sum(acc);
        if (lane == 0) out[i] = ok ? (l2 ? acc : -acc) : __int_as_float(0x7fc00000);
    }
}

__global__ void check_ids_kernel(const uint32_t *__restrict__ ids, const uint32_t *__restrict__ qmap, int total_n,
                                 size_t num, int nq, int *__restrict__ bad) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_n) return;
    if ((ids && (size_t)ids[i] >= num) || (qmap && qmap[i] >= (uint32_t)nq)) atomicExch(bad, 1);
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct diskann_cuda_table {
    int device = 0;
    size_t num = 0;
    int dim = 0;
    bool sq8 = false;
    bool owns_rows = false;
    void *rows = nullptr;  // float* or uint8_t*
    float *mins = nullptr;
    float *scale = nullptr;
    float *norms = nullptr;  // SQ8 with dim % 16 == 0, dim <= 512: sum_d (scale_d / 255 * code_d)^2 per row
};

namespace {

// One launch for one batch (batches == nullptr) or for nbatches of them (descriptors on the
// device; total_n is then the largest batch and nq / queries / ids / qmap / out are unused).
int launch_distance(const diskann_cuda_table &t, const float *queries, int nq, const uint32_t *ids,
                    const uint32_t *qmap, int total_n, int metric, float *out, cudaStream_t stream,
                    const diskann_cuda_batch *batches = nullptr, int nbatches = 1, bool aligned16 = true,
                    const int *group_off = nullptr, const int *row_off = nullptr, long long rows_all = 0) {
    const int sms = sm_count(t.device);
    unsigned gy = (unsigned)(batches ? nbatches : 1);
    // blocks per batch: enough to fill the GPU alone, fewer when many batches share it
    auto blocks_for = [&](long long want, long long cap) -> unsigned {
        if (batches) cap = std::max<long long>(1, std::min<long long>(cap, (2 * cap + nbatches - 1) / nbatches));
        return (unsigned)std::max<long long>(1, std::min(want, cap));
    };
    const bool q16 = batches ? aligned16 : ((reinterpret_cast<uintptr_t>(queries) & 15) == 0);
    if (!t.sq8) {
        const float *rows = static_cast<const float *>(t.rows);
        const bool vec = (t.dim % 4 == 0) && ((reinterpret_cast<uintptr_t>(rows) & 15) == 0) && q16;
        // fewer rows than resident warps: put four warps on each row
        const bool small = (batches ? rows_all : (long long)total_n) < sms * 16;
        if (batches && !small) {
            // exactly one wave of blocks for all batches together
            int per_sm = 0;
            if (vec)
                ANN_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, batch_distance_f32_multi_kernel<true>,
                                                                           kWarpsPerBlock * 32, 0));
            else
                ANN_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, batch_distance_f32_multi_kernel<false>,
                                                                           kWarpsPerBlock * 32, 0));
            const dim3 grid((unsigned)std::min<long long>((rows_all + kWarpsPerBlock - 1) / kWarpsPerBlock,
                                                          (long long)sms * std::max(per_sm, 1)));
            if (vec)
                batch_distance_f32_multi_kernel<true><<<grid, kWarpsPerBlock * 32, 0, stream>>>(rows, t.num, t.dim, batches,
                                                                                                row_off, nbatches, metric);
            else
                batch_distance_f32_multi_kernel<false><<<grid, kWarpsPerBlock * 32, 0, stream>>>(rows, t.num, t.dim, batches,
                                                                                                 row_off, nbatches, metric);
            count_launch();
            ANN_CUDA_TRY(cudaGetLastError());
            return 0;
        }
        const int wpr = small ? 4 : 1;
        const int rows_per_block = kWarpsPerBlock / wpr;
        dim3 grid(blocks_for(((long long)total_n + rows_per_block - 1) / rows_per_block, (long long)sms * 32), gy);
        dim3 block(kWarpsPerBlock * 32);
        if (small) {
            if (vec)
                batch_distance_f32_kernel<4, true><<<grid, block, 0, stream>>>(rows, t.num, t.dim, queries, nq, ids, qmap,
                                                                                total_n, metric, out, batches);
            else
                batch_distance_f32_kernel<4, false><<<grid, block, 0, stream>>>(rows, t.num, t.dim, queries, nq, ids,
                                                                                 qmap, total_n, metric, out, batches);
        } else {
            if (vec)
                batch_distance_f32_kernel<1, true><<<grid, block, 0, stream>>>(rows, t.num, t.dim, queries, nq, ids, qmap,
                                                                                total_n, metric, out, batches);
            else
                batch_distance_f32_kernel<1, false><<<grid, block, 0, stream>>>(rows, t.num, t.dim, queries, nq, ids,
                                                                                 qmap, total_n, metric, out, batches);
        }
    } else {
        const uint8_t *codes = static_cast<const uint8_t *>(t.rows);
        // words (4 codes) per lane: the smallest count that covers the row with 32 lanes
        int wpl = 0;
        for (int c = 1; c <= 4 && !wpl; c++)
            if (t.dim <= 128 * c && t.dim % (4 * c) == 0) wpl = c;
        const bool regs = wpl != 0 && ((reinterpret_cast<uintptr_t>(codes) & 3) == 0) && q16;
        const bool pipe = t.norms && (t.dim % 16 == 0) && t.dim <= kPipeMaxDim && total_n >= 4096 &&
                          ((reinterpret_cast<uintptr_t>(codes) & 15) == 0) && q16;
        const long long groups = ((long long)total_n + kSq8RowsPerWarp - 1) / kSq8RowsPerWarp;
        const long long group_blocks = (groups + kWarpsPerBlock - 1) / kWarpsPerBlock;
        if (pipe) {
            const size_t smem = (size_t)kWarpsPerBlock * kPipeStages * kSq8RowsPerWarp * t.dim;
            // several batches: one grid of two blocks per SM walks the groups of all of them
            const dim3 g(batches ? (unsigned)(sms * 2) : blocks_for(group_blocks, (long long)sms * 2), 1);
            const unsigned b = kWarpsPerBlock * 32;
#define ANN_LAUNCH_PIPE3(W, L2, FULL)                                                                          \
    do {                                                                                                       \
        ANN_CUDA_TRY(cudaFuncSetAttribute(batch_distance_sq8_dp4a_kernel<W, L2, FULL>,                         \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));            \
        batch_distance_sq8_dp4a_kernel<W, L2, FULL><<<g, b, smem, stream>>>(                                   \
            codes, t.norms, t.num, t.dim, t.mins, t.scale, queries, nq, ids, qmap, total_n, out, batches,      \
            group_off, nbatches);                                                                              \
    } while (0)
#define ANN_LAUNCH_PIPE(W)                                         \
    do {                                                           \
        const bool full = t.dim == 128 * (W);                      \
        if (metric == 0) {                                         \
            if (full) ANN_LAUNCH_PIPE3(W, true, true);             \
            else ANN_LAUNCH_PIPE3(W, true, false);                 \
        } else {                                                   \
            if (full) ANN_LAUNCH_PIPE3(W, false, true);            \
            else ANN_LAUNCH_PIPE3(W, false, false);                \
        }                                                          \
    } while (0)
            // words per lane when lane l owns words l, l + 32, ...
            switch ((t.dim / 4 + 31) / 32) {
            case 1: ANN_LAUNCH_PIPE(1); break;
            case 2: ANN_LAUNCH_PIPE(2); break;
            case 3: ANN_LAUNCH_PIPE(3); break;
            default: ANN_LAUNCH_PIPE(4); break;
            }
#undef ANN_LAUNCH_PIPE3
#undef ANN_LAUNCH_PIPE
        } else if (regs) {
            const dim3 g(blocks_for(group_blocks, (long long)sms * 4), gy);
            const unsigned b = kWarpsPerBlock * 32;
            switch (wpl) {
            case 1: batch_distance_sq8_regs_kernel<1><<<g, b, 0, stream>>>(codes, t.num, t.dim, t.mins, t.scale, queries, nq, ids, qmap, total_n, metric, out, batches); break;
            case 2: batch_distance_sq8_regs_kernel<2><<<g, b, 0, stream>>>(codes, t.num, t.dim, t.mins, t.scale, queries, nq, ids, qmap, total_n, metric, out, batches); break;
            case 3: batch_distance_sq8_regs_kernel<3><<<g, b, 0, stream>>>(codes, t.num, t.dim, t.mins, t.scale, queries, nq, ids, qmap, total_n, metric, out, batches); break;
            default: batch_distance_sq8_regs_kernel<4><<<g, b, 0, stream>>>(codes, t.num, t.dim, t.mins, t.scale, queries, nq, ids, qmap, total_n, metric, out, batches); break;
            }
        } else {
            const dim3 g(blocks_for(((long long)total_n + kWarpsPerBlock - 1) / kWarpsPerBlock, (long long)sms * 32), gy);
            batch_distance_sq8_generic_kernel<<<g, kWarpsPerBlock * 32, 0, stream>>>(
                codes, t.num, t.dim, t.mins, t.scale, queries, nq, ids, qmap, total_n, metric, out, batches);
        }
    }
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

// One call's worth of device staging for the host-pointer entry points.  The
// reference's bridge shares one ring of buffers between all threads with no
// lock (src/metal_diskann_bridge.mm:52-53,118-120); here every call takes a
// private context from a pool, so concurrent callers never share buffers.
struct CallCtx {
    int device = 0;
    cudaStream_t stream = nullptr;
    GrowBuf q, cand, ids, map, out, flag;
    GrowBuf desc;                // descriptor image of an asynchronous multi-batch launch
    cudaEvent_t done = nullptr;  // recorded after the launch that last read `desc`
};

struct BridgeState {
    std::mutex mu;
    bool probed = false;
    bool available = false;
    int device = 0;
    std::vector<CallCtx *> free_list;

    bool probe() {
        std::lock_guard<std::mutex> lock(mu);
        if (probed) return available;
        probed = true;
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
            cudaGetLastError();
            set_error("no CUDA device");
            return false;
        }
        const char *env = getenv("ANN_CUDA_DEVICE");
        device = env ? atoi(env) : 0;
        if (device < 0 || device >= count) device = 0;
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return false;
        if (prop.major != 10) {
            set_error("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
            return false;
        }
        available = true;
        return true;
    }

    CallCtx *acquire(int dev) {
        {
            std::lock_guard<std::mutex> lock(mu);
            for (size_t i = 0; i < free_list.size(); i++) {
                if (free_list[i]->device == dev) {
                    CallCtx *c = free_list[i];
                    free_list.erase(free_list.begin() + i);
                    return c;
                }
            }
        }
        CallCtx *c = new CallCtx();
        c->device = dev;
        if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete c;
            return nullptr;
        }
        return c;
    }
    void release(CallCtx *c) {
        std::lock_guard<std::mutex> lock(mu);
        free_list.push_back(c);
    }
};

BridgeState &state() {
    static BridgeState *s = new BridgeState();  // intentionally leaked: safe at process exit
    return *s;
}

struct CtxLease {
    CallCtx *ctx;
    explicit CtxLease(int dev) : ctx(state().acquire(dev)) {}
    ~CtxLease() {
        if (ctx) state().release(ctx);
    }
};

int host_call(const diskann_cuda_table *table, const float *gathered, const float *queries, int nq,
              const uint32_t *ids, const uint32_t *qmap, int total_n, int dim, int metric, float *out) {
    const int dev = table ? table->device : state().device;
    DeviceGuard guard(dev);
    if (!guard.ok) return set_error("cudaSetDevice(%d) failed", dev);
    CtxLease lease(dev);
    CallCtx *c = lease.ctx;
    if (!c) return set_error("could not create a CUDA stream");
    const size_t qbytes = (size_t)nq * dim * sizeof(float);
    const size_t obytes = (size_t)total_n * sizeof(float);
    if (c->q.ensure(qbytes) || c->out.ensure(obytes) || c->flag.ensure(sizeof(int))) return -1;
    ANN_CUDA_TRY(cudaMemcpyAsync(c->q.ptr, queries, qbytes, cudaMemcpyHostToDevice, c->stream));
    const uint32_t *d_ids = nullptr, *d_map = nullptr;
    if (ids) {
        if (c->ids.ensure((size_t)total_n * 4)) return -1;
        ANN_CUDA_TRY(cudaMemcpyAsync(c->ids.ptr, ids, (size_t)total_n * 4, cudaMemcpyHostToDevice, c->stream));
        d_ids = c->ids.as<uint32_t>();
    }
    if (qmap) {
        if (c->map.ensure((size_t)total_n * 4)) return -1;
        ANN_CUDA_TRY(cudaMemcpyAsync(c->map.ptr, qmap, (size_t)total_n * 4, cudaMemcpyHostToDevice, c->stream));
        d_map = c->map.as<uint32_t>();
    }
    diskann_cuda_table tmp;
    const diskann_cuda_table *t = table;
    if (!t) {
        const size_t cbytes = (size_t)total_n * dim * sizeof(float);
        if (c->cand.ensure(cbytes)) return -1;
        ANN_CUDA_TRY(cudaMemcpyAsync(c->cand.ptr, gathered, cbytes, cudaMemcpyHostToDevice, c->stream));
        tmp.device = dev;
        tmp.num = (size_t)total_n;
        tmp.dim = dim;
        tmp.rows = c->cand.ptr;
        t = &tmp;
    }
    ANN_CUDA_TRY(cudaMemsetAsync(c->flag.ptr, 0, sizeof(int), c->stream));
    if (d_ids || d_map) {
        check_ids_kernel<<<(total_n + 255) / 256, 256, 0, c->stream>>>(d_ids, d_map, total_n, t->num, nq,
                                                                      c->flag.as<int>());
        count_launch();
        ANN_CUDA_TRY(cudaGetLastError());
    }
    if (launch_distance(*t, c->q.as<float>(), nq, d_ids, d_map, total_n, metric, c->out.as<float>(), c->stream))
        return -1;
    int bad = 0;
    ANN_CUDA_TRY(cudaMemcpyAsync(out, c->out.ptr, obytes, cudaMemcpyDeviceToHost, c->stream));
    ANN_CUDA_TRY(cudaMemcpyAsync(&bad, c->flag.ptr, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    ANN_CUDA_TRY(cudaStreamSynchronize(c->stream));
    if (bad) return set_error("row id or query_map entry out of range");
    return 0;
}

int make_table(int device, const void *rows, bool rows_on_device, const float *mins, const float *scale, size_t num,
               int dim, bool sq8, diskann_cuda_table **out) {
    if (!out) return set_error("null output handle");
    *out = nullptr;
    if (!rows || num == 0 || dim <= 0 || (sq8 && (!mins || !scale))) return set_error("invalid table arguments");
    if (num > 0xffffffffull) return set_error("row ids are 32-bit: at most 2^32 rows");
    if (!state().probe()) return -1;
    DeviceGuard guard(device);
    if (!guard.ok) return set_error("cudaSetDevice(%d) failed", device);
    std::unique_ptr<diskann_cuda_table> t(new diskann_cuda_table());
    t->device = device;
    t->num = num;
    t->dim = dim;
    t->sq8 = sq8;
    const size_t bytes = num * (size_t)dim * (sq8 ? 1 : sizeof(float));
    if (rows_on_device) {
        t->rows = const_cast<void *>(rows);
    } else {
        ANN_CUDA_TRY(cudaMalloc(&t->rows, bytes));
        t->owns_rows = true;
        cudaError_t e = cudaMemcpy(t->rows, rows, bytes, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            cudaFree(t->rows);
            return set_error("table upload failed: %s", cudaGetErrorString(e));
        }
    }
    if (sq8) {
        cudaError_t e1 = cudaMalloc(&t->mins, (size_t)dim * 4), e2 = cudaMalloc(&t->scale, (size_t)dim * 4);
        if (e1 == cudaSuccess && e2 == cudaSuccess) {
            e1 = cudaMemcpy(t->mins, mins, (size_t)dim * 4, cudaMemcpyHostToDevice);
            e2 = cudaMemcpy(t->scale, scale, (size_t)dim * 4, cudaMemcpyHostToDevice);
        }
        if (e1 != cudaSuccess || e2 != cudaSuccess) {
            diskann_cuda_unregister(t.release());
            return set_error("SQ8 parameter upload failed");
        }
        if (dim % 16 == 0 && dim <= kPipeMaxDim && (reinterpret_cast<uintptr_t>(t->rows) & 15) == 0) {
            // per-row constants of the integer dot-product kernel, 4 bytes per row
            if (cudaMalloc(&t->norms, num * sizeof(float)) != cudaSuccess) {
                cudaGetLastError();
                diskann_cuda_unregister(t.release());
                return set_error("out of device memory for the SQ8 row norms");
            }
            size_t blocks = (num + kWarpsPerBlock - 1) / kWarpsPerBlock;
            const size_t cap = (size_t)sm_count(device) * 32;
            if (blocks > cap) blocks = cap;
            sq8_row_norms_kernel<<<(unsigned)blocks, kWarpsPerBlock * 32>>>(static_cast<const uint8_t *>(t->rows), num,
                                                                           dim, t->scale, t->norms);
            count_launch();
            cudaError_t e = cudaGetLastError();
            if (e == cudaSuccess) e = cudaDeviceSynchronize();
            if (e != cudaSuccess) {
                diskann_cuda_unregister(t.release());
                return set_error("SQ8 row norms failed: %s", cudaGetErrorString(e));
            }
        }
    }
    *out = t.release();
    return 0;
}

}  // namespace

extern "C" {

const char *diskann_cuda_last_error(void) { return last_error_ref().c_str(); }

int diskann_metal_available(void) { return state().probe() ? 1 : 0; }

int diskann_metal_batch_distances(const float *query, const float *candidates, int n, int dim, int metric,
                                  float *out_distances) {
    if (!query || !candidates || !out_distances || n <= 0 || dim <= 0) return set_error("invalid arguments");
    if (!state().probe()) return -1;
    return host_call(nullptr, candidates, query, 1, nullptr, nullptr, n, dim, metric, out_distances);
}

int diskann_metal_multi_batch_distances(const float *queries, const float *candidates, const unsigned int *query_map,
                                        int total_n, int nq, int dim, int metric, float *out_distances) {
    if (!queries || !candidates || !query_map || !out_distances || total_n <= 0 || nq <= 0 || dim <= 0)
        return set_error("invalid arguments");
    if (!state().probe()) return -1;
    return host_call(nullptr, candidates, queries, nq, nullptr, query_map, total_n, dim, metric, out_distances);
}

int diskann_cuda_register_table(int device, const float *host_rows, size_t num, int dim, diskann_cuda_table **out) {
    return make_table(device, host_rows, false, nullptr, nullptr, num, dim, false, out);
}

int diskann_cuda_register_table_device(int device, const float *device_rows, size_t num, int dim,
                                       diskann_cuda_table **out) {
    return make_table(device, device_rows, true, nullptr, nullptr, num, dim, false, out);
}

int diskann_cuda_register_sq8(int device, const uint8_t *codes, const float *mins, const float *scale, size_t num,
                              int dim, diskann_cuda_table **out) {
    return make_table(device, codes, false, mins, scale, num, dim, true, out);
}

int diskann_cuda_register_sq8_device(int device, const uint8_t *device_codes, const float *mins, const float *scale,
                                     size_t num, int dim, diskann_cuda_table **out) {
    return make_table(device, device_codes, true, mins, scale, num, dim, true, out);
}

int diskann_cuda_unregister(diskann_cuda_table *t) {
    if (!t) return 0;
    DeviceGuard guard(t->device);
    if (t->owns_rows && t->rows) cudaFree(t->rows);
    if (t->mins) cudaFree(t->mins);
    if (t->scale) cudaFree(t->scale);
    if (t->norms) cudaFree(t->norms);
    delete t;
    return 0;
}

int diskann_cuda_batch_distances_by_id(const diskann_cuda_table *table, const float *queries, int nq,
                                       const uint32_t *ids, const uint32_t *query_map, int total_n, int metric,
                                       float *out_distances) {
    if (!table || !queries || !ids || !out_distances || total_n <= 0 || nq <= 0)
        return set_error("invalid arguments");
    if (!query_map && nq != 1) return set_error("query_map may be NULL only when nq == 1");
    return host_call(table, nullptr, queries, nq, ids, query_map, total_n, table->dim, metric, out_distances);
}

int diskann_cuda_batch_distances_by_id_device(const diskann_cuda_table *table, const float *queries, int nq,
                                              const uint32_t *ids, const uint32_t *query_map, int total_n,
                                              int metric, float *out_distances, void *stream) {
    if (!table || !queries || !ids || !out_distances || total_n <= 0 || nq <= 0)
        return set_error("invalid arguments");
    if (!query_map && nq != 1) return set_error("query_map may be NULL only when nq == 1");
    DeviceGuard guard(table->device);
    if (!guard.ok) return set_error("cudaSetDevice(%d) failed", table->device);
    return launch_distance(*table, queries, nq, ids, query_map, total_n, metric, out_distances,
                           static_cast<cudaStream_t>(stream));
}

int diskann_cuda_batch_distances_by_id_device_multi(const diskann_cuda_table *table, const diskann_cuda_batch *batches,
                                                    int nbatches, int metric, void *stream) {
    if (!table || !batches || nbatches <= 0) return set_error("invalid arguments");
    if (nbatches > 65535) return set_error("at most 65535 batches per call");
    int max_n = 0;
    bool aligned16 = true;
    for (int i = 0; i < nbatches; i++) {
        const diskann_cuda_batch &b = batches[i];
        if (!b.queries || !b.ids || !b.out_distances || b.total_n <= 0 || b.nq <= 0)
            return set_error("batch %d: invalid arguments", i);
        if (!b.query_map && b.nq != 1) return set_error("batch %d: query_map may be NULL only when nq == 1", i);
        max_n = std::max(max_n, b.total_n);
        aligned16 = aligned16 && (reinterpret_cast<uintptr_t>(b.queries) & 15) == 0;
    }
    DeviceGuard guard(table->device);
    if (!guard.ok) return set_error("cudaSetDevice(%d) failed", table->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // stream-ordered copy of the descriptors: the host array is free on return, the device
    // copy is released after the kernel
    // device image: descriptors, then first group (8 rows) and first row of every batch in the
    // sequence of all batches
    const size_t desc_bytes = (size_t)nbatches * sizeof(diskann_cuda_batch);
    const size_t bytes = desc_bytes + 2 * (size_t)(nbatches + 1) * sizeof(int);
    std::vector<unsigned char> image(bytes);
    std::memcpy(image.data(), batches, desc_bytes);
    int *group_off = reinterpret_cast<int *>(image.data() + desc_bytes), *row_off = group_off + nbatches + 1;
    long long groups = 0, rows = 0;
    for (int i = 0; i < nbatches; i++) {
        group_off[i] = (int)groups;
        row_off[i] = (int)rows;
        groups += (batches[i].total_n + kSq8RowsPerWarp - 1) / kSq8RowsPerWarp;
        rows += batches[i].total_n;
    }
    if (rows > 0x7fffffffLL) return set_error("more than 2^31 rows in one call");
    group_off[nbatches] = (int)groups;
    row_off[nbatches] = (int)rows;
    // The device copy lives in a pooled per-call context (no allocation in the steady state);
    // an event recorded behind the launch keeps the next user of that context from overwriting
    // the image while this launch may still read it.
    CallCtx *c = state().acquire(table->device);
    if (!c) return set_error("could not create a call context");
    int rc = 0;
    if (c->done && cudaEventSynchronize(c->done) != cudaSuccess) rc = set_error("device error before the launch");
    if (rc == 0 && !c->done && cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming) != cudaSuccess)
        rc = set_error("could not create an event");
    if (rc == 0 && c->desc.ensure(bytes)) rc = -1;
    if (rc == 0) {
        unsigned char *dev = static_cast<unsigned char *>(c->desc.ptr);
        const cudaError_t e = cudaMemcpyAsync(dev, image.data(), bytes, cudaMemcpyHostToDevice, s);
        if (e != cudaSuccess) rc = set_error("descriptor upload failed: %s", cudaGetErrorString(e));
        if (rc == 0)
            rc = launch_distance(*table, nullptr, 0, nullptr, nullptr, max_n, metric, nullptr, s,
                                 reinterpret_cast<const diskann_cuda_batch *>(dev), nbatches, aligned16,
                                 reinterpret_cast<const int *>(dev + desc_bytes),
                                 reinterpret_cast<const int *>(dev + desc_bytes) + nbatches + 1, rows);
        cudaEventRecord(c->done, s);
    }
    state().release(c);
    return rc;
}

int diskann_cuda_parse_index(const void *image, size_t len, diskann_cuda_index_info *info) {
    if (!image || !info) return set_error("invalid arguments");
    const unsigned char *p = static_cast<const unsigned char *>(image);
    auto u32 = [&](size_t off) -> uint32_t {
        return (uint32_t)p[off] | ((uint32_t)p[off + 1] << 8) | ((uint32_t)p[off + 2] << 16) | ((uint32_t)p[off + 3] << 24);
    };
    std::memset(info, 0, sizeof *info);
    if (len < 32) return set_error("index image too small: %zu bytes, the header alone is 32", len);
    if (std::memcmp(p, "DANN", 4) != 0) return set_error("bad magic: not a .diskann image");
    if (u32(4) != 2) return set_error("unsupported .diskann version %u (2 expected)", u32(4));
    info->num_vectors = u32(8);
    info->dimension = u32(12);
    info->max_degree = u32(16);
    info->num_entry_points = u32(20);
    info->metric = p[24];
    info->build_complexity = u32(28);
    if (info->dimension == 0) return set_error("dimension 0 in the header");
    if (info->metric > 1) return set_error("unknown metric %u in the header", info->metric);
    info->entry_points_offset = 32;
    info->vectors_offset = 32 + (uint64_t)info->num_entry_points * 4;
    const uint64_t vec_bytes = (uint64_t)info->num_vectors * info->dimension * 4;
    info->adjacency_offset = info->vectors_offset + vec_bytes;
    info->standard_size = info->adjacency_offset + (uint64_t)info->num_vectors * info->max_degree * 4;
    if (info->standard_size > len)
        return set_error("index image truncated: %llu bytes needed, %zu given", (unsigned long long)info->standard_size, len);
    // optional SQ8 trailer
    const uint64_t t = info->standard_size;
    if (len > t + 4 && std::memcmp(p + t, "SQ8\0", 4) == 0) {
        if (len < t + 16) return set_error("SQ8 trailer truncated");
        const uint32_t sq_dim = u32(t + 4);
        const uint64_t qlen = (uint64_t)u32(t + 8) | ((uint64_t)u32(t + 12) << 32);
        if (sq_dim != info->dimension)
            return set_error("SQ8 trailer has dimension %u, the header %u", sq_dim, info->dimension);
        if (qlen != (uint64_t)info->num_vectors * info->dimension)
            return set_error("SQ8 trailer holds %llu code bytes, %llu expected", (unsigned long long)qlen,
                             (unsigned long long)info->num_vectors * info->dimension);
        info->sq8_min_offset = t + 16;
        info->sq8_scale_offset = info->sq8_min_offset + (uint64_t)sq_dim * 4;
        info->sq8_codes_offset = info->sq8_scale_offset + (uint64_t)sq_dim * 4;
        info->sq8_codes_size = qlen;
        if (info->sq8_codes_offset + qlen > len)
            return set_error("SQ8 section truncated: need %llu bytes, have %zu",
                             (unsigned long long)(info->sq8_codes_offset + qlen), len);
        info->has_sq8 = 1;
    }
    return 0;
}

int diskann_cuda_load_index(int device, const void *image, size_t len, diskann_cuda_index_info *info,
                            diskann_cuda_table **vectors, diskann_cuda_table **sq8) {
    if (!vectors) return set_error("null output handle");
    *vectors = nullptr;
    if (sq8) *sq8 = nullptr;
    diskann_cuda_index_info local;
    if (!info) info = &local;
    if (diskann_cuda_parse_index(image, len, info)) return -1;
    if (info->num_vectors == 0) return set_error("the index holds no vectors");
    if (info->dimension > 0x7fffffffu) return set_error("dimension too large");
    const unsigned char *p = static_cast<const unsigned char *>(image);
    // the segments sit at arbitrary byte offsets: copy through aligned host vectors
    std::vector<float> rows((size_t)info->num_vectors * info->dimension);
    std::memcpy(rows.data(), p + info->vectors_offset, rows.size() * 4);
    if (make_table(device, rows.data(), false, nullptr, nullptr, info->num_vectors, (int)info->dimension, false, vectors))
        return -1;
    if (sq8 && info->has_sq8) {
        std::vector<float> mins(info->dimension), scale(info->dimension);
        std::memcpy(mins.data(), p + info->sq8_min_offset, mins.size() * 4);
        std::memcpy(scale.data(), p + info->sq8_scale_offset, scale.size() * 4);
        if (make_table(device, p + info->sq8_codes_offset, false, mins.data(), scale.data(), info->num_vectors,
                       (int)info->dimension, true, sq8)) {
            diskann_cuda_unregister(*vectors);
            *vectors = nullptr;
            return -1;
        }
    }
    return 0;
}

int diskann_cuda_load_index_file(int device, const char *path, diskann_cuda_index_info *info,
                                 diskann_cuda_table **vectors, diskann_cuda_table **sq8) {
    if (!path) return set_error("null path");
    FILE *f = std::fopen(path, "rb");
    if (!f) return set_error("cannot open %s", path);
    std::vector<unsigned char> buf;
    if (std::fseek(f, 0, SEEK_END) == 0) {
        const long size = std::ftell(f);
        if (size > 0) buf.resize((size_t)size);
        std::rewind(f);
    }
    const size_t got = buf.empty() ? 0 : std::fread(buf.data(), 1, buf.size(), f);
    std::fclose(f);
    if (got != buf.size() || buf.empty()) return set_error("cannot read %s", path);
    return diskann_cuda_load_index(device, buf.data(), buf.size(), info, vectors, sq8);
}

}  // extern "C"
