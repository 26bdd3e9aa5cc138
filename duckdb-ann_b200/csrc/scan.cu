// Exact-fp32 scan of row ranges with fused warp k-selection.
//
// One warp owns one (query, row range) item: it streams the rows with 16-byte
// coalesced loads (lanes across the dimension), reduces each row's distance with
// warp shuffles and keeps the k best in a register-resident replace-max list, so
// no distance ever goes to memory.  Two callers:
//   - IVFFlat list scan: the item is (query, probed inverted list); this replaces
//     the reference's per-query host gather + distance + select
//     (faiss-metal/src/MetalIndexIVFFlat.mm:149-250) with lists resident in HBM;
//   - the "simt" flat kernel: items are (query, database chunk); same arithmetic as
//     the reference's fused_l2_topk_min / fused_ip_topk_max shaders
//     (faiss-metal/shaders/fused_l2_topk.metal:18,135) and used as an on-device
//     cross-check of the tensor-core path.
// Distances are the direct forms sum (q-x)^2 and sum q*x in fp32.
//
// Further down: the threshold scan of the flat search's exact tier (compact_flagged_kernel,
// scan_flagged_kernel), which cuts the work by rows instead of by query.
#include "common.cuh"
#include "kernels.h"
#include "select.cuh"

#include <algorithm>

namespace anncuda {
namespace {

constexpr int kWarps = 8;
constexpr int kRows = 8;  // rows in flight per warp

__device__ __forceinline__ float4 ld_row4(const float4 *p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}

template <int KR>
__global__ void __launch_bounds__(kWarps * 32)
scan_items_kernel(const float *__restrict__ x, const float *__restrict__ xlo, int dp, int d,
                  const float *__restrict__ queries, int q_stride, const int32_t *__restrict__ item_query,
                  const int64_t *__restrict__ range_begin, const int64_t *__restrict__ range_end, int64_t n_items,
                  int k, int metric, float *__restrict__ part_key, int32_t *__restrict__ part_idx,
                  uint32_t *__restrict__ qtau, const int *gate, int elem) {
    extern __shared__ float4 smem_q4[];
    if (gate && *gate != kScreenOverflow) return;  // a fallback pass that is not needed
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *myq = reinterpret_cast<float *>(smem_q4) + (size_t)warp * dp;
    const float4 *myq4 = reinterpret_cast<const float4 *>(myq);
    const bool l2 = metric != 0;  // FAISS codes: 1 = L2, 0 = inner product
    const int n4 = dp >> 2;
    for (int64_t item = (int64_t)blockIdx.x * kWarps + warp; item < n_items; item += (int64_t)gridDim.x * kWarps) {
        const int q = item_query[item];
        if (q == kItemSkip) continue;  // a query this pass does not repair: its lists are never read
        const int64_t begin = range_begin[item], end = range_end[item];
        float *lk = part_key + item * (int64_t)k;
        int32_t *li = part_idx + item * (int64_t)k;
        WarpList<KR> list;
        list.fill_empty(k, lane);
        for (int slot = lane; slot < k; slot += 32) li[slot] = -1;
        float m;
        int pos;
        list.argmax(lane, m, pos);
        // thr: a key must be below it to matter.  It is the smaller of this list's current
        // maximum and, when qtau is given, the best k-th key any other item of the same
        // query has published (items of one query scan different lists at different times).
        float thr = m, published = kInf;
        if (q >= 0 && begin < end) {
            __syncwarp();
            for (int c = lane; c < dp; c += 32) myq[c] = c < d ? queries[(int64_t)q * q_stride + c] : 0.f;
            __syncwarp();
            for (int64_t row0 = begin; row0 < end; row0 += kRows) {
                const int nrows = (int)((end - row0) < kRows ? (end - row0) : kRows);
                if (qtau) {
                    const uint32_t tg = __ldcg(qtau + q);
                    if (tg < float_to_ordered(thr)) thr = ordered_to_float(tg);
                }
                float acc[kRows];
#pragma unroll
                for (int r = 0; r < kRows; r++) acc[r] = 0.f;
                for (int c4 = lane; c4 < n4; c4 += 32) {
                    const float4 qv = myq4[c4];
                    float4 xv[kRows];
#pragma unroll
                    for (int r = 0; r < kRows; r++) {
                        if (r < nrows) {
                            const int64_t off = (row0 + r) * (int64_t)n4 + c4;
                            if (elem != kElemF32) {  // 16-bit rows: four elements are eight bytes
                                const uint2 b = __ldg(reinterpret_cast<const uint2 *>(x) + off);
                                xv[r].x = h16_to_float((uint16_t)(b.x & 0xffffu), elem);
                                xv[r].y = h16_to_float((uint16_t)(b.x >> 16), elem);
                                xv[r].z = h16_to_float((uint16_t)(b.y & 0xffffu), elem);
                                xv[r].w = h16_to_float((uint16_t)(b.y >> 16), elem);
                                continue;
                            }
                            xv[r] = ld_row4(reinterpret_cast<const float4 *>(x) + off);
                            if (xlo) {
                                float4 t = ld_row4(reinterpret_cast<const float4 *>(xlo) + off);
                                xv[r].x += t.x; xv[r].y += t.y; xv[r].z += t.z; xv[r].w += t.w;
                            }
                        }
                    }
#pragma unroll
                    for (int r = 0; r < kRows; r++) {
                        if (r < nrows) {
                            if (l2) {
                                float a = qv.x - xv[r].x, b = qv.y - xv[r].y, c = qv.z - xv[r].z, e = qv.w - xv[r].w;
                                acc[r] = fmaf(a, a, acc[r]);
                                acc[r] = fmaf(b, b, acc[r]);
                                acc[r] = fmaf(c, c, acc[r]);
                                acc[r] = fmaf(e, e, acc[r]);
                            } else {
                                acc[r] = fmaf(qv.x, xv[r].x, acc[r]);
                                acc[r] = fmaf(qv.y, xv[r].y, acc[r]);
                                acc[r] = fmaf(qv.z, xv[r].z, acc[r]);
                                acc[r] = fmaf(qv.w, xv[r].w, acc[r]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int r = 0; r < kRows; r++) acc[r] = warp_sum(acc[r]);
#pragma unroll
                for (int r = 0; r < kRows; r++) {
                    if (r < nrows) {
                        const float key = l2 ? acc[r] : -acc[r];
                        if (key < thr) {  // warp-uniform: every lane holds the same sum
                            if (lane == (pos & 31)) li[pos] = (int32_t)(row0 + r);
                            list.set(pos, key, lane);
                            list.argmax(lane, m, pos);
                            thr = fminf(thr, m);
                        }
                    }
                }
                if (qtau && m < published) {  // the list holds k rows: its maximum bounds the query's k-th best
                    published = m;
                    if (lane == 0) atomicMin(qtau + q, float_to_ordered(m));
                }
            }
        }
        list.store(lk, k, lane);
    }
}

// ---- threshold scan of the flagged queries ---------------------------------------------------
// The exact tier behind a tensor-core tier: that tier has already left k real rows with their exact
// distances in the output arrays of every query, flagged or not, so the k-th of them bounds the true
// k-th distance from above.  The flagged queries are compacted into a list, and one CTA takes one
// (row tile, group of QB flagged queries) item: the group's queries sit in shared memory, the warps
// share out the tile's rows (RB = 32 / QB rows at a time each), every lane accumulates its slice of the
// RB x QB dot products, a transposing butterfly (31 shuffles for 32 sums) leaves each lane with one
// finished (row, query) distance, and the lane appends the row to the query's candidate buffer if the
// distance is at or below the query's bound.  The parallelism comes from the rows, so a single flagged
// query is scanned by the whole device, and a row is read once for QB queries.  A query whose buffer
// overflows (more rows inside the bound than the buffer holds: duplicates by the thousand) or whose
// bound is not usable is left to the item scan above.
constexpr int kFilterTile = 256;  // rows of one work item

__device__ __forceinline__ float4 ld_row_any(const float *__restrict__ x, const float *__restrict__ xlo, int64_t off,
                                             int elem) {
    float4 v;
    if (elem != kElemF32) {  // 16-bit rows: four elements are eight bytes
        const uint2 b = __ldg(reinterpret_cast<const uint2 *>(x) + off);
        v.x = h16_to_float((uint16_t)(b.x & 0xffffu), elem);
        v.y = h16_to_float((uint16_t)(b.x >> 16), elem);
        v.z = h16_to_float((uint16_t)(b.y & 0xffffu), elem);
        v.w = h16_to_float((uint16_t)(b.y >> 16), elem);
        return v;
    }
    v = __ldg(reinterpret_cast<const float4 *>(x) + off);
    if (xlo) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(xlo) + off);
        v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
    }
    return v;
}

// Sums v[i] over the warp for all 32 i at once: lane l returns the total of v[l].
__device__ __forceinline__ float transpose_sum32(float (&v)[32], int lane) {
#pragma unroll
    for (int half = 16; half >= 1; half >>= 1) {
        const bool upper = (lane & half) != 0;
#pragma unroll
        for (int i = 0; i < half; i++) {
            const float send = upper ? v[i] : v[i + half];
            const float keep = upper ? v[i + half] : v[i];
            v[i] = keep + __shfl_xor_sync(kFullMask, send, half);
        }
    }
    return v[0];
}

// aux[0] = number of flagged queries, aux[1 + r] = the r-th of them; rank_of[q] = r or -1;
// counts[r] = 0 for the ranks that get a candidate buffer.
__global__ void __launch_bounds__(1024)
compact_flagged_kernel(const int32_t *__restrict__ over_q, int64_t nq, int *__restrict__ aux,
                       int32_t *__restrict__ rank_of, int *__restrict__ counts, int r_max, const int *gate) {
    __shared__ int warp_tot[32];
    __shared__ int base_s;
    if (gate && *gate != kScreenOverflow) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) base_s = 0;
    __syncthreads();
    for (int64_t start = 0; start < nq; start += 1024) {
        const int64_t i = start + tid;
        const bool f = i < nq && over_q[i] != 0;
        const unsigned b = __ballot_sync(kFullMask, f);
        if (lane == 0) warp_tot[warp] = __popc(b);
        __syncthreads();
        int off = base_s;
        for (int w = 0; w < warp; w++) off += warp_tot[w];
        off += __popc(b & ((1u << lane) - 1u));
        if (i < nq) rank_of[i] = f ? off : -1;
        if (f) {
            aux[1 + off] = (int)i;
            if (off < r_max) counts[off] = 0;
        }
        __syncthreads();
        if (tid == 0) {
            int t = 0;
            for (int w = 0; w < 32; w++) t += warp_tot[w];
            base_s += t;
        }
        __syncthreads();
    }
    if (tid == 0) aux[0] = base_s;
}

template <int QB>
__global__ void __launch_bounds__(kWarps * 32, 3)
scan_flagged_kernel(const float *__restrict__ x, const float *__restrict__ xlo, int dp, int d, int64_t n,
                    const float *__restrict__ queries, int q_stride, const int *__restrict__ aux, int *counts, int r_max,
                    int cap, int k_out, int k_last, const float *__restrict__ out_d, const int64_t *__restrict__ out_i,
                    const unsigned *__restrict__ x_max_norm2, int metric, float *__restrict__ cand_key,
                    int32_t *__restrict__ cand_idx, const int *gate, int elem, int round_tiles) {
    constexpr int RB = 32 / QB;  // rows a warp has in flight: RB x QB sums fill the butterfly
    extern __shared__ float4 smem_q4[];
    __shared__ float s_thr[QB];
    __shared__ int s_rank[QB];
    if (gate && *gate != kScreenOverflow) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *sq = reinterpret_cast<float *>(smem_q4);
    const bool l2 = metric != 0;
    const int n4 = dp >> 2;
    int nf = aux[0];
    if (nf > r_max) nf = r_max;
    if (nf <= 0) return;
    const int n_groups = (nf + QB - 1) / QB;
    const int64_t n_tiles = (n + kFilterTile - 1) / kFilterTile;
    const int64_t n_items = n_tiles * n_groups;
    // Both this scan and the re-ranking that left the bound sum d products in fp32, each within
    // ~d 2^-24 of the exact value relative to the sum of the terms' magnitudes: twice that, doubled.
    const float eps = 4.f * (float)(d + 4) * 5.9604645e-8f;
    const float xm2 = __uint_as_float(*x_max_norm2);
    const int my_r = lane / QB, my_qi = lane % QB;  // the (row, query) pair whose sum this lane ends up with
    // Order of the items: the tiles go in rounds of round_tiles (a few dozen MB of rows); within a round every
    // group takes all its tiles before the next group starts.  CTAs that run together are thus spread over
    // many tiles (and L2 slices), and the later groups of a round find its rows in L2.
    const int64_t round_items = (int64_t)round_tiles * n_groups;
    for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
        const int64_t round = item / round_items;
        const int64_t rem = item - round * round_items;
        const int64_t first = round * round_tiles;
        const int64_t tcount = n_tiles - first < round_tiles ? n_tiles - first : round_tiles;
        const int g = (int)(rem / tcount);
        const int64_t tile = first + (rem - g * tcount);
        __syncthreads();  // the item before is done with the queries and bounds
        for (int qi = warp; qi < QB; qi += kWarps) {
            int r = g * QB + qi;
            if (r >= nf || __ldcg(counts + r) > cap) r = -1;  // (a buffer that has overflowed is a lost cause)
            const int q = r >= 0 ? aux[1 + r] : -1;
            float qn = 0.f;
            for (int c = lane; c < dp; c += 32) {
                const float v = (q >= 0 && c < d) ? queries[(int64_t)q * q_stride + c] : 0.f;
                sq[qi * dp + c] = v;
                qn = fmaf(v, v, qn);
            }
            qn = warp_sum(qn);
            float t = -kInf;  // nothing passes
            if (q >= 0) {
                const float dist = out_d[(int64_t)q * k_out + k_last];
                const int64_t label = out_i[(int64_t)q * k_out + k_last];
                const float key = l2 ? dist : -dist;
                const float slack = l2 ? key * eps : eps * sqrtf(qn * xm2);
                // no k-th row, or a distance that is no number: every row passes and the buffer overflows
                t = (label >= 0 && key == key && fabsf(key) < kInf) ? key + slack : kInf;
            }
            if (lane == 0) {
                s_rank[qi] = r;
                s_thr[qi] = t;
            }
        }
        __syncthreads();
        const int rank = s_rank[my_qi];
        const float thr = s_thr[my_qi];
        const float4 *sq4 = reinterpret_cast<const float4 *>(sq);
        const int64_t begin = tile * kFilterTile;
        const int64_t end = begin + kFilterTile < n ? begin + kFilterTile : n;
        for (int64_t row0 = begin + warp * RB; row0 < end; row0 += kWarps * RB) {
            float acc[32];
#pragma unroll
            for (int i = 0; i < 32; i++) acc[i] = 0.f;
            float4 xn[RB];
#pragma unroll
            for (int r = 0; r < RB; r++)
                xn[r] = (row0 + r < end && lane < n4) ? ld_row_any(x, xlo, (row0 + r) * (int64_t)n4 + lane, elem)
                                                      : make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c4 = lane; c4 < n4; c4 += 32) {
                float4 xv[RB];
#pragma unroll
                for (int r = 0; r < RB; r++) {
                    xv[r] = xn[r];
                    if (c4 + 32 < n4 && row0 + r < end) xn[r] = ld_row_any(x, xlo, (row0 + r) * (int64_t)n4 + c4 + 32, elem);
                }
#pragma unroll
                for (int qi = 0; qi < QB; qi++) {
                    const float4 qv = sq4[qi * n4 + c4];
#pragma unroll
                    for (int r = 0; r < RB; r++) {
                        float s = acc[r * QB + qi];
                        if (l2) {
                            const float a = qv.x - xv[r].x, b = qv.y - xv[r].y, c = qv.z - xv[r].z, e = qv.w - xv[r].w;
                            s = fmaf(a, a, s);
                            s = fmaf(b, b, s);
                            s = fmaf(c, c, s);
                            s = fmaf(e, e, s);
                        } else {
                            s = fmaf(qv.x, xv[r].x, s);
                            s = fmaf(qv.y, xv[r].y, s);
                            s = fmaf(qv.z, xv[r].z, s);
                            s = fmaf(qv.w, xv[r].w, s);
                        }
                        acc[r * QB + qi] = s;
                    }
                }
            }
            const float sum = transpose_sum32(acc, lane);  // of pair (my_r, my_qi)
            const float key = l2 ? sum : -sum;
            if (row0 + my_r < end && rank >= 0 && key <= thr) {
                const int pos = atomicAdd(counts + rank, 1);
                if (pos < cap) {
                    cand_key[(int64_t)rank * cap + pos] = key;
                    cand_idx[(int64_t)rank * cap + pos] = (int32_t)(row0 + my_r);
                }
            }
        }
    }
}

// ---- items of the exact flat scan -------------------------------------------------------------
__global__ void fill_chunk_items_kernel(int32_t *__restrict__ item_query, int64_t *__restrict__ range_begin,
                                        int64_t *__restrict__ range_end, int64_t n_items, int chunks, int64_t per,
                                        int64_t n, const int32_t *__restrict__ only_q) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_items) return;
    const int64_t q = i / chunks, c = i - q * chunks;
    item_query[i] = (only_q && !only_q[q]) ? kItemSkip : (int32_t)q;
    range_begin[i] = c * per;
    range_end[i] = (c + 1) * per < n ? (c + 1) * per : n;
}

// ---- IVF item construction ------------------------------------------------------------------
// With list_off given, probes of lists that hold no rows here (empty, or stored on another shard)
// are not counted: they get no query tile and no work item.
__global__ void ivf_count_kernel(const int32_t *__restrict__ probes, int64_t n, int64_t nlist, int *counts,
                                 const int64_t *__restrict__ list_off) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int l = probes[i];
    const bool ok = l >= 0 && l < nlist;
    if (ok && list_off && list_off[l + 1] == list_off[l]) return;
    atomicAdd(&counts[ok ? l : nlist], 1);
}

// Exclusive scan of nlist+1 counters by one block; cursors[i] = start of bucket i.
__global__ void ivf_scan_kernel(const int *__restrict__ counts, int *__restrict__ cursors, int64_t nbuckets) {
    __shared__ int carry;
    __shared__ int warp_tot[32];
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t base = 0; base < nbuckets; base += blockDim.x) {
        int64_t i = base + threadIdx.x;
        int v = i < nbuckets ? counts[i] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(kFullMask, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = lane < (int)(blockDim.x >> 5) ? warp_tot[lane] : 0;
            int wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int t = __shfl_up_sync(kFullMask, wi, o);
                if (lane >= o) wi += t;
            }
            warp_tot[lane] = wi - w;  // exclusive prefix of the warp totals
        }
        __syncthreads();
        int excl = carry + warp_tot[warp] + incl - v;
        if (i < nbuckets) cursors[i] = excl;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = excl + v;
        __syncthreads();
    }
}

__global__ void ivf_place_kernel(const int32_t *__restrict__ probes, int64_t n, int nprobe, int64_t nlist,
                                 const int64_t *__restrict__ list_off, int *cursors,
                                 int32_t *__restrict__ item_query, int64_t *__restrict__ range_begin,
                                 int64_t *__restrict__ range_end, int32_t *__restrict__ item_slot) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int l = probes[i];
    const bool ok = l >= 0 && l < nlist;
    int slot = atomicAdd(&cursors[ok ? l : nlist], 1);
    item_slot[i] = slot;
    item_query[slot] = ok ? (int32_t)(i / nprobe) : -1;
    range_begin[slot] = ok ? list_off[l] : 0;
    range_end[slot] = ok ? list_off[l + 1] : 0;
}

// ---- grouping of probes by list for the tensor-core list scan ---------------------------------
// counts[l] = queries probing list l -> tiles[l] = ceil(counts / 128); exclusive scan of tiles.
__global__ void group_tiles_kernel(const int *__restrict__ counts, int *__restrict__ tile_off, int64_t nlist,
                                   int *__restrict__ n_tiles) {
    __shared__ int carry;
    __shared__ int warp_tot[32];
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t base = 0; base < nlist; base += blockDim.x) {
        const int64_t i = base + threadIdx.x;
        const int v = i < nlist ? (counts[i] + 127) / 128 : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(kFullMask, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const int w = lane < (int)(blockDim.x >> 5) ? warp_tot[lane] : 0;
            int wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(kFullMask, wi, o);
                if (lane >= o) wi += t;
            }
            warp_tot[lane] = wi - w;
        }
        __syncthreads();
        const int excl = carry + warp_tot[warp] + incl - v;
        if (i < nlist) tile_off[i] = excl;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = excl + v;
        __syncthreads();
    }
    if (threadIdx.x == 0) *n_tiles = carry;
}

__global__ void group_items_kernel(const int *__restrict__ counts, const int *__restrict__ tile_off, int64_t nlist,
                                   const int64_t *__restrict__ list_off, int4 *__restrict__ items) {
    const int64_t l = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (l >= nlist) return;
    const int tiles = (counts[l] + 127) / 128;
    for (int t = 0; t < tiles; t++)
        items[tile_off[l] + t] = make_int4(tile_off[l] + t, (int)list_off[l], (int)list_off[l + 1], (int)l);
}

__global__ void group_place_kernel(const int32_t *__restrict__ probes, int64_t n, int nprobe, int64_t nlist,
                                   const int64_t *__restrict__ list_off, const int *__restrict__ tile_off,
                                   int *cursors, int32_t *__restrict__ qrow_query, int32_t *__restrict__ gslot) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int l = probes[i];
    // an invalid probe or an empty list contributes nothing: no list slot is ever written for it
    if (l < 0 || l >= nlist || list_off[l + 1] == list_off[l]) {
        gslot[i] = -1;
        return;
    }
    const int pos = atomicAdd(&cursors[l], 1);
    const int g = tile_off[l] * 128 + pos;
    qrow_query[g] = (int32_t)(i / nprobe);
    gslot[i] = g;
}

template <int KR>
int launch_scan_kr(const float *x, const float *xlo, int dp, int d, const float *queries, int q_stride,
                   const int32_t *item_query, const int64_t *rb, const int64_t *re, int64_t n_items, int k,
                   int metric, float *part_key, int32_t *part_idx, uint32_t *qtau, int device, cudaStream_t stream,
                   const int *gate, int elem) {
    const size_t smem = (size_t)kWarps * dp * sizeof(float);
    if (smem > 48 * 1024) {
        ANN_CUDA_TRY(cudaFuncSetAttribute(scan_items_kernel<KR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem));
    }
    int64_t blocks = (n_items + kWarps - 1) / kWarps;
    const int64_t cap = (int64_t)sm_count(device) * 16;
    if (blocks > cap) blocks = cap;
    scan_items_kernel<KR><<<(unsigned)blocks, kWarps * 32, smem, stream>>>(
        x, xlo, dp, d, queries, q_stride, item_query, rb, re, n_items, k, metric, part_key, part_idx, qtau, gate, elem);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

struct FlaggedScanArgs {
    const float *x, *xlo;
    int dp, d;
    int64_t n;
    const float *queries;
    int q_stride;
    const int *aux;
    int *counts;
    int r_max, cap, k_out, k_last;
    const float *out_d;
    const int64_t *out_i;
    const unsigned *x_max_norm2;
    int metric;
    float *cand_key;
    int32_t *cand_idx;
    const int *gate;
    int elem;
    int round_tiles;
};

template <int QB>
int launch_scan_flagged_qb(const FlaggedScanArgs &a, int64_t blocks, size_t smem, cudaStream_t stream) {
    if (smem > 40 * 1024)  // (the kernel's static arrays count toward the 48 KB a launch gets unasked)
        ANN_CUDA_TRY(cudaFuncSetAttribute(scan_flagged_kernel<QB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    scan_flagged_kernel<QB><<<(unsigned)blocks, kWarps * 32, smem, stream>>>(
        a.x, a.xlo, a.dp, a.d, a.n, a.queries, a.q_stride, a.aux, a.counts, a.r_max, a.cap, a.k_out, a.k_last, a.out_d,
        a.out_i, a.x_max_norm2, a.metric, a.cand_key, a.cand_idx, a.gate, a.elem, a.round_tiles);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

}  // namespace

int scan_flagged_group(int dp) {
    for (int qb = 16; qb >= 8; qb >>= 1)
        if ((size_t)qb * dp * sizeof(float) <= 200 * 1024) return qb;
    return 0;
}

int launch_scan_items(const float *x, const float *xlo, int dp, int d, const float *queries, int q_stride,
                      const int32_t *item_query, const int64_t *range_begin, const int64_t *range_end,
                      int64_t n_items, int k, int metric, float *part_key, int32_t *part_idx, uint32_t *qtau,
                      int device, cudaStream_t stream, const int *gate, int elem) {
    if (n_items <= 0) return 0;
    if (k <= 0 || k > kMaxK) return set_error("k must be in [1, %d]", kMaxK);
    if ((size_t)kWarps * dp * sizeof(float) > 200 * 1024) return set_error("dimension %d too large for the scan kernel", d);
    if (k <= 32)
        return launch_scan_kr<1>(x, xlo, dp, d, queries, q_stride, item_query, range_begin, range_end, n_items, k,
                                 metric, part_key, part_idx, qtau, device, stream, gate, elem);
    if (k <= 128)
        return launch_scan_kr<4>(x, xlo, dp, d, queries, q_stride, item_query, range_begin, range_end, n_items, k,
                                 metric, part_key, part_idx, qtau, device, stream, gate, elem);
    if (k <= 512)
        return launch_scan_kr<16>(x, xlo, dp, d, queries, q_stride, item_query, range_begin, range_end, n_items, k,
                                  metric, part_key, part_idx, qtau, device, stream, gate, elem);
    return launch_scan_kr<64>(x, xlo, dp, d, queries, q_stride, item_query, range_begin, range_end, n_items, k, metric,
                              part_key, part_idx, qtau, device, stream, gate, elem);
}

int launch_scan_flagged(const float *x, const float *xlo, int dp, int d, int64_t n, const float *queries, int q_stride,
                        const int32_t *over_q, int64_t nq, int *aux, int32_t *rank_of, int *counts, int r_max, int cap,
                        int k_out, int k_last, const float *out_d, const int64_t *out_i, const unsigned *x_max_norm2,
                        int metric, float *cand_key, int32_t *cand_idx, int device, cudaStream_t stream, const int *gate,
                        int elem) {
    if (nq <= 0 || n <= 0) return 0;
    const int qb = scan_flagged_group(dp);
    if (qb == 0) return set_error("dimension %d too large for the scan kernel", d);
    compact_flagged_kernel<<<1, 1024, 0, stream>>>(over_q, nq, aux, rank_of, counts, r_max, gate);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    const size_t smem = (size_t)qb * dp * sizeof(float);
    const int64_t n_tiles = (n + kFilterTile - 1) / kFilterTile;
    const int64_t max_groups = (std::min<int64_t>(nq, r_max) + qb - 1) / qb;
    int64_t blocks = n_tiles * max_groups;
    const int64_t most = (int64_t)sm_count(device) * 3;  // three CTAs fit an SM
    if (blocks > most) blocks = most;
    // a round of tiles: ~24 MB of rows, a fraction of L2
    const int64_t tile_bytes = (int64_t)kFilterTile * dp * (elem != kElemF32 ? 2 : (xlo ? 8 : 4));
    const int64_t round_tiles = std::max<int64_t>(4, std::min<int64_t>(512, (24ll << 20) / tile_bytes));
    const FlaggedScanArgs a{x, xlo, dp, d, n, queries, q_stride, aux, counts, r_max, cap, k_out, k_last, out_d, out_i,
                            x_max_norm2, metric, cand_key, cand_idx, gate, elem, (int)round_tiles};
    if (qb == 16) return launch_scan_flagged_qb<16>(a, blocks, smem, stream);
    return launch_scan_flagged_qb<8>(a, blocks, smem, stream);
}

int launch_fill_chunk_items(int32_t *item_query, int64_t *range_begin, int64_t *range_end, int64_t nq, int chunks,
                            int64_t per, int64_t n, cudaStream_t stream, const int32_t *only_q) {
    const int64_t n_items = nq * chunks;
    if (n_items <= 0) return 0;
    fill_chunk_items_kernel<<<(unsigned)((n_items + 255) / 256), 256, 0, stream>>>(item_query, range_begin, range_end,
                                                                                   n_items, chunks, per, n, only_q);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_build_ivf_items(const int32_t *probes, int64_t nq, int nprobe, int64_t nlist, const int64_t *list_off,
                           int32_t *item_query, int64_t *range_begin, int64_t *range_end, int32_t *item_slot,
                           int *scratch, cudaStream_t stream) {
    const int64_t n = nq * nprobe;
    if (n <= 0) return 0;
    int *counts = scratch, *cursors = scratch + (nlist + 1);
    ANN_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int) * (size_t)(nlist + 1), stream));
    const unsigned blocks = (unsigned)((n + 255) / 256);
    ivf_count_kernel<<<blocks, 256, 0, stream>>>(probes, n, nlist, counts, nullptr);
    ivf_scan_kernel<<<1, 1024, 0, stream>>>(counts, cursors, nlist + 1);
    ivf_place_kernel<<<blocks, 256, 0, stream>>>(probes, n, nprobe, nlist, list_off, cursors, item_query,
                                                 range_begin, range_end, item_slot);
    count_launch(3);
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_group_probes(const int32_t *probes, int64_t nq, int nprobe, int64_t nlist, const int64_t *list_off,
                        int *scratch, int *n_tiles, int4 *items, int32_t *qrow_query, int32_t *gslot,
                        cudaStream_t stream) {
    const int64_t n = nq * nprobe;
    if (n <= 0) return 0;
    int *counts = scratch, *second = scratch + (nlist + 1);  // second: tile offsets, then placement cursors
    ANN_CUDA_TRY(cudaMemsetAsync(scratch, 0, sizeof(int) * (size_t)(nlist + 1) * 2, stream));
    const unsigned blocks = (unsigned)((n + 255) / 256);
    ivf_count_kernel<<<blocks, 256, 0, stream>>>(probes, n, nlist, counts, list_off);
    // tile offsets live in `second`; the placement cursors reuse `counts` after it is consumed
    group_tiles_kernel<<<1, 1024, 0, stream>>>(counts, second, nlist, n_tiles);
    group_items_kernel<<<(unsigned)((nlist + 255) / 256), 256, 0, stream>>>(counts, second, nlist, list_off, items);
    ANN_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int) * (size_t)(nlist + 1), stream));
    group_place_kernel<<<blocks, 256, 0, stream>>>(probes, n, nprobe, nlist, list_off, second, counts, qrow_query, gslot);
    count_launch(4);
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

}  // namespace anncuda
