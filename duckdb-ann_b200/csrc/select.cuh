// Warp-level k-selection primitives shared by the search kernels.
//
// All kernels select on a float KEY where smaller is better:
//   L2:  key = |x|^2 - 2 q.x   (the query norm is constant per query and is
//        added when the result is finalised), or the full squared distance;
//   IP:  key = -q.x.
// A "list" is k (key, index) slots in memory, unsorted; the selection keeps the
// k smallest keys by replacing the current maximum.  Empty slots hold key +inf
// and index -1, so a list is always "full" and needs no fill phase.
//
// These take the role of the reference's warp_select / block_select shaders
// (faiss-metal/shaders/warp_select.metal:11,71, block_select.metal:66,162) but,
// unlike block_select (which keeps 8 per thread and can drop true neighbours),
// the replace-max list is exact for every k.
#pragma once

#include "common.cuh"

namespace anncuda {

constexpr unsigned kFullMask = 0xffffffffu;

// Order-preserving map float -> uint32 (handles negatives and infinities).
__device__ __forceinline__ uint32_t float_to_ordered(float f) {
    uint32_t u = __float_as_uint(f);
    return u ^ ((uint32_t)((int32_t)u >> 31) | 0x80000000u);
}
__device__ __forceinline__ float ordered_to_float(uint32_t u) {
    return __uint_as_float(u ^ (((u >> 31) - 1u) | 0x80000000u));
}

// A list of k keys held by one warp in registers: lane l owns slots l, l+32, ...
// Slots >= k hold -inf (never the maximum).
template <int KR>
struct WarpList {
    float v[KR];

    __device__ __forceinline__ void load(const float *keys, int k, int lane) {
#pragma unroll
        for (int i = 0; i < KR; i++) {
            int slot = i * 32 + lane;
            v[i] = slot < k ? keys[slot] : -kInf;
        }
    }
    __device__ __forceinline__ void fill_empty(int k, int lane) {
#pragma unroll
        for (int i = 0; i < KR; i++) v[i] = (i * 32 + lane) < k ? kInf : -kInf;
    }
    __device__ __forceinline__ void store(float *keys, int k, int lane) const {
#pragma unroll
        for (int i = 0; i < KR; i++) {
            int slot = i * 32 + lane;
            if (slot < k) keys[slot] = v[i];
        }
    }
    // Maximum key over the warp and the slot that holds it (lowest lane wins ties).
    __device__ __forceinline__ void argmax(int lane, float &m, int &pos) const {
        float best = v[0];
        int bi = 0;
#pragma unroll
        for (int i = 1; i < KR; i++) {
            if (v[i] > best) {
                best = v[i];
                bi = i;
            }
        }
        uint32_t u = float_to_ordered(best);
        uint32_t mu = __reduce_max_sync(kFullMask, u);
        unsigned who = __ballot_sync(kFullMask, u == mu);
        int src = __ffs(who) - 1;
        int slot = bi * 32 + lane;
        pos = __shfl_sync(kFullMask, slot, src);
        m = ordered_to_float(mu);
    }
    // Overwrites slot `pos` (owner lane only changes its register).
    __device__ __forceinline__ void set(int pos, float key, int lane) {
        if (lane == (pos & 31)) {
            int r = pos >> 5;
#pragma unroll
            for (int i = 0; i < KR; i++)
                if (i == r) v[i] = key;
        }
    }
};

}  // namespace anncuda
