// Shared host/device helpers of the CUDA search library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

namespace anncuda {

// ---- per-thread error text ---------------------------------------------------
inline std::string &last_error_ref() {
    static thread_local std::string msg;
    return msg;
}

inline int set_error(const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    last_error_ref() = buf;
    return -1;
}

#define ANN_CUDA_TRY(expr)                                                                          \
    do {                                                                                            \
        cudaError_t err__ = (expr);                                                                 \
        if (err__ != cudaSuccess) {                                                                 \
            return ::anncuda::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__),  \
                                        __FILE__, __LINE__);                                        \
        }                                                                                           \
    } while (0)

// Sets the device for the current scope and restores the caller's on exit, so
// library calls never change the calling thread's current device.
struct DeviceGuard {
    int prev = -1;
    bool ok = false;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        ok = (cudaSetDevice(device) == cudaSuccess);
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// A device buffer that only grows (next power of two), reused across calls.
struct GrowBuf {
    void *ptr = nullptr;
    size_t cap = 0;
    int ensure(size_t bytes) {
        if (bytes <= cap) return 0;
        size_t want = 4096;
        while (want < bytes) want <<= 1;
        if (ptr) cudaFree(ptr);
        ptr = nullptr;
        cap = 0;
        ANN_CUDA_TRY(cudaMalloc(&ptr, want));
        cap = want;
        return 0;
    }
    void release() {
        if (ptr) cudaFree(ptr);
        ptr = nullptr;
        cap = 0;
    }
    template <class T>
    T *as() const {
        return static_cast<T *>(ptr);
    }
};

inline int sm_count(int device) {
    static int cached[64];
    static std::once_flag once;
    std::call_once(once, [] { memset(cached, 0, sizeof cached); });
    if (device < 0 || device >= 64) return 148;
    if (cached[device] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || v <= 0) v = 148;
        cached[device] = v;
    }
    return cached[device];
}

// ---- device helpers -----------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

constexpr float kInf = __builtin_huge_valf();

// Error slack of tensor-core ranking keys.  Twice the bound E' on |ranking key - exact key| for a
// query with qn = |q - mu|^2 (L2) or |q|^2 (IP) against a store whose largest row norm squared is
// xm2.  The dot product the tensor cores form differs from the exact one by at most rel |q||x|:
//   screened search (q_hi.x_hi only): each operand rounded to 11 significant bits,
//       rel = 2^-10 (1 + 2^-11) + d 2^-23;
//   split product (q_hi.x_hi + q_hi.x_lo + q_lo.x_hi): the dropped q_lo.x_lo term is <= 2^-22, the
//       lo operands lose up to 2^-10 of themselves when the MMA reads them as TF32 (2 x 2^-21),
//       rel = 1.25 2^-20 + 3 d 2^-23.
// The d 2^-23 terms bound the fp32 accumulation in tensor memory (one rounding of at most one ulp
// of |q||x| per product added, three products per element for the split form).  An L2 key is
// |x - mu|^2 - 2 (q - mu).x, so it carries twice the dot-product error plus the fp32 rounding of
// the stored norm (<= (d / 32 + 6) 2^-24 of a value that is at most 4 xm2).
// If K is the k-th smallest ranking key of a query, its exact k-th best key is <= K + E' and a row
// can be among the exact k best only if its ranking key is <= K + 2E' = K + slack.
//
// 16-bit stores (elem = kElemF16 / kElemBF16: rows kept as fp16 or bf16, exact in that type; only the
// query is rounded).  One 16-bit part of the query per product ("screened"): each query element is off
// by at most 2^-11 (fp16) or 2^-8 (bf16) of itself, fp16 elements below 2^-14 by at most 2^-25
// absolutely, so the dot product is off by at most  rel |q||x| + 2^-25 sqrt(d) |x|  with
//   rel = 2^-11 (1 + 2^-11) + d 2^-23 (fp16),  2^-8 (1 + 2^-8) + d 2^-23 (bf16);
// two parts (q = q_hi + q_lo, "split"): rel = 2^-22 + 2 d 2^-23 (fp16), 2^-16 + 2 d 2^-23 (bf16).
// Products of two 16-bit values are exact in fp32; the d 2^-23 terms bound the accumulation as above.
constexpr int kElemF32 = 0, kElemF16 = 1, kElemBF16 = 2;
__host__ __device__ inline float key_slack(float qn, float xm2, int d, bool l2, bool screened, int elem = kElemF32) {
    float rel, abs_term = 0.f;
    if (elem == kElemF32) {
        rel = screened ? 9.8e-4f + (float)d * 1.2e-7f : 1.2e-6f + (float)d * 3.6e-7f;
    } else if (elem == kElemF16) {
        rel = screened ? 4.9e-4f + (float)d * 1.2e-7f : 2.4e-7f + (float)d * 2.4e-7f;
        abs_term = 3.0e-8f * sqrtf((float)d * xm2);
    } else {
        rel = screened ? 3.93e-3f + (float)d * 1.2e-7f : 1.53e-5f + (float)d * 2.4e-7f;
    }
    const float e = rel * sqrtf(qn * xm2) + abs_term;
    return 2.f * (l2 ? 2.f * e + ((float)d * (1.f / 32.f) + 6.f) * 6e-8f * 4.f * xm2 : e);
}
__host__ __device__ inline float screen_slack(float qn, float xm2, int d, bool l2) {
    return key_slack(qn, xm2, d, l2, true);
}

#ifdef __CUDACC__
// 16-bit row elements <-> float (elem = kElemF16 or kElemBF16).  Round to nearest even, as
// faiss-metal/src/MetalIndexFlat.mm:211-236 converts rows on add; widening is exact.
__device__ __forceinline__ float h16_to_float(uint16_t b, int elem) {
    return elem == kElemBF16 ? __uint_as_float((uint32_t)b << 16) : __half2float(__ushort_as_half(b));
}
__device__ __forceinline__ uint16_t float_to_h16(float v, int elem) {
    return elem == kElemBF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}
#endif

}  // namespace anncuda
