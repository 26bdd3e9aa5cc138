// Flat (exhaustive) search on the Blackwell tensor cores: split-TF32 GEMM fused
// with k-selection.  sm_100a only.
//
// What it replaces: the reference computes a full (queries x rows) distance
// matrix with a GEMM and then runs a separate selection pass over it
// (faiss-metal/src/MetalIndexFlat.mm:336-345, faiss-metal/src/MetalDistance.mm:206-288,
// faiss-metal/shaders/simdgroup_gemm.metal:143-252 for the fused-norm epilogue,
// faiss-metal/src/MetalSelect.mm:31-74).  Here the distance tile never leaves the
// SM: accumulators live in tensor memory and the epilogue warps select from them.
//
// Arithmetic.  q.x is evaluated as q_hi.x_hi + q_hi.x_lo + q_lo.x_hi with
// hi = TF32-rounded value and lo = value - hi (three tcgen05.mma kind::tf32 per
// K step, fp32 accumulation in TMEM), which keeps ~21 mantissa bits per product.
// L2 uses key = |x|^2 - 2 q.x (the query norm is constant per query); inner
// product uses key = -q.x.  Smaller key is better.
//
// Decomposition.  A work unit is (tile of 128 queries) x (chunk of database
// tiles, 256 rows each).  CTAs are persistent and walk units round-robin, query
// tile fastest, so the CTAs running at any moment read the same database rows
// and share them through L2.  Per unit the kernel leaves 128 unsorted k-lists in
// global memory; merge.cu reduces the chunks of a query to the final top-k.
//
// CTA layout (192 threads, one CTA per SM):
//   warp 0     TMA producer: per K block of 32 floats, four tiled loads
//              (q_hi, q_lo: 128 x 32; x_hi, x_lo: 256 x 32; 128-byte swizzle)
//              into a 2-stage shared-memory ring, signalled by mbarriers;
//   warp 1     allocates 512 TMEM columns (two 128 x 256 fp32 accumulators) and
//              issues the MMAs; tcgen05.commit releases ring stages and hands
//              finished accumulators to the epilogue;
//   warps 2-5  epilogue: thread t owns query row t (TMEM lane t), reads the
//              accumulator 16 columns at a time with tcgen05.ld, forms keys and
//              selects.  k <= 16: the k-list sits in shared memory, one column of
//              it per thread.  k > 16: keys below the row's current threshold go
//              to a 16-deep per-row queue in shared memory; when a queue would
//              overflow the warp folds its queues into the rows' k-lists in
//              global memory (L2-resident) with a register-held replace-max list.
//              The epilogue warps share nothing, so they need no barrier between them.
// Every wait on an mbarrier is bounded: after ~2 s without progress the kernel
// writes a code to *status and all roles leave their loops.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "select.cuh"

namespace anncuda {
namespace {

constexpr int BM = 128;           // queries per tile (TMEM lanes)
constexpr int BN = 256;           // database rows per tile (TMEM columns)
constexpr int BK = 32;            // floats per K block = one 128-byte swizzled row
constexpr int kStages = 2;
constexpr int kABytes = BM * BK * 4;                    // 16 KB
constexpr int kBBytes = BN * BK * 4;                    // 32 KB
constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;  // hi + lo of both operands: 96 KB
constexpr int kQueueDepth = 16;   // per-row candidate queue, also the small-k list capacity
constexpr int kThreads = 192;

struct SmemLayout {
    static constexpr int stages = 0;
    static constexpr int queue_key = kStages * kStageBytes;
    static constexpr int queue_idx = queue_key + kQueueDepth * BM * 4;
    static constexpr int xnorm = queue_idx + kQueueDepth * BM * 4;
    static constexpr int barriers = xnorm + 4 * 2 * BN * 4;  // (after a private norm copy per epilogue warp)
    // barriers: full[2] empty[2] tmem_full[2] tmem_empty[2]
    static constexpr int tmem_ptr = barriers + 8 * 8;
    static constexpr int abort_flag = tmem_ptr + 4;
    static constexpr int total = abort_flag + 4;
};
constexpr int kSmemBytes = SmemLayout::total + 1024;  // + slack to align the ring to 1024 B
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

// tcgen05 instruction descriptor, kind::tf32: D fp32, A and B TF32, both K-major,
// N = 256, M = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                ((uint32_t)(BM >> 4) << 24);

// ---- PTX wrappers -----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false when another role has already given up or when
// this wait itself runs out (~2 s); the caller then leaves its loop.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                            int code) {
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - t0 > 2000000000ull) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                          int code) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, code);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int32_t c0, int32_t c1,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128
// bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kInstrDesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float *v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

// ---- selection helpers ------------------------------------------------------------------------
// Folds the queues of this warp's 32 rows into their k-lists in global memory.
template <int KR>
__device__ __noinline__ void flush_queues(float *unit_key, int32_t *unit_idx, int k, int row0, const float *qkey,
                                          const int32_t *qidx, int &cnt, float &tau, int lane) {
    for (int r = 0; r < 32; r++) {
        const int c = __shfl_sync(kFullMask, cnt, r);
        if (c == 0) continue;
        const int row = row0 + r;
        float *lk = unit_key + (size_t)row * k;
        int32_t *li = unit_idx + (size_t)row * k;
        WarpList<KR> list;
        list.load(lk, k, lane);
        float m;
        int pos;
        list.argmax(lane, m, pos);
        for (int j = 0; j < c; j++) {
            const float ck = qkey[j * BM + row];
            if (ck < m) {
                if (lane == (pos & 31)) li[pos] = qidx[j * BM + row];
                list.set(pos, ck, lane);
                list.argmax(lane, m, pos);
            }
        }
        list.store(lk, k, lane);
        if (lane == r) {
            tau = m;
            cnt = 0;
        }
    }
    __syncwarp();
}

struct KernelArgs {
    const float *xnorm;
    int64_t n;
    int64_t nq;
    int kblocks;  // dp / BK
    int k;
    int l2;
    int nq_tiles, chunks, tiles_per_chunk, units;
    int64_t ntiles;
    float *part_key;
    int32_t *part_idx;
    int *status;
    int debug;  // measurement only: bit 0 = epilogue skips selection, bit 1 = MMA issuer skips the MMAs
};

template <int KR, bool SMALLK>
__global__ void __launch_bounds__(kThreads, 1)
flat_tc_kernel(const __grid_constant__ CUtensorMap map_qhi, const __grid_constant__ CUtensorMap map_qlo,
               const __grid_constant__ CUtensorMap map_xhi, const __grid_constant__ CUtensorMap map_xlo,
               const KernelArgs args) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    float *qkey = reinterpret_cast<float *>(smem + SmemLayout::queue_key);
    int32_t *qidx = reinterpret_cast<int32_t *>(smem + SmemLayout::queue_idx);
    float *xn_all = reinterpret_cast<float *>(smem + SmemLayout::xnorm);
    const uint32_t bar_full = smem_base + SmemLayout::barriers;
    const uint32_t bar_empty = bar_full + 8 * kStages;
    const uint32_t bar_tfull = bar_empty + 8 * kStages;
    const uint32_t bar_tempty = bar_tfull + 16;
    volatile uint32_t *tmem_ptr_s = reinterpret_cast<volatile uint32_t *>(smem + SmemLayout::tmem_ptr);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + SmemLayout::abort_flag);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(bar_tfull + 8 * b, 1);
            mbar_init(bar_tempty + 8 * b, 4);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_base + SmemLayout::tmem_ptr),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem_base = *tmem_ptr_s;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            for (int u = blockIdx.x; u < args.units; u += gridDim.x) {
                const int qt = u % args.nq_tiles, chunk = u / args.nq_tiles;
                const int64_t t_begin = (int64_t)chunk * args.tiles_per_chunk;
                int64_t t_end = t_begin + args.tiles_per_chunk;
                if (t_end > args.ntiles) t_end = args.ntiles;
                for (int64_t tile = t_begin; tile < t_end; tile++) {
                    for (int kb = 0; kb < args.kblocks; kb++) {
                        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, args.status, 1)) goto done;
                        const uint32_t full = bar_full + 8 * stage;
                        const uint32_t base = smem_base + stage * kStageBytes;
                        mbar_expect_tx(full, kStageBytes);
                        tma_load_2d(base, &map_qhi, kb * BK, qt * BM, full);
                        tma_load_2d(base + kABytes, &map_qlo, kb * BK, qt * BM, full);
                        tma_load_2d(base + 2 * kABytes, &map_xhi, kb * BK, (int32_t)(tile * BN), full);
                        tma_load_2d(base + 2 * kABytes + kBBytes, &map_xlo, kb * BK, (int32_t)(tile * BN), full);
                        if (++stage == kStages) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t it = 0;  // tiles issued by this CTA
            for (int u = blockIdx.x; u < args.units; u += gridDim.x) {
                const int chunk = u / args.nq_tiles;
                const int64_t t_begin = (int64_t)chunk * args.tiles_per_chunk;
                int64_t t_end = t_begin + args.tiles_per_chunk;
                if (t_end > args.ntiles) t_end = args.ntiles;
                for (int64_t tile = t_begin; tile < t_end; tile++, it++) {
                    const uint32_t buf = it & 1;
                    if (!mbar_wait(bar_tempty + 8 * buf, ((it >> 1) & 1) ^ 1, abort_flag, args.status, 2)) goto done;
                    tmem_fence_after();
                    const uint32_t tmem_d = tmem_base + buf * BN;
                    for (int kb = 0; kb < args.kblocks; kb++) {
                        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, args.status, 3)) goto done;
                        tmem_fence_after();
                        const uint32_t base = smem_base + stage * kStageBytes;
#pragma unroll
                        for (int ks = 0; ks < BK / 8; ks++) {
                            const uint64_t a_hi = make_smem_desc(base + ks * 32);
                            const uint64_t a_lo = make_smem_desc(base + kABytes + ks * 32);
                            const uint64_t b_hi = make_smem_desc(base + 2 * kABytes + ks * 32);
                            const uint64_t b_lo = make_smem_desc(base + 2 * kABytes + kBBytes + ks * 32);
                            if (args.debug & 2) continue;
                            mma_tf32(tmem_d, a_hi, b_lo, (kb | ks) != 0);
                            mma_tf32(tmem_d, a_lo, b_hi, 1);
                            mma_tf32(tmem_d, a_hi, b_hi, 1);
                        }
                        mma_commit(bar_empty + 8 * stage);  // stage is free once these MMAs have read it
                        if (++stage == kStages) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                    mma_commit(bar_tfull + 8 * buf);  // accumulator complete
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue / selection
        const int quarter = warp & 3;          // TMEM lanes this warp may read
        const int row = quarter * 32 + lane;   // query row inside the tile
        // Each epilogue warp keeps its own copy of the tile's row norms, so the four
        // warps never have to meet at a barrier (a warp that gave up on a wait can
        // leave without stranding the others).
        float *xn_s = xn_all + quarter * (2 * BN);
        const int k = args.k;
        uint32_t it = 0;
        for (int u = blockIdx.x; u < args.units; u += gridDim.x) {
            const int qt = u % args.nq_tiles, chunk = u / args.nq_tiles;
            const int64_t t_begin = (int64_t)chunk * args.tiles_per_chunk;
            int64_t t_end = t_begin + args.tiles_per_chunk;
            if (t_end > args.ntiles) t_end = args.ntiles;
            const bool row_valid = (int64_t)qt * BM + row < args.nq;
            float *unit_key = args.part_key + (size_t)u * BM * k;
            int32_t *unit_idx = args.part_idx + (size_t)u * BM * k;
            float tau = row_valid ? kInf : -kInf;
            int cnt = 0;   // queue fill (large k)
            int pos = 0;   // slot of the current maximum (small k)
            if (SMALLK) {
                for (int s = 0; s < k; s++) {
                    qkey[s * BM + row] = kInf;
                    qidx[s * BM + row] = -1;
                }
            } else {
                for (int r = 0; r < 32; r++) {
                    const size_t base = (size_t)(quarter * 32 + r) * k;
                    for (int s = lane; s < k; s += 32) {
                        unit_key[base + s] = kInf;
                        unit_idx[base + s] = -1;
                    }
                }
            }
            for (int64_t tile = t_begin; tile < t_end; tile++, it++) {
                const uint32_t buf = it & 1;
                if (args.l2) {
                    for (int j = lane; j < BN; j += 32) {
                        const int64_t col = tile * BN + j;
                        xn_s[buf * BN + j] = col < args.n ? __ldg(args.xnorm + col) : 0.f;
                    }
                    __syncwarp();
                }
                if (!mbar_wait(bar_tfull + 8 * buf, (it >> 1) & 1, abort_flag, args.status, 4)) goto done;
                tmem_fence_after();
                const int64_t rem = args.n - tile * BN;
                const int ncols = rem < BN ? (int)rem : BN;
                const int32_t col0 = (int32_t)(tile * BN);
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
                for (int cb = 0; cb < BN / 16; cb++) {
                    if (cb * 16 >= ncols || (args.debug & 1)) break;
                    float key[16];
                    tmem_ld16(taddr + cb * 16, key);
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        key[j] = args.l2 ? fmaf(-2.f, key[j], xn_s[buf * BN + cb * 16 + j]) : -key[j];
                    const int nvalid = ncols - cb * 16;  // >= 1
                    if (SMALLK) {
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            if (j < nvalid && key[j] < tau) {
                                qkey[pos * BM + row] = key[j];
                                qidx[pos * BM + row] = col0 + cb * 16 + j;
                                float m = -kInf;
                                for (int s = 0; s < k; s++) {
                                    const float v = qkey[s * BM + row];
                                    if (v > m) {
                                        m = v;
                                        pos = s;
                                    }
                                }
                                tau = m;
                            }
                        }
                    } else {
                        uint32_t mask = 0;
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (j < nvalid && key[j] < tau) mask |= 1u << j;
                        const bool overflow = cnt + __popc(mask) > kQueueDepth;
                        if (__any_sync(kFullMask, overflow)) {
                            flush_queues<KR>(unit_key, unit_idx, k, quarter * 32, qkey, qidx, cnt, tau, lane);
                            mask = 0;
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (j < nvalid && key[j] < tau) mask |= 1u << j;
                        }
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            if (mask & (1u << j)) {
                                qkey[cnt * BM + row] = key[j];
                                qidx[cnt * BM + row] = col0 + cb * 16 + j;
                                cnt++;
                            }
                        }
                    }
                }
                tmem_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
            }
            if (SMALLK) {
                for (int s = 0; s < k; s++) {
                    unit_key[(size_t)row * k + s] = qkey[s * BM + row];
                    unit_idx[(size_t)row * k + s] = qidx[s * BM + row];
                }
            } else {
                if (__any_sync(kFullMask, cnt > 0))
                    flush_queues<KR>(unit_key, unit_idx, k, quarter * 32, qkey, qidx, cnt, tau, lane);
            }
        }
    }
done:
    tmem_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Row-major (rows x dp) fp32 matrix, boxes of box_rows x 32 floats, 128-byte
// swizzle.  Rows past `rows` read as zero.
int make_map(CUtensorMap *map, const float *base, int64_t rows, int dp, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error("cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)dp, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)dp * sizeof(float)};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error("cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

template <int KR, bool SMALLK>
int launch_variant(const FlatPlan &plan, const CUtensorMap maps[4], const KernelArgs &args, cudaStream_t stream) {
    ANN_CUDA_TRY(cudaFuncSetAttribute(flat_tc_kernel<KR, SMALLK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemBytes));
    flat_tc_kernel<KR, SMALLK><<<plan.grid, kThreads, kSmemBytes, stream>>>(maps[0], maps[1], maps[2], maps[3], args);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

}  // namespace

FlatPlan make_flat_plan(int64_t nq, int64_t n, int k, int sms) {
    FlatPlan p;
    p.nq_tiles = (int)((nq + BM - 1) / BM);
    const int64_t ntiles = (n + BN - 1) / BN;
    int64_t max_chunks = 8192 / (k > 0 ? k : 1);  // the merge sorts chunks * k candidates per query
    if (max_chunks < 1) max_chunks = 1;
    if (max_chunks > ntiles) max_chunks = ntiles;
    int64_t chunks = 1;
    for (int waves = 8; waves >= 1; waves >>= 1) {
        chunks = (int64_t)sms * waves / p.nq_tiles;  // rounded down: units fill at most `waves` full waves
        if (chunks < 1) chunks = 1;
        if (waves == 1 || ntiles / chunks >= 32) break;
    }
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks < 1) chunks = 1;
    p.tiles_per_chunk = (int)((ntiles + chunks - 1) / chunks);
    p.chunks = (int)((ntiles + p.tiles_per_chunk - 1) / p.tiles_per_chunk);
    p.units = p.nq_tiles * p.chunks;
    p.grid = p.units < sms ? p.units : sms;
    p.part_entries = (size_t)p.units * BM * (size_t)k;
    return p;
}

int launch_flat_tc(const FlatPlan &plan, const float *xhi, const float *xlo, const float *xnorm, int64_t n,
                   const float *qhi, const float *qlo, int64_t nq, int dp, int k, int metric, float *part_key,
                   int32_t *part_idx, int *status, int device, cudaStream_t stream) {
    (void)device;
    if (n <= 0 || nq <= 0) return 0;
    if (k <= 0 || k > kMaxK) return set_error("k must be in [1, %d]", kMaxK);
    if (dp % BK != 0) return set_error("padded dimension must be a multiple of %d", BK);
    if (n > 0x7fffffffll - BN) return set_error("a flat shard holds at most 2^31 rows");
    CUtensorMap maps[4];
    if (make_map(&maps[0], qhi, nq, dp, BM) || make_map(&maps[1], qlo, nq, dp, BM) ||
        make_map(&maps[2], xhi, n, dp, BN) || make_map(&maps[3], xlo, n, dp, BN))
        return -1;
    KernelArgs a;
    a.xnorm = xnorm;
    a.n = n;
    a.nq = nq;
    a.kblocks = dp / BK;
    a.k = k;
    a.l2 = metric != 0;
    a.nq_tiles = plan.nq_tiles;
    a.chunks = plan.chunks;
    a.tiles_per_chunk = plan.tiles_per_chunk;
    a.units = plan.units;
    a.ntiles = (n + BN - 1) / BN;
    a.part_key = part_key;
    a.part_idx = part_idx;
    a.status = status;
    {
        const char *e = getenv("ANN_CUDA_TC_DEBUG");
        a.debug = e ? atoi(e) : 0;
    }
    if (k <= kQueueDepth) return launch_variant<1, true>(plan, maps, a, stream);
    if (k <= 32) return launch_variant<1, false>(plan, maps, a, stream);
    if (k <= 128) return launch_variant<4, false>(plan, maps, a, stream);
    if (k <= 512) return launch_variant<16, false>(plan, maps, a, stream);
    return launch_variant<64, false>(plan, maps, a, stream);
}

}  // namespace anncuda
