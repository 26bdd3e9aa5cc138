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
// Shared threshold.  Once a chunk holds k rows for a query, its k-th best key
// bounds the query's final k-th best, so rows of ANY chunk above it cannot be in
// the answer.  Each chunk publishes that key with atomicMin to a per-query word
// and reads the word at every tile; the number of list insertions per query then
// grows like k log N for the whole database instead of per chunk.
//
// Decomposition.  Work is handed out dynamically.  The database is cut into
// chunks of a few 256-row tiles; every tile of 128 queries has a counter of
// chunks not yet taken.  A CTA adopts a query tile (its home tile first), takes
// chunks of it one by one with atomicAdd, and keeps ONE k-list per row for as long
// as it stays with that query tile, so a list sees a long stream of rows and
// settles after the first few tiles.  When a query tile has no chunks left the CTA
// moves to another one and starts a new list there.  At the end each query has
// one k-list per CTA that worked on its tile (at most lists_per_qt); merge.cu
// reduces them to the final top-k.
//
// The screened search of a large store is walked with a STATIC schedule instead (see
// choose_static): every CTA owns the same share of each chunk of the store, so all
// CTAs stay within two chunks of one another (an arrival counter per chunk paces
// them) and a row tile comes from DRAM once, from L2 for the other query tiles.
// Handing chunks out per query tile cannot do that: 148 CTAs do not divide evenly
// over the query tiles, the tiles with one CTA more run ahead, and a 20M x 768
// store was read from DRAM ~11 times per search (3 TB/s) - power the SMs then did
// not get under the board's cap.  A CTA's share touches at most two query tiles;
// it alternates between their two lists, keeping the one it is not working on
// parked (its fill counts in global memory).
//
// Pair mode of the static schedule (even number of query tiles and of SMs): the kernel is launched
// as clusters of two CTAs, and a PAIR owns a share of the (pair of query tiles, row tile) units.
// Both CTAs work on the same 256-row tile, each for its own query tile: a CTA stages its own 128
// queries and HALF of the rows, the leader issues tcgen05.mma.cta_group::2 (M = 256 over the two
// tensor memories, the two halves of the row tile read from both shared memories), and each CTA's
// epilogue selects from its own accumulator.  A K block then costs a CTA 32 KB of shared-memory
// fill instead of 48 KB, which is what bounded the one-CTA kernel.  Barriers: "stage full" lives in
// the leader (both CTAs' loads count their bytes there), "stage empty" and "accumulator full" are
// signalled in both CTAs by one multicast tcgen05.commit, "accumulator empty" collects the eight
// epilogue warps of the pair in the leader.  No load is multicast.
//
// This file is compiled three times: as it stands (TF32 operands, K blocks of 16 floats), through
// flat_tc_bk32.cu (K blocks of 32 floats: the screened search) and through flat_tc_h16.cu (fp16 / bf16
// operands, tcgen05.mma kind::f16: stores that keep their rows in 16 bits).
//
// Inverted-list scans read their rows as ONE plane of plain fp32 values (KernelArgs::derive_lo): such
// launches have two more warps (256 threads) that turn each row tile, once it has landed in shared
// memory, into its TF32 hi / lo parts in place - see the converter role below.
//
// CTA layout (192 threads, one CTA per SM):
//   warp 0     scheduler + TMA producer: takes the next chunk, announces it to the
//              other roles through a small descriptor ring, then per K block
//              issues four tiled loads (q_hi, q_lo: 128 rows; x_hi, x_lo: 256 rows;
//              swizzled) into the shared-memory ring, signalled by mbarriers;
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
// This file is compiled twice: as it stands (K blocks of 16 floats, four 48 KB stages: best for
// the three-MMA product and for the list scan, which want a deep ring) and, through
// flat_tc_bk32.cu, with K blocks of 32 floats for the screened search, whose single MMA per K
// step is otherwise dominated by the per-block bookkeeping of the issuing thread.
// A third build (flat_tc_h16.cu) is the same kernel over 16-bit operands (rows stored as fp16 or
// bf16, queries rounded to the same type): tcgen05.mma kind::f16, K blocks of 64 elements = the
// same 128-byte rows, 16 elements per MMA instead of 8 - twice the flops per byte staged.
#if defined(ANN_TC_VARIANT_H16) || defined(ANN_TC_VARIANT_BK32)
#define ANN_TC_SECONDARY 1  // a second or third build of this file: kernels and their launcher only
#endif
#if defined(ANN_TC_VARIANT_H16)
#define ANN_TC_BK 64
#define ANN_TC_ELEM_BYTES 2
#define ANN_TC_KIND "kind::f16"
#define ANN_TC_LAUNCH launch_flat_tc_h16
#elif defined(ANN_TC_VARIANT_BK32)
#define ANN_TC_BK 32
#define ANN_TC_LAUNCH launch_flat_tc_bk32
#else
#define ANN_TC_LAUNCH launch_flat_tc
#endif
#ifndef ANN_TC_BK
#define ANN_TC_BK 16
#endif
#ifndef ANN_TC_ELEM_BYTES
#define ANN_TC_ELEM_BYTES 4
#define ANN_TC_KIND "kind::tf32"
#endif
constexpr int BK = ANN_TC_BK;     // elements per K block: one 128-byte swizzled row (32 floats, 64 halves) or one 64-byte row (16 floats)
constexpr int kElemBytes = ANN_TC_ELEM_BYTES;
constexpr bool kH16 = kElemBytes == 2;
constexpr int kMmaK = 32 / kElemBytes;  // elements of K per MMA instruction: always 32 bytes of each operand row
static_assert(BK * kElemBytes == 128 || BK * kElemBytes == 64, "K block is one 128-byte or one 64-byte swizzled row");
constexpr int kStages = 256 / (BK * kElemBytes);  // the ring always holds 256 bytes of K per row: 2 x 96 KB or 4 x 48 KB
// Screened mode needs the hi planes only: the lo half of every stage serves as a stage of its own,
// so the ring is twice as deep (stage s = planes s & 1 of the physical stage s >> 1).
constexpr int kMaxStages = 2 * kStages;
// Pair mode (screened search with the static schedule): two CTAs of a cluster work on one 256-row
// tile with tcgen05.mma.cta_group::2.  Each CTA stages its own 128 queries and HALF of the row
// tile, so a K block costs a CTA kABytes + kBBytes / 2 of operand traffic instead of kABytes +
// kBBytes, and the ring holds more, smaller stages.
constexpr int kPairStages = 6;
constexpr int kPairStagesSplit2 = 4;  // 16-bit build, both parts of the queries staged: 48 KB per stage
constexpr int kBarStages = kMaxStages > kPairStages ? kMaxStages : kPairStages;
constexpr int kRowBytes = BK * kElemBytes;
constexpr bool kWideRows = kRowBytes == 128;                // the builds that have the pair mode
constexpr uint64_t kDescLayout = kWideRows ? 2ull : 4ull;   // SWIZZLE_128B : SWIZZLE_64B
constexpr uint64_t kDescSbo = (8 * kRowBytes) >> 4;         // 8-row group stride, in 16-byte units
constexpr int kABytes = BM * kRowBytes;                 // 16 KB
constexpr int kBBytes = BN * kRowBytes;                 // 32 KB
constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;  // hi + lo of both operands: 96 KB
constexpr int kPairStageBytes = kABytes + kBBytes / 2;  // pair mode: own queries + half of the row tile
static_assert(kPairStages * kPairStageBytes <= kStages * kStageBytes, "the pair ring fits into the stage memory");
static_assert(kPairStagesSplit2 * (kPairStageBytes + kABytes) <= kStages * kStageBytes, "and so does the two-part one");
constexpr int kQueueDepth = kSmemListMax;   // per-row candidate queue, also the small-k list capacity
constexpr int kThreads = 192;
// Launches whose rows come as one plain fp32 plane (KernelArgs::derive_lo) add two converter warps
// that split every row tile into TF32 hi / lo parts in shared memory.
constexpr int kConvWarps = 2;
constexpr int kThreadsDerive = kThreads + 32 * kConvWarps;
constexpr int kPaceSpins = 10000;  // polls of ~100 ns a CTA of the static schedule waits for the others, once
constexpr int kWorkRing = 4;       // chunk descriptors in flight between the scheduler and the other roles

struct SmemLayout {
    static constexpr int stages = 0;
    static constexpr int queue_key = kStages * kStageBytes;
    static constexpr int queue_idx = queue_key + kQueueDepth * BM * 4;
    static constexpr int xnorm = queue_idx + kQueueDepth * BM * 4;
    static constexpr int barriers = xnorm + 4 * 2 * BN * 4;  // (after a private norm copy per epilogue warp)
    // barriers: full[kBarStages] empty[kBarStages] tmem_full[2] tmem_empty[2] converted[kBarStages]
    static constexpr int work_bars = barriers + (3 * kBarStages + 4) * 8;  // wfull[kWorkRing] wempty[kWorkRing]
    static constexpr int work_ring = work_bars + 2 * kWorkRing * 8;    // kWorkRing descriptors of 32 bytes
    static constexpr int tmem_ptr = work_ring + kWorkRing * 32;
    static constexpr int abort_flag = tmem_ptr + 4;
    static constexpr int total = abort_flag + 4;
};
constexpr int kSmemBytes = SmemLayout::total + 1024;  // + slack to align the ring to 1024 B
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

// tcgen05 instruction descriptor, kind::tf32: D fp32, A and B TF32, both K-major,
// N = 256, M = 128.
// (16-bit build: the operand format, 0 = fp16, 1 = bf16, is added at run time - see operand_format)
constexpr uint32_t kOperandTf32 = kH16 ? 0u : 2u;
constexpr uint32_t kInstrDesc = (1u << 4) | (kOperandTf32 << 7) | (kOperandTf32 << 10) | ((uint32_t)(BN >> 3) << 17) |
                                ((uint32_t)(BM >> 4) << 24);
// The same for cta_group::2: M = 256, 128 rows of it in the tensor memory of each CTA of the pair.
constexpr uint32_t kInstrDescPair = (1u << 4) | (kOperandTf32 << 7) | (kOperandTf32 << 10) | ((uint32_t)(BN >> 3) << 17) |
                                    ((uint32_t)((2 * BM) >> 4) << 24);
__host__ __device__ constexpr uint32_t operand_format(int bf16) { return bf16 ? ((1u << 7) | (1u << 10)) : 0u; }

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
// this wait itself runs out (limit_ns, 2 s unless the host lowered it); the caller then
// leaves its loop.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                            uint64_t limit_ns, int code) {
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - t0 > limit_ns) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                          uint64_t limit_ns, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, limit_ns, code);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int32_t c0, int32_t c1,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, rows of kRowBytes with the
// matching swizzle, 8-row groups 8 * kRowBytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | (kDescSbo << 32) | (1ull << 46) | (kDescLayout << 61);
}

// (fmt: operand_format() of the 16-bit build, 0 otherwise)
__device__ __forceinline__ void mma_issue(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate,
                                         uint32_t fmt = 0) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1." ANN_TC_KIND " [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kInstrDesc | fmt), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// ---- pair mode (a cluster of two CTAs, tcgen05 cta_group::2) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of this CTA's shared address `addr` in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// All threads of both CTAs meet (not .aligned: roles arrive from different paths).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// Tiled load whose completion is counted on a barrier of the pair's leader CTA (`bar` is an address
// in the cluster window).  No multicast: each CTA fetches what it stages.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int32_t c0, int32_t c1,
                                                 uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// One MMA over both CTAs of the pair: A = 2 x 128 queries (each CTA's own), B = 2 x 128 rows (half
// of the tile in each CTA), D = 128 x 256 in each CTA's tensor memory.  Issued by the leader only.
__device__ __forceinline__ void mma_issue_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate,
                                              uint32_t fmt = 0) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2." ANN_TC_KIND " [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kInstrDescPair | fmt), "r"(accumulate)
        : "memory");
}
// Arrives, once the MMAs issued so far are complete, on the barrier at the same address in BOTH CTAs.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"((uint16_t)3)
        : "memory");
}

// value rounded to TF32 (10 mantissa bits, to nearest, ties away from zero): what the row planes hold
__device__ __forceinline__ float round_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

__device__ __forceinline__ void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Asynchronous read of 32 accumulator columns of this thread's TMEM lane.  The
// registers are valid only after tmem_ld_wait, which names them as in/out operands so
// the compiler cannot move their uses above the wait.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
// Waits for every TMEM read this thread has in flight, naming no registers.  Needed before code
// with calls, loops or jumps while a read into another register buffer is still in flight: the
// compiler believes those registers were written when the read was ISSUED and may copy or save
// them at any point after that - a copy taken before the data has landed is stale.
__device__ __forceinline__ void tmem_ld_wait_all() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                   "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                   "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// Stores that execute only where `p` is set, as predicated instructions (no branch).
__device__ __forceinline__ void st_global_if(bool p, float *addr, float v) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %0, 0;\n\t@q st.global.f32 [%1], %2;\n\t}" ::"r"((int)p), "l"(addr),
                 "f"(v)
                 : "memory");
}
__device__ __forceinline__ void st_global_if(bool p, int32_t *addr, int32_t v) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %0, 0;\n\t@q st.global.s32 [%1], %2;\n\t}" ::"r"((int)p), "l"(addr),
                 "r"(v)
                 : "memory");
}

// One append: key and row number stored together, or not at all (one predicate for both).
__device__ __forceinline__ void st_global_pair_if(bool p, float *kaddr, float key, int32_t *iaddr, int32_t idx) {
    asm volatile(
        "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %0, 0;\n\t@q st.global.f32 [%1], %2;\n\t@q st.global.s32 [%3], %4;\n\t}" ::"r"(
            (int)p),
        "l"(kaddr), "f"(key), "l"(iaddr), "r"(idx)
        : "memory");
}

// ---- selection helpers ------------------------------------------------------------------------
// Folds the queues of this warp's 32 rows into their k-lists in global memory.
template <int KR>
__device__ __noinline__ void flush_queues(float *unit_key, int32_t *unit_idx, int k, int row0, const float *qkey,
                                          const int32_t *qidx, int &cnt, float &tau, int lane, uint32_t *qtau_word,
                                          float koff) {
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
            // m is the k-th best key of this chunk so far: no row of any chunk with a
            // larger key can be in the query's final top-k, so it is published for all
            tau = fminf(tau, m);
            cnt = 0;
            if (m < kInf) atomicMin(qtau_word, float_to_ordered(__fadd_ru(m, koff)));
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
    int nq_tiles, nchunks, tiles_per_chunk, lists_per_qt;
    int64_t ntiles;
    int *next_chunk;  // [nq_tiles] chunks handed out so far (zero on entry)
    int *nlists;      // [nq_tiles] lists started so far (zero on entry)
    // Grouped mode (IVF list scan): work items are given, one per tile of gathered queries.
    const int4 *items;          // {gathered query tile, first row, end row, unused}; null = flat mode
    const int *n_items;         // device count of items
    int *item_counter;          // zero on entry
    // Static schedule (see FlatPlan::static_g): arrivals[c] counts the CTAs that have started
    // chunk c (zero on entry); slot_cnt[list * 128 + row] keeps the fill count of a row's append
    // buffer while its CTA works for its other query tile
    int static_g, static_chunks, pace_window;
    int *arrivals;
    int *slot_cnt;
    const int32_t *qrow_query;  // gathered row -> query (its threshold word), -1 = padding row
    // Grouped L2 with residual queries (may be null): constant K of every gathered row such that
    // key + K is comparable between the lists of one query; keys inside the kernel leave it out
    const float *qrow_const;
    // Grouped append mode (may be null): a finished row leaves its append buffer unsorted and
    // writes its fill count here (index = slot * 128 + row); the merge filters and sorts
    int32_t *part_cnt;
    // Screened mode (flat search, append selection; 0 = off).  The tensor cores form q_hi.x_hi
    // only: one MMA per K step instead of three, and only the hi planes travel through shared
    // memory.  That dot product is within  E = (2^-10 + d 2^-23) |q||x|  of the exact one (each
    // operand is rounded to 11 significant bits; fp32 accumulation), so all keys of a query are
    // within E' (E for IP, 2E for L2) of the exact ones, |x| taken as the largest norm in the
    // store.  If K is the k_rank-th smallest coarse key, the exact k_rank-th best is at most
    // K + E', and a row can be among the k_rank best only if its coarse key is <= K + 2E'.  The
    // lists therefore keep k > k_rank entries, the threshold is the k_rank-th key + 2E', and the
    // caller re-ranks the k candidates it gets back by their exact fp32 distance.
    int screen;                   // one-MMA keys
    int banded;                   // lists pruned by the k_rank-th key + slack (screen implies banded)
    int k_rank;                   // = k when not banded
    const float *q_norm2;         // per query |q - mu|^2 (L2, mu = the store's reference point) or |q|^2 (IP)
    const unsigned *x_max_norm2;  // bits of the largest |x|^2 in the store
    int d;
    float *part_key;
    int32_t *part_idx;
    uint32_t *qtau;  // per query: smallest k-th-best key any chunk has published (ordered-uint form)
    int *status;
    uint64_t wait_ns;     // limit of every bounded wait
    int withhold_after;   // test hook (-1 = off): see flat_test_withhold_after in kernels.h
    const int *gate;      // may be null: run only if *gate == kScreenOverflow (a fallback pass)
    int pair;             // launched as clusters of two CTAs that share row tiles (screened, static schedule)
    int bf16;             // 16-bit build: operands are bf16 (else fp16)
    int derive_lo;        // rows come as one plain fp32 plane; converter warps split them in shared memory
    int split2;           // 16-bit build, pair mode: both 16-bit parts of the queries (q_hi.x + q_lo.x)
#ifdef ANN_CUDA_MEASURE
    unsigned long long *stats;  // see kStat* below
    int debug;  // bit 0 = epilogue skips selection, bit 1 = MMA issuer skips the MMAs, bit 2 = no appends, bit 3 = consume only
#endif
};

// Counters and stage switches for profiling exist only in builds with -DANN_CUDA_MEASURE; in the
// product build both read as constants and the code behind them is dropped.
#ifdef ANN_CUDA_MEASURE
__device__ __forceinline__ unsigned long long *kstats(const KernelArgs &a) { return a.stats; }
__device__ __forceinline__ int kdebug(const KernelArgs &a) { return a.debug; }
#else
__device__ __forceinline__ unsigned long long *kstats(const KernelArgs &) { return nullptr; }
__device__ __forceinline__ int kdebug(const KernelArgs &) { return 0; }
#endif

// How the epilogue keeps the k best keys of a row:
//   kSelSmem    k <= 16: the list sits in shared memory, one column per thread;
//   kSelAppend  16 < k <= 128: every key below the row's threshold is appended to a
//               512-slot buffer of the row in global memory (a plain store, no
//               dependent work); when a buffer is nearly full the warp sorts it in
//               registers (bitonic, 16 keys per lane), keeps the best k and tightens
//               the threshold to the k-th.  Buffers fill at n = 512, ~2.5k, ~13k, ...
//               rows seen, so a row is compacted a handful of times per search;
//   kSelReplace k > 128: 16-deep queue in shared memory folded into a replace-max
//               list in global memory (exact for any k, slower).
// Slots of the optional statistics array (cycle counts are summed over CTAs / warps).
enum { kStatCompactRows = 0, kStatAppends = 1, kStatCompactCycles = 2, kStatEpiWaitCycles = 3, kStatMmaWaitTmem = 4,
       kStatMmaWaitSmem = 5, kStatEpiTileCycles = 6, kStatTiles = 7, kStatSlowGroups = 8, kStatSlowCycles = 9,
       kStatLdWaitCycles = 10, kStatCount = 12 };

enum SelMode { kSelSmem = 0, kSelAppend = 1, kSelReplace = 2 };
constexpr int kBuf = kAppendBuffer;  // candidate slots per row in append mode
static_assert(kAppendMaxK <= kBuf / 2 && kScreenMaxList <= kBuf / 2, "a compacted row must leave room for new candidates");

// ---- bitonic sort of (key, idx) pairs held by a warp, E per lane ---------------------------------
// Keys are order-preserving uint32 images of the float keys.  Element e lives in lane e / E,
// register e % E, so exchanges at distance < E stay inside a thread and larger ones are one shuffle.
// Every compare-exchange is written without a conditional on the direction (the
// direction is an XOR mask), so the code is straight-line selects, no branches.
__device__ __forceinline__ void ce_swap(uint32_t &ka, int32_t &ia, uint32_t &kb, int32_t &ib, uint32_t dm) {
    const bool sw = (ka ^ dm) > (kb ^ dm);  // dm = 0: ascending, ~0: descending
    const uint32_t ta = sw ? kb : ka, tb = sw ? ka : kb;
    const int32_t ua = sw ? ib : ia, ub = sw ? ia : ib;
    ka = ta; kb = tb; ia = ua; ib = ub;
}
// Sorts 32 * E pairs, E per lane (element e lives in lane e / E, register e % E).
template <int E>
__device__ __forceinline__ void warp_sort(uint32_t (&key)[E], int32_t (&idx)[E], int lane) {
    // sizes 2..E: all exchanges are inside a lane
#pragma unroll
    for (int size = 2; size <= E; size <<= 1) {
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
#pragma unroll
            for (int i = 0; i < E; i++) {
                if ((i & stride) == 0) {
                    const uint32_t dm = size == E ? (0u - (uint32_t)(lane & 1)) : ((i & size) ? 0xffffffffu : 0u);
                    ce_swap(key[i], idx[i], key[i | stride], idx[i | stride], dm);
                }
            }
        }
    }
    // sizes 2E..32E: the direction is the same for all elements of a lane
#pragma unroll 1
    for (int size = 2 * E; size <= 32 * E; size <<= 1) {
        const uint32_t dm = ((lane * E) & size) ? 0xffffffffu : 0u;
#pragma unroll 1
        for (int ls = size / (2 * E); ls > 0; ls >>= 1) {
            // the lower lane of a pair keeps the smaller key when ascending
            const uint32_t km = ((lane & ls) ? 0xffffffffu : 0u) ^ dm;  // 0: keep min, ~0: keep max
#pragma unroll
            for (int i = 0; i < E; i++) {
                const uint32_t ok = __shfl_xor_sync(kFullMask, key[i], ls);
                const int32_t oi = __shfl_xor_sync(kFullMask, idx[i], ls);
                const bool take = (ok ^ km) < (key[i] ^ km);
                key[i] = take ? ok : key[i];
                idx[i] = take ? oi : idx[i];
            }
        }
#pragma unroll
        for (int stride = E / 2; stride > 0; stride >>= 1) {
#pragma unroll
            for (int i = 0; i < E; i++)
                if ((i & stride) == 0) ce_swap(key[i], idx[i], key[i | stride], idx[i | stride], dm);
        }
    }
}

// Largest of 32 accumulator values (three-input max: 16 instructions, four levels deep).
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float max32(const uint32_t (&raw)[32]) {
    float m[11];
#pragma unroll
    for (int i = 0; i < 10; i++)
        m[i] = max3(__uint_as_float(raw[3 * i]), __uint_as_float(raw[3 * i + 1]), __uint_as_float(raw[3 * i + 2]));
    m[10] = fmaxf(__uint_as_float(raw[30]), __uint_as_float(raw[31]));
    const float a = max3(m[0], m[1], m[2]), b = max3(m[3], m[4], m[5]), c = max3(m[6], m[7], m[8]);
    return max3(max3(a, b, c), m[9], m[10]);
}

// raw[j] for a j known only at run time: registers cannot be indexed, so the value is chosen by a
// select tree on the bits of j (16 + 8 + 4 + 2 + 1 selects, five levels deep).
__device__ __forceinline__ uint32_t select32(const uint32_t (&raw)[32], int j) {
    const bool b4 = (j & 16) != 0, b3 = (j & 8) != 0, b2 = (j & 4) != 0, b1 = (j & 2) != 0, b0 = (j & 1) != 0;
    uint32_t a[16], b[8], c[4], d[2];
#pragma unroll
    for (int i = 0; i < 16; i++) a[i] = b4 ? raw[i + 16] : raw[i];
#pragma unroll
    for (int i = 0; i < 8; i++) b[i] = b3 ? a[i + 8] : a[i];
#pragma unroll
    for (int i = 0; i < 4; i++) c[i] = b2 ? b[i + 4] : b[i];
#pragma unroll
    for (int i = 0; i < 2; i++) d[i] = b1 ? c[i + 2] : c[i];
    return b0 ? d[1] : d[0];
}

// Sorts the first 32 * E slots of one row's append buffer (c <= 32 * E of them filled) and writes
// back, in order, those of the best k that lie within `slack` of the k_rank-th best key (nothing
// above that can reach the final top k_rank; index -1 in the slots up to k that stay empty).
// Returns the k_rank-th best key (k_rank <= k; meaningful only if c >= k_rank) and, in `kept`,
// how many entries the row keeps.
template <int E>
__device__ __forceinline__ float compact_one(float *bk, int32_t *bi, int c, int k, int k_rank, float slack, int lane,
                                             int &kept) {
    uint32_t key[E];
    int32_t idx[E];
    if (E >= 4) {
#pragma unroll
        for (int v = 0; v < E / 4; v++) {
            const float4 kk = *reinterpret_cast<const float4 *>(bk + lane * E + v * 4);
            const int4 ii = *reinterpret_cast<const int4 *>(bi + lane * E + v * 4);
            key[v * 4 + 0] = float_to_ordered(kk.x); key[v * 4 + 1] = float_to_ordered(kk.y);
            key[v * 4 + 2] = float_to_ordered(kk.z); key[v * 4 + 3] = float_to_ordered(kk.w);
            idx[v * 4 + 0] = ii.x; idx[v * 4 + 1] = ii.y; idx[v * 4 + 2] = ii.z; idx[v * 4 + 3] = ii.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < E; i++) {
            key[i] = float_to_ordered(bk[lane * E + i]);
            idx[i] = bi[lane * E + i];
        }
    }
#pragma unroll
    for (int i = 0; i < E; i++) {
        const bool stale = lane * E + i >= c;  // slots past the fill hold old data
        key[i] = stale ? 0xff800000u : key[i];  // +inf
        idx[i] = stale ? -1 : idx[i];
    }
    warp_sort<E>(key, idx, lane);
    float kth = kInf;
#pragma unroll
    for (int i = 0; i < E; i++) kth = (lane * E + i == k_rank - 1) ? ordered_to_float(key[i]) : kth;
    kth = 32 * E < k_rank ? kInf : __shfl_sync(kFullMask, kth, (k_rank - 1) / E);
    // fewer than k_rank entries (their tail sorts as +inf): no threshold yet, everything stays
    const float cut = (c >= k_rank) ? kth + slack : kInf;
    int mine = 0;
#pragma unroll
    for (int i = 0; i < E; i++) {
        const int e = lane * E + i;
        const float kf = ordered_to_float(key[i]);
        const bool keep = e < k && idx[i] >= 0 && kf <= cut;
        st_global_if(e < k, bk + e, kf);
        st_global_if(e < k, bi + e, keep ? idx[i] : -1);
        mine += keep ? 1 : 0;
    }
    if (32 * E < k)  // the sorted part is shorter than the list: mark the rest empty
        for (int e = 32 * E + lane; e < k; e += 32) bi[e] = -1;
    kept = __reduce_add_sync(kFullMask, mine);
    return kth;
}

// Compaction of a full append buffer (up to 512 entries) WITHOUT sorting it.  A radix select over
// the order-preserving integer images of the keys (two bits per round, the three counters of a
// round packed into one warp reduction) finds the k_rank-th smallest key; everything within
// `slack` of it moves to the front of the buffer, in no particular order, the rest is dropped.
// ~2.5k cycles against ~14k for the 512-wide sorting network - and a row is compacted five or six
// times per list.  Returns the k_rank-th key; kept = entries that stay, or -1 when more than k lie
// inside the band (the caller then takes the sorting path, which cuts at k).
__device__ __forceinline__ float select_one(float *bk, int32_t *bi, int c, int k, int k_rank, float slack, int lane,
                                            int &kept) {
    constexpr int E = 16;
    uint32_t key[E];
    int32_t idx[E];
#pragma unroll
    for (int v = 0; v < E / 4; v++) {
        const float4 kk = *reinterpret_cast<const float4 *>(bk + lane * E + v * 4);
        const int4 ii = *reinterpret_cast<const int4 *>(bi + lane * E + v * 4);
        key[v * 4 + 0] = float_to_ordered(kk.x); key[v * 4 + 1] = float_to_ordered(kk.y);
        key[v * 4 + 2] = float_to_ordered(kk.z); key[v * 4 + 3] = float_to_ordered(kk.w);
        idx[v * 4 + 0] = ii.x; idx[v * 4 + 1] = ii.y; idx[v * 4 + 2] = ii.z; idx[v * 4 + 3] = ii.w;
    }
#pragma unroll
    for (int i = 0; i < E; i++) {
        const bool stale = lane * E + i >= c;  // slots past the fill hold old data
        key[i] = stale ? 0xffffffffu : key[i];
        idx[i] = stale ? -1 : idx[i];
    }
    if (c < k_rank) {  // fewer entries than the rank asked for: no threshold yet, everything stays (warp-uniform)
        kept = c;
        return kInf;
    }
    uint32_t prefix = 0;
    int need = k_rank;  // rank of the wanted key among the entries that match the prefix so far
#pragma unroll 1
    for (int shift = 30; shift >= 0; shift -= 2) {
        const uint32_t hi_mask = shift == 30 ? 0u : (0xffffffffu << (shift + 2));
        uint32_t packed = 0;  // counts of digits 0, 1, 2 among the matching entries, 10 bits each
#pragma unroll
        for (int i = 0; i < E; i++) {
            const uint32_t digit = (key[i] >> shift) & 3u;
            const uint32_t one = ((key[i] & hi_mask) == prefix && digit != 3u) ? (1u << (10u * digit)) : 0u;
            packed += one;
        }
        packed = __reduce_add_sync(kFullMask, packed);
        const int c0 = (int)(packed & 1023u), c1 = (int)((packed >> 10) & 1023u), c2 = (int)((packed >> 20) & 1023u);
        uint32_t digit;
        if (need <= c0) digit = 0;
        else if (need <= c0 + c1) { digit = 1; need -= c0; }
        else if (need <= c0 + c1 + c2) { digit = 2; need -= c0 + c1; }
        else { digit = 3; need -= c0 + c1 + c2; }
        prefix |= digit << shift;
    }
    const float kth = ordered_to_float(prefix);
    const uint32_t cut = float_to_ordered(kth + slack);
    int mine = 0;
#pragma unroll
    for (int i = 0; i < E; i++) mine += (idx[i] >= 0 && key[i] <= cut) ? 1 : 0;
    const int total = __reduce_add_sync(kFullMask, mine);
    if (total > k) {
        kept = -1;
        return kth;
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(kFullMask, incl, o);
        incl += lane >= o ? t : 0;
    }
    int pos = incl - mine;
    __syncwarp();  // every lane holds its part of the buffer in registers before anything is overwritten
#pragma unroll
    for (int i = 0; i < E; i++) {
        const bool keep = idx[i] >= 0 && key[i] <= cut;
        st_global_if(keep, bk + pos, ordered_to_float(key[i]));
        st_global_if(keep, bi + pos, idx[i]);
        pos += keep ? 1 : 0;
    }
    kept = total;
    return kth;
}

// The same compaction for BANDED lists, which have room to spare (k - k_rank >= 32 slots): the threshold need
// not be the k_rank-th key itself, any key that at least k_rank entries do not exceed will do - it only
// prunes, the merge and the exact re-ranking that follow decide.  32 sample keys (one per lane) are sorted
// across the warp and a binary search over them finds the smallest sample that has k_rank entries at or below
// it: five counting rounds of 16 compares each instead of sixteen radix rounds - ~2k cycles instead of ~11k,
// and a list is compacted two or three times, all 32 rows of a warp at once, before its threshold settles.
// Returns that sample (an upper bound of the k_rank-th key, a few entries above it at most); kept = -1 when
// the samples hold no such key or more than k entries lie inside the band (the caller then sorts).
__device__ __forceinline__ float select_one_sampled(float *bk, int32_t *bi, int c, int k, int k_rank, float slack, int lane,
                                                    int &kept) {
    constexpr int E = 16;
    uint32_t key[E];
    int32_t idx[E];
#pragma unroll
    for (int v = 0; v < E / 4; v++) {
        const float4 kk = *reinterpret_cast<const float4 *>(bk + lane * E + v * 4);
        const int4 ii = *reinterpret_cast<const int4 *>(bi + lane * E + v * 4);
        key[v * 4 + 0] = float_to_ordered(kk.x); key[v * 4 + 1] = float_to_ordered(kk.y);
        key[v * 4 + 2] = float_to_ordered(kk.z); key[v * 4 + 3] = float_to_ordered(kk.w);
        idx[v * 4 + 0] = ii.x; idx[v * 4 + 1] = ii.y; idx[v * 4 + 2] = ii.z; idx[v * 4 + 3] = ii.w;
    }
#pragma unroll
    for (int i = 0; i < E; i++) {
        const bool stale = lane * E + i >= c;  // slots past the fill hold old data
        key[i] = stale ? 0xffffffffu : key[i];
        idx[i] = stale ? -1 : idx[i];
    }
    if (c < k_rank) {  // fewer entries than the rank asked for: no threshold yet, everything stays (warp-uniform)
        kept = c;
        return kInf;
    }
    // the samples, sorted ascending across the lanes (bitonic network on one value per lane)
    uint32_t smp = key[0];
#pragma unroll
    for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const uint32_t other = __shfl_xor_sync(kFullMask, smp, stride);
            const bool keep_min = ((lane & stride) == 0) == ((lane & size) == 0);
            smp = keep_min ? (other < smp ? other : smp) : (other > smp ? other : smp);
        }
    }
    auto count_le = [&](uint32_t p) {
        int mine = 0;
#pragma unroll
        for (int i = 0; i < E; i++) mine += (key[i] <= p) ? 1 : 0;
        return __reduce_add_sync(kFullMask, mine);
    };
    int lo = 0, hi = 31;
#pragma unroll 1
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (count_le(__shfl_sync(kFullMask, smp, mid)) >= k_rank) hi = mid;
        else lo = mid + 1;
    }
    const uint32_t pivot = __shfl_sync(kFullMask, smp, lo);
    if (pivot == 0xffffffffu || count_le(pivot) < k_rank) {  // (the largest sample ranks below k_rank: not with these sizes)
        kept = -1;
        return kInf;
    }
    const float kth = ordered_to_float(pivot);
    const uint32_t cut = float_to_ordered(kth + slack);
    int mine = 0;
#pragma unroll
    for (int i = 0; i < E; i++) mine += (idx[i] >= 0 && key[i] <= cut) ? 1 : 0;
    const int total = __reduce_add_sync(kFullMask, mine);
    if (total > k) {
        kept = -1;
        return kth;
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(kFullMask, incl, o);
        incl += lane >= o ? t : 0;
    }
    int pos = incl - mine;
    __syncwarp();  // every lane holds its part of the buffer in registers before anything is overwritten
#pragma unroll
    for (int i = 0; i < E; i++) {
        const bool keep = idx[i] >= 0 && key[i] <= cut;
        st_global_if(keep, bk + pos, ordered_to_float(key[i]));
        st_global_if(keep, bi + pos, idx[i]);
        pos += keep ? 1 : 0;
    }
    kept = total;
    return kth;
}

// Compacts the append buffers of the rows in `need` (bit r = row row0 + r of this warp): a full
// buffer by select_one (unsorted), a partly filled one (and a band that holds more than k) down to
// their best k, sorted.  The sort is as wide as the row's fill needs: a full buffer takes the
// 512-wide network (~14k cycles); the few dozen entries typical when a list is closed behind a
// tight threshold take the 32- or 64-wide one (a few hundred cycles).
__device__ __noinline__ void compact_rows(float *slot_key, int32_t *slot_idx, int k, int row0, unsigned need, int &cnt,
                                          float &tau, int lane, uint32_t *qtau_word, float koff, int k_rank,
                                          float slack) {
    __syncwarp();  // the appends of every lane are visible to the whole warp
    while (need) {
        const int r = __ffs(need) - 1;
        need &= need - 1;
        const int c = __shfl_sync(kFullMask, cnt, r);
        // every lane works on row r's buffer now: the band is row r's, not the lane's own row's
        const float row_slack = __shfl_sync(kFullMask, slack, r);
        float *bk = slot_key + (size_t)(row0 + r) * kBuf;
        int32_t *bi = slot_idx + (size_t)(row0 + r) * kBuf;
        float kth;
        int kept;
        if (c > 256) {
            kth = (k - k_rank >= 32) ? select_one_sampled(bk, bi, c, k, k_rank, row_slack, lane, kept)
                                     : select_one(bk, bi, c, k, k_rank, row_slack, lane, kept);
            if (kept < 0) kth = compact_one<16>(bk, bi, c, k, k_rank, row_slack, lane, kept);
        } else if (c > 128) kth = compact_one<8>(bk, bi, c, k, k_rank, row_slack, lane, kept);
        else if (c > 64) kth = compact_one<4>(bk, bi, c, k, k_rank, row_slack, lane, kept);
        else if (c > 32) kth = compact_one<2>(bk, bi, c, k, k_rank, row_slack, lane, kept);
        else kth = compact_one<1>(bk, bi, c, k, k_rank, row_slack, lane, kept);
        if (lane == r) {
            cnt = kept;
            if (c >= k_rank) {
                // the k_rank-th best key so far (plus this row's error slack when the keys are
                // coarse): nothing above it can reach the final top k_rank
                const float thr = kth + slack;
                tau = fminf(tau, thr);
                atomicMin(qtau_word, float_to_ordered(__fadd_ru(thr, koff)));
            }
        }
    }
    __syncwarp();
}

// PAIR: the kernel of the pair mode, launched as clusters of two CTAs.  A kernel of its own because
// code that holds cta_group::2 instructions can only be launched with a cluster size that fits them.
template <int KR, int MODE, bool PAIR>
__global__ void __launch_bounds__(kThreadsDerive, 1)
flat_tc_kernel(const __grid_constant__ CUtensorMap map_qhi, const __grid_constant__ CUtensorMap map_qlo,
               const __grid_constant__ CUtensorMap map_xhi, const __grid_constant__ CUtensorMap map_xlo,
               const KernelArgs args) {
    constexpr bool SMALLK = (MODE == kSelSmem);
    constexpr bool APPEND = (MODE == kSelAppend);
    extern __shared__ uint8_t smem_raw[];
    // a fallback pass whose predecessor found nothing to repair: leave before anything is set up
    if (args.gate && *args.gate != kScreenOverflow) return;
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    float *qkey = reinterpret_cast<float *>(smem + SmemLayout::queue_key);
    int32_t *qidx = reinterpret_cast<int32_t *>(smem + SmemLayout::queue_idx);
    float *xn_all = reinterpret_cast<float *>(smem + SmemLayout::xnorm);
    const uint32_t bar_full = smem_base + SmemLayout::barriers;
    const uint32_t bar_empty = bar_full + 8 * kBarStages;
    const uint32_t bar_tfull = bar_empty + 8 * kBarStages;
    // (pair mode with both 16-bit parts of the queries staged, split2: stages of A_hi, A_lo and half a row tile)
    const uint32_t pair_stage_bytes = args.split2 ? kPairStageBytes + kABytes : kPairStageBytes;
    const uint32_t nstages = PAIR ? (args.split2 ? kPairStagesSplit2 : kPairStages) : args.screen ? kMaxStages : kStages;
    // pair mode: rank of this CTA in its cluster of two; rank 0 (the leader) issues the MMAs of both
    const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
    const bool leader = crank == 0;
    const uint32_t bar_tempty = bar_tfull + 16;
    const uint32_t bar_conv = bar_tempty + 16;  // derive_lo: the converter warps are done with the stage
    volatile uint32_t *tmem_ptr_s = reinterpret_cast<volatile uint32_t *>(smem + SmemLayout::tmem_ptr);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + SmemLayout::abort_flag);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kBarStages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int s = 0; s < kBarStages; s++) mbar_init(bar_conv + 8 * s, kConvWarps);
        for (int b = 0; b < 2; b++) {
            mbar_init(bar_tfull + 8 * b, 1);
            // one arrival per epilogue warp (pair mode: of both CTAs, on the leader's barrier)
            mbar_init(bar_tempty + 8 * b, PAIR ? 8 : 4);
        }
        for (int w = 0; w < kWorkRing; w++) {
            mbar_init(smem_base + SmemLayout::work_bars + 8 * w, 1);                    // written by the scheduler
            // read by MMA + 4 epilogue warps (+ the converter warps)
            mbar_init(smem_base + SmemLayout::work_bars + 8 * (kWorkRing + w), 5 + (args.derive_lo ? kConvWarps : 0));
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        // pair mode: the same warp of both CTAs allocates the same columns in both tensor memories
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_base + SmemLayout::tmem_ptr),
                         "r"(512u)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_base + SmemLayout::tmem_ptr),
                         "r"(512u)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tmem_fence_before();
    __syncthreads();
    // pair mode: the peer's barriers are initialised before anything of this CTA signals them
    if (PAIR) cluster_sync_all();
    tmem_fence_after();
    const uint32_t tmem_base = *tmem_ptr_s;

    struct Work {
        int qt, row_begin, row_end, slot, fresh, pad[3];
    };
    volatile Work *ring = reinterpret_cast<volatile Work *>(smem + SmemLayout::work_ring);
    const uint32_t bar_wfull = smem_base + SmemLayout::work_bars;
    const uint32_t bar_wempty = bar_wfull + 8 * kWorkRing;

    if (warp == 0) {
        // ---------------------------------------------------------------- scheduler + TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            int issued = 0;   // K blocks loaded so far (test hook only)
            uint32_t wi = 0;  // work items announced
            int cur = -1, slot = -1, fresh = 0;
            // Adopts query tile t if it still has chunks and a free list slot.
            auto adopt = [&](int t) -> bool {
                if (*reinterpret_cast<volatile int *>(args.next_chunk + t) >= args.nchunks) return false;
                const int j = atomicAdd(args.nlists + t, 1);
                if (j >= args.lists_per_qt) return false;
                cur = t;
                slot = t * args.lists_per_qt + j;
                fresh = 1;
                return true;
            };
            const int home = blockIdx.x % args.nq_tiles;
            bool have = false;
            if (!args.items && !args.static_g)
                for (int i = 0; i < args.nq_tiles && !have; i++) have = adopt((home + i) % args.nq_tiles);
            const int n_items = args.items ? *args.n_items : 0;
            // static schedule: this CTA's share [ulo, uhi) of the units of every chunk, the (at
            // most two) query tiles it falls into, their list slots
            // (pair mode: the schedule is the pair's - both CTAs compute the same one - over PAIRS of
            // query tiles; this CTA's query tile of schedule tile t is 2 t + rank)
            const int G = args.static_g;
            const int sched_id = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
            const int sched_n = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
            const int sched_qt = PAIR ? args.nq_tiles >> 1 : args.nq_tiles;
            const long long U = (long long)sched_qt * G;
            const int ulo = G ? (int)(sched_id * U / sched_n) : 0;
            const int uhi = G ? (int)((sched_id + 1) * U / sched_n) : 0;
            const int t_first = G ? ulo / G : 0, t_last = G ? (uhi - 1) / G : -1;
            int st_slot[2] = {-1, -1};
            int st_chunk = 0, st_tile = t_first, st_active = -1, st_close = 0;
            bool st_arrived = false, st_paced = true;
            for (;;) {
                int64_t r_begin, r_end;
                if (G) {
                    bool got = false;
                    while (!got && st_chunk < args.static_chunks) {
                        if (st_tile > t_last) {
                            st_chunk++;
                            st_tile = t_first;
                            st_arrived = false;
                            continue;
                        }
                        if (!st_arrived) {
                            // nobody starts chunk c before everybody has started chunk c - pace_window:
                            // the CTAs stay within two chunks of one another in the store.  Bounded:
                            // pacing is an optimisation, never a condition for progress.
                            if (st_paced && st_chunk >= args.pace_window) {
                                const volatile int *prev = args.arrivals + (st_chunk - args.pace_window);
                                int spins = 0;
                                while (*prev < (int)gridDim.x && spins < kPaceSpins) {
                                    __nanosleep(100);
                                    spins++;
                                }
                                // a CTA of this grid that is a millisecond late is not running (its SM
                                // is held by another kernel): stop waiting for good, not chunk by chunk
                                if (spins >= kPaceSpins) st_paced = false;
                            }
                            atomicAdd(args.arrivals + st_chunk, 1);
                            st_arrived = true;
                        }
                        const int t = st_tile++;
                        const int a = ulo > t * G ? ulo : t * G, b = uhi < (t + 1) * G ? uhi : (t + 1) * G;
                        if (a >= b) continue;
                        r_begin = ((int64_t)st_chunk * G + (a - t * G)) * BN;
                        r_end = ((int64_t)st_chunk * G + (b - t * G)) * BN;
                        if (r_begin >= args.n) continue;
                        if (r_end > args.n) r_end = args.n;
                        const int si = t - t_first;
                        const int my_qt = PAIR ? 2 * t + (int)crank : t;
                        if (st_slot[si] < 0) {
                            const int j = atomicAdd(args.nlists + my_qt, 1);
                            if (j >= args.lists_per_qt) {  // cannot happen with the plan's list count
                                atomicExch(args.status, 9);
                                *abort_flag = 1;
                                goto done;
                            }
                            st_slot[si] = my_qt * args.lists_per_qt + j;
                            fresh = 1;
                        } else {
                            fresh = st_active != t ? 2 : 0;
                        }
                        st_active = t;
                        cur = my_qt;
                        slot = st_slot[si];
                        got = true;
                    }
                    if (!got) {
                        // all chunks done: one empty item per list, which closes it
                        while (st_close < 2 && st_slot[st_close] < 0) st_close++;
                        if (st_close >= 2) break;
                        cur = PAIR ? 2 * (t_first + st_close) + (int)crank : t_first + st_close;
                        slot = st_slot[st_close];
                        fresh = (st_active != t_first + st_close ? 2 : 0) | 4;
                        st_active = t_first + st_close;
                        st_close++;
                        r_begin = r_end = 0;
                    }
                } else if (args.items) {
                    // grouped mode: items are independent, each with its own lists
                    const int i = atomicAdd(args.item_counter, 1);
                    if (i >= n_items) break;
                    const int4 it4 = args.items[i];
                    cur = it4.x;
                    slot = it4.x;
                    fresh = 1;
                    r_begin = it4.y;
                    r_end = it4.z;
                    if (r_end <= r_begin) continue;  // empty list: the slot stays empty
                } else {
                    if (!have) break;
                    const int c = atomicAdd(args.next_chunk + cur, 1);
                    if (c >= args.nchunks) {  // this query tile is finished: look for another one
                        have = false;
                        const int from = cur;
                        for (int i = 1; i < args.nq_tiles && !have; i++) have = adopt((from + i) % args.nq_tiles);
                        continue;
                    }
                    r_begin = (int64_t)c * args.tiles_per_chunk * BN;
                    r_end = r_begin + (int64_t)args.tiles_per_chunk * BN;
                    if (r_end > args.n) r_end = args.n;
                }
                {
                    const uint32_t w = wi % kWorkRing;
                    if (!mbar_wait(bar_wempty + 8 * w, ((wi / kWorkRing) & 1) ^ 1, abort_flag, args.status, args.wait_ns, 5)) goto done;
                    ring[w].qt = cur;
                    ring[w].row_begin = (int)r_begin;
                    ring[w].row_end = (int)r_end;
                    ring[w].slot = slot;
                    ring[w].fresh = fresh;
                    fresh = 0;
                    __threadfence_block();
                    mbar_arrive(bar_wfull + 8 * w);
                    wi++;
                }
                for (int64_t trow = r_begin; trow < r_end; trow += BN) {
                    for (int kb = 0; kb < args.kblocks; kb++) {
                        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, args.status, args.wait_ns, 1)) goto done;
                        // test hook: from this K block on nothing is loaded, so the MMA issuer's
                        // wait for the stage runs out and the give-up path is exercised
                        if (args.withhold_after >= 0 && issued++ >= args.withhold_after) goto done;
                        const uint32_t full = bar_full + 8 * stage;
                        if (PAIR) {
                            // own queries + this CTA's half of the row tile; the bytes of both CTAs are
                            // counted on the LEADER's barrier, which its MMA issuer waits on
                            const uint32_t base = smem_base + stage * pair_stage_bytes;
                            const uint32_t full_leader = map_to_cta(full, 0);
                            if (leader) mbar_expect_tx(full, 2 * pair_stage_bytes);
                            tma_load_2d_pair(base, &map_qhi, kb * BK, cur * BM, full_leader);
                            if (args.split2) tma_load_2d_pair(base + kABytes, &map_qlo, kb * BK, cur * BM, full_leader);
                            tma_load_2d_pair(base + (args.split2 ? 2 : 1) * kABytes, &map_xlo, kb * BK,
                                             (int32_t)trow + (int32_t)crank * (BN / 2), full_leader);
                        } else if (args.screen) {  // hi planes only, into plane set stage & 1 of stage >> 1
                            const uint32_t base = smem_base + (stage >> 1) * kStageBytes;
                            mbar_expect_tx(full, kABytes + kBBytes);
                            tma_load_2d(base + (stage & 1) * kABytes, &map_qhi, kb * BK, cur * BM, full);
                            tma_load_2d(base + 2 * kABytes + (stage & 1) * kBBytes, &map_xhi, kb * BK, (int32_t)trow, full);
                        } else {
                            const uint32_t base = smem_base + stage * kStageBytes;
                            // (16-bit build: no lo plane of the rows exists; derive_lo: it is formed in shared memory)
                            const bool one_row_plane = kH16 || args.derive_lo;
                            mbar_expect_tx(full, one_row_plane ? 2 * kABytes + kBBytes : kStageBytes);
                            tma_load_2d(base, &map_qhi, kb * BK, cur * BM, full);
                            tma_load_2d(base + kABytes, &map_qlo, kb * BK, cur * BM, full);
                            tma_load_2d(base + 2 * kABytes, &map_xhi, kb * BK, (int32_t)trow, full);
                            if (!one_row_plane) tma_load_2d(base + 2 * kABytes + kBBytes, &map_xlo, kb * BK, (int32_t)trow, full);
                        }
                        if (++stage == nstages) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
            }
            {  // end marker
                const uint32_t w = wi % kWorkRing;
                if (!mbar_wait(bar_wempty + 8 * w, ((wi / kWorkRing) & 1) ^ 1, abort_flag, args.status, args.wait_ns, 5)) goto done;
                ring[w].qt = -1;
                __threadfence_block();
                mbar_arrive(bar_wfull + 8 * w);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t it = 0;  // tiles issued by this CTA
            const uint32_t fmt = kH16 ? operand_format(args.bf16) : 0u;
            for (uint32_t wi = 0;; wi++) {
                const uint32_t w = wi % kWorkRing;
                if (!mbar_wait(bar_wfull + 8 * w, (wi / kWorkRing) & 1, abort_flag, args.status, args.wait_ns, 6)) goto done;
                const int qt = ring[w].qt;
                const int64_t r_begin = ring[w].row_begin, r_end = ring[w].row_end;
                mbar_arrive(bar_wempty + 8 * w);
                if (qt < 0) break;
                if (PAIR && !leader) continue;  // the leader issues the MMAs of both CTAs
                for (int64_t trow = r_begin; trow < r_end; trow += BN, it++) {
                    const uint32_t buf = it & 1;
                    long long t0 = kstats(args) ? clock64() : 0;
                    if (!mbar_wait(bar_tempty + 8 * buf, ((it >> 1) & 1) ^ 1, abort_flag, args.status, args.wait_ns, 2)) goto done;
                    if (kstats(args)) atomicAdd(kstats(args) + kStatMmaWaitTmem, (unsigned long long)(clock64() - t0));
                    tmem_fence_after();
                    const uint32_t tmem_d = tmem_base + buf * BN;
                    for (int kb = 0; kb < args.kblocks; kb++) {
                        t0 = kstats(args) ? clock64() : 0;
                        if (!mbar_wait((args.derive_lo ? bar_conv : bar_full) + 8 * stage, phase, abort_flag, args.status,
                                       args.wait_ns, 3))
                            goto done;
                        if (kstats(args)) atomicAdd(kstats(args) + kStatMmaWaitSmem, (unsigned long long)(clock64() - t0));
                        tmem_fence_after();
                        if (PAIR) {
                            const uint32_t base = smem_base + stage * pair_stage_bytes;
                            const uint64_t a0 = make_smem_desc(base);
                            const uint64_t b0 = make_smem_desc(base + (args.split2 ? 2 : 1) * kABytes);
                            if (args.split2) {
                                // 16-bit rows are exact: the query alone is split, q = q_hi + q_lo
                                const uint64_t a1 = make_smem_desc(base + kABytes);
#pragma unroll
                                for (int ks = 0; ks < BK / kMmaK; ks++) {
                                    mma_issue_pair(tmem_d, a1 + 2 * ks, b0 + 2 * ks, (kb | ks) != 0, fmt);
                                    mma_issue_pair(tmem_d, a0 + 2 * ks, b0 + 2 * ks, 1, fmt);
                                }
                            } else if (!(kdebug(args) & 2)) {
                                mma_issue_pair(tmem_d, a0, b0, kb != 0, fmt);
#pragma unroll
                                for (int ks = 1; ks < BK / kMmaK; ks++) mma_issue_pair(tmem_d, a0 + 2 * ks, b0 + 2 * ks, 1, fmt);
                            }
                            mma_commit_pair(bar_empty + 8 * stage);  // frees the stage in both CTAs
                            if (++stage == nstages) {
                                stage = 0;
                                phase ^= 1;
                            }
                            continue;
                        }
                        if (args.screen) {
                            // One MMA per K step: the loop of this single thread is what paces the
                            // tensor pipe, so the descriptors are formed once per K block and only
                            // their address field moves (32 bytes = 2 units of 16 per K step).
                            const uint32_t base = smem_base + (stage >> 1) * kStageBytes;
                            const uint64_t a0 = make_smem_desc(base + (stage & 1) * kABytes);
                            const uint64_t b0 = make_smem_desc(base + 2 * kABytes + (stage & 1) * kBBytes);
                            if (!(kdebug(args) & 2)) {
                                mma_issue(tmem_d, a0, b0, kb != 0, fmt);
#pragma unroll
                                for (int ks = 1; ks < BK / kMmaK; ks++) mma_issue(tmem_d, a0 + 2 * ks, b0 + 2 * ks, 1, fmt);
                            }
                        } else {
                            const uint32_t base = smem_base + stage * kStageBytes;
#pragma unroll
                            for (int ks = 0; ks < BK / kMmaK; ks++) {
                                const uint64_t a_hi = make_smem_desc(base + ks * 32);
                                const uint64_t a_lo = make_smem_desc(base + kABytes + ks * 32);
                                const uint64_t b_hi = make_smem_desc(base + 2 * kABytes + ks * 32);
                                const uint64_t b_lo = make_smem_desc(base + 2 * kABytes + kBBytes + ks * 32);
                                if (kdebug(args) & 2) continue;
                                if (kH16) {
                                    // 16-bit rows are exact: the query alone is split, q = q_hi + q_lo
                                    mma_issue(tmem_d, a_lo, b_hi, (kb | ks) != 0, fmt);
                                    mma_issue(tmem_d, a_hi, b_hi, 1, fmt);
                                } else {
                                    mma_issue(tmem_d, a_hi, b_lo, (kb | ks) != 0);
                                    mma_issue(tmem_d, a_lo, b_hi, 1);
                                    mma_issue(tmem_d, a_hi, b_hi, 1);
                                }
                            }
                        }
                        mma_commit(bar_empty + 8 * stage);  // stage is free once these MMAs have read it
                        if (++stage == nstages) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                    // accumulator complete (pair mode: in both CTAs' tensor memories)
                    if (PAIR) mma_commit_pair(bar_tfull + 8 * buf);
                    else mma_commit(bar_tfull + 8 * buf);
                }
            }
        }
    } else if (warp >= 2 + 4) {
        // ---------------------------------------------------------------- row-plane converter (derive_lo launches only)
        // The row tile arrives as plain fp32 values.  Each converter warp takes its share of the
        // stage's row slot, writes hi = the value rounded to TF32 back in place and lo = value - hi
        // into the lo slot (same swizzled offsets: the operation is element-wise), makes the writes
        // visible to the tensor core's reads and arrives on the stage's "converted" barrier.
        const int cw = warp - (2 + 4);
        uint32_t stage = 0, phase = 0;
        for (uint32_t wi = 0;; wi++) {
            const uint32_t w = wi % kWorkRing;
            if (!mbar_wait(bar_wfull + 8 * w, (wi / kWorkRing) & 1, abort_flag, args.status, args.wait_ns, 10)) goto done;
            const int qt = ring[w].qt;
            const int64_t r_begin = ring[w].row_begin, r_end = ring[w].row_end;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_wempty + 8 * w);
            if (qt < 0) break;
            for (int64_t trow = r_begin; trow < r_end; trow += BN) {
                for (int kb = 0; kb < args.kblocks; kb++) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, args.status, args.wait_ns, 11)) goto done;
                    constexpr int kVecs = kBBytes / 16 / kConvWarps;  // float4 per converter warp
                    float4 *hi4 = reinterpret_cast<float4 *>(smem + (size_t)stage * kStageBytes + 2 * kABytes) + cw * kVecs;
                    float4 *lo4 = hi4 + kBBytes / 16;
                    // all loads first: a store to the lo slot in between would keep the compiler from
                    // moving the next load up (it cannot see that the slots do not overlap)
                    static_assert(kVecs % 32 == 0, "whole rounds of the warp");
                    float4 v[kVecs / 32];
#pragma unroll
                    for (int j = 0; j < kVecs / 32; j++) v[j] = hi4[lane + 32 * j];
#pragma unroll
                    for (int j = 0; j < kVecs / 32; j++) {
                        const float4 h = make_float4(round_tf32(v[j].x), round_tf32(v[j].y), round_tf32(v[j].z), round_tf32(v[j].w));
                        hi4[lane + 32 * j] = h;
                        lo4[lane + 32 * j] = make_float4(v[j].x - h.x, v[j].y - h.y, v[j].z - h.z, v[j].w - h.w);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_conv + 8 * stage);
                    if (++stage == nstages) {
                        stage = 0;
                        phase ^= 1;
                    }
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
        // state of the current list (one per row, kept while the CTA stays with a query tile)
        float *unit_key = nullptr;
        int32_t *unit_idx = nullptr;
        uint32_t *qtau_word = nullptr;  // this row's shared-threshold word
        float koff = 0.f;               // published key = key + koff (residual-query mode), else 0
        bool row_valid = false;
        float tau = -kInf;       // a key must be below this to matter
        float list_max = kInf;   // small k: current maximum of this row's list
        float published = kInf;
        int cnt = 0;             // queue fill (large k)
        int pos = 0;             // slot of the current maximum (small k)
        const int stride = APPEND ? kBuf : k;  // slots per row in the list memory
        int cur_slot = 0;
        float slack = 0.f;  // screened mode: twice the error bound of this row's coarse keys
        const int k_rank = (APPEND && args.banded) ? args.k_rank : k;
        auto close_list = [&]() {
            if (!unit_key) return;
            if (APPEND && args.part_cnt) {
                // the per-query merge sees the final threshold of the query and throws most of
                // these entries away before it sorts: nothing to do here but say how many there are
                // (flat search: index = list slot * 128 + row as well)
                args.part_cnt[(size_t)cur_slot * BM + row] = row_valid ? cnt : 0;

            } else if (APPEND) {
                const unsigned need = __ballot_sync(kFullMask, cnt > 0);
                if (need) compact_rows(unit_key, unit_idx, k, quarter * 32, need, cnt, tau, lane, qtau_word, koff, k_rank, slack);
                if (!((need >> lane) & 1u)) {  // no candidate ever reached this row: an empty list
                    for (int s = 0; s < k; s++) unit_idx[(size_t)row * kBuf + s] = -1;
                }
            } else if (SMALLK) {
                for (int s = 0; s < k; s++) {
                    unit_key[(size_t)row * k + s] = qkey[s * BM + row];
                    unit_idx[(size_t)row * k + s] = qidx[s * BM + row];
                }
            } else {
                if (__any_sync(kFullMask, cnt > 0))
                    flush_queues<KR>(unit_key, unit_idx, k, quarter * 32, qkey, qidx, cnt, tau, lane, qtau_word, koff);
            }
        };
        for (uint32_t wi = 0;; wi++) {
            const uint32_t w = wi % kWorkRing;
            if (!mbar_wait(bar_wfull + 8 * w, (wi / kWorkRing) & 1, abort_flag, args.status, args.wait_ns, 7)) goto done;
            const int qt = ring[w].qt, slot = ring[w].slot, fresh = ring[w].fresh;
            const int64_t r_begin = ring[w].row_begin, r_end = ring[w].row_end;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_wempty + 8 * w);
            if (qt < 0) break;
            if (fresh & 3) {
                if (args.static_g) {
                    // static schedule: the list left behind is taken up again later; only its fill
                    // count has to survive (the buffer is in global memory, thresholds are shared)
                    if (APPEND && unit_key) args.slot_cnt[(size_t)cur_slot * BM + row] = cnt;
                } else {
                    close_list();
                }
                cur_slot = slot;
                unit_key = args.part_key + (size_t)slot * BM * stride;
                unit_idx = args.part_idx + (size_t)slot * BM * stride;
                if (args.items) {
                    // grouped mode: the row's threshold word belongs to its query, shared by all
                    // the lists that query probes; padding rows carry -1
                    const int32_t q = args.qrow_query[(size_t)qt * BM + row];
                    row_valid = q >= 0;
                    qtau_word = args.qtau + (row_valid ? q : 0);
                    koff = (args.qrow_const && row_valid) ? args.qrow_const[(size_t)qt * BM + row] : 0.f;
                } else {
                    row_valid = (int64_t)qt * BM + row < args.nq;
                    qtau_word = args.qtau + (size_t)qt * BM + row;
                    if (APPEND && args.banded && row_valid) {
                        slack = key_slack(args.q_norm2[(size_t)qt * BM + row], __uint_as_float(*args.x_max_norm2), args.d,
                                          args.l2 != 0, args.screen != 0,
                                          kH16 ? (args.bf16 ? kElemBF16 : kElemF16) : kElemF32);
                    }
                }
                tau = row_valid ? kInf : -kInf;
                list_max = kInf;
                published = kInf;
                cnt = (APPEND && (fresh & 2)) ? args.slot_cnt[(size_t)slot * BM + row] : 0;
                pos = 0;
                if (APPEND) {
                    // nothing to initialise: a row's buffer is valid up to its fill count
                } else if (SMALLK) {
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
            }
            for (int64_t trow = r_begin; trow < r_end; trow += BN, it++) {
                const uint32_t buf = it & 1;
                if (args.l2) {
                    for (int j = lane; j < BN; j += 32) {
                        const int64_t col = trow + j;
                        xn_s[buf * BN + j] = col < r_end ? __ldg(args.xnorm + col) : 0.f;
                    }
                    __syncwarp();
                }
                long long t0 = (kstats(args) && lane == 0) ? clock64() : 0;
                if (!mbar_wait(bar_tfull + 8 * buf, (it >> 1) & 1, abort_flag, args.status, args.wait_ns, 4)) goto done;
                long long t1 = 0;
                if (kstats(args) && lane == 0) {
                    t1 = clock64();
                    atomicAdd(kstats(args) + kStatEpiWaitCycles, (unsigned long long)(t1 - t0));
                    atomicAdd(kstats(args) + kStatTiles, 1ull);
                }
                tmem_fence_after();
                if (row_valid) {
                    // thresholds published by the other CTAs working on this query (L2-coherent read)
                    // (rounded up after taking the row's constant out: never tighter than published)
                    const float tg = __fadd_ru(ordered_to_float(__ldcg(qtau_word)), -koff);
                    if (tg < tau) tau = tg;
                }
                const int64_t rem = r_end - trow;
                const int ncols = rem < BN ? (int)rem : BN;
                const int32_t col0 = (int32_t)trow;
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
                // Selection over 32 accumulator columns (raw: the registers of one TMEM read).
                // The common case - no column beats the threshold - is branch-free: with one
                // warp per scheduler a branch per column would cost far more than the
                // arithmetic.  Keys are formed and compared with predicated instructions into
                // a bit mask; one warp vote then decides whether anything has to be done.
                auto key_of = [&](const uint32_t (&raw)[32], int g, int j) -> float {
                    const float acc = __uint_as_float(raw[j]);
                    return args.l2 ? fmaf(-2.f, acc, xn_s[buf * BN + g * 32 + j]) : -acc;
                };
                auto beat_mask = [&](const uint32_t (&raw)[32], int g, uint32_t valid) -> uint32_t {
                    uint32_t mask = 0;
#pragma unroll
                    for (int j = 0; j < 32; j++) mask |= (key_of(raw, g, j) < tau) ? (1u << j) : 0u;
                    return mask & valid;
                };
                // key of column j, j known only at run time: the accumulator comes out of a select tree
                auto pick = [&](const uint32_t (&raw)[32], int g, int j) -> float {
                    const float acc = __uint_as_float(select32(raw, j));
                    return args.l2 ? fmaf(-2.f, acc, xn_s[buf * BN + g * 32 + j]) : -acc;
                };
                auto process32 = [&](const uint32_t (&raw)[32], int g) {
                    const int nvalid = ncols - g * 32;
                    if (nvalid <= 0) return;
                    const uint32_t valid = nvalid >= 32 ? 0xffffffffu : ((1u << nvalid) - 1u);
                    if (kdebug(args) & 8) {  // measurement only: consume the registers, no selection
                        uint32_t x = 0;
#pragma unroll
                        for (int j = 0; j < 32; j++) x ^= raw[j];
                        if (x == 0x12345678u) tau = 0.f;
                        return;
                    }
                    // inner product: key = -acc, so no column of the 32 beats the threshold unless their
                    // largest accumulator does - 16 instructions instead of the 64 that form the mask
                    if (!args.l2 && !__any_sync(kFullMask, max32(raw) > -tau)) return;
                    uint32_t mask = beat_mask(raw, g, valid);
                    if (!__any_sync(kFullMask, mask != 0)) return;
                    // some row has a candidate: what follows has loops, jumps and a call, and the read of
                    // the next 32 columns is in flight into the other register buffer - let it land first
                    const long long s0 = kstats(args) ? clock64() : 0;
                    tmem_ld_wait_all();
                    const long long s1 = kstats(args) ? clock64() : 0;
                    const int32_t colg = col0 + g * 32;
                    if (APPEND) {
                        const unsigned need = __ballot_sync(kFullMask, cnt + __popc(mask) > kBuf);
                        if (need) {
                            const long long c0 = kstats(args) ? clock64() : 0;
                            compact_rows(unit_key, unit_idx, k, quarter * 32, need, cnt, tau, lane, qtau_word, koff, k_rank, slack);
                            if (kstats(args) && lane == 0) {
                                atomicAdd(kstats(args) + kStatCompactCycles, (unsigned long long)(clock64() - c0));
                                atomicAdd(kstats(args) + kStatCompactRows, (unsigned long long)__popc(need));
                            }
                            mask = beat_mask(raw, g, valid);
                        }
                        if (kdebug(args) & 4) mask = 0;
                        if (kstats(args) && mask) atomicAdd(kstats(args) + kStatAppends, (unsigned long long)__popc(mask));
                        float *bk = unit_key + (size_t)row * kBuf;
                        int32_t *bi = unit_idx + (size_t)row * kBuf;
                        if (!__any_sync(kFullMask, __popc(mask) > 4)) {
                            // Sparse hits (the steady state: about one per row and tile): every lane walks its
                            // own hits, so the warp makes one or two rounds per 32 columns.  The column of a hit
                            // is known only at run time and registers cannot be indexed: the value comes out of
                            // a five-level select tree over the 32 registers (31 selects, no dependency chain
                            // longer than five).
                            while (__any_sync(kFullMask, mask != 0)) {
                                const bool p = mask != 0;
                                const int j = p ? __ffs(mask) - 1 : 0;
                                mask &= mask - 1;
                                st_global_pair_if(p, bk + cnt, pick(raw, g, j), bi + cnt, colg + j);
                                cnt += p ? 1 : 0;
                            }
                        } else {
                            // Dense hits (a list that has no threshold yet, or a short one): all 32 columns in
                            // straight-line code, a predicated pair of stores each - ~25 cycles per column
                            // whatever it holds.  (A warp-uniform loop over the columns that have a hit, with a
                            // jump table on the column number, cost ~160 cycles per column it visited.)
#pragma unroll
                            for (int j = 0; j < 32; j++) {
                                const bool p = (mask >> j) & 1u;
                                st_global_pair_if(p, bk + cnt, key_of(raw, g, j), bi + cnt, colg + j);
                                cnt += p ? 1 : 0;
                            }
                        }
                        if (kstats(args) && lane == 0) {
                            atomicAdd(kstats(args) + kStatSlowGroups, 1ull);
                            atomicAdd(kstats(args) + kStatSlowCycles, (unsigned long long)(clock64() - s0));
                            atomicAdd(kstats(args) + kStatLdWaitCycles, (unsigned long long)(s1 - s0));
                        }
                    } else if (SMALLK) {
                        while (mask) {
                            const int j = __ffs(mask) - 1;
                            mask &= mask - 1;
                            const float key = pick(raw, g, j);
                            if (key < tau) {  // tau may have dropped since the mask was formed
                                qkey[pos * BM + row] = key;
                                qidx[pos * BM + row] = colg + j;
                                float m = -kInf;
                                for (int s = 0; s < k; s++) {
                                    const float v = qkey[s * BM + row];
                                    if (v > m) {
                                        m = v;
                                        pos = s;
                                    }
                                }
                                list_max = m;
                                tau = fminf(tau, m);
                            }
                        }
                    } else {
                        // the queue holds 16 entries: take the 32 columns in two halves
#pragma unroll 1
                        for (int half = 0; half < 2; half++) {
                            uint32_t hm = (mask >> (16 * half)) & 0xffffu;
                            const bool overflow = cnt + __popc(hm) > kQueueDepth;
                            if (__any_sync(kFullMask, overflow)) {
                                flush_queues<KR>(unit_key, unit_idx, k, quarter * 32, qkey, qidx, cnt, tau, lane,
                                                 qtau_word, koff);
                                mask = beat_mask(raw, g, valid);
                                hm = (mask >> (16 * half)) & 0xffffu;
                            }
                            while (hm) {
                                const int j = __ffs(hm) - 1 + 16 * half;
                                hm &= hm - 1;
                                qkey[cnt * BM + row] = pick(raw, g, j);
                                qidx[cnt * BM + row] = colg + j;
                                cnt++;
                            }
                        }
                    }
                };
                if (!(kdebug(args) & 1)) {
                    // Two register buffers: the read of the next 32 columns is in flight while
                    // the current 32 are scanned.
                    uint32_t ra[32], rb[32];
                    tmem_ld32_issue(taddr, ra);
#pragma unroll 1
                    for (int g = 0; g < BN / 32; g += 2) {
                        tmem_ld_wait(ra);
                        tmem_ld32_issue(taddr + (g + 1) * 32, rb);
                        process32(ra, g);
                        tmem_ld_wait(rb);
                        if (g + 2 < BN / 32) tmem_ld32_issue(taddr + (g + 2) * 32, ra);
                        process32(rb, g + 1);
                    }
                }
                tmem_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * buf, 0));
                    else mbar_arrive(bar_tempty + 8 * buf);
                }
                if (kstats(args) && lane == 0) atomicAdd(kstats(args) + kStatEpiTileCycles, (unsigned long long)(clock64() - t1));
                if (SMALLK && list_max < published) {
                    published = list_max;
                    atomicMin(qtau_word, float_to_ordered(__fadd_ru(list_max, koff)));
                }
            }
            if (fresh & 4) {  // static schedule, after the last chunk: this list is complete
                close_list();
                unit_key = nullptr;
            }
        }
        close_list();
    }
done:
    tmem_fence_before();
    __syncthreads();
    // pair mode: neither CTA frees its tensor memory or leaves while the other may still signal its
    // barriers or (the leader) write its accumulators
    if (PAIR) cluster_sync_all();
    if (warp == 1) {
        tmem_fence_after();
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
        else
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

// Row-major (rows x dp) fp32 matrix, boxes of box_rows x BK floats, swizzled by
// row width.  Rows past `rows` read as zero.
int make_map(CUtensorMap *map, const float *base, int64_t rows, int dp, int box_rows, bool bf16 = false) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error("cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)dp, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)dp * kElemBytes};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    // (16-bit build: `base` points at fp16 or bf16 elements)
    const CUtensorMapDataType type = !kH16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                     : bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                            : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = fn(map, type, 2, const_cast<float *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, kWideRows ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error("cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

template <int KR, int MODE>
int launch_variant(const FlatPlan &plan, const CUtensorMap maps[4], const KernelArgs &args, cudaStream_t stream) {
    if constexpr (KR == 1 && MODE == kSelAppend && kWideRows) {
      if (args.pair) {  // clusters of two CTAs
        ANN_CUDA_TRY(cudaFuncSetAttribute(flat_tc_kernel<KR, MODE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kSmemBytes));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)plan.grid);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        ANN_CUDA_TRY(cudaLaunchKernelEx(&cfg, flat_tc_kernel<KR, MODE, true>, maps[0], maps[1], maps[2], maps[3], args));
        count_launch();
        return 0;
      }
    }
    if (args.pair) return set_error("internal: pair mode asked of a kernel variant that has none");
    ANN_CUDA_TRY(cudaFuncSetAttribute(flat_tc_kernel<KR, MODE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemBytes));
    flat_tc_kernel<KR, MODE, false><<<plan.grid, args.derive_lo ? kThreadsDerive : kThreads, kSmemBytes, stream>>>(
        maps[0], maps[1], maps[2], maps[3], args);
    count_launch();
    ANN_CUDA_TRY(cudaGetLastError());
    return 0;
}

// Whether grid / 2 clusters of two CTAs of the append kernel can be resident at once (every SM
// takes one CTA of this kernel; the pairs must find two free SMs side by side).  Asked once.
bool pair_clusters_fit(int grid) {
  if constexpr (!kWideRows) {
    (void)grid;
    return false;
  } else {
    static int max_clusters = [] {
        int n = 0;
        if (cudaFuncSetAttribute(flat_tc_kernel<1, kSelAppend, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
            cudaSuccess)
            return 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, flat_tc_kernel<1, kSelAppend, true>, &cfg) != cudaSuccess) {
            cudaGetLastError();
            return 0;
        }
        return n;
    }();
    return 2 * max_clusters >= grid;
  }
}

}  // namespace

#ifndef ANN_TC_SECONDARY
constexpr int64_t kMaxTilesPerChunk = 2;

namespace {
int gcd_int(int a, int b) { return b ? gcd_int(b, a % b) : a; }

// Static schedule for the screened search of a large store.  (Measured with the three-MMA product
// as well, 5M x 768 rows, 4096 queries, k = 10: 149 ms against 126 ms with dynamic chunks - that
// kernel is bound by the tensor pipe and gains nothing from the saved DRAM reads - so it is not
// used there.)  A chunk is G row tiles; its
// nq_tiles * G units (query tile t = u / G, row tile u % G) are dealt to the CTAs in equal
// contiguous shares, the same for every chunk, so that
//  - every CTA does the same work per chunk and all of them walk the store together: a row tile
//    comes from DRAM once and from L2 for the other query tiles (with chunks handed out per query
//    tile the tiles that have one CTA more run ahead, and the store was read ~11 times);
//  - a CTA works for at most two query tiles, alternating between their two lists.
// G = sms / gcd(sms, nq_tiles) makes the shares exact.
void choose_static(FlatPlan &p, int64_t n, int sms, bool screened) {
    p.static_g = 0;
    p.static_chunks = 0;
    p.pair = false;
    p.sched_ints = (size_t)p.nq_tiles * 2;
    static const bool off = [] { const char *e = getenv("ANN_CUDA_STATIC"); return e && atoi(e) == 0; }();
    static const bool pair_off = [] { const char *e = getenv("ANN_CUDA_PAIR"); return e && atoi(e) == 0; }();
    if (!screened || off || p.nq_tiles > sms) return;
    const int64_t ntiles = (n + BN - 1) / BN;
    // CTA pairs (sms / 2 of them over nq_tiles / 2 pairs of query tiles) when both are even
    const bool pair = !pair_off && sms % 2 == 0 && p.nq_tiles % 2 == 0;
    const int g = pair ? (sms / 2) / gcd_int(sms / 2, p.nq_tiles / 2) : sms / gcd_int(sms, p.nq_tiles);
    const int ctas_per_qt = (sms + p.nq_tiles - 1) / p.nq_tiles;
    if (ntiles < 16 * (int64_t)g || p.lists_per_qt < ctas_per_qt + 1) return;  // short stores: the ragged last chunk would cost more
    p.static_g = g;
    p.static_chunks = (int)((ntiles + g - 1) / g);
    p.pair = pair;
    p.grid = sms;
    // + one arrival counter per chunk, + one fill count per (list, row)
    p.sched_ints += (size_t)p.static_chunks + (size_t)p.nq_tiles * p.lists_per_qt * BM;
}
}  // namespace

FlatPlan make_flat_plan(int64_t nq, int64_t n, int k, int sms) {
    FlatPlan p;
    p.nq_tiles = (int)((nq + BM - 1) / BM);
    const int64_t ntiles = (n + BN - 1) / BN;
    // CTAs that will share one query tile, and chunks small enough that they finish together
    const int ctas_per_qt = (sms + p.nq_tiles - 1) / p.nq_tiles;
    int64_t tpc = ntiles / ((int64_t)ctas_per_qt * 8);
    if (tpc < 1) tpc = 1;
    // ... and short enough that all CTAs stay within a few MB of one another in the store: the
    // CTAs of one query tile pull consecutive chunks and every query tile starts at row 0, so a row
    // tile is fetched from DRAM by the first CTA that needs it and from L2 by the others, as long
    // as they are no more than a few tens of microseconds apart.  With long chunks (hundreds of
    // tiles) the 148 CTAs spread over gigabytes and every query tile streamed the store from DRAM
    // by itself (measured on 20M x 768 rows, 4096 queries: 14.0k queries/s with chunks of up to
    // 512 tiles, 14.4k with 4, 15.3k with 3, 16.0-16.5k with 2 or 1; the SM clock under the power
    // cap rises with every byte that does not come from DRAM).
    if (tpc > kMaxTilesPerChunk) tpc = kMaxTilesPerChunk;
    p.tiles_per_chunk = (int)tpc;
    p.nchunks = (int)((ntiles + tpc - 1) / tpc);
    // one k-list per CTA that ever works on a query tile; the merge sorts lists * k candidates
    int lists = 2 * ctas_per_qt + 2;
    const int cap = kMergeCandidates / (k > 0 ? k : 1);
    if (lists > cap) lists = cap;
    if (lists > p.nchunks) lists = p.nchunks;
    if (lists < 1) lists = 1;
    p.lists_per_qt = lists;
    const int64_t work = (int64_t)p.nq_tiles * p.nchunks;
    p.grid = (int)(work < sms ? work : sms);
    p.list_stride = (k > kQueueDepth && k <= kAppendMaxK) ? kBuf : k;
    p.lists_sorted = (k > kQueueDepth && k <= kAppendMaxK);
    p.part_entries = (size_t)p.nq_tiles * lists * BM * (size_t)p.list_stride;
    choose_static(p, n, sms, false);
    return p;
}

FlatPlan make_flat_plan_screened(int64_t nq, int64_t n, int k, int sms) {
    auto screened_plan = [&](int64_t nq_planned) {
        FlatPlan p = make_flat_plan(nq_planned, n, k, sms);
        // lists of up to kScreenMaxList entries, kept by the append selection
        p.list_stride = kBuf;
        p.lists_sorted = true;
        p.part_entries = (size_t)p.nq_tiles * p.lists_per_qt * BM * (size_t)p.list_stride;
        choose_static(p, n, sms, true);
        return p;
    };
    FlatPlan p = screened_plan(nq);
    // An odd number of query tiles has no pair mode.  With eleven tiles or more, one more tile that holds no
    // query (its rows are never looked at, its lists stay empty) costs less than pair mode gains: the plan is
    // made for the even count; the kernel's callers size their per-tile memory by plan.nq_tiles.
    if (p.static_g && !p.pair && p.nq_tiles % 2 == 1 && p.nq_tiles >= 11) {
        const FlatPlan padded = screened_plan((int64_t)(p.nq_tiles + 1) * BM);
        if (padded.pair) return padded;
    }
    return p;
}

FlatPlan make_grouped_plan(int64_t max_query_tiles, int k, int sms) {
    FlatPlan p;
    p.nq_tiles = (int)max_query_tiles;
    p.tiles_per_chunk = 0;
    p.nchunks = 0;
    p.lists_per_qt = 1;  // a gathered query tile is scanned by exactly one CTA
    p.grid = (int)(max_query_tiles < sms ? max_query_tiles : sms);
    if (p.grid < 1) p.grid = 1;
    p.list_stride = (k > kQueueDepth && k <= kAppendMaxK) ? kBuf : k;
    p.lists_sorted = (k > kQueueDepth && k <= kAppendMaxK);
    p.part_entries = (size_t)max_query_tiles * BM * (size_t)p.list_stride;
    p.sched_ints = 16;
    return p;
}

#endif  // !ANN_TC_SECONDARY

int ANN_TC_LAUNCH(const FlatPlan &plan, const float *xhi, const float *xlo, const float *xnorm, int64_t n,
                   const float *qhi, const float *qlo, int64_t nq, int dp, int k, int metric, float *part_key,
                   int32_t *part_idx, uint32_t *qtau, int *sched, int *status, int device, cudaStream_t stream,
                   const GroupedWork *grouped, const ScreenInput *screen, const int *gate, int32_t *flat_part_cnt) {
    (void)device;
    if (n <= 0 || nq <= 0) return 0;
    static_assert(kMaxListK <= 66 * 32, "the widest replace-max list covers every list length");
    if (k <= 0 || k > kMaxListK) return set_error("k must be in [1, %d]", kMaxListK);
#ifndef ANN_TC_SECONDARY
    // the screened (one-MMA) search runs in the build of this file with K blocks of 32 floats
    if (screen && screen->one_mma && !grouped && screen->k_rank >= 1 && screen->k_rank <= k && k <= kScreenMaxList &&
        k > kSmemListMax && dp % 32 == 0)
        return launch_flat_tc_bk32(plan, xhi, xlo, xnorm, n, qhi, qlo, nq, dp, k, metric, part_key, part_idx, qtau, sched,
                                   status, device, stream, grouped, screen, gate, flat_part_cnt);
#endif
    if (dp % BK != 0) return set_error("padded dimension must be a multiple of %d", BK);
    if (n > 0x7fffffffll - BN) return set_error("a flat shard holds at most 2^31 rows");
    CUtensorMap maps[4];
    const bool bf16 = kH16 && screen && screen->elem == kElemBF16;
    // (16-bit build: there is no lo plane of the rows; the fourth map repeats the third)
    // The query planes are allocated in whole tiles of 128 rows (the rows past nq hold anything: their
    // accumulator rows are never looked at), so no query load ever reaches past the end of its tensor.
    const int64_t nq_rows = grouped ? nq : (int64_t)plan.nq_tiles * BM;
    if (make_map(&maps[0], qhi, nq_rows, dp, BM, bf16) || make_map(&maps[1], qlo ? qlo : qhi, nq_rows, dp, BM, bf16) ||
        make_map(&maps[2], xhi, n, dp, BN, bf16) || make_map(&maps[3], (kH16 || !xlo) ? xhi : xlo, n, dp, BN, bf16))
        return -1;
    KernelArgs a;
    a.xnorm = xnorm;
    a.n = n;
    a.nq = nq;
    a.kblocks = dp / BK;
    a.k = k;
    a.l2 = metric != 0;
    a.nq_tiles = plan.nq_tiles;
    a.nchunks = plan.nchunks;
    a.tiles_per_chunk = plan.tiles_per_chunk;
    a.lists_per_qt = plan.lists_per_qt;
    a.next_chunk = sched;
    a.nlists = sched + plan.nq_tiles;
    a.ntiles = (n + BN - 1) / BN;
    a.part_key = part_key;
    a.part_idx = part_idx;
    a.qtau = qtau;
    a.status = status;
    a.items = grouped ? grouped->items : nullptr;
    a.n_items = grouped ? grouped->n_items : nullptr;
    a.item_counter = grouped ? grouped->item_counter : nullptr;
    a.static_chunks = plan.static_chunks;
    a.pace_window = 1;  // measured at 20M x 768: 19.0k queries/s with 1, 18.4k with 2 or 3, 13.8k unpaced
    a.arrivals = sched + 2 * plan.nq_tiles;
    a.slot_cnt = a.arrivals + plan.static_chunks;
    a.qrow_query = grouped ? grouped->qrow_query : nullptr;
    a.qrow_const = grouped ? grouped->qrow_const : nullptr;
    a.part_cnt = grouped ? grouped->part_cnt : flat_part_cnt;
    const bool use_band = screen && !grouped && screen->k_rank >= 1 && screen->k_rank <= k && k <= kScreenMaxList &&
                          k > kQueueDepth;  // banded lists are append buffers
    const bool use_screen = use_band && screen->one_mma;
    a.screen = use_screen ? 1 : 0;
    a.banded = use_band ? 1 : 0;
    // the static schedule parks and resumes append buffers; it pays for the screened search only
    // (16-bit build: the two-part product of banded lists takes it too, in pair mode)
    const bool two_part = kH16 && use_band && !use_screen;
    a.static_g = (use_screen || two_part) ? plan.static_g : 0;
    // pair mode: the fourth map becomes the hi plane of the rows in boxes of HALF a tile
    a.pair = (a.static_g && plan.pair && kWideRows && plan.grid % 2 == 0 && pair_clusters_fit(plan.grid)) ? 1 : 0;
    a.split2 = (two_part && a.pair) ? 1 : 0;
    if (two_part && !a.pair) a.static_g = 0;  // (the one-CTA static path stages hi planes only)
    if (a.pair && make_map(&maps[3], xhi, n, dp, BN / 2, bf16)) return -1;
    a.bf16 = bf16 ? 1 : 0;
    a.derive_lo = (grouped && grouped->derive_lo && !kH16) ? 1 : 0;
    a.k_rank = use_band ? screen->k_rank : k;
    a.q_norm2 = use_band ? screen->q_norm2 : nullptr;
    a.x_max_norm2 = use_band ? screen->x_max_norm2 : nullptr;
    a.d = use_band ? screen->d : dp;
    a.wait_ns = flat_wait_limit_ns();
    a.withhold_after = flat_test_withhold_after();
    a.gate = gate;
#ifdef ANN_CUDA_MEASURE
    {
        static const int debug_bits = [] { const char *e = getenv("ANN_CUDA_TC_DEBUG"); return e ? atoi(e) : 0; }();
        a.debug = debug_bits;
    }
    a.stats = nullptr;
    static unsigned long long *stats_dev = nullptr;
    static const bool want_stats = getenv("ANN_CUDA_TC_STATS") != nullptr;
    if (want_stats) {  // synchronises and prints
        if (!stats_dev) ANN_CUDA_TRY(cudaMalloc(&stats_dev, kStatCount * sizeof(unsigned long long)));
        ANN_CUDA_TRY(cudaMemsetAsync(stats_dev, 0, kStatCount * sizeof(unsigned long long), stream));
        a.stats = stats_dev;
    }
#endif
    int rc;
    if (k <= kQueueDepth) rc = launch_variant<1, kSelSmem>(plan, maps, a, stream);
    else if (k <= kAppendMaxK || use_band) rc = launch_variant<1, kSelAppend>(plan, maps, a, stream);
    else if (k <= 17 * 32) rc = launch_variant<17, kSelReplace>(plan, maps, a, stream);
    else if (k <= 33 * 32) rc = launch_variant<33, kSelReplace>(plan, maps, a, stream);
    else rc = launch_variant<66, kSelReplace>(plan, maps, a, stream);
#ifdef ANN_CUDA_MEASURE
    if (rc == 0 && a.stats) {
        unsigned long long h[kStatCount];
        ANN_CUDA_TRY(cudaStreamSynchronize(stream));
        ANN_CUDA_TRY(cudaMemcpy(h, a.stats, sizeof h, cudaMemcpyDeviceToHost));
        fprintf(stderr,
                "[flat_tc stats] grid %d k %d tiles(x4 warps) %llu | compact rows %llu cycles %llu | appends %llu | "
                "epilogue: wait %llu work %llu cycles | mma wait: tmem %llu smem %llu cycles | slow groups %llu cycles %llu "
                "(of which waiting for the load in flight %llu)\n",
                plan.grid, k, h[kStatTiles], h[kStatCompactRows], h[kStatCompactCycles], h[kStatAppends],
                h[kStatEpiWaitCycles], h[kStatEpiTileCycles], h[kStatMmaWaitTmem], h[kStatMmaWaitSmem], h[kStatSlowGroups],
                h[kStatSlowCycles], h[kStatLdWaitCycles]);
    }
#endif
    return rc;
}

}  // namespace anncuda
