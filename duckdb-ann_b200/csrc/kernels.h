// Launchers shared between the translation units of the CUDA search library.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace anncuda {

// Rows are stored padded to a multiple of kDimPad floats so that every row is a
// whole number of 128-byte TMA boxes.
constexpr int kDimPad = 32;
constexpr int kMaxK = 2048;  // largest k a search accepts
// Longest list a first-stage kernel keeps: the split-product search selects k + kSplitSpare
// candidates so that near ties at the k-th place can be settled by exact fp32 re-ranking.
constexpr int kSplitSpare = 32;
constexpr int kMaxListK = kMaxK + 2 * kSplitSpare;

inline int pad_dim(int d) { return (d + kDimPad - 1) / kDimPad * kDimPad; }

uint64_t launch_count_value();
void count_launch(int n = 1);

// Limit of every bounded wait inside the tensor-core kernel (process-wide; 2 s by default).
uint64_t flat_wait_limit_ns();
void set_flat_wait_limit_ns(uint64_t ns);
// Test hook, off (-1) by default: with a value >= 0 the TMA producer of every CTA stops loading
// after that many K blocks, so the MMA issuer's wait for the next stage runs out after the wait
// limit, the kernel records the give-up code and every role leaves in order.  The search then
// fails with an error; it never returns partial results as success.
int flat_test_withhold_after();
void set_flat_test_withhold_after(int k_blocks);

// ---- prep.cu -----------------------------------------------------------------------------
// x (n x d, row stride d) -> hi, lo (n x dp each): hi = x rounded to TF32, lo = x - hi
// (exact in fp32, so hi + lo reconstructs x bit for bit); pad columns are zero;
// norms[i] = sum x^2 in fp32 (may be nullptr).
// With `mu` (d floats, device) the norms are |x - mu|^2; with `center_rows` the planes hold
// x - mu too (queries), otherwise x itself (database rows).
// max_norm2_bits (optional, device word, zero before the first rows): raised to the bit pattern of
// the largest |x|^2 seen (not centred).
int launch_split_rows(const float *x, int64_t n, int d, int dp, float *hi, float *lo, float *norms,
                      cudaStream_t stream, const float *mu = nullptr, bool center_rows = false,
                      unsigned *max_norm2_bits = nullptr);
// mu[c] = mean over the n rows of x[r][c]
int launch_column_mean(const float *x, int64_t n, int d, float *mu, cudaStream_t stream);
// x (n x d) -> out (n x dp) zero padded, norms (may be nullptr).
int launch_pad_rows(const float *x, int64_t n, int d, int dp, float *out, float *norms, cudaStream_t stream);
// out (n x d) <- hi + lo (n x dp)
// (elem != kElemF32: `hi` holds n x dp 16-bit elements of that type, `lo` is unused)
int launch_join_rows(const float *hi, const float *lo, int64_t n, int d, int dp, float *out, cudaStream_t stream,
                     int elem = 0);
// Rows or queries of a 16-bit store (see prep_rows_h16_kernel): hi (and lo, queries only) are n x dp 16-bit
// elements; overflow (may be null) points at the status words of the two tensor-core tiers.
int launch_split_rows_h16(const float *x, int64_t n, int d, int dp, void *hi, void *lo, float *norms, cudaStream_t stream,
                          const float *mu, bool center_rows, unsigned *max_norm2_bits, int elem, int *overflow,
                          int32_t *bad_row = nullptr);

// ---- flat_tc.cu --------------------------------------------------------------------------
constexpr int kSmemListMax = 16;         // lists up to this length are kept in shared memory
constexpr int kAppendMaxK = 256;         // largest k the append-and-compact selection handles
constexpr int kMergeCandidates = 16384;  // most (list, slot) candidates per query the merge kernel sorts
// Threshold scan of the exact tier: entries of one flagged query's candidate buffer (at least two k), and
// of all buffers of a query block together (8 bytes each)
constexpr int kFlaggedCandidates = 4096;
constexpr int64_t kFlaggedEntries = 16 << 20;

struct FlatPlan {
    int nq_tiles = 0;         // ceil(nq / 128)
    int tiles_per_chunk = 0;  // 256-row tiles handed out at a time
    int nchunks = 0;          // chunks per query tile
    int lists_per_qt = 0;     // k-lists a query tile can end up with (one per CTA that worked on it)
    int grid = 0;
    int list_stride = 0;      // slots per row in the list memory (k, or the append buffer size)
    size_t part_entries = 0;  // nq_tiles * lists_per_qt * 128 * list_stride
    bool lists_sorted = false;  // every finished k-list is sorted best first (append mode)
    // Static schedule (append selection on large stores; 0 = chunks are handed out dynamically):
    // the store is walked in chunks of static_g row tiles and every CTA owns a fixed share of the
    // nq_tiles * static_g (query tile, row tile) units of each chunk.
    int static_g = 0, static_chunks = 0;
    // Static schedule over PAIRS of CTAs (clusters of two that share every row tile through
    // tcgen05 cta_group::2): needs an even number of query tiles and of SMs.
    bool pair = false;
    size_t sched_ints = 0;    // ints of scheduler memory (zero on entry)
};
// Chooses the decomposition for nq queries against n rows on a device with `sms` SMs.
FlatPlan make_flat_plan(int64_t nq, int64_t n, int k, int sms);

// Scratch of one flat_tc launch, set up by ONE kernel (gated like the launch it serves): the per-query
// threshold words to "no threshold yet" (all ones), the scheduler memory and the fill counts of the append
// lists (cnt, may be null) to zero, and - for the selections that write whole lists (idx non-null) - row
// number -1 in the first k slots of each of the `lists` lists of `list_stride` slots.
int launch_flat_scratch_init(uint32_t *qtau, size_t qtau_words, int *sched, size_t sched_ints, int32_t *cnt,
                             size_t cnt_words, int32_t *idx, size_t lists, int list_stride, int k, cudaStream_t stream,
                             const int *gate, int32_t *over_q = nullptr, size_t nq = 0);

// Fused split-TF32 GEMM + k-selection on the tensor cores.  Inputs are hi/lo row
// stores of the database (n x dp) and the queries (nq x dp, in buffers that hold whole tiles of 128
// rows: plan.nq_tiles * 128 x dp elements each - plan.nq_tiles may be one more than ceil(nq / 128) - the
// rows past nq unspecified), plus row norms for L2.
// Writes 128 unsorted lists of k (key, local row) pairs per list slot
// (slot = query tile * lists_per_qt + j, j < sched[nq_tiles + query tile]).
// Flat search with the append selection (FlatPlan::lists_sorted) and flat_part_cnt given: a list
// stays UNSORTED in the first flat_part_cnt[slot * 128 + row] slots of its row's buffer, for
// launch_merge_filtered (layout 0); nothing has to be cleared in the list memory then.
// On entry: part_idx all -1 (bytes 0xFF); qtau (nq_tiles * 128 words, the per-query shared
// threshold) all bytes 0xFF; sched (2 * nq_tiles ints: chunks taken, lists started) all zero.
// status: device int, set non-zero if a bounded wait inside the kernel ran out.
// Grouped mode (IVF list scan): `grouped` names device arrays of work items, one per tile
// of 128 gathered queries: {query tile, first row, end row} of the inverted list those
// queries probe.  The query stores then hold the GATHERED queries (query tile t = rows
// 128 t ..), list slot = query tile, and qrow_query maps a gathered row to its query
// (-1 = padding), whose word of `qtau` it shares with the query's other probes.
struct GroupedWork {
    const int4 *items;
    const int *n_items;
    int *item_counter;  // zero on entry
    const int32_t *qrow_query;
    const float *qrow_const = nullptr;  // per gathered row: add to a key to compare across lists (null = 0)
    // append mode only (16 < k <= kAppendMaxK), may be null: finished rows keep their append
    // buffer unsorted and write its fill count to part_cnt[gathered row]; use launch_merge_filtered
    int32_t *part_cnt = nullptr;
    // The rows are ONE plane of plain fp32 values (xhi; xlo is not read): two more warps of every CTA
    // split each row tile into its TF32 hi / lo parts in shared memory, between the load and the MMAs -
    // the same operands as with two stored planes, for half the bytes from DRAM.
    bool derive_lo = false;
};
FlatPlan make_grouped_plan(int64_t max_query_tiles, int k, int sms);

// Screened flat search (see KernelArgs::screen in flat_tc.cu).  The lists the kernel keeps are
// `k` long as always; `k_rank` (< k) is the rank whose key, plus the error slack, is the
// threshold: the caller asks for k = k_rank + spare candidates and re-ranks them exactly.
struct ScreenInput {
    int k_rank;                   // the caller's k
    const float *q_norm2;         // per query |q - mu|^2 (L2) or |q|^2 (IP)
    const unsigned *x_max_norm2;  // device word: bits of the largest |x|^2 in the store
    int d;                        // true dimension
    // true: one-MMA keys (q_hi.x_hi only; the build with 32-float K blocks, static schedule on
    // large stores).  false: the three-MMA split product with the same banded lists - the slack is
    // then the split product's much smaller one (see key_slack).
    bool one_mma = true;
    // 16-bit build only (launch_flat_tc_h16): kElemF16 or kElemBF16 operands.  There the rows are exact in
    // their 16-bit type and only the query is rounded (one_mma) or split in two 16-bit parts.
    int elem = 0;
};
constexpr int kScreenMaxList = 256;  // longest list (k_rank + spare) the screened mode keeps
constexpr int kScreenMaxK = kScreenMaxList - kSplitSpare;  // largest k searched with screening
constexpr int kScreenOverflow = 100;  // status code: more rows inside the error band than the spare holds
// Band check of a tensor-core ranking (screened = one-MMA keys, else split-product keys; see
// key_slack): sets *overflow (if still 0) to kScreenOverflow when the last of the k_list merged
// candidates of some query is still within the slack of its k_rank-th key - rows that belong
// among the exact k_rank best may then have been left out.  *overflow_count (may be null) is
// incremented once per launch that flags.
// Every launcher that takes a `gate` runs its kernel only if gate is null or *gate ==
// kScreenOverflow on the device when the kernel starts: that is how a fallback pass is enqueued
// behind the pass it repairs without a host round trip.
int launch_screen_check(const float *sel_key, int64_t nq, int k_list, int k_rank, const float *q_norm2,
                        const unsigned *x_max_norm2, int d, int metric, bool screened, int *overflow,
                        int *overflow_count, cudaStream_t stream, const int *gate = nullptr);

int launch_flat_tc(const FlatPlan &plan, const float *xhi, const float *xlo, const float *xnorm, int64_t n,
                   const float *qhi, const float *qlo, int64_t nq, int dp, int k, int metric, float *part_key,
                   int32_t *part_idx, uint32_t *qtau, int *sched, int *status, int device, cudaStream_t stream,
                   const GroupedWork *grouped = nullptr, const ScreenInput *screen = nullptr,
                   const int *gate = nullptr, int32_t *flat_part_cnt = nullptr);
// The same kernel built with K blocks of 32 floats (flat_tc_bk32.cu); launch_flat_tc hands the
// screened searches to it.
int launch_flat_tc_bk32(const FlatPlan &plan, const float *xhi, const float *xlo, const float *xnorm, int64_t n,
                        const float *qhi, const float *qlo, int64_t nq, int dp, int k, int metric, float *part_key,
                        int32_t *part_idx, uint32_t *qtau, int *sched, int *status, int device, cudaStream_t stream,
                        const GroupedWork *grouped, const ScreenInput *screen, const int *gate, int32_t *flat_part_cnt);
// The same kernel over 16-bit operands (flat_tc_h16.cu; tcgen05.mma kind::f16): xhi = rows as fp16 or bf16
// (n x dp elements, dp a multiple of 64), qhi / qlo = the two 16-bit parts of the queries, xlo unused.
// Banded lists only (screen non-null): one_mma -> q_hi.x, static schedule and pair mode as in the
// 32-float build; else q_hi.x + q_lo.x with dynamic chunks.
int launch_flat_tc_h16(const FlatPlan &plan, const float *xhi, const float *xlo, const float *xnorm, int64_t n,
                       const float *qhi, const float *qlo, int64_t nq, int dp, int k, int metric, float *part_key,
                       int32_t *part_idx, uint32_t *qtau, int *sched, int *status, int device, cudaStream_t stream,
                       const GroupedWork *grouped, const ScreenInput *screen, const int *gate, int32_t *flat_part_cnt);
// make_flat_plan for a screened search: lists of `k` (up to kScreenMaxList) in append mode
FlatPlan make_flat_plan_screened(int64_t nq, int64_t n, int k, int sms);

// IVF grouping: from probes (nq x nprobe list numbers, -1 = none) builds, on the device,
//   tile_off[l]     first gathered query tile of list l (lists padded to whole tiles of 128),
//   n_tiles         total gathered tiles (device int),
//   items[t]        {t, list_off[l], list_off[l+1], l} for every gathered tile t,
//   qrow_query[g]   query of gathered row g (-1 padding; caller pre-fills with 0xFF),
//   gslot[q*nprobe+p] gathered row of probe p of query q (-1 if that probe is invalid).
// scratch: 2 * (nlist + 1) ints.
int launch_group_probes(const int32_t *probes, int64_t nq, int nprobe, int64_t nlist, const int64_t *list_off,
                        int *scratch, int *n_tiles, int4 *items, int32_t *qrow_query, int32_t *gslot,
                        cudaStream_t stream);

// hi/lo split of gathered query rows: row g takes query qrow_query[g] of x (zeros if < 0),
// for g < 128 * *n_tiles.
// With `items` and the centroid planes given, gathered row g is written as the residual of its
// query against the centroid of list items[g / 128].w and qconst[g] = |v|^2 + 2 v.c.
int launch_split_gathered(const float *x, int d, int dp, const int32_t *qrow_query, const int *n_tiles,
                          int64_t max_rows, float *hi, float *lo, cudaStream_t stream, const int4 *items = nullptr,
                          const float *cent_hi = nullptr, const float *cent_lo = nullptr, float *qconst = nullptr);

// out[r] = |x_r - c|^2 for every row of a store grouped by list (CSR list_off), c = the
// centroid (cent_hi + cent_lo) of the row's list.
int launch_residual_norms(const float *xhi, const float *xlo, int64_t n, int d, int dp, const int64_t *list_off,
                          int nlist, const float *cent_hi, const float *cent_lo, float *out, cudaStream_t stream);

// ---- scan.cu -----------------------------------------------------------------------------
// Exact-fp32 scan of row ranges with warp k-selection: one warp per (query, range)
// item.  Item i scans rows [range_begin[i], range_end[i]) for query item_query[i] and
// writes an unsorted list of k (key, row) at part_*[i * k ...].  Rows are read from
// `x` (n x dp); when `xlo` is non-null the row is x + xlo (a split store).
// key = squared L2 distance, or negated dot.  qtau (optional, one word per query, all
// bytes 0xFF on entry): items of the same query share their k-th best key through it,
// so later items skip rows that cannot reach the query's final top-k.
// (elem != kElemF32: x holds 16-bit elements of that type, dp of them per row, xlo is unused)
int launch_scan_items(const float *x, const float *xlo, int dp, int d, const float *queries, int q_stride,
                      const int32_t *item_query, const int64_t *range_begin, const int64_t *range_end,
                      int64_t n_items, int k, int metric, float *part_key, int32_t *part_idx, uint32_t *qtau,
                      int device, cudaStream_t stream, const int *gate = nullptr, int elem = 0);

// Items of the exact flat scan, built on the device: item q * chunks + c = query q against rows
// [c * per, min(n, (c + 1) * per)).  With only_q (one word per query) the items of queries whose word is zero
// are marked "skip" (kItemSkip): the scan neither works on them nor writes their lists.
constexpr int32_t kItemSkip = -2;
int launch_fill_chunk_items(int32_t *item_query, int64_t *range_begin, int64_t *range_end, int64_t nq, int chunks,
                            int64_t per, int64_t n, cudaStream_t stream, const int32_t *only_q = nullptr);

// Exact tier behind a tensor-core tier, for the queries flagged in over_q (one word per query): the k-th
// distance that tier left in out_d / out_i (k_out per query, the k-th at k_last) bounds the true k-th, so one
// pass over the store appends every row at or below it (plus the rounding of two fp32 sums) to the query's
// candidate buffer (cap entries at cand_*[rank * cap], rank = the query's place among the flagged ones, the
// first r_max of them get a buffer).  Work is cut by rows, so one flagged query occupies the whole device, and
// a row is read once for 16 queries (8 when the dimension leaves no room for more).  Scratch: aux (1 + nq ints), rank_of (nq), counts (r_max).
// launch_select_flagged then sorts each buffer and writes the k best of it; left_q[q] = 1 for the flagged
// queries it could not settle (buffer overflowed, no buffer, bound not usable), which the item scan takes;
// the same kernel lays out that scan's items (as launch_fill_chunk_items would, with only_q = left_q).
int scan_flagged_group(int dp);  // queries per group: 16 or 8 by shared memory; 0: the dimension is too large
int launch_scan_flagged(const float *x, const float *xlo, int dp, int d, int64_t n, const float *queries, int q_stride,
                        const int32_t *over_q, int64_t nq, int *aux, int32_t *rank_of, int *counts, int r_max, int cap,
                        int k_out, int k_last, const float *out_d, const int64_t *out_i, const unsigned *x_max_norm2,
                        int metric, float *cand_key, int32_t *cand_idx, int device, cudaStream_t stream, const int *gate,
                        int elem);
int launch_select_flagged(const float *cand_key, const int32_t *cand_idx, const int *counts, const int32_t *rank_of,
                          const int32_t *over_q, int r_max, int cap, int64_t nq, int k, float *out_key, int32_t *out_idx,
                          int32_t *left_q, int32_t *item_query, int64_t *range_begin, int64_t *range_end, int chunks,
                          int64_t per, int64_t n, cudaStream_t stream, const int *gate);

// Builds the (query, list) items of an IVF search from the coarse result:
// probes (nq x nprobe) int32 list numbers (-1 = none); items are grouped by list so
// that warps scanning the same list run together.  Outputs arrays of nq*nprobe items;
// the item of (q, p) is written at slot perm[q*nprobe+p].  `scratch` needs
// (nlist + 1) * 2 ints.
int launch_build_ivf_items(const int32_t *probes, int64_t nq, int nprobe, int64_t nlist, const int64_t *list_off,
                           int32_t *item_query, int64_t *range_begin, int64_t *range_end, int32_t *item_slot,
                           int *scratch, cudaStream_t stream);

// ---- merge.cu ----------------------------------------------------------------------------
// Per query: the k best of `nparts` unsorted lists, sorted best first.
// The list of (query q, part p) starts at part_*[(p * part_stride_p + q_major(q)) * k].
// Layout kinds: 0 = flat list slots (slot = (q / 128) * nparts + p, row q % 128; only the first
//                   min(nparts, lists_started[q / 128]) slots of a query tile are read),
//               1 = item slots (slot_of[q * nparts + p], or q * nparts + p if null).
// A list holds its k entries in the first k of `list_stride` slots.  With `lists_sorted` every
// list is already sorted best first (entries past its end have index -1) and the lists are
// merged pairwise instead of sorted from scratch.  `slot_key_offset[slot * 128-row index]`
// (layout 1 only, may be null) is added to every key of that list as it is read.
int launch_merge_parts(const float *part_key, const int32_t *part_idx, int layout, const int *lists_started,
                       const int32_t *slot_of, int nparts, int64_t nq, int k, int list_stride, float *out_key,
                       int32_t *out_idx, int device, cudaStream_t stream, bool lists_sorted = false,
                       const float *slot_key_offset = nullptr, const int *gate = nullptr, const int32_t *only_q = nullptr,
                       int k_out = 0, float *complete_to = nullptr);

// Grouped list scan: per query, the k best of the lists of its nparts probes (gathered row
// slot_of[q * nparts + p], -1 = none), sorted best first.  A row's list is the first part_cnt[row]
// of list_stride slots at part_*[row * list_stride] (append buffers left unsorted by the scan), or,
// with part_cnt null, list_stride slots of which the empty ones carry index -1.  Entries above the
// query's final threshold qtau[q] (ordered-uint form, key + slot_key_offset[row]) are dropped as
// they are read, so any number of probes can be merged.
constexpr int kAppendBuffer = 512;
// With lists_started given (flat search, see launch_flat_tc): the lists of query q are the first
// min(nparts, lists_started[q / 128]) list slots of its query tile, row q % 128 of each.
int launch_merge_filtered(const float *part_key, const int32_t *part_idx, const int32_t *part_cnt,
                          const int32_t *slot_of, const float *slot_key_offset, const uint32_t *qtau, int nparts,
                          int64_t nq, int k, int list_stride, float *out_key, int32_t *out_idx,
                          cudaStream_t stream, const int *lists_started = nullptr, const int *gate = nullptr);

// Optional input of launch_refine_finalize: the candidates were ranked by tensor-core keys
// (key[q * k_sel + j], ascending) under the slack of key_slack.
//  cut: only the candidates within the slack of the rank-th key can be among the exact `rank` best; the others
//       are not re-evaluated.
//  check_rank > 0: the band check of the pass that selected them - if the LAST candidate of a query lies within
//       the slack of its check_rank-th key, rows that were not kept could belong to the answer: *overflow (0 so
//       far) becomes kScreenOverflow and *overflow_count (optional) counts it once per pass.
struct RefineBand {
    const float *key;
    int rank;
    const float *q_norm2;
    const unsigned *x_max_norm2;
    int d;
    bool one_mma;
    int elem;  // kElemF32, or the 16-bit type of the store (rows and slack, see key_slack)
    bool cut;
    int check_rank;
    int *overflow;
    int *overflow_count;
    int32_t *over_q;          // optional, one word per query: set to 1 for every query whose band check fails
    const int32_t *only_q;    // optional: re-rank (and write results for) the queries with a non-zero word only
    const int32_t *bad_q;     // optional: queries whose keys are meaningless (non-zero word): their check fails
    // optional, per query: the candidates are the best of a UNION of lists and are known to be complete only
    // for keys below this bound (launch_merge_parts, complete_to); the check takes the smaller of it and the
    // last candidate's key
    const float *complete_to;
};

// Flat: recomputes the distance of every selected (query, row) pair in exact fp32
// from the split store, sorts the k results best first and writes the user-facing
// distances (squared L2 / raw dot) and int64 labels (row + label_offset, or
// ids[row] when ids is non-null).  Empty slots -> (+-inf, -1).
// With approx_key (L2 list scan in residual form: approx_key[q * k_sel + j] is the scan's own
// squared distance, rnorm[row] = |x - c|^2, xnorm[row] = |x|^2) a pair is recomputed only if its
// distance is small against the error bound of the scan's dot product; the others keep approx_key.
// With out_row the k_out best ROW NUMBERS (int32, -1 = none) are written there and nothing else.
int launch_refine_finalize(const float *xhi, const float *xlo, int dp, int d, const float *queries, int q_stride,
                           const int32_t *sel_idx, int64_t nq, int k_sel, int k_out, int metric,
                           const int64_t *ids, int64_t label_offset, float *out_d, int64_t *out_i, int device,
                           cudaStream_t stream, const float *approx_key = nullptr, const float *rnorm = nullptr,
                           const float *xnorm = nullptr, int32_t *out_row = nullptr, const int *gate = nullptr,
                           const RefineBand *band = nullptr);

// Already-exact keys: just convert to user-facing values and labels, padding to k_out.
int launch_finalize(const float *sel_key, const int32_t *sel_idx, int64_t nq, int k_sel, int k_out, int metric,
                    const int64_t *ids, int64_t label_offset, float *out_d, int64_t *out_i, cudaStream_t stream);

// Multi-GPU: k best of nparts sorted (distance, label) runs per query.
int launch_merge_results(const float *parts_d, const int64_t *parts_i, int nparts, int64_t nq, int k, int metric,
                         float *out_d, int64_t *out_i, int device, cudaStream_t stream);

// Fills n (distance, label) slots with the "missing" sentinel.
int launch_fill_missing(float *d, int64_t *i, int64_t n, int metric, cudaStream_t stream);

// IVF add: scatter rows into the split store.  dst_row[i] is the destination row (or -1 to drop).
int launch_scatter_rows(const float *x, int64_t n, int d, int dp, const int64_t *dst_row, float *hi, float *lo,
                        float *norms, cudaStream_t stream);

}  // namespace anncuda
