// Paged prefill / chunked-prefill attention on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory) for 16-bit pools, page_size 128,
// head_dim 128 or 64 (the comments speak of 128; with 64 the Q, K and V tiles are one 64-element column block of 16 KiB
// instead of two, Q.K^T has four K = 16 steps instead of eight, and O is 64 columns wide).
//
// Mask.  The reference's prefill mask (falcon_perception/paged_attention.py:343-362,
// falcon_perception/attention.py:75-96) lets query t see key u of the same
// sequence iff u <= t, or t and u lie in the same image span.  An image span
// is a contiguous run of positions that contains t, so the visible set of a
// query is always a PREFIX of its own sequence: [0, extent_t) with
//     extent_t = pos_t + 1                      outside an image span,
//     extent_t = end of t's image span          inside one.
// The host passes extent_t per packed token (0 for pad tokens) and the kernel
// needs nothing else: block sparsity is "key tiles below ceil(max extent/128)",
// the element mask is "key position < extent of the row".
//
// Keys and values are read from the page pool through the page table (the
// sequence's K/V, including the later positions of an image span, must have
// been appended before its queries run), so the same kernel serves a whole
// prompt, a chunk of one, or a step that mixes both.
//
// Work item = one 128-row query tile of a PAIR of query heads that share a stored
// head (a single head when the GQA ratio is odd): the K/V tile staged in shared
// memory feeds both heads, which halves the L2 traffic per FLOP.  A key tile is
// worked through in two halves of 64 keys; per half and head:
//     S = Q K^T    128x64x128,  A = Q (shared, K-major), B = 64 rows of the K tile (shared, K-major) -> TMEM
//     O += P V     128x128x64,  A = P (TMEM, written over the first half of the S columns), B = 64 rows of the V
//                               tile (shared, MN-major) -> TMEM
// Tensor memory holds S/P and O of both heads (4 x 128 columns = all 512).  The
// two halves of a head's score columns are independent buffers: as soon as the
// P.V of one half is issued, the next key tile's Q.K^T over the same 64 keys is
// issued behind it, so the scores of a half are ready again by the time the
// softmax threads have dealt with the other half.  Four chains  S -> softmax ->
// P.V -> next S  are in flight per SM (two heads x two halves).
//   * The CTAs are persistent: one per SM, each walking its share of the items
//     (longest first, dealt out boustrophedon).  Every barrier carries its phase
//     across items, so the copies and the first Q.K^T of the next item run while
//     the softmax warps still write the previous item's output.
//   * Warps 0-3 are the softmax group of head 0, warps 4-7 of head 1: one thread
//     per query row, 64 scores per step (load, row maximum, exponentials, packed
//     P store, hand-over).  The groups run independently, so that one group's
//     loads and barrier traffic overlap the other group's exponentials.
//   * Warp 8 is the TMA producer (2-stage K and V rings running across items).
//   * Warps 9 and 10 issue the MMAs, one warp per head: the tensor pipe takes the
//     MMAs of a thread one after the other and idles through whatever else that
//     thread does, so each head gets its own issuer.
//   * Warp 11 prepares the next item while the current one runs: slot, visible
//     extent of every row, page ids of all key tiles (two descriptor buffers).
//   * An item of a SINGLE head (odd GQA ratio, a pool with one stored head per query head, a split pool) runs the
//     same machinery with the pair's two sides taken by the even and the odd key tiles of the one head: softmax
//     group g and MMA issuer g work through tiles g, g + 2, ..., each side with its own score columns, reference
//     maximum, row sum and O accumulator, and the two partial results are merged in the epilogue (each group
//     writes half of the output columns).
// The running maximum is only raised when a half exceeds it by more than 2^8
// (probabilities stay below 256, exact in fp32 and harmless in bf16), so O in
// TMEM is rarely rescaled.  Each thread owns a whole output row; 32 columns of
// a warp's 32 rows at a time are staged in shared memory (64-byte swizzle) and
// leave as one bulk tensor store.
// Every wait is a bounded mbarrier wait; on expiry the CTA raises
// FPKV_STATUS_TIMEOUT, every role leaves its loops, the copies and MMAs in
// flight are drained (bounded), TMEM is freed and the kernel returns.

#include <cuda.h>
#include <string.h>
#include <type_traits>
#include "common.cuh"

namespace fpkv {
namespace {

constexpr int kTileM = 128, kTileN = 128, kPage = 128;
constexpr int kTileBytes = 128 * 128 * 2;              // a 128 x 128 16-bit tile: the size of every tile buffer (head_dim 64 fills half)
constexpr int kHalfBytes = kTileBytes / 2;             // 64 columns (128 bytes) x 128 rows
constexpr int kStages = 2;                             // K ring, and V ring of head-pair items
constexpr int kStagesVMax = 3;                         // V ring of single-head items: the unused second query buffer is its third stage
constexpr int kSoftmaxWarps = 4;                       // per head: warps 0-3 are head 0's softmax group, warps 4-7 head 1's
constexpr int kLoadWarp = 8, kMmaWarp = 9;              // warps 9 and 10 issue the MMAs of head 0 and head 1 of the pair
constexpr int kScoutWarp = 11;                         // prepares the next item's descriptor
constexpr int kPrefillThreads = 12 * 32;
constexpr int kMaxKeyTiles = 512;                      // 65 536 keys per sequence
constexpr uint32_t kSpin = 1u << 22;
constexpr uint32_t kTmemCols = 512;                    // S/P head 0, S/P head 1, O head 0, O head 1: 128 columns each
constexpr float kRescaleThreshold = 8.f;

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t bar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kSpin; ++i) {
        if (bar_try(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void tma_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}

// ---- tcgen05 --------------------------------------------------------------
// Shared-memory operand descriptor, 128-byte swizzle, version 1 (sm_100).
//   K-major tile  (rows of 128 bytes = 64 elements of the contraction dim):
//       SBO = 1024 (8 rows), LBO unused.
//   MN-major tile (rows of 128 bytes = 64 elements of the M/N dim, one row per contraction index):
//       SBO = 1024 (8 contraction indices), LBO = distance between 64-element column groups.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;                            // descriptor version
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}
// Instruction descriptor for kind::f16: D = f32, A/B = bf16 or f16, M = 128, N = 128.
__device__ __forceinline__ uint32_t umma_idesc(bool bf16, bool b_mn_major, int n = kTileN) {
    uint32_t d = 0;
    d |= 1u << 4;                                      // accumulator format f32
    d |= (bf16 ? 1u : 0u) << 7;                        // A format
    d |= (bf16 ? 1u : 0u) << 10;                       // B format
    d |= (b_mn_major ? 1u : 0u) << 16;                 // B major: 0 = K, 1 = MN
    d |= (uint32_t)(n >> 3) << 17;
    d |= (uint32_t)(kTileM >> 4) << 24;
    return d;
}
// The issuing thread shares its scheduler with softmax warps, so the issue loop is kept to a few
// instructions per MMA: the descriptors' high words are constants, the low words (start address >> 4)
// advance by a compile-time step.
__device__ __forceinline__ void umma(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                     uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
                 "setp.ne.b32 p, %6, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
                 ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate));
}
// A operand from tensor memory (128 lanes x 8 columns of packed 16-bit pairs per K = 16 step), B from shared memory.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tmov.b64 db, {%2, %3};\n\tsetp.ne.b32 p, %5, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate));
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 32 lanes x 32 columns of 32-bit: thread t of the warp gets lane (warp%4)*32 + t, columns [col, col+32)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32_nowait(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float max3f(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    uint32_t w;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(b), "f"(a));      // first source lands in the upper half
    return w;
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    uint32_t w;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(b), "f"(a));
    return w;
}
// Two output values rounded to the storage type (and, with the sink gate on, multiplied by the gate and rounded
// again, the reference's two-step value), as one packed word.  Conversions go through a unit as narrow as the
// exponential unit, so they are done two at a time.
template <typename T> __device__ __forceinline__ uint32_t gated_pair(float a, float b, float gate, bool on);
template <> __device__ __forceinline__ uint32_t gated_pair<__nv_bfloat16>(float a, float b, float gate, bool on) {
    uint32_t w = pack2<__nv_bfloat16>(a, b);
    if (on) w = pack2<__nv_bfloat16>(__uint_as_float(w << 16) * gate, __uint_as_float(w & 0xffff0000u) * gate);
    return w;
}
template <> __device__ __forceinline__ uint32_t gated_pair<__half>(float a, float b, float gate, bool on) {
    uint32_t w = pack2<__half>(a, b);
    if (on) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
        w = pack2<__half>(f.x * gate, f.y * gate);
    }
    return w;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed fp32 pairs: one instruction scales two scores or adds two probabilities into the row sums.
struct F2 { float x, y; };
__device__ __forceinline__ F2 fma2(F2 a, F2 b, F2 c) {
    F2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ F2 add2(F2 a, F2 b) {
    F2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}


// O += P V over one half of a key tile (64 keys, four K = 16 steps): P from tensor memory (8 packed columns per 16
// keys, starting at `a`), V rows from shared memory (MN-major, 16 rows = 2 KiB per step, starting at row 64 * kHalf).
// `acc_first` is the accumulate flag of the first MMA.
template <int kHalf>
__device__ __forceinline__ void issue_pv_half(uint32_t d, uint32_t a, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t acc_first) {
#pragma unroll
    for (int k = 0; k < 4; ++k)
        umma_ts(d, a + k * 8, b_lo + (kHalf * 4 + k) * ((16 * 128) >> 4), hi, idesc, k > 0 ? 1u : acc_first);
}
// S half = Q K^T over 64 keys (N = 64): the K tile's rows [64 * kHalf, +64), i.e. 8 KiB into each 64-element column block.
template <int kHalf, int D>
__device__ __forceinline__ void issue_qk_half(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t bar) {
#pragma unroll
    for (int k = 0; k < D / 16; ++k) {
        const uint32_t off = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
        umma(d, a_lo + off, hi, b_lo + off + ((kHalf * 64 * 128) >> 4), hi, idesc, k > 0);
    }
    umma_commit(bar);
}

struct PrefillParams {
    const int64_t* page_table;
    const int64_t* p2l;
    const int64_t* batch_idx;   // [L] slot of each packed token (0 = pad)
    const int32_t* extent;      // [L] number of visible keys of each packed token
    void* out;                  // (Hq, L, D) contiguous, or (L, Hq, D) when token-major
    float* lse;                 // (Hq, L)
    int32_t* status;
    int L, Hq, Hkv, n_pages, max_batch;
    int rows_per_plane;         // n_pages * page_size
    float scale_log2;
    int heads_per_item;         // 2: both query heads of a GQA pair share the staged K/V tiles; 1 otherwise
    int split;                  // split pool layout: kv_map covers the first K halves, khw_map the second halves (per query
                                // head), v_map the values; an item is then a single query head (its K tile is its own)
    int n_qtiles, n_pairs, n_items;
    Epilogue epi;
};

// What every role needs to know about a work item, prepared one item ahead by the scout warp.
struct ItemDesc {
    int valid;                  // 0: no more work for this CTA
    int t0;                     // first packed token of the query tile
    int hq0;                    // first query head of the item
    int n_tiles;                // key tiles any row of the tile sees
    int max_extent;             // largest visible-prefix length among the rows
    int first_bad;              // first key tile whose page is unmapped (n_tiles when all are mapped)
    int pad_[2];
    int extent[kTileM];         // visible keys of each row (0: pad, or a row the tile may not hold)
    int page_row[kMaxKeyTiles]; // pool row of the K tile of key tile j (reserved page 0 when unmapped)
    unsigned char page_ok[kMaxKeyTiles];
};

// 64 scores (two 32-column pieces) -> 32 packed probability words, row sum into rs.  valid_cols: how many of the 64
// columns exist for this row (all of them on the fast path).
template <typename T, bool kFull>
__device__ __forceinline__ void probabilities64(const uint32_t (&sv)[2][32], uint32_t (&pk)[32], F2 (&rs)[2], float scale_log2,
                                                float neg_m, int valid_cols) {
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2) {
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
            // scale and reference maximum for both scores of the pair in one packed FMA
            const F2 x = fma2(F2{__uint_as_float(sv[c2][c]), __uint_as_float(sv[c2][c + 1])}, F2{scale_log2, scale_log2},
                              F2{neg_m, neg_m});
            F2 p;
            p.x = ex2(x.x); p.y = ex2(x.y);
            if (!kFull) {
                if (c2 * 32 + c >= valid_cols) p.x = 0.f;
                if (c2 * 32 + c + 1 >= valid_cols) p.y = 0.f;
            }
            rs[(c >> 1) & 1] = add2(rs[(c >> 1) & 1], p);                      // packed row sums, two accumulators
            pk[c2 * 16 + c / 2] = pack2<T>(p.x, p.y);
        }
    }
}
template <bool kFull>
__device__ __forceinline__ float max64(const uint32_t (&sv)[2][32], int valid_cols) {
    if (kFull) {
        float m2[2];
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
            m2[c2] = max3f(__uint_as_float(sv[c2][0]), __uint_as_float(sv[c2][1]), __uint_as_float(sv[c2][2]));
#pragma unroll
            for (int c = 3; c + 1 < 32; c += 2) m2[c2] = max3f(m2[c2], __uint_as_float(sv[c2][c]), __uint_as_float(sv[c2][c + 1]));
            m2[c2] = fmaxf(m2[c2], __uint_as_float(sv[c2][31]));
        }
        return fmaxf(m2[0], m2[1]);
    }
    float mx = -INFINITY;
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2)
#pragma unroll
        for (int c = 0; c < 32; ++c) if (c2 * 32 + c < valid_cols) mx = fmaxf(mx, __uint_as_float(sv[c2][c]));
    return mx;
}

template <typename T, int D, bool kSolo>
__global__ void __launch_bounds__(kPrefillThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                  const __grid_constant__ CUtensorMap khw_map, const __grid_constant__ CUtensorMap v_map,
                  const __grid_constant__ CUtensorMap o_map, const PrefillParams prm)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem;                                   // 2 x 32 KiB: the query tile of each head of the pair
    uint8_t* k_s = q_s + 2 * kTileBytes;                   // kStages x 32 KiB
    uint8_t* v_s = k_s + kStages * kTileBytes;             // kStages x 32 KiB
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + kStages * kTileBytes);
    int* ints = reinterpret_cast<int*>(bars + 48);
    volatile int* abort_flag = ints;                       // [0] abort, [1] TMEM base
    int* tmem_slot = ints + 1;
    ItemDesc* desc = reinterpret_cast<ItemDesc*>(ints + 16);   // [2]
    float* xch = reinterpret_cast<float*>(desc + 2);       // [2][2 groups][128 rows][m, l]: merge of single-head items
    uint8_t* ostage = reinterpret_cast<uint8_t*>(xch + 2 * 2 * kTileM * 2);   // [8 softmax warps][32 rows][64 bytes]: output transposition
    static_assert((48 * 8 + 16 * 4 + 2 * sizeof(ItemDesc) + 2 * 2 * kTileM * 8) % 512 == 0,
                  "the output staging buffers must start on a 512-byte boundary (64-byte swizzle pattern of the bulk stores)");

    // mbarriers; every one keeps its phase across items
    const uint32_t desc_full0 = s32(bars + 0), desc_empty0 = s32(bars + 2);            // [2] descriptor buffers
    const uint32_t q_full0 = s32(bars + 4), q_empty0 = s32(bars + 6);                  // [2] per head
    const uint32_t k_full0 = s32(bars + 8), v_full0 = s32(bars + 8 + kStages);
    const uint32_t k_empty0 = s32(bars + 8 + kStages + kStagesVMax), v_empty0 = s32(bars + 8 + 2 * kStages + kStagesVMax);
    const uint32_t s_half0 = s32(bars + 8 + 2 * kStages + 2 * kStagesVMax);           // [head][half] scores of 64 keys are in TMEM
    const uint32_t p_half0 = s_half0 + 32;                                             // [head][half] P of 64 keys written
    const uint32_t pv_done0 = s_half0 + 64;                                            // [2] a half's P.V has completed (one phase per half)
    const uint32_t all_done0 = s_half0 + 80, o_free0 = s_half0 + 96;                   // [2] last P.V complete / O read by the epilogue
    const uint32_t drain0 = s_half0 + 112;                                             // [2] give-up path: a head's MMAs have completed
    const uint32_t merge0 = s_half0 + 128;                                             // single-head items: both groups have published (m, l)

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    constexpr int kTileBytesD = kTileM * D * 2;            // bytes a Q, K or V tile really holds
    constexpr bool solo = kSolo;                           // single-head items: the two sides take the even and the odd key tiles
    // Single-head items consume two key tiles at once (one per side), so a two-stage ring leaves no room to fetch
    // ahead.  K is needed late (see the issuer), V is not: its ring gets the second query buffer, which such items
    // do not use, as a third stage.
    constexpr int kStagesV = kSolo ? kStagesVMax : kStages;
    auto v_stage = [&](uint32_t st) -> uint8_t* { return (kSolo && st == 2) ? q_s + kTileBytes : v_s + st * kTileBytes; };
    constexpr int heads = kSolo ? 1 : 2;                   // query heads of one stored head in an item
    const int n_rep = prm.Hq / prm.Hkv;

    // ---- set-up, once per CTA ------------------------------------------------
    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            bar_init(desc_full0 + 8 * b, 1); bar_init(desc_empty0 + 8 * b, 3 + 2 * kSoftmaxWarps);
            bar_init(q_full0 + 8 * b, 1); bar_init(q_empty0 + 8 * b, solo ? 2 : 1);      // single head: both issuers read the one query tile
            for (int hf = 0; hf < 2; ++hf) { bar_init(s_half0 + 16 * b + 8 * hf, 1); bar_init(p_half0 + 16 * b + 8 * hf, kSoftmaxWarps); }
            bar_init(pv_done0 + 8 * b, 1); bar_init(all_done0 + 8 * b, 1);
            bar_init(o_free0 + 8 * b, solo ? 2 * kSoftmaxWarps : kSoftmaxWarps);
            bar_init(drain0 + 8 * b, 1);
        }
        bar_init(merge0, 2 * kSoftmaxWarps);
        for (int s = 0; s < kStages; ++s) { bar_init(k_full0 + 8 * s, 1); bar_init(k_empty0 + 8 * s, heads); }   // one commit per MMA warp that reads the tile
        for (int s = 0; s < kStagesV; ++s) { bar_init(v_full0 + 8 * s, 1); bar_init(v_empty0 + 8 * s, heads); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {                                // TMEM allocation is a whole-warp operation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = (uint32_t)*tmem_slot;
    // tensor memory: S/P of head 0 [0,128), S/P of head 1 [128,256), O of head 0 [256,384), O of head 1 [384,512);
    // within a head's 128 columns the scores of keys 0-63 take [0,64), those of keys 64-127 [64,128); the packed P of a
    // half (32 columns) goes over the first half of its own score columns
    bool alive = true;
    // copies requested so far by the producer thread (for the give-up path)
    uint32_t k_requested = 0, v_requested = 0, q_requested[2] = {0, 0};

    if (warp == kScoutWarp) {
        // ============================== scout ===================================
        // Items are numbered longest first (query tiles from the end of the packed row backwards: under a causal
        // mask the later tiles see more keys; all head pairs of a tile before the next tile) and dealt to the CTAs
        // in rounds, forwards and backwards alternately, so that every CTA gets a similar mix.
        const int G = gridDim.x, rounds = (prm.n_items + G - 1) / G;
        uint32_t it = 0;
        for (int k = 0; k <= rounds && alive; ++k) {
            int idx = -1;
            if (k < rounds) {
                idx = k * G + ((k & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x);
                if (idx >= prm.n_items) continue;
            }
            const uint32_t b = it & 1u;
            if (lane == 0) alive = bar_wait(desc_empty0 + 8 * b, ((it >> 1) & 1u) ^ 1u, abort_flag);
            alive = __shfl_sync(0xffffffffu, alive, 0);
            if (!alive) break;
            ItemDesc* d = desc + b;
            if (idx < 0) {
                if (lane == 0) d->valid = 0;
            } else {
                const int y = idx / prm.n_pairs, x = idx - y * prm.n_pairs;
                const int t0 = (prm.n_qtiles - 1 - y) * kTileM, hq0 = x * heads, hkv = hq0 / n_rep;
                int sl[4], ex[4], smax = 0;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int tk = t0 + lane + 32 * r;
                    long long s = 0; int e = 0;
                    if (tk < prm.L) { s = prm.batch_idx[tk]; e = prm.extent[tk]; }     // both loads in flight together
                    if (s < 0 || s >= prm.max_batch) { raise_status(prm.status, FPKV_STATUS_BAD_SLOT); s = 0; }
                    sl[r] = (int)s; ex[r] = (s > 0 && e > 0) ? e : 0;
                    smax = max(smax, sl[r]);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) smax = max(smax, __shfl_xor_sync(0xffffffffu, smax, o));   // pads are slot 0
                int emax = 0;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    if (sl[r] != 0 && sl[r] != smax) { raise_status(prm.status, FPKV_STATUS_BAD_SLOT); ex[r] = 0; }   // two live sequences in one tile
                    if ((long long)ex[r] > (long long)prm.n_pages * kPage) { raise_status(prm.status, FPKV_STATUS_BAD_POS); ex[r] = 0; }
                    if (ex[r] > kMaxKeyTiles * kTileN) { raise_status(prm.status, FPKV_STATUS_BAD_POS); ex[r] = kMaxKeyTiles * kTileN; }
                    d->extent[lane + 32 * r] = ex[r];
                    emax = max(emax, ex[r]);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) emax = max(emax, __shfl_xor_sync(0xffffffffu, emax, o));
                const int n_tiles = (emax + kTileN - 1) / kTileN;
                // page ids of all key tiles, resolved once (coalesced) instead of one dependent load per tile
                const long long trow = (long long)smax * prm.n_pages;
                int first_bad = n_tiles;
                for (int j = lane; j < n_tiles; j += 32) {
                    const long long pg = prm.page_table[trow + j];
                    bool ok = pg >= 0 && pg < prm.n_pages;
                    if (pg >= prm.n_pages) raise_status(prm.status, FPKV_STATUS_BAD_PAGE);
                    if (ok) ok = prm.p2l[trow + pg] >= 0;
                    d->page_row[j] = hkv * prm.rows_per_plane + (ok ? (int)pg : 0) * kPage;   // unmapped: reserved page 0, masked
                    d->page_ok[j] = ok;
                    if (!ok) first_bad = min(first_bad, j);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) first_bad = min(first_bad, __shfl_xor_sync(0xffffffffu, first_bad, o));
                if (lane == 0) { d->valid = 1; d->t0 = t0; d->hq0 = hq0; d->n_tiles = n_tiles; d->max_extent = emax; d->first_bad = first_bad; }
            }
            __syncwarp();
            if (lane == 0) bar_arrive(desc_full0 + 8 * b);
            ++it;
        }
    } else if (warp == kLoadWarp) {
        // ============================== TMA producer ========================
        if (lane == 0) {
            uint32_t gk = 0, wit = 0;                      // key tiles requested, items with work so far
            for (uint32_t it = 0; alive; ++it) {
                const uint32_t b = it & 1u;
                if (!bar_wait(desc_full0 + 8 * b, (it >> 1) & 1u, abort_flag)) { alive = false; break; }
                const ItemDesc* d = desc + b;
                if (!d->valid) break;
                const int n = d->n_tiles;
                if (n > 0) {
                    for (int h = 0; h < heads && alive; ++h) {           // the head's query buffer is free once its last Q.K^T is through
                        if (!bar_wait(q_empty0 + 8 * h, (wit & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                        bar_expect_tx(q_full0 + 8 * h, kTileBytesD);
                        tma_4d(s32(q_s + h * kTileBytes), &q_map, 0, d->t0, 0, d->hq0 + h, q_full0 + 8 * h);
                        q_requested[h] = wit + 1;
                    }
                    // The K ring and the V ring advance independently: a K stage frees up when the tile's Q.K^T is
                    // through, long before its V stage does (P.V comes a softmax later), so whichever ring has room
                    // gets its next copy; waiting for them strictly in turn would hold K copies back behind V.
                    int jk = 0, jv = 0;
                    uint32_t idle = 0;
                    while ((jk < n || jv < n) && alive) {
                        bool progress = false;
                        if (jk < n) {
                            const uint32_t g = gk + jk, st = g % kStages;
                            if (bar_try(k_empty0 + 8 * st, ((g / kStages) & 1u) ^ 1u)) {
                                bar_expect_tx(k_full0 + 8 * st, kTileBytesD);
                                if (!prm.split) {
                                    tma_3d(s32(k_s + st * kTileBytes), &kv_map, 0, d->page_row[jk], 0, k_full0 + 8 * st);
                                } else {                   // shared first half and this query head's second half, side by side
                                    tma_3d(s32(k_s + st * kTileBytes), &kv_map, 0, d->page_row[jk], 0, k_full0 + 8 * st);
                                    tma_3d(s32(k_s + st * kTileBytes + kHalfBytes), &khw_map, 0,
                                           d->page_row[jk] + (d->hq0 - d->hq0 / n_rep) * prm.rows_per_plane, 0, k_full0 + 8 * st);
                                }
                                k_requested = g + 1; ++jk; progress = true;
                            }
                        }
                        if (jv < n) {
                            const uint32_t g = gk + jv, st = g % kStagesV;
                            if (bar_try(v_empty0 + 8 * st, ((g / kStagesV) & 1u) ^ 1u)) {
                                bar_expect_tx(v_full0 + 8 * st, kTileBytesD);
                                if (!prm.split) tma_3d(s32(v_stage(st)), &kv_map, 0, d->page_row[jv] + prm.Hkv * prm.rows_per_plane, 0, v_full0 + 8 * st);
                                else tma_3d(s32(v_stage(st)), &v_map, 0, d->page_row[jv], 0, v_full0 + 8 * st);
                                v_requested = g + 1; ++jv; progress = true;
                            }
                        }
                        if (progress) idle = 0;
                        else if (++idle > kSpin || ((idle & 255u) == 255u && *abort_flag)) alive = false;
                    }
                    gk += n;
                    ++wit;
                }
                if (alive) bar_arrive(desc_empty0 + 8 * b);
            }
        }
    } else if (warp >= kMmaWarp && warp < kMmaWarp + 2) {
        // ============================== MMA issuers =========================
        // Two issuing warps.  The tensor pipe takes the MMAs of one thread strictly one after the other, and
        // whatever else that thread does (barrier waits, commits) is time the pipe idles for it; with two issuers
        // the other one's MMAs fill those gaps, and each side's chain  S -> softmax -> P.V -> next S  advances on its
        // own.  With a head pair, issuer g has head g and both read the one staged K / V tile; with a single head,
        // issuer g has the key tiles g, g + 2, ... of that head.
        const int g = warp - kMmaWarp;
        if (lane == 0) {
            const bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
            const uint32_t idesc_qk = umma_idesc(is_bf16, false, 64);
            const uint32_t idesc_pv = umma_idesc(is_bf16, true, D);
            // descriptor words: low = start address >> 4 (| LBO for MN-major), high = SBO 1024 | version | 128-byte swizzle
            const uint32_t desc_hi = (uint32_t)(umma_desc(0, 0, 1024) >> 32);
            const int qb = solo ? 0 : g;                   // query buffer (and its barriers) this issuer reads
            constexpr int step = solo ? 2 : 1;             // distance between this issuer's key tiles
            const int j0 = solo ? g : 0;                   // its first key tile of an item
            const uint32_t q_lo = ((s32(q_s) & 0x3FFFF) >> 4) + qb * (kTileBytes >> 4), k_lo = (s32(k_s) & 0x3FFFF) >> 4;
            // V stage descriptors (MN-major: LBO = distance between the 64-column groups); the third stage of single-head items lies apart
            const uint32_t v_lo0 = ((s32(v_s) & 0x3FFFF) >> 4) | (uint32_t)umma_desc(0, kHalfBytes, 1024);
            const uint32_t v_lo2 = ((s32(q_s + kTileBytes) & 0x3FFFF) >> 4) | (uint32_t)umma_desc(0, kHalfBytes, 1024);
            const uint32_t t_s = tmem + g * kTileN, t_o = tmem + 256 + g * kTileN;
            const uint32_t s_lo = s_half0 + 16 * g, s_hi = s_lo + 8, p_lo = p_half0 + 16 * g, p_hi = p_lo + 8;
            const uint32_t pv_done = pv_done0 + 8 * g;
            uint32_t gk = 0, th = 0, wit = 0, wg = 0;      // key tiles of all items, this issuer's tiles, items with work, items with work for this issuer
            for (uint32_t it = 0; alive; ++it) {
                const uint32_t b = it & 1u;
                if (!bar_wait(desc_full0 + 8 * b, (it >> 1) & 1u, abort_flag)) { alive = false; break; }
                const ItemDesc* d = desc + b;
                if (!d->valid) break;
                const int n = d->n_tiles;
                if (n > j0) {
                    const uint32_t c0 = gk + j0, st0 = c0 % kStages;
                    alive = bar_wait(q_full0 + 8 * qb, wit & 1u, abort_flag) &&
                            bar_wait(k_full0 + 8 * st0, (c0 / kStages) & 1u, abort_flag);
                    if (!alive) break;
                    tc_fence_after();
                    issue_qk_half<0, D>(t_s, q_lo, k_lo + st0 * (kTileBytes >> 4), desc_hi, idesc_qk, s_lo);
                    issue_qk_half<1, D>(t_s + 64, q_lo, k_lo + st0 * (kTileBytes >> 4), desc_hi, idesc_qk, s_hi);
                    umma_commit(k_empty0 + 8 * st0);
                    if (j0 + step >= n) umma_commit(q_empty0 + 8 * qb);    // that was this issuer's only Q.K^T of the item
                    for (int j = j0; j < n; j += step) {
                        const uint32_t cur = gk + j, nxt = cur + step;
                        const uint32_t sv = cur % kStagesV, sn = nxt % kStages;
                        const bool more = j + step < n;
                        // the operand tiles first: they arrived long ago, and waiting for them here costs nothing
                        // while the softmax group is still busy.  (Single head: the next K tile of this side goes into
                        // the stage its present tile has just left, so it is waited for only where it is needed.)
                        if (!bar_wait(v_full0 + 8 * sv, (cur / kStagesV) & 1u, abort_flag)) { alive = false; break; }
                        if (!solo && more && !bar_wait(k_full0 + 8 * sn, (nxt / kStages) & 1u, abort_flag)) { alive = false; break; }
                        // O of the previous item must have been read by its epilogue before the first P.V overwrites it
                        if (j == j0 && !bar_wait(o_free0 + 8 * g, (wg & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                        // keys 0-63: P.V, then at once the next tile's scores of the same half (its columns are free again)
                        if (!bar_wait(p_lo, th & 1u, abort_flag)) { alive = false; break; }
                        tc_fence_after();
                        const uint32_t v_lo = (solo && sv == 2) ? v_lo2 : v_lo0 + sv * (kTileBytes >> 4);
                        issue_pv_half<0>(t_o, t_s, v_lo, desc_hi, idesc_pv, j > j0);
                        umma_commit(pv_done);
                        if (solo && more && !bar_wait(k_full0 + 8 * sn, (nxt / kStages) & 1u, abort_flag)) { alive = false; break; }
                        if (more) issue_qk_half<0, D>(t_s, q_lo, k_lo + sn * (kTileBytes >> 4), desc_hi, idesc_qk, s_lo);
                        // keys 64-127
                        if (!bar_wait(p_hi, th & 1u, abort_flag)) { alive = false; break; }
                        tc_fence_after();
                        issue_pv_half<1>(t_o, t_s + 64, v_lo, desc_hi, idesc_pv, 1u);
                        umma_commit(pv_done);
                        umma_commit(v_empty0 + 8 * sv);
                        ++th;
                        if (more) {
                            issue_qk_half<1, D>(t_s + 64, q_lo, k_lo + sn * (kTileBytes >> 4), desc_hi, idesc_qk, s_hi);
                            umma_commit(k_empty0 + 8 * sn);
                            if (j + 2 * step >= n) umma_commit(q_empty0 + 8 * qb);     // that was this issuer's last Q.K^T of the item
                        }
                    }
                    if (!alive) break;
                    umma_commit(all_done0 + 8 * g);
                    ++wg;
                } else if (n > 0) {
                    bar_arrive(q_empty0 + 8 * qb);         // single head, one key tile: nothing for this issuer, only its share of the hand-back
                }
                if (n > 0) { gk += n; ++wit; }
                bar_arrive(desc_empty0 + 8 * b);
            }
            if (!alive) {
                // Gave up: tensor memory is freed and the CTA's shared memory handed on after the last barrier
                // below, so wait (bounded, ignoring the abort flag) for the MMAs already in the pipe.
                umma_commit(drain0 + 8 * g);
                for (uint32_t k = 0; k < kSpin && !bar_try(drain0 + 8 * g, 0); ++k) {}
            }
        }
    } else if (warp < 2 * kSoftmaxWarps && (warp < kSoftmaxWarps || heads == 2 || solo)) {
        // ============================== softmax groups ======================
        // Group g (warps 4g .. 4g+3): one thread per query row, warp w reaches tensor-memory lanes [32 (w % 4), +32).
        // With a head pair, group g owns head g.  With a single head, group g owns the key tiles g, g + 2, ... of
        // that head, with its own score columns, reference maximum, row sum and accumulator (those of group 1 live
        // in the columns the second head would use).  The groups do not synchronise with each other inside an
        // item: while one exponentiates, the other one's score loads, maximum, P store and barrier traffic -- and
        // the MMAs -- run underneath.
        const int grp = warp / kSoftmaxWarps, quarter = warp % kSoftmaxWarps;
        const int h = solo ? 0 : grp;                                  // head of the item this group works on
        constexpr int step = solo ? 2 : 1;                             // distance between this group's key tiles
        const int j0 = solo ? grp : 0;                                 // its first key tile of an item
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t ts = tmem + grp * kTileN + lane_base;          // this group's scores: keys 0-63 in columns [0,64), keys 64-127 in [64,128)
        const uint32_t to = tmem + 256 + grp * kTileN + lane_base;    // this group's accumulator
        const uint32_t pv_done = pv_done0 + 8 * grp;
        uint32_t gk = 0, th = 0, wit = 0, wg = 0;          // key tiles of all items, this group's tiles, items with work, items with work for this group
        for (uint32_t it = 0; alive; ++it) {
            const uint32_t b = it & 1u;
            if (!bar_wait(desc_full0 + 8 * b, (it >> 1) & 1u, abort_flag)) { alive = false; break; }
            const ItemDesc* d = desc + b;
            if (!d->valid) break;
            const int n = d->n_tiles, max_extent = d->max_extent, my_extent = d->extent[row];
            const int tk = d->t0 + row, hq = d->hq0 + h;
            float m_ref = -INFINITY, l = 0.f;
            uint32_t sv[2][32], pk[32];
            // per-item constants of the tile loop: tiles below `wfull` are fully visible to every row of this warp
            const int first_bad = d->first_bad;
            int wfull = my_extent / kTileN;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) wfull = min(wfull, __shfl_xor_sync(0xffffffffu, wfull, o));
            wfull = min(wfull, first_bad);
            const int zero_from = min(first_bad, (max_extent % kTileN) ? n - 1 : n);   // first tile with value rows to clear
            for (int j = j0; j < n && alive; j += step) {
                const bool page_ok = j < first_bad || d->page_ok[j];
                // Value rows past the last key any row of this tile sees (the tail of the last key tile, or all of
                // an unmapped page's stand-in) were fetched but possibly never appended: the pool may hold anything
                // there, and 0 x NaN would poison O.  Clear them in shared memory before this group's first P.V of
                // the tile (every group that reads the tile does, each ahead of its own hand-over; the tensor cores
                // read shared memory through the async proxy, hence the proxy fence).
                if (j >= zero_from) {
                    const int tile_rows = page_ok ? min(kTileN, max_extent - j * kTileN) : 0;
                    const uint32_t cur = gk + j, st = cur % kStagesV;
                    if (!bar_wait(v_full0 + 8 * st, (cur / kStagesV) & 1u, abort_flag)) { alive = false; break; }
                    for (int i = row; i < (kTileN - tile_rows) * (D / 8); i += kSoftmaxWarps * 32) {
                        const int r = tile_rows + i / (D / 8), c = i % (D / 8);  // token row, 16-byte piece of its D * 2 bytes
                        *reinterpret_cast<uint4*>(v_stage(st) + (c >> 3) * kHalfBytes + r * 128 + ((c & 7) << 4)) =
                            make_uint4(0u, 0u, 0u, 0u);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                const bool full = j < wfull;
                const int valid_row = full ? kTileN : (page_ok ? min(kTileN, my_extent - j * kTileN) : 0);   // visible keys of this row in the tile
                // The tile is worked through in two halves of 64 keys.  Each half has its own score columns, and the
                // MMA warp refills a half (next tile's Q.K^T over the same 64 keys) as soon as that half's P.V is
                // issued: the scores of the next half are there when this group comes back for them.
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const uint32_t unit = 2 * th + hf;                          // halves this group has gone through so far
                    const int valid_cols = valid_row - 64 * hf;
                    if (!bar_wait(s_half0 + 16 * grp + 8 * hf, th & 1u, abort_flag)) { alive = false; break; }
                    tc_fence_after();
                    tmem_ld32_nowait(ts + 64 * hf, sv[0]);
                    tmem_ld32_nowait(ts + 64 * hf + 32, sv[1]);
                    tmem_wait_ld();
                    // The reference maximum is raised lazily: only when a score lies more than 2^8 above it (the
                    // probabilities stay below 256, exact in fp32 and harmless in 16 bits), so that O in tensor memory
                    // is rarely rescaled.  O is stable only once every P.V issued so far has completed.
                    const float mx = (full ? max64<true>(sv, 64) : max64<false>(sv, valid_cols)) * prm.scale_log2;   // scale > 0: max commutes with it
                    const bool raise = mx > m_ref + kRescaleThreshold || (m_ref == -INFINITY && mx > -INFINITY);
                    if (__any_sync(0xffffffffu, raise)) {  // tensor-memory access is a whole-warp operation
                        const float m_new = raise ? mx : m_ref;
                        const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
                        if (j > j0 || hf > 0) {            // rescale this row of O in tensor memory (nothing is in it before the group's first P.V)
                            if (!bar_wait(pv_done, (unit - 1) & 1u, abort_flag)) { alive = false; break; }
                            tc_fence_after();
#pragma unroll 1
                            for (int c4 = 0; c4 < D / 32; ++c4) {
                                tmem_ld32(to + c4 * 32, pk);
#pragma unroll
                                for (int c = 0; c < 32; ++c) pk[c] = __float_as_uint(__uint_as_float(pk[c]) * alpha);
                                tmem_st32(to + c4 * 32, pk);
                            }
                        }
                        l *= alpha;
                        m_ref = m_new;
                    }
                    const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
                    F2 rs[2] = {F2{0.f, 0.f}, F2{0.f, 0.f}};
                    if (full) probabilities64<T, true>(sv, pk, rs, prm.scale_log2, neg_m, 64);
                    else probabilities64<T, false>(sv, pk, rs, prm.scale_log2, neg_m, valid_cols);
                    tmem_st32_nowait(ts + 64 * hf, pk);    // P of these 64 keys over the first half of their own score columns
                    l += (rs[0].x + rs[0].y) + (rs[1].x + rs[1].y);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) bar_arrive(p_half0 + 16 * grp + 8 * hf);
                }
                ++th;
            }
            if (!alive) break;
            gk += n;
            // ---- epilogue: O / l -> out, lse; every thread owns one row of 256 contiguous bytes ----
            const bool own_tiles = n > j0;                 // this group's accumulator holds something
            const bool oth_tiles = solo && n > (j0 ^ 1);   // single head: so does the other group's
            if (own_tiles) {
                if (!bar_wait(all_done0 + 8 * grp, wg & 1u, abort_flag)) { alive = false; break; }
                tc_fence_after();
                ++wg;
            }
            float w_own = 1.f, w_oth = 0.f;                // single head: weights of the two groups' partial results
            if (solo && n > 0) {
                // The two groups went through disjoint sets of key tiles, each with its own reference maximum: tell
                // each other (m, l) -- each after its own last P.V has completed, so that both accumulators are final
                // once both have told -- then every thread scales both accumulators of its row to the common maximum.
                float2* told = reinterpret_cast<float2*>(xch) + (wit & 1u) * (2 * kTileM);   // two buffers, used in turn
                told[grp * kTileM + row] = make_float2(m_ref, l);
                __syncwarp();
                if (lane == 0) bar_arrive(merge0);
                if (!bar_wait(merge0, wit & 1u, abort_flag)) { alive = false; break; }
                tc_fence_after();
                const float2 oth = told[(grp ^ 1) * kTileM + row];
                const float m = fmaxf(m_ref, oth.x);
                w_own = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m);
                w_oth = (oth.x == -INFINITY) ? 0.f : exp2f(oth.x - m);
                l = l * w_own + oth.y * w_oth;
                m_ref = m;
            }
            if (n > 0) ++wit;
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const float lse_nat = l > 0.f ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
            const bool gate_on = prm.epi.sinks != nullptr;
            const float gate = sink_gate(prm.epi, hq, lse_nat);
            // A thread owns a row, so a plain store instruction of the warp would touch 32 rows with 16 bytes each.
            // 32 columns (64 bytes per row) at a time go into a per-warp staging buffer instead, in the 64-byte
            // swizzle pattern (conflict-free for the row-per-lane writes), and leave as one bulk tensor store of
            // 32 rows x 64 bytes: the warp does not wait for the memory system, only -- before it refills the buffer
            // -- for the copy engine to have read it.  Rows past the end of the packed row fall outside the tensor
            // map and are dropped by the copy.
            uint8_t* stage = ostage + warp * 2048;
            auto put_rows = [&](const uint32_t (&w)[16], int col) {
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous copy has read the buffer
                __syncwarp();
#pragma unroll
                for (int c = 0; c < 4; ++c)                // 16-byte chunk c of row `lane`
                    *reinterpret_cast<uint4*>(stage + lane * 64 + ((c ^ ((lane >> 1) & 3)) << 4)) =
                        make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // every writer, ahead of the copy engine's read
                __syncwarp();
                const int row0 = d->t0 + quarter * 32;     // first packed token of this warp's rows
                if (lane == 0 && row0 < prm.L) {
                    const int c1 = prm.epi.token_major ? hq : row0, c2 = prm.epi.token_major ? row0 : hq;
                    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                                 ::"l"(reinterpret_cast<uint64_t>(&o_map)), "r"(col), "r"(c1), "r"(c2), "r"(s32(stage)) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            };
            if (!solo) {
#pragma unroll 1
                for (int c2 = 0; c2 < D / 64; ++c2) {
                    if (n > 0) {
                        tmem_ld32_nowait(to + c2 * 64, sv[0]);
                        tmem_ld32_nowait(to + c2 * 64 + 32, sv[1]);
                        tmem_wait_ld();
                        if (c2 == D / 64 - 1) {            // O is in registers: the next item's first P.V may overwrite it
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) bar_arrive(o_free0 + 8 * grp);
                        }
                    }
#pragma unroll
                    for (int q16 = 0; q16 < 2; ++q16) {
                        uint32_t w[16];
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const float a = (n > 0 && l > 0.f) ? __uint_as_float(sv[q16][2 * e]) * inv : 0.f;
                            const float bb = (n > 0 && l > 0.f) ? __uint_as_float(sv[q16][2 * e + 1]) * inv : 0.f;
                            w[e] = gated_pair<T>(a, bb, gate, gate_on);
                        }
                        put_rows(w, c2 * 64 + q16 * 32);
                    }
                }
            } else {
                // single head: this group writes columns [grp * D/2, +D/2) of the row, from both accumulators
                constexpr int kCols = D / 2;
                const uint32_t to_oth = tmem + 256 + (grp ^ 1) * kTileN + lane_base;
#pragma unroll 1
                for (int c2 = 0; c2 < kCols / 32; ++c2) {
                    const int col0 = grp * kCols + c2 * 32;
                    // (an accumulator that got no key tile of this item holds whatever was there: it is not read)
                    if (own_tiles) tmem_ld32_nowait(to + col0, sv[0]);
                    if (oth_tiles) tmem_ld32_nowait(to_oth + col0, sv[1]);
                    if (own_tiles || oth_tiles) tmem_wait_ld();
                    if (c2 == kCols / 32 - 1 && (own_tiles || oth_tiles)) {   // read: the next item's P.V may overwrite them
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0 && own_tiles) bar_arrive(o_free0 + 8 * grp);
                        if (lane == 0 && oth_tiles) bar_arrive(o_free0 + 8 * (grp ^ 1));
                    }
                    uint32_t w[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int c = 2 * e;
                        const bool some = n > 0 && l > 0.f;
                        const float a0 = own_tiles ? __uint_as_float(sv[0][c]) * w_own : 0.f, a1 = oth_tiles ? __uint_as_float(sv[1][c]) * w_oth : 0.f;
                        const float b0 = own_tiles ? __uint_as_float(sv[0][c + 1]) * w_own : 0.f, b1 = oth_tiles ? __uint_as_float(sv[1][c + 1]) * w_oth : 0.f;
                        const float a = some ? (a0 + a1) * inv : 0.f;
                        const float bb = some ? (b0 + b1) * inv : 0.f;
                        w[e] = gated_pair<T>(a, bb, gate, gate_on);
                    }
                    put_rows(w, col0);
                }
            }
            if (tk < prm.L && (!solo || grp == 0)) prm.lse[(size_t)hq * prm.L + tk] = lse_nat;
            __syncwarp();
            if (lane == 0) bar_arrive(desc_empty0 + 8 * b);
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the staging buffer is shared memory the next CTA gets
    }
    if (!alive && lane == 0) {
        if (!*abort_flag) raise_status(prm.status, FPKV_STATUS_TIMEOUT);
        *abort_flag = 1;
    }
    // ---- teardown: everyone meets here, then the allocating warp frees TMEM ---
    tc_fence_before();
    __syncthreads();
    if (warp == kLoadWarp && lane == 0 && *abort_flag) {
        // Copies still in flight target this CTA's shared memory, which the next CTA on this SM gets: wait
        // (bounded) for the last copy requested into every buffer, on the phase that copy completes.
        for (int h = 0; h < 2; ++h)
            if (q_requested[h] > 0) for (uint32_t k = 0; k < kSpin && !bar_try(q_full0 + 8 * h, (q_requested[h] - 1) & 1u); ++k) {}
        for (uint32_t s = 0; s < (uint32_t)kStages; ++s) {
            if (k_requested > s) {
                const uint32_t last = ((k_requested - 1 - s) / kStages) * kStages + s;    // last key tile requested into stage s
                for (uint32_t k = 0; k < kSpin && !bar_try(k_full0 + 8 * s, (last / kStages) & 1u); ++k) {}
            }
        }
        for (uint32_t s = 0; s < (uint32_t)kStagesV; ++s) {
            if (v_requested > s) {
                const uint32_t last = ((v_requested - 1 - s) / kStagesV) * kStagesV + s;
                for (uint32_t k = 0; k < kSpin && !bar_try(v_full0 + 8 * s, (last / kStagesV) & 1u); ++k) {}
            }
        }
    }
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encoder() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

int prefill_sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v > 0 ? v : 148;
    }();
    return n;
}

constexpr int kPrefillSmem = 1024 + (2 + 2 * kStages) * kTileBytes + 48 * 8 + 16 * 4 + 2 * (int)sizeof(ItemDesc) +
                             2 * 2 * kTileM * 8 + 8 * 2048 + 64;   // Q x2, K and V x kStages, barriers, flags, descriptors, merge and output staging buffers

}  // namespace


bool prefill_tc_supported(const PoolView& pv, int Hq)
{
    if (pv.split_hq && (Hq != pv.split_hq || pv.D != 128)) return false;   // half rows of a split pool must fill a 128-byte swizzle row
    if (pv.dtype != FPKV_BF16 && pv.dtype != FPKV_F16) return false;
    if (pv.P != kPage || (pv.D != 128 && pv.D != 64)) return false;
    if (Hq % pv.H) return false;
    // TMA coordinates are 32-bit token rows within one layer's K and V planes (more rows than 180 GB can hold)
    if ((long long)2 * pv.H * pv.n_pages * pv.P >= (1ll << 31)) return false;
    return encoder() != nullptr;
}

int launch_prefill_tc(const PoolView& pv, int layer, void* out, float* lse, const void* q, long long q_stride_h,
                      long long q_stride_t, const int64_t* batch_idx, const int32_t* extent, int L, int Hq,
                      float sm_scale, const Epilogue& epi, int32_t* status, cudaStream_t stream)
{
    if (L == 0) return FPKV_OK;
    const CUtensorMapDataType dt = pv.dtype == FPKV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap kv_map, khw_map, v_map, q_map;
    memset(&khw_map, 0, sizeof(khw_map)); memset(&v_map, 0, sizeof(v_map));
    // a tensor of `rows` token rows of `halves` 64-element column groups, seen through a box of one page
    auto encode_pages = [&](CUtensorMap* m, void* base, unsigned long long rows, int halves) {
        const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)halves};
        const cuuint64_t strides[2] = {(cuuint64_t)halves * 128, 128};
        const cuuint32_t box[3] = {64, (cuuint32_t)kPage, (cuuint32_t)halves};
        const cuuint32_t es[3] = {1, 1, 1};
        return encoder()(m, dt, 3, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    const unsigned long long R = (unsigned long long)pv.n_pages * pv.P;
    if (!pv.split_hq) {     // one layer's K and V planes as one tensor
        if (!encode_pages(&kv_map, pv.plane(layer, 0, 0), 2ull * pv.H * R, pv.D / 64)) return FPKV_ELAUNCH;
    } else {                // first K halves (per KV head), second K halves (per query head), values (per KV head)
        if (!encode_pages(&kv_map, pv.kt_plane(layer, 0), (unsigned long long)pv.H * R, 1) ||
            !encode_pages(&khw_map, pv.khw_plane(layer, 0), (unsigned long long)pv.split_hq * R, 1) ||
            !encode_pages(&v_map, pv.v_plane(layer, 0), (unsigned long long)pv.H * R, 2))
            return FPKV_ELAUNCH;
    }
    {   // queries: (64 elements, L tokens, head_dim / 64, Hq heads); rows past L read as zeros
        const cuuint64_t dims[4] = {64, (cuuint64_t)L, (cuuint64_t)(pv.D / 64), (cuuint64_t)Hq};
        const cuuint64_t strides[3] = {(cuuint64_t)q_stride_t * 2, 128, (cuuint64_t)q_stride_h * 2};
        const cuuint32_t box[4] = {64, (cuuint32_t)kTileM, (cuuint32_t)(pv.D / 64), 1};
        const cuuint32_t es[4] = {1, 1, 1, 1};
        if (encoder()(&q_map, dt, 4, const_cast<void*>(q), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return FPKV_ELAUNCH;
    }
    CUtensorMap o_map;
    {   // output rows: (head_dim, Hq heads, L tokens) or (head_dim, L tokens, Hq heads), written 32 rows x 64 bytes at a time
        const bool tm = epi.token_major;
        const cuuint64_t dims[3] = {(cuuint64_t)pv.D, (cuuint64_t)(tm ? Hq : L), (cuuint64_t)(tm ? L : Hq)};
        const cuuint64_t strides[2] = {(cuuint64_t)pv.D * 2, (cuuint64_t)(tm ? Hq : L) * pv.D * 2};
        const cuuint32_t box[3] = {32, tm ? 1u : 32u, tm ? 32u : 1u};
        const cuuint32_t es[3] = {1, 1, 1};
        if (encoder()(&o_map, dt, 3, out, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                      CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return FPKV_ELAUNCH;
    }
    PrefillParams prm;
    prm.page_table = pv.page_table; prm.p2l = pv.p2l; prm.batch_idx = batch_idx; prm.extent = extent;
    prm.out = out; prm.lse = lse; prm.status = status;
    prm.L = L; prm.Hq = Hq; prm.Hkv = pv.H; prm.n_pages = pv.n_pages; prm.max_batch = pv.max_batch;
    prm.rows_per_plane = pv.n_pages * pv.P;
    prm.scale_log2 = sm_scale * kLog2e;
    prm.split = pv.split_hq ? 1 : 0;
    prm.heads_per_item = (!prm.split && (Hq / pv.H) % 2 == 0) ? 2 : 1;
    prm.n_qtiles = (L + kTileM - 1) / kTileM;
    prm.n_pairs = Hq / prm.heads_per_item;
    const long long n_items = (long long)prm.n_qtiles * prm.n_pairs;
    if (n_items >= (1ll << 30)) return FPKV_ESHAPE;
    prm.n_items = (int)n_items;
    prm.epi = epi;
    const int grid = prm.n_items < prefill_sm_count() ? prm.n_items : prefill_sm_count();    // persistent: one CTA per SM
    auto launch = [&](auto kern) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem) != cudaSuccess) return false;
        kern<<<grid, kPrefillThreads, kPrefillSmem, stream>>>(q_map, kv_map, khw_map, v_map, o_map, prm);
        return true;
    };
    bool ok;
    if (prm.heads_per_item == 2) {
        if (pv.dtype == FPKV_BF16) ok = pv.D == 128 ? launch(prefill_tc_kernel<__nv_bfloat16, 128, false>) : launch(prefill_tc_kernel<__nv_bfloat16, 64, false>);
        else ok = pv.D == 128 ? launch(prefill_tc_kernel<__half, 128, false>) : launch(prefill_tc_kernel<__half, 64, false>);
    } else {
        if (pv.dtype == FPKV_BF16) ok = pv.D == 128 ? launch(prefill_tc_kernel<__nv_bfloat16, 128, true>) : launch(prefill_tc_kernel<__nv_bfloat16, 64, true>);
        else ok = pv.D == 128 ? launch(prefill_tc_kernel<__half, 128, true>) : launch(prefill_tc_kernel<__half, 64, true>);
    }
    if (!ok) return FPKV_ELAUNCH;
    return cudaGetLastError() == cudaSuccess ? FPKV_OK : FPKV_ELAUNCH;
}

}  // namespace fpkv
