// Paged prefill / chunked-prefill attention on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory) for 16-bit pools, page_size 128,
// head_dim 128.
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
// One CTA = one 128-row query tile of a PAIR of query heads that share a stored
// head (a single head when the GQA ratio is odd): the K/V tile staged in shared
// memory feeds both heads, which halves the L2 traffic per FLOP.  Per key tile
// and head:
//     S = Q K^T    128x128x128, A = Q (shared, K-major), B = K tile (shared, K-major) -> TMEM
//     O += P V     128x128x128, A = P (TMEM, written in place over S), B = V tile (shared, MN-major) -> TMEM
// Tensor memory holds S/P and O of both heads (4 x 128 columns = all 512), so
// each head is one dependent chain  S -> softmax -> P.V -> next S  and only two
// chains are in flight.  Two resources bound a (tile, head pair) at 2048 clocks
// each: the tensor pipe (32 MMAs of 64 clocks) and the exponential unit (2 x
// 128 x 128 results at 16 per clock per SM); the kernel is about keeping both
// busy at once.
//   * Warps 0-7 do the softmax, all eight on ONE head's tile at a time, two
//     threads per query row (warps w and w + 4 reach the same 32 TMEM lanes and
//     take 64 key columns each).  Two warps per scheduler keep the exponential
//     unit saturated; a quarter of the exponentials run as a polynomial on the
//     FMA pipe instead.  While they work on one head, the other head's MMAs run.
//   * Warp 8 is the TMA producer (2-stage K and V rings).
//   * Warps 9 and 10 issue the MMAs, one warp per head: the tensor pipe takes the
//     MMAs of a thread one after the other and idles through whatever else that
//     thread does (a barrier wait costs it ~30-100 clocks), so each head gets its
//     own issuer and waits for operand tiles before it waits for P.
// The running maximum is only raised when a tile exceeds it by more than 2^8
// (probabilities stay below 256, exact in fp32 and harmless in bf16), so O in
// TMEM is rarely rescaled.  The output tile is staged through the idle query
// buffer so that rows leave in whole lines.
// Every wait is a bounded mbarrier wait; on expiry the CTA raises
// FPKV_STATUS_TIMEOUT, the MMA and copy warps leave their loops, the softmax
// warps run theirs to the end without waiting (they meet at named barriers),
// TMEM is freed and the kernel returns.

#include <cuda.h>
#include <type_traits>
#include "common.cuh"

namespace fpkv {
namespace {

constexpr int kTileM = 128, kTileN = 128, kHeadDim = 128, kPage = 128;
constexpr int kTileBytes = 128 * 128 * 2;              // any 128 x 128 16-bit tile
constexpr int kHalfBytes = kTileBytes / 2;             // 64 columns (128 bytes) x 128 rows
constexpr int kStages = 2;
constexpr int kSoftmaxWarps = 4;                       // per key-column half: warps 0-3 take columns [0,64), warps 4-7 [64,128)
constexpr int kLoadWarp = 8, kMmaWarp = 9;              // warps 9 and 10 issue the MMAs of head 0 and head 1 of the pair
constexpr int kPrefillThreads = 12 * 32;               // warp 11 idles: registers are granted per four warps anyway
constexpr int kMaxKeyTiles = 512;                      // 65 536 keys per sequence
constexpr uint32_t kSpin = 1u << 22;
constexpr uint32_t kTmemCols = 512;                    // S/P head 0, S/P head 1, O head 0, O head 1: 128 columns each
constexpr float kRescaleThreshold = 8.f;
#ifndef FPKV_POLY_EVERY
#define FPKV_POLY_EVERY 4
#endif
constexpr int kPolyEvery = FPKV_POLY_EVERY;            // one pair in this many takes the polynomial 2^x (0x7fffffff: none)

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
__device__ __forceinline__ uint32_t umma_idesc(bool bf16, bool b_mn_major) {
    uint32_t d = 0;
    d |= 1u << 4;                                      // accumulator format f32
    d |= (bf16 ? 1u : 0u) << 7;                        // A format
    d |= (bf16 ? 1u : 0u) << 10;                       // B format
    d |= (b_mn_major ? 1u : 0u) << 16;                 // B major: 0 = K, 1 = MN
    d |= (uint32_t)(kTileN >> 3) << 17;
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

// 2^x for a pair of arguments on the FMA and integer pipes instead of the exponential unit, which is the narrow
// resource of the softmax phase (16 results per clock per SM): round to the nearest integer with the
// 1.5 * 2^23 trick, a degree-3 polynomial on the remainder in [-0.5, 0.5] (maximum relative error 7.5e-5, far
// below the 16-bit rounding of the probabilities), the integer added into the exponent bits.  Arguments
// are clamped below at -126; they never exceed 8 here.  Packed f32x2 arithmetic halves the instruction count.
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
__device__ __forceinline__ F2 ex2_poly2(F2 x) {
    x.x = fmaxf(x.x, -126.f); x.y = fmaxf(x.y, -126.f);
    const F2 fl = add2(x, F2{12582912.f, 12582912.f});
    const F2 n = add2(fl, F2{-12582912.f, -12582912.f});
    const F2 f = add2(x, F2{-n.x, -n.y});
    F2 p = fma2(f, F2{0.05517164617776871f, 0.05517164617776871f}, F2{0.2426111251115799f, 0.2426111251115799f});
    p = fma2(p, f, F2{0.6932609677314758f, 0.6932609677314758f});
    p = fma2(p, f, F2{0.9999280571937561f, 0.9999280571937561f});
    F2 r;
    r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(fl.x) << 23));
    r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(fl.y) << 23));
    return r;
}


// S = Q K^T: eight K = 16 steps (32 bytes along the 128-byte swizzled rows, second 64-element half 16 KiB on), then
// the commit that tells the softmax group.
__device__ __forceinline__ void issue_qk_gemm(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t bar) {
#pragma unroll
    for (int k = 0; k < kHeadDim / 16; ++k) {
        const uint32_t off = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
        umma(d, a_lo + off, hi, b_lo + off, hi, idesc, k > 0);
    }
    umma_commit(bar);
}
// O += P V: P from tensor memory (8 packed columns per 16 keys), V rows from shared memory (MN-major, 16 rows = 2 KiB per step).
// Issued in two halves of four steps (keys 0-63, 64-127) so that the first can run while the softmax group still
// exponentiates the second half of the tile.
template <int kHalf>
__device__ __forceinline__ void issue_pv_gemm(uint32_t d, uint32_t a, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t acc0) {
#pragma unroll
    for (int k = kHalf * 4; k < kHalf * 4 + 4; ++k)
        umma_ts(d, a + k * 8, b_lo + k * ((16 * 128) >> 4), hi, idesc, k > 0 ? 1u : acc0);
}


struct PrefillParams {
    const int64_t* page_table;
    const int64_t* p2l;
    const int64_t* batch_idx;   // [L] slot of each packed token (0 = pad)
    const int32_t* extent;      // [L] number of visible keys of each packed token
    void* out;                  // (Hq, L, D) contiguous
    float* lse;                 // (Hq, L)
    int32_t* status;
    int L, Hq, Hkv, n_pages, max_batch;
    int rows_per_plane;         // n_pages * page_size
    float scale_log2;
    int is_bf16;
    int heads_per_cta;          // 2: both query heads of a GQA pair share the staged K/V tiles; 1 otherwise
    Epilogue epi;
};

template <typename T>
__global__ void __launch_bounds__(kPrefillThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                  const PrefillParams prm)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem;                                   // 2 x 32 KiB: the query tile of each head of the pair
    uint8_t* k_s = q_s + 2 * kTileBytes;                   // kStages x 32 KiB
    uint8_t* v_s = k_s + kStages * kTileBytes;             // kStages x 32 KiB
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + kStages * kTileBytes);
    int* ints = reinterpret_cast<int*>(bars + 24);
    volatile int* abort_flag = ints;                       // [0] abort, [1] TMEM base
    int* tmem_slot = ints + 1;
    int* warp_red = ints + 4;                              // [8] per-warp reductions of the prologue
    int* page_row = ints + 16;                             // [kMaxKeyTiles] pool row of key tile j (page 0 when unmapped)
    unsigned char* page_ok = reinterpret_cast<unsigned char*>(page_row + kMaxKeyTiles);   // [kMaxKeyTiles]
    float* xch = reinterpret_cast<float*>(page_ok + kMaxKeyTiles);                         // [2][2][128] row max / row sum exchange

    const uint32_t q_full = s32(bars + 0);
    const uint32_t k_full0 = s32(bars + 1), v_full0 = s32(bars + 3), k_empty0 = s32(bars + 5), v_empty0 = s32(bars + 7);
    const uint32_t s_full0 = s32(bars + 9);                // [2] one per head of the pair
    const uint32_t p_full0 = s32(bars + 11);               // [2] P of the tile written (all eight softmax warps arrive)
    const uint32_t all_done0 = s32(bars + 13);             // [2] one per head

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    // Query tiles are taken from the end of the packed row backwards, all head pairs of a tile before the next tile:
    // under a causal mask the later tiles of a sequence see more keys, and the long CTAs should start first.
    const int t0 = (int)(gridDim.y - 1 - blockIdx.y) * kTileM;   // first packed token of the query tile
    const int heads = prm.heads_per_cta;                   // 1 or 2 query heads of one stored head
    const int hq0 = blockIdx.x * heads;
    const int hkv = hq0 / (prm.Hq / prm.Hkv);
    const bool is_softmax = warp < 2 * kSoftmaxWarps;

    // ---- prologue ----------------------------------------------------------
    if (tid == 0) {
        bar_init(q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            bar_init(k_full0 + 8 * s, 1); bar_init(v_full0 + 8 * s, 1);
            bar_init(k_empty0 + 8 * s, heads); bar_init(v_empty0 + 8 * s, heads);     // one commit per head's MMA warp
        }
        for (int g = 0; g < 2; ++g) { bar_init(s_full0 + 8 * g, 1); bar_init(p_full0 + 8 * g, 2 * kSoftmaxWarps); }
        bar_init(all_done0, 1); bar_init(all_done0 + 8, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {                                // TMEM allocation is a whole-warp operation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // slot and extent of this thread's row (both softmax groups look at the same 128 rows);
    // the tile's slot is the largest one (pads are slot 0)
    const int row = tid % kTileM;
    int my_slot = 0, my_extent = 0;
    if (is_softmax && t0 + row < prm.L) {
        const long long s = prm.batch_idx[t0 + row];
        const int e = prm.extent[t0 + row];                // both loads in flight together
        if (s < 0 || s >= prm.max_batch) raise_status(prm.status, FPKV_STATUS_BAD_SLOT);
        else { my_slot = (int)s; my_extent = s > 0 ? e : 0; }
        if (my_extent < 0) my_extent = 0;
    }
    {
        int sl = my_slot;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sl = max(sl, __shfl_xor_sync(0xffffffffu, sl, o));
        if (lane == 0 && warp < kSoftmaxWarps) warp_red[warp] = sl;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const int slot = max(max(warp_red[0], warp_red[1]), max(warp_red[2], warp_red[3]));
    // The copy warp starts as early as it can: the query tile depends on nothing (issued now), the first K / V
    // tile only on the sequence's first page id (load started now, used after the next barrier), so that the first
    // Q.K^T does not wait for the rest of the set-up.
    const bool early = warp == kLoadWarp && lane == 0 && slot > 0;
    long long early_pg = -1;
    if (early) {
        bar_expect_tx(q_full, heads * kTileBytes);
        for (int g = 0; g < heads; ++g) tma_4d(s32(q_s + g * kTileBytes), &q_map, 0, t0, 0, hq0 + g, q_full);
        early_pg = prm.page_table[(long long)slot * prm.n_pages];
    }
    if (my_slot != 0 && my_slot != slot) {                 // two live sequences in one query tile: not supported
        raise_status(prm.status, FPKV_STATUS_BAD_SLOT);
        my_extent = 0;
    }
    if ((long long)my_extent > (long long)prm.n_pages * kPage) { raise_status(prm.status, FPKV_STATUS_BAD_POS); my_extent = 0; }
    {
        int ex = my_extent;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ex = max(ex, __shfl_xor_sync(0xffffffffu, ex, o));
        if (lane == 0 && warp < kSoftmaxWarps) warp_red[4 + warp] = ex;
    }
    __syncthreads();
    const int max_extent = max(max(warp_red[4], warp_red[5]), max(warp_red[6], warp_red[7]));
    int n_tiles = (max_extent + kTileN - 1) / kTileN;
    if (n_tiles > kMaxKeyTiles) { if (tid == 0) raise_status(prm.status, FPKV_STATUS_BAD_POS); n_tiles = kMaxKeyTiles; }
    int k_requested = 0, v_requested = 0;                  // key / value tiles the copy thread has requested so far
    if (early && n_tiles > 0) {                            // first K and V tile (an unmapped first page is masked later)
        k_requested = v_requested = 1;
        const int row0 = hkv * prm.rows_per_plane + ((early_pg >= 0 && early_pg < prm.n_pages) ? (int)early_pg : 0) * kPage;
        bar_expect_tx(k_full0, kTileBytes);
        tma_3d(s32(k_s), &kv_map, 0, row0, 0, k_full0);
        bar_expect_tx(v_full0, kTileBytes);
        tma_3d(s32(v_s), &kv_map, 0, row0 + prm.Hkv * prm.rows_per_plane, 0, v_full0);
    }
    // page ids of all key tiles, resolved once (coalesced) instead of one dependent load per tile
    for (int j = tid; j < n_tiles; j += kPrefillThreads) {
        const long long trow = (long long)slot * prm.n_pages;
        const long long pg = prm.page_table[trow + j];
        bool ok = pg >= 0 && pg < prm.n_pages;
        if (pg >= prm.n_pages) raise_status(prm.status, FPKV_STATUS_BAD_PAGE);
        if (ok) ok = prm.p2l[trow + pg] >= 0;
        page_row[j] = hkv * prm.rows_per_plane + (ok ? (int)pg : 0) * kPage;   // unmapped: reserved page 0 (finite junk, masked)
        page_ok[j] = ok;
    }
    __syncthreads();
    const uint32_t tmem = (uint32_t)*tmem_slot;
    // tensor memory: S/P of head 0 [0,128), S/P of head 1 [128,256), O of head 0 [256,384), O of head 1 [384,512)
    bool alive = true;

    if (warp == kLoadWarp) {
        // ============================== TMA producer ========================
        if (lane == 0 && n_tiles > 0) {
            if (!early) {
                bar_expect_tx(q_full, heads * kTileBytes);
                for (int g = 0; g < heads; ++g) tma_4d(s32(q_s + g * kTileBytes), &q_map, 0, t0, 0, hq0 + g, q_full);
            }
            for (int j = early ? 1 : 0; j < n_tiles; ++j) {
                const int st = j % kStages;
                const uint32_t ph = (j / kStages) & 1u;
                if (!bar_wait(k_empty0 + 8 * st, ph ^ 1u, abort_flag)) { alive = false; break; }
                bar_expect_tx(k_full0 + 8 * st, kTileBytes);
                tma_3d(s32(k_s + st * kTileBytes), &kv_map, 0, page_row[j], 0, k_full0 + 8 * st);
                k_requested = j + 1;
                if (!bar_wait(v_empty0 + 8 * st, ph ^ 1u, abort_flag)) { alive = false; break; }
                bar_expect_tx(v_full0 + 8 * st, kTileBytes);
                tma_3d(s32(v_s + st * kTileBytes), &kv_map, 0, page_row[j] + prm.Hkv * prm.rows_per_plane, 0, v_full0 + 8 * st);
                v_requested = j + 1;
            }
        }
    } else if (warp >= kMmaWarp && warp < kMmaWarp + heads) {
        // ============================== MMA issuers =========================
        // One issuing warp per head of the pair.  The tensor pipe takes the MMAs of one thread strictly one
        // after the other, and whatever else that thread does (barrier waits, commits) is time the pipe
        // idles for it; with an issuer per head the other head's MMAs fill those gaps, and each head's
        // chain  S -> softmax -> P.V -> next S  advances on its own.  Both heads read the one staged K / V tile.
        const int g = warp - kMmaWarp;
        if (lane == 0 && n_tiles > 0) {
            const uint32_t idesc_qk = umma_idesc(prm.is_bf16 != 0, false);
            const uint32_t idesc_pv = umma_idesc(prm.is_bf16 != 0, true);
            // descriptor words: low = start address >> 4 (| LBO for MN-major), high = SBO 1024 | version | 128-byte swizzle
            const uint32_t desc_hi = (uint32_t)(umma_desc(0, 0, 1024) >> 32);
            const uint32_t q_lo = ((s32(q_s) & 0x3FFFF) >> 4) + g * (kTileBytes >> 4), k_lo = (s32(k_s) & 0x3FFFF) >> 4;
            const uint32_t v_lo = ((s32(v_s) & 0x3FFFF) >> 4) | (uint32_t)umma_desc(0, kHalfBytes, 1024);
            const uint32_t t_s = tmem + g * kTileN, t_o = tmem + 256 + g * kTileN;
            const uint32_t s_full = s_full0 + 8 * g, p_full = p_full0 + 8 * g;
            alive = bar_wait(q_full, 0, abort_flag) && bar_wait(k_full0, 0, abort_flag);
            if (alive) {
                tc_fence_after();
                issue_qk_gemm(t_s, q_lo, k_lo, desc_hi, idesc_qk, s_full);
                umma_commit(k_empty0);
            }
            for (int j = 0; j < n_tiles && alive; ++j) {
                const int st = j % kStages, sn = (j + 1) % kStages;
                // the operand tiles first: they arrived long ago, and waiting for them here costs nothing
                // while the softmax group is still busy
                if (!bar_wait(v_full0 + 8 * st, (j / kStages) & 1u, abort_flag)) { alive = false; break; }
                if (j + 1 < n_tiles && !bar_wait(k_full0 + 8 * sn, ((j + 1) / kStages) & 1u, abort_flag)) { alive = false; break; }
                if (!bar_wait(p_full, j & 1u, abort_flag)) { alive = false; break; }
                tc_fence_after();
                issue_pv_gemm<0>(t_o, t_s, v_lo + st * (kTileBytes >> 4), desc_hi, idesc_pv, j > 0);
                issue_pv_gemm<1>(t_o, t_s, v_lo + st * (kTileBytes >> 4), desc_hi, idesc_pv, 1u);
                umma_commit(v_empty0 + 8 * st);
                if (j + 1 < n_tiles) {
                    issue_qk_gemm(t_s, q_lo, k_lo + sn * (kTileBytes >> 4), desc_hi, idesc_qk, s_full);
                    umma_commit(k_empty0 + 8 * sn);
                }
            }
            umma_commit(all_done0 + 8 * g);                // arrives when every MMA this thread issued has completed
            if (!alive) {
                // Gave up: tensor memory is freed and the CTA's shared memory handed on after the last barrier
                // below, so wait (bounded, ignoring the abort flag) for the MMAs already in the pipe.
                for (uint32_t k = 0; k < kSpin && !bar_try(all_done0 + 8 * g, 0); ++k) {}
            }
        }
    } else if (is_softmax) {
        // ============================== softmax warps =======================
        // All eight warps work on ONE head's score tile at a time, two threads per query row: warps w and
        // w + 4 reach the same 32 tensor-memory lanes, warp w / 4 takes key columns [0,64) or [64,128).  The
        // exponential unit (16 results per clock per SM) bounds this phase; with two warps per scheduler
        // it stays saturated, and a head's tile is through in half the time a single thread per row needs,
        // which is what the chain  S -> softmax -> P.V -> next S  of each head waits for.  The heads alternate
        // (tile j of head 0, tile j of head 1, tile j + 1 of head 0, ...) while the other head's MMAs run.
        const int quarter = warp % 4, colhalf = warp / 4;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        float m_ref[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        uint32_t v[32];
        uint32_t xslot = 0;                                // exchange buffer parity
        // (the two warps of a row quarter meet at their own named barrier, 1 + quarter)
        auto exchange_max = [&](float mine) {              // maximum over the two threads of a row
            float* buf = xch + (xslot & 1u) * 256;
            buf[colhalf * 128 + row] = mine;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
            const float other = buf[(1 - colhalf) * 128 + row];
            ++xslot;
            return fmaxf(mine, other);
        };
        for (int j = 0; j < n_tiles; ++j) {
            // Value rows past the last key any row of this tile sees (the tail of the last key tile, or all of
            // an unmapped page's stand-in) were fetched but possibly never appended: the pool may hold anything
            // there, and 0 x NaN would poison O.  Clear them in shared memory before the first P.V of the tile
            // (the tensor cores read shared memory through the async proxy, hence the proxy fence).
            const int tile_rows = page_ok[j] ? min(kTileN, max_extent - j * kTileN) : 0;
            if (tile_rows < kTileN) {
                const int st = j % kStages;
                if (alive && !bar_wait(v_full0 + 8 * st, (j / kStages) & 1u, abort_flag)) alive = false;
                for (int i = tid; i < (kTileN - tile_rows) * 16; i += 2 * kSoftmaxWarps * 32) {
                    const int r = tile_rows + (i >> 4), c = i & 15;         // token row, 16-byte piece of its 256 bytes
                    *reinterpret_cast<uint4*>(v_s + st * kTileBytes + (c >> 3) * kHalfBytes + r * 128 + ((c & 7) << 4)) =
                        make_uint4(0u, 0u, 0u, 0u);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            const int valid_row = page_ok[j] ? min(kTileN, my_extent - j * kTileN) : 0;   // visible keys of this row in the tile
            const int valid_cols = valid_row - colhalf * 64;                               // ... among this thread's 64 columns
            const bool full = __all_sync(0xffffffffu, valid_cols >= 64);
            for (int h = 0; h < heads; ++h) {
                const uint32_t ts = tmem + h * kTileN + lane_base;          // S, then P, of this head
                const uint32_t to = tmem + 256 + h * kTileN + lane_base + colhalf * 64;   // this thread's half of the O row
                // s_full also tells that P.V of tile j-1 is complete: O is stable and the P columns are free.
                // A wait that runs out does not leave the loop: every thread must reach the named barrier below.
                if (alive && !bar_wait(s_full0 + 8 * h, j & 1u, abort_flag)) alive = false;
                tc_fence_after();
                uint32_t sv[2][32];
                tmem_ld32_nowait(ts + colhalf * 64, sv[0]);
                tmem_ld32_nowait(ts + colhalf * 64 + 32, sv[1]);
                tmem_wait_ld();
                float mx;
                if (full) {
                    float m2[2];
#pragma unroll
                    for (int c2 = 0; c2 < 2; ++c2) {
                        m2[c2] = max3f(__uint_as_float(sv[c2][0]), __uint_as_float(sv[c2][1]), __uint_as_float(sv[c2][2]));
#pragma unroll
                        for (int c = 3; c + 1 < 32; c += 2)
                            m2[c2] = max3f(m2[c2], __uint_as_float(sv[c2][c]), __uint_as_float(sv[c2][c + 1]));
                        m2[c2] = fmaxf(m2[c2], __uint_as_float(sv[c2][31]));
                    }
                    mx = fmaxf(m2[0], m2[1]);
                } else {
                    mx = -INFINITY;
#pragma unroll
                    for (int c2 = 0; c2 < 2; ++c2)
#pragma unroll
                        for (int c = 0; c < 32; ++c) if (c2 * 32 + c < valid_cols) mx = fmaxf(mx, __uint_as_float(sv[c2][c]));
                }
                // after this barrier both threads of the row hold all their scores in registers, so the packed
                // P columns may overwrite either thread's score columns
                mx = exchange_max(mx) * prm.scale_log2;    // scale > 0: max commutes with it
                // raise the reference maximum only when this tile is far above it (both threads of a row decide alike)
                const bool raise = mx > m_ref[h] + kRescaleThreshold || (m_ref[h] == -INFINITY && mx > -INFINITY);
                if (__any_sync(0xffffffffu, raise)) {      // tensor-memory access is a whole-warp operation
                    const float m_new = raise ? mx : m_ref[h];
                    const float alpha = (m_ref[h] == -INFINITY) ? 0.f : exp2f(m_ref[h] - m_new);
                    if (j > 0) {                           // rescale this thread's half of the O row in tensor memory
#pragma unroll 1
                        for (int c2 = 0; c2 < 2; ++c2) {
                            tmem_ld32(to + c2 * 32, v);
#pragma unroll
                            for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * alpha);
                            tmem_st32(to + c2 * 32, v);
                        }
                    }
                    l[h] *= alpha;
                    m_ref[h] = m_new;
                }
                // probabilities, packed two per 32-bit column: this thread's 64 scores become packed columns
                // [colhalf * 32, colhalf * 32 + 32) of the region
                float r4[4] = {0.f, 0.f, 0.f, 0.f};
                const float neg_m = (m_ref[h] == -INFINITY) ? 0.f : -m_ref[h];
                uint32_t pk[32];
                auto probabilities = [&](auto full_tag) {
                    constexpr bool kFull = decltype(full_tag)::value;
#pragma unroll
                    for (int c2 = 0; c2 < 2; ++c2) {
#pragma unroll
                        for (int c = 0; c < 32; c += 2) {
                            float p0, p1;
                            if ((c >> 1) % kPolyEvery == kPolyEvery - 1) {     // every fourth pair off the exponential unit
                                const F2 p = ex2_poly2(fma2(F2{__uint_as_float(sv[c2][c]), __uint_as_float(sv[c2][c + 1])},
                                                            F2{prm.scale_log2, prm.scale_log2}, F2{neg_m, neg_m}));
                                p0 = p.x; p1 = p.y;
                            } else {
                                p0 = ex2(fmaf(__uint_as_float(sv[c2][c]), prm.scale_log2, neg_m));
                                p1 = ex2(fmaf(__uint_as_float(sv[c2][c + 1]), prm.scale_log2, neg_m));
                            }
                            if (!kFull) {
                                if (c2 * 32 + c >= valid_cols) p0 = 0.f;
                                if (c2 * 32 + c + 1 >= valid_cols) p1 = 0.f;
                            }
                            r4[(c >> 1) & 1] += p0;
                            r4[2 + ((c >> 1) & 1)] += p1;
                            pk[c2 * 16 + c / 2] = pack2<T>(p0, p1);
                        }
                    }
                };
                if (full) probabilities(std::true_type{}); else probabilities(std::false_type{});
                tmem_st32_nowait(ts + colhalf * 32, pk);
                l[h] += (r4[0] + r4[1]) + (r4[2] + r4[3]);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) bar_arrive(p_full0 + 8 * h);
            }
        }
        // ---- epilogue: O / l -> out, lse --------------------------------------
        // Each thread holds 64 of the 128 output values of its row.  Storing them straight from registers
        // would touch 32 different lines per warp instruction; the two warps of a row quarter stage their 32
        // rows in the (now idle) query tile of the head, 16-byte chunks XOR-swizzled by row so that neither
        // side has bank conflicts, and write them out two whole rows per instruction.
        T* out = reinterpret_cast<T*>(prm.out);
        for (int h = 0; h < heads; ++h) {
            const int hq = hq0 + h;
            const uint32_t to = tmem + 256 + h * kTileN + lane_base + colhalf * 64;
            if (n_tiles > 0) {
                if (alive && !bar_wait(all_done0 + 8 * h, 0, abort_flag)) alive = false;
                tc_fence_after();
            }
            // row sum over both threads of the row
            float* buf = xch + (xslot & 1u) * 256;
            buf[colhalf * 128 + row] = l[h];
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
            const float lsum = l[h] + buf[(1 - colhalf) * 128 + row];
            ++xslot;
            const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
            const float lse_nat = lsum > 0.f ? (m_ref[h] + log2f(lsum)) * kLn2 : -INFINITY;
            const bool gate_on = prm.epi.sinks != nullptr;
            const float gate = sink_gate(prm.epi, hq, lse_nat);
            uint8_t* slab = q_s + h * kTileBytes + quarter * (32 * 256);
#pragma unroll 1
            for (int c2 = 0; c2 < 2; ++c2) {
                if (n_tiles > 0) tmem_ld32(to + c2 * 32, v);
#pragma unroll
                for (int c = 0; c < 32; c += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float a = (n_tiles > 0 && lsum > 0.f) ? __uint_as_float(v[c + 2 * e]) * inv : 0.f;
                        const float b = (n_tiles > 0 && lsum > 0.f) ? __uint_as_float(v[c + 2 * e + 1]) * inv : 0.f;
                        w[e] = gated_pair<T>(a, b, gate, gate_on);
                    }
                    const int chunk = colhalf * 8 + c2 * 4 + c / 8;
                    *reinterpret_cast<uint4*>(slab + lane * 256 + ((chunk ^ (lane & 15)) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");         // both column halves of every row are staged
#pragma unroll 4
            for (int i = 0; i < 8; ++i) {                  // this warp writes out 16 of the quarter's 32 rows
                const int rr = colhalf * 16 + 2 * i + (lane >> 4), chunk = lane & 15;
                const uint4 val = *reinterpret_cast<const uint4*>(slab + rr * 256 + ((chunk ^ (rr & 15)) * 16));
                const int tk = t0 + quarter * 32 + rr;
                if (tk < prm.L) {
                    T* dst = out + (prm.epi.token_major ? ((size_t)tk * prm.Hq + hq) : ((size_t)hq * prm.L + tk)) * kHeadDim + chunk * 8;
                    *reinterpret_cast<uint4*>(dst) = val;
                }
            }
            if (colhalf == 0 && t0 + row < prm.L) prm.lse[(size_t)hq * prm.L + t0 + row] = lse_nat;
        }
    }
    if (!alive && lane == 0) {
        if (!*abort_flag) raise_status(prm.status, FPKV_STATUS_TIMEOUT);
        *abort_flag = 1;
    }
    // ---- teardown: everyone meets here, then the allocating warp frees TMEM ---
    tc_fence_before();
    __syncthreads();
    if (early && n_tiles == 0) {                          // the query tile was requested before it turned out that no row sees a key
        for (uint32_t k = 0; k < (1u << 20) && !bar_try(q_full, 0); ++k) {}
    }
    if (warp == kLoadWarp && lane == 0 && *abort_flag) {
        // Copies still in flight target this CTA's shared memory, which the next CTA on this SM gets: wait
        // (bounded) for the last copy requested into every stage, on the phase that copy completes.
        if (n_tiles > 0) for (uint32_t k = 0; k < kSpin && !bar_try(q_full, 0); ++k) {}
        for (int s = 0; s < kStages; ++s) {
            const int jk = ((k_requested - 1 - s) / kStages) * kStages + s;       // last key tile requested into stage s
            if (k_requested > s) for (uint32_t k = 0; k < kSpin && !bar_try(k_full0 + 8 * s, (jk / kStages) & 1u); ++k) {}
            const int jv = ((v_requested - 1 - s) / kStages) * kStages + s;
            if (v_requested > s) for (uint32_t k = 0; k < kSpin && !bar_try(v_full0 + 8 * s, (jv / kStages) & 1u); ++k) {}
        }
    }
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

constexpr int kPrefillSmem = 1024 + (2 + 2 * kStages) * kTileBytes + 24 * 8 + 16 * 4 + kMaxKeyTiles * 5 + 2 * 2 * 128 * 4 + 64;   // Q x2, K and V x kStages

}  // namespace


bool prefill_tc_supported(const PoolView& pv, int Hq)
{
    if (pv.dtype != FPKV_BF16 && pv.dtype != FPKV_F16) return false;
    if (pv.P != kPage || pv.D != kHeadDim) return false;
    if (Hq % pv.H) return false;
    if ((long long)2 * pv.H * pv.n_pages * pv.P >= (1ll << 31)) return false;
    return encoder() != nullptr;
}

int launch_prefill_tc(const PoolView& pv, int layer, void* out, float* lse, const void* q, long long q_stride_h,
                      long long q_stride_t, const int64_t* batch_idx, const int32_t* extent, int L, int Hq,
                      float sm_scale, const Epilogue& epi, int32_t* status, cudaStream_t stream)
{
    if (L == 0) return FPKV_OK;
    const CUtensorMapDataType dt = pv.dtype == FPKV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap kv_map, q_map;
    {   // one layer's K and V planes: (64 elements, token rows, head_dim / 64)
        const cuuint64_t dims[3] = {64, (cuuint64_t)2 * pv.H * pv.n_pages * pv.P, (cuuint64_t)(pv.D / 64)};
        const cuuint64_t strides[2] = {(cuuint64_t)pv.D * 2, 128};
        const cuuint32_t box[3] = {64, (cuuint32_t)kPage, (cuuint32_t)(pv.D / 64)};
        const cuuint32_t es[3] = {1, 1, 1};
        if (encoder()(&kv_map, dt, 3, pv.plane(layer, 0, 0), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
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
    PrefillParams prm;
    prm.page_table = pv.page_table; prm.p2l = pv.p2l; prm.batch_idx = batch_idx; prm.extent = extent;
    prm.out = out; prm.lse = lse; prm.status = status;
    prm.L = L; prm.Hq = Hq; prm.Hkv = pv.H; prm.n_pages = pv.n_pages; prm.max_batch = pv.max_batch;
    prm.rows_per_plane = pv.n_pages * pv.P;
    prm.scale_log2 = sm_scale * kLog2e;
    prm.is_bf16 = pv.dtype == FPKV_BF16;
    prm.heads_per_cta = ((Hq / pv.H) % 2 == 0) ? 2 : 1;
    prm.epi = epi;
    if ((L + kTileM - 1) / kTileM > 65535) return FPKV_ESHAPE;
    dim3 grid(Hq / prm.heads_per_cta, (L + kTileM - 1) / kTileM);
    if (pv.dtype == FPKV_BF16) {
        auto kern = prefill_tc_kernel<__nv_bfloat16>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem) != cudaSuccess) return FPKV_ELAUNCH;
        kern<<<grid, kPrefillThreads, kPrefillSmem, stream>>>(q_map, kv_map, prm);
    } else {
        auto kern = prefill_tc_kernel<__half>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem) != cudaSuccess) return FPKV_ELAUNCH;
        kern<<<grid, kPrefillThreads, kPrefillSmem, stream>>>(q_map, kv_map, prm);
    }
    return cudaGetLastError() == cudaSuccess ? FPKV_OK : FPKV_ELAUNCH;
}

}  // namespace fpkv
