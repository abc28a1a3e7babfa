// Paged decode attention for 16-bit pools on sm_100a: TMA-staged KV pages,
// mbarrier ring, tensor-core dot products, warp-shuffle online softmax.
//
// The kernel is bound by HBM reads of K and V.  Everything is arranged so that
// every SM streams an equal share of the batch's pages at full rate:
//
//  * "Tile" = one page of one stored head of one row: a K tile and a V tile of
//    page_size x head_dim elements, each contiguous in the pool (32 KiB at
//    page 128, head_dim 128, 16-bit).  Tiles are numbered row-major over
//    (row b, stored head h, logical page).
//  * SMs do not all pull the same bandwidth, so equal static shares leave the
//    fast ones idle at the end (measured: exits spread over 150..190 us).  The
//    flat tile range is therefore cut into "units" of decreasing size (five
//    phases, each covering half of what is left with gridDim.x units) and the
//    persistent CTAs, one per SM, claim units in order from an atomic counter.
//  * A unit can start and end in the middle of a (b, h) segment; such a piece
//    leaves an unnormalised partial (m, l, acc) in the workspace.  A second,
//    small kernel, launched with programmatic stream serialisation so that its
//    CTAs are already resident when the main grid drains, merges the partials
//    of every cut segment in parallel.  (Merging inside the main kernel with
//    arrival tickets was measured: a fence + atomic round trip costs ~5 us
//    under a saturated memory system and the merges pile up at the end.)
//    Segments inside one unit are normalised and written directly.  The unit
//    counter must be zero on entry and is left zero, so the workspace is
//    zero-filled once, not per call.
//  * Warp roles: a scout warp claims units, publishes them to the consumers
//    and resolves each tile to a pool row through the page table and its
//    inverse (32 tiles per coalesced read, up to 256 tiles ahead, so the
//    dependent global loads are off the critical path); an issue warp turns
//    resolved tiles into TMA tensor copies, one per K or V tile, into a ring
//    of shared-memory slots.  A copy lands with the 128-byte swizzle so that
//    ldmatrix reads are free of bank conflicts, and targets this CTA's own
//    shared memory only.  The last, partly filled page of a row is fetched in
//    groups of 16 token rows (one consumer warp's share) up to the row's length,
//    and the warps whose rows were not fetched skip the tile.
//  * Eight consumer warps each own page_size/8 token rows of every tile.  The
//    GQA group's query heads are the M rows of mma.sync.m16n8k16 (zero padded
//    to 16), so all query heads of a stored head consume the one staged tile.
//    Scores stay in registers; the row maximum is a two-step quad shuffle;
//    probabilities are repacked in place as the A operand of the P.V product.
//  * Every wait in the kernel is a bounded mbarrier wait (the consumers'
//    CTA-level barrier included): when a limit is hit the CTA raises
//    FPKV_STATUS_TIMEOUT, every role leaves its loop, the issue warp drains the
//    copies it has in flight (again bounded) and the kernel returns.
//
// Semantics: the reference's decode mask + FlexAttention call
// (falcon_perception/paged_inference.py:783-826,
//  falcon_perception/paged_attention.py:234-333, falcon_perception/model.py:156-162).

#include <cuda.h>          // CUtensorMap (types only; the encoder is fetched at run time)
#include <string.h>
#include "common.cuh"

namespace fpkv {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kIssueWarp = kConsumerWarps, kScoutWarp = kConsumerWarps + 1;
constexpr int kThreads = (kConsumerWarps + 2) * 32;
#ifndef FPKV_DECODE_PHASES
#define FPKV_DECODE_PHASES 5
#endif
constexpr int kPhases = FPKV_DECODE_PHASES;           // unit sizes halve from phase to phase
#ifndef FPKV_SMALL_PHASE_TILES
#define FPKV_SMALL_PHASE_TILES 8
#endif
constexpr int kSmallPhaseTiles = FPKV_SMALL_PHASE_TILES;   // a remainder of at most this many tiles per unit is not halved again
// Tiles taken by phase p when `rem` are left: half of them, or all of them in the last phase and when halving
// would leave units of a tile or two (small batches: each piece of a segment costs a partial and a merge step).
__device__ __forceinline__ int phase_step(int rem, int p, int G) {
    return (p == kPhases - 1 || rem <= kSmallPhaseTiles * G) ? rem : (rem + 1) / 2;
}
constexpr int kDescBlocks = 8;                 // resolved-tile blocks (32 tiles each) between scout and issue warp
constexpr int kUnitQueue = 8;                  // claimed units in flight between scout and consumers
constexpr int kClaimAhead = 3;                 // the scout claims the next unit when this few resolved tiles are unissued
constexpr int kMaxGrid = 256;
constexpr int kMaxBatchPerLaunch = 512;
constexpr uint32_t kSpinLimit = 1u << 22;      // try_wait attempts before giving up
constexpr int kSmemBudget = 227 * 1024;

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Bounded wait.  Returns false when the limit ran out or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
template <typename T> struct Mma;
template <> struct Mma<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
};
template <> struct Mma<__half> {
    static __device__ __forceinline__ void run(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
};
// ------------------------------------------------------------ shared layout
template <int D, int P, int NREP>
struct Layout {
    static constexpr int kTileBytes = P * D * 2;                       // one K or V tile
    static constexpr int kMergeFloats = kConsumerWarps * NREP * (D + 2);
    static constexpr int kBarWords = 80;                                // mbarriers (8 bytes each)
    static constexpr int kSmallInts = kDescBlocks * 33 + kUnitQueue + 16 + 4 + (kPhases + 1) + 3;
    static constexpr int kBatchInts = (kMaxBatchPerLaunch + 1) + 2 * kMaxBatchPerLaunch + (kPhases * kMaxGrid + 1);
    static constexpr int kFixedBytes = 2 * kMergeFloats * 4 + kBarWords * 8 + (kSmallInts + kBatchInts) * 4 + 64;
    static constexpr int kSlotsFit = (kSmemBudget - 1024 - kFixedBytes) / kTileBytes;
    static constexpr int kSlots = (kSlotsFit > 12 ? 12 : kSlotsFit) & ~1;   // K and V alternate: even
    static constexpr int kSmemBytes = 1024 + kSlots * kTileBytes + kFixedBytes;
    static_assert(kSlots >= 4, "ring too small");
};

struct Params {
    const int64_t* page_table;
    const int64_t* p2l;
    const int64_t* batch_idx;
    const void* pos;
    const void* q;
    void* out;
    float* lse;
    int* counters;             // [0] unit counter, zero between calls
    int4* seginfo;             // [B * Hkv] per segment: first unit, last unit, slot of the first piece | has-empty-units << 1, total tiles
    float* ws;                 // partials [units][2][NREP][D+2]
    int32_t* status;
    long long q_stride_b, q_stride_h;
    int B, Hkv, n_pages, max_batch;
    int after_append;          // 1: the preceding kernel on the stream is this library's append and writes only the pool
    int rows_per_plane;        // n_pages * P: token rows of one (K|V, head) plane
    float scale_log2;
    Epilogue epi;
};


// Unit schedule.  Phase p covers half of the tiles left after phase p-1 (the last one all of them) and
// is cut into G equal units; unit id u = p * G + j.  ub[u] = first flat tile of unit u, ub[NU] = total;
// the table is filled once per CTA so that every later use is a shared-memory read.
__device__ __forceinline__ int unit_of(const int* ub, int NU, int t) {     // ub[u] <= t < ub[u+1], t < ub[NU]
    int lo = 0, hi = NU;
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (ub[mid] <= t) lo = mid; else hi = mid; }
    return lo;
}

// ------------------------------------------------------------------ kernel
// Tensor maps of one layer.  Uniform layout: `kv` covers the K and V planes (box = one page), `kv_rows` the
// same tensor with a box of one consumer warp's rows of one 64-element column group.  Split layout (16-bit,
// head_dim 128): the first K halves, the second K halves and V are three tensors, each with a page box and
// a row-group box; a half-plane row is 64 elements = one 128-byte swizzle row, so a first half and a second
// half copied side by side form the same shared-memory tile as a whole K page of the uniform layout.
struct TileMaps {
    CUtensorMap kv, kv_rows;
    CUtensorMap kt, kt_rows, khw, khw_rows, v, v_rows;
};

template <typename T, int D, int P, int NREP, typename PosT, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1)
decode_tma_kernel(const __grid_constant__ TileMaps maps, const Params prm)
{
    // ring slots one tile takes: K and V, or (split) K of the group's first query head, the second K half of each
    // further query head, and V
    constexpr int kSlotsPerTile = SPLIT ? NREP + 1 : 2;
    static_assert(!SPLIT || (D == 128 && NREP >= 2), "the split layout needs head_dim 128 and a real GQA group");
    using L = Layout<D, P, NREP>;
    constexpr int NS = L::kSlots;
    constexpr int kTile = L::kTileBytes;
    constexpr int RW = P / kConsumerWarps;            // token rows per consumer warp (16 at P=128)
    constexpr int NB = RW / 8;                        // n8 score blocks per warp
    static_assert(RW % 16 == 0, "page_size must be a multiple of 128 rows / 8 warps * 16");
    static_assert(NREP <= 8, "query heads per stored head must fit the lower 8 MMA rows");
    static_assert(2 * NS + 2 * kDescBlocks + 2 * kUnitQueue + 1 <= L::kBarWords, "barrier area too small");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    float* merge = reinterpret_cast<float*>(ring + NS * kTile);               // [2][W][NREP][D+2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(merge + 2 * L::kMergeFloats);
    int* ints = reinterpret_cast<int*>(bars + L::kBarWords);
    int* dcount = ints;                               // [kDescBlocks] tiles in the block, -1 = end of work
    int* drow = dcount + kDescBlocks;                 // [kDescBlocks][32] pool row of the K tile | (16-row groups to fetch - 1), -1 = unmapped page
    int* uq = drow + kDescBlocks * 32;                // [kUnitQueue] claimed unit ids, -1 = end of work
    int* slot_valid = uq + kUnitQueue;                // [16] per ring slot: row groups present (0 = unmapped page, 8 = whole tile)
    volatile int* abort_flag = slot_valid + 16;       // [4]: abort flag, tiles issued so far
    volatile int* issued = abort_flag + 1;
    int* pb = const_cast<int*>(abort_flag) + 4;       // [kPhases + 1] phase boundaries
    int* cum = pb + kPhases + 1;                      // [B + 1] tiles before row b
    int* slot_of = cum + kMaxBatchPerLaunch + 1;      // [B] slot of row b
    int* nkeys_of = slot_of + kMaxBatchPerLaunch;     // [B] visible keys of row b (position + 1)
    int* ub = nkeys_of + kMaxBatchPerLaunch;          // [kPhases * G + 1] first tile of each unit

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int B = prm.B, Hkv = prm.Hkv;
    const int G = gridDim.x;
    const int NU = kPhases * G;
    // Launched with programmatic stream serialisation.  Standalone, nothing may be read before the
    // preceding kernel is complete.  Behind this library's append kernel (which writes only the pool)
    // everything up to the first pool read may overlap it; the issue warp waits before its first copy.
    if (!prm.after_append) asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * NS;
    const uint32_t dfull0 = empty0 + 8 * NS, dempty0 = dfull0 + 8 * kDescBlocks;
    const uint32_t ufull0 = dempty0 + 8 * kDescBlocks, uempty0 = ufull0 + 8 * kUnitQueue;
    const uint32_t cbar = uempty0 + 8 * kUnitQueue;   // CTA-level barrier of the consumer warps

    // ---- prologue: barriers, per-row page counts, exclusive scan -----------
    if (tid == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, kConsumerWarps); }
        for (int s = 0; s < kDescBlocks; ++s) { mbar_init(dfull0 + 8 * s, 1); mbar_init(dempty0 + 8 * s, 1); }
        for (int s = 0; s < kUnitQueue; ++s) { mbar_init(ufull0 + 8 * s, 1); mbar_init(uempty0 + 8 * s, kConsumerWarps); }
        mbar_init(cbar, kConsumerWarps);
        *abort_flag = 0;
        *issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int b = tid; b < B; b += kThreads) {
        const long long slot = prm.batch_idx[b];
        const long long p = load_pos<PosT>(prm.pos, b);
        int npg = 0;
        if (slot < 0 || slot >= prm.max_batch) raise_status(prm.status, FPKV_STATUS_BAD_SLOT);
        else if (p < 0 || p / P >= prm.n_pages) raise_status(prm.status, FPKV_STATUS_BAD_POS);
        else npg = (int)(p / P) + 1;
        slot_of[b] = (npg > 0) ? (int)slot : 0;
        nkeys_of[b] = (npg > 0) ? (int)p + 1 : 0;
        cum[b + 1] = npg * Hkv;                        // scanned below
    }
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int base = 0; base < B; base += 32) {
            const int i = base + lane;
            int v = (i < B) ? cum[i + 1] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
            if (i < B) cum[i + 1] = v + carry;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
        if (lane == 0) {
            cum[0] = 0;
            int at = 0;                                // phase p takes half of what is left, the last one all of it
            for (int p = 0; p < kPhases; ++p) { pb[p] = at; at += phase_step(carry - at, p, G); }
            pb[kPhases] = carry;
        }
    }
    __syncthreads();
    for (int u = tid; u <= NU; u += kThreads) {
        const int p = u / G, j = u - p * G;
        ub[u] = (p >= kPhases) ? pb[kPhases] : pb[p] + (int)((long long)(pb[p + 1] - pb[p]) * j / G);
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;");   // the finish kernel may take its seats now
    // rows without any tile (bad slot or position): out = 0, lse = -inf, one CTA per such row
    {
        const int Hq = Hkv * NREP;
        T* out0 = reinterpret_cast<T*>(prm.out);
        for (int b = blockIdx.x; b < B; b += G) {
            if (cum[b + 1] != cum[b]) continue;
            for (int e = tid; e < Hq * D; e += kThreads) out0[(size_t)b * Hq * D + e] = ElemTraits<T>::from_float(0.f);
            for (int e = tid; e < Hq; e += kThreads) prm.lse[(size_t)b * Hq + e] = -INFINITY;
        }
    }

    // Row that owns flat tile t (cum[b] <= t < cum[b+1]); B >= 1 and t < Ttot.
    auto row_of = [&](int t) {
        int lo = 0, hi = B;                            // invariant: cum[lo] <= t < cum[hi]
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (cum[mid] <= t) lo = mid; else hi = mid; }
        return lo;
    };
    auto give_up = [&]() {                             // a bounded wait ran out (or another role gave up)
        if (!*abort_flag) raise_status(prm.status, FPKV_STATUS_TIMEOUT);
        *abort_flag = 1;
    };

    if (warp == kScoutWarp) {
        // ============================ scout warp ============================
        // The first unit of a CTA is its own index; later ones come from the grid-wide counter, claimed
        // only when the issue warp is about to run out of resolved tiles, so that a slow SM does not
        // hoard work that a fast one could take.
        uint32_t qn = 0, blk = 0;                      // units published, descriptor blocks written
        int resolved = 0;                              // tiles handed to the issue warp so far
        int u = blockIdx.x;
        bool ok = true;
        while (ok) {
            if (u >= NU) {                             // nothing left; the very last claim of the grid rearms the counter
                if (lane == 0 && u == NU + G - 1) prm.counters[0] = 0;
                u = -1;
            }
            int r0 = 0, r1 = 0;
            if (u >= 0) { r0 = ub[u]; r1 = ub[u + 1]; }
            if (u >= 0 && r1 == r0) {
                // An empty unit (small batches) leaves a neutral partial, so that the finish kernel can read
                // every unit of a segment's range without working out which ones hold tiles.
                if (lane < NREP) __stcg(reinterpret_cast<float2*>(prm.ws + (((size_t)u * 2) * NREP + lane) * (D + 2)),
                                        make_float2(-INFINITY, 0.f));
            }
            if (u < 0 || r1 > r0) {                    // empty units are not handed to the consumers
                if (lane == 0) {
                    const uint32_t s = qn % kUnitQueue, ph = (qn / kUnitQueue) & 1u;
                    ok = mbar_wait(uempty0 + 8 * s, ph ^ 1u, abort_flag);
                    if (ok) { uq[s] = u; mbar_arrive(ufull0 + 8 * s); }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                ++qn;
            }
            if (!ok || u < 0) break;
            for (int base = r0; base < r1 && ok; base += 32) {
                const int t = base + lane;
                int row_k = -1;
                if (t < r1) {
                    const int b = row_of(t);
                    const int npg = (cum[b + 1] - cum[b]) / Hkv;
                    const int rel = t - cum[b];
                    const int h = rel / npg;
                    const long long trow = (long long)slot_of[b] * prm.n_pages;
                    const long long pg = prm.page_table[trow + (rel - h * npg)];
                    if (pg >= prm.n_pages) raise_status(prm.status, FPKV_STATUS_BAD_PAGE);
                    else if (pg >= 0 && prm.p2l[trow + pg] >= 0) {
                        // the row's last page is fetched only as far as it is filled, in groups of RW rows
                        const int n_here = min(P, nkeys_of[b] - (rel - h * npg) * P);
                        row_k = (h * prm.rows_per_plane + (int)pg * P) | ((n_here + RW - 1) / RW - 1);
                    }
                }
                const uint32_t s = blk % kDescBlocks, ph = (blk / kDescBlocks) & 1u;
                if (lane == 0) ok = mbar_wait(dempty0 + 8 * s, ph ^ 1u, abort_flag);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                drow[s * 32 + lane] = row_k;
                if (lane == 0) dcount[s] = min(32, r1 - base);
                __syncwarp();
                if (lane == 0) mbar_arrive(dfull0 + 8 * s);
                ++blk;
            }
            if (!ok) break;
            resolved += r1 - r0;
            // Claim the next unit as late as the lookups allow: when the issue warp has only a few resolved
            // tiles left.  A CTA then never sits on work that a faster SM could take (measured: claiming one
            // unit ahead cost 3 % through the tail), and three tiles of streaming cover the claim and the two
            // dependent table reads.
            if (lane == 0) {
                uint32_t spins = 0;
                while (resolved - *issued > kClaimAhead && !*abort_flag && ++spins < kSpinLimit) __nanosleep(100);
                ok = spins < kSpinLimit && !*abort_flag;
                if (ok) u = G + atomicAdd(prm.counters, 1);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            u = __shfl_sync(0xffffffffu, u, 0);
        }
        if (lane == 0) {
            if (!ok) give_up();
            else {                                     // end marker for the issue warp
                const uint32_t s = blk % kDescBlocks, ph = (blk / kDescBlocks) & 1u;
                if (mbar_wait(dempty0 + 8 * s, ph ^ 1u, abort_flag)) { dcount[s] = -1; mbar_arrive(dfull0 + 8 * s); }
                else give_up();
            }
        }
        return;
    }

    if (warp == kIssueWarp) {
        // ============================ issue warp ============================
        if (lane != 0) return;
        if (prm.after_append) asm volatile("griddepcontrol.wait;" ::: "memory");   // the appended rows are in the pool
        uint32_t it = 0, blk = 0;                      // ring position (one per slot filled), descriptor block
        int tiles_issued = 0;
        bool ok = true;
        while (ok) {
            const uint32_t ds = blk % kDescBlocks, dph = (blk / kDescBlocks) & 1u;
            if (!mbar_wait(dfull0 + 8 * ds, dph, abort_flag)) { ok = false; break; }
            const int cnt = dcount[ds];
            if (cnt < 0) break;
            for (int j = 0; j < cnt && ok; ++j) {
                const int desc = drow[ds * 32 + j];
                const int rk = desc < 0 ? -1 : (desc & ~(P - 1));
                const int groups = desc < 0 ? 0 : (desc & (P - 1)) + 1;
                if constexpr (!SPLIT) {
#pragma unroll
                    for (int kv = 0; kv < 2; ++kv, ++it) {
                        const uint32_t s = it % NS, ph = (it / NS) & 1u;
                        if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag)) { ok = false; break; }
                        slot_valid[s] = groups;
                        const int row = rk + kv * Hkv * prm.rows_per_plane;
                        const uint32_t dst = smem_u32(ring + s * kTile);
                        if (groups == kConsumerWarps) {                     // whole page: one copy
                            mbar_arrive_expect_tx(full0 + 8 * s, kTile);
                            tma_load_3d(dst, &maps.kv, 0, row, 0, full0 + 8 * s);
                        } else if (groups > 0) {                            // filled part of a row's last page
                            mbar_arrive_expect_tx(full0 + 8 * s, groups * RW * D * 2);
                            for (int g = 0; g < groups; ++g)
#pragma unroll
                                for (int half = 0; half < D / 64; ++half)
                                    tma_load_3d(dst + half * (P * 128) + g * (RW * 128), &maps.kv_rows, 0, row + g * RW, half,
                                                full0 + 8 * s);
                        } else {
                            mbar_arrive(full0 + 8 * s);
                        }
                    }
                } else {
                    // rk = stored head * rows + page * P: the row in the first-half tensor and in the V tensor; the
                    // second half of query head r of the group lives (head * (NREP - 1) + r) planes further on
                    const int hkv = rk < 0 ? 0 : rk / prm.rows_per_plane;
#pragma unroll
                    for (int part = 0; part < kSlotsPerTile; ++part, ++it) {
                        const uint32_t s = it % NS, ph = (it / NS) & 1u;
                        if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag)) { ok = false; break; }
                        slot_valid[s] = groups;
                        const uint32_t dst = smem_u32(ring + s * kTile);
                        const uint32_t bar = full0 + 8 * s;
                        if (groups == 0) { mbar_arrive(bar); continue; }
                        const bool whole = groups == kConsumerWarps;
                        if (part < NREP) {                                  // K: part 0 brings the shared first half too
                            const int row_hw = rk + (hkv * (NREP - 1) + part) * prm.rows_per_plane;
                            const int halves = part == 0 ? 2 : 1;
                            mbar_arrive_expect_tx(bar, halves * groups * RW * 64 * 2);
                            if (whole) {
                                if (part == 0) tma_load_3d(dst, &maps.kt, 0, rk, 0, bar);
                                tma_load_3d(dst + P * 128, &maps.khw, 0, row_hw, 0, bar);
                            } else {
                                for (int g = 0; g < groups; ++g) {
                                    if (part == 0) tma_load_3d(dst + g * (RW * 128), &maps.kt_rows, 0, rk + g * RW, 0, bar);
                                    tma_load_3d(dst + P * 128 + g * (RW * 128), &maps.khw_rows, 0, row_hw + g * RW, 0, bar);
                                }
                            }
                        } else {                                            // V
                            mbar_arrive_expect_tx(bar, groups * RW * D * 2);
                            if (whole) tma_load_3d(dst, &maps.v, 0, rk, 0, bar);
                            else
                                for (int g = 0; g < groups; ++g)
#pragma unroll
                                    for (int half = 0; half < 2; ++half)
                                        tma_load_3d(dst + half * (P * 128) + g * (RW * 128), &maps.v_rows, 0, rk + g * RW, half, bar);
                        }
                    }
                }
                ++tiles_issued;
                *issued = tiles_issued;                // tiles issued so far: paces the scout's claims
            }
            mbar_arrive(dempty0 + 8 * ds);
            ++blk;
        }
        if (!ok) {
            give_up();
            // drain: every copy issued has an expect_tx on its full barrier; wait for each once
            const uint32_t first = it > (uint32_t)NS ? it - NS : 0;
            for (uint32_t i = first; i < it; ++i) {
                const uint32_t s = i % NS, ph = (i / NS) & 1u;
                for (uint32_t k = 0; k < kSpinLimit && !mbar_try_wait(full0 + 8 * s, ph); ++k) {}
            }
        }
        return;
    }

    // ============================ consumer warps ============================
    // While the first tiles are in flight: tell the finish kernel which units hold each segment.
    bool has_empty_units = false;                      // a phase shorter than the grid leaves some units without tiles
#pragma unroll
    for (int p = 0; p < kPhases; ++p) has_empty_units |= (pb[p + 1] - pb[p]) < G;
    for (int sgi = blockIdx.x + G * tid; sgi < B * Hkv; sgi += G * kConsumerWarps * 32) {
        const int b = sgi / Hkv, h = sgi - b * Hkv;
        const int npg = (cum[b + 1] - cum[b]) / Hkv;
        int4 info = make_int4(-1, -1, 0, cum[B]);
        if (npg > 0) {
            const int seg0 = cum[b] + h * npg;
            info.x = unit_of(ub, NU, seg0);
            info.y = unit_of(ub, NU, seg0 + npg - 1);
            info.z = ((seg0 <= ub[info.x]) ? 0 : 1) | (has_empty_units ? 2 : 0);
        }
        __stcg(prm.seginfo + sgi, info);
    }
    const int g = lane >> 2, tq = lane & 3;            // MMA row group / thread-in-quad
    const T* qbase = reinterpret_cast<const T*>(prm.q);
    T* out = reinterpret_cast<T*>(prm.out);
    const int Hq = Hkv * NREP;
    uint32_t it = 0, qn = 0, nbar = 0;
    int piece = 0;
    bool alive = true;
    // CTA-level barrier of the consumer warps, bounded like every other wait
    auto consumer_bar = [&]() -> bool {
        __syncwarp();
        if (lane == 0) mbar_arrive(cbar);
        const bool ok = mbar_wait(cbar, nbar & 1u, abort_flag);
        ++nbar;
        return ok;
    };

    while (alive) {
        // ---- next unit claimed by the scout --------------------------------
        int u;
        {
            const uint32_t s = qn % kUnitQueue, ph = (qn / kUnitQueue) & 1u;
            if (!mbar_wait(ufull0 + 8 * s, ph, abort_flag)) { alive = false; break; }
            u = uq[s];
            __syncwarp();
            if (lane == 0) mbar_arrive(uempty0 + 8 * s);
            ++qn;
        }
        if (u < 0) break;
        const int r0 = ub[u], r1 = ub[u + 1];

        for (int t = r0; t < r1 && alive; ++piece) {
            // ---- piece = part of one (b, h) segment inside this unit -------
            const int b = row_of(t);
            const int npg = (cum[b + 1] - cum[b]) / Hkv;
            const int rel = t - cum[b];
            const int h = rel / npg, pg0 = rel - h * npg;
            const int seg0 = cum[b] + h * npg, seg1 = seg0 + npg;
            const int piece_end = min(seg1, r1);
            const bool direct = seg0 >= r0 && seg1 <= r1;
            const int ws_slot = (t == r0) ? 0 : 1;
            const long long n_keys = load_pos<PosT>(prm.pos, b) + 1;

            // query fragments: rows g < NREP are heads h*NREP + g, the rest zero
            uint32_t qa[D / 16][2];
            {
                const T* qrow = qbase + b * prm.q_stride_b + (long long)(h * NREP + g) * prm.q_stride_h;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    qa[kk][0] = (g < NREP) ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + 2 * tq) : 0u;
                    qa[kk][1] = (g < NREP) ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + 8 + 2 * tq) : 0u;
                }
            }
            float m = -INFINITY, l = 0.f;
            float o[D / 8][2];
#pragma unroll
            for (int n = 0; n < D / 8; ++n) { o[n][0] = 0.f; o[n][1] = 0.f; }

            for (int pg = pg0; pg < pg0 + (piece_end - t); ++pg) {
                // ---------------- S = Q K^T for this warp's RW tokens -------
                uint32_t s = it % NS, ph = (it / NS) & 1u;
                if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) { alive = false; break; }
                const bool valid = warp < slot_valid[s];               // this warp's rows were fetched
                float sc[NB][4];
#pragma unroll
                for (int j = 0; j < NB; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f; }
                if (valid) {
                    const uint32_t kt = smem_u32(ring + s * kTile);
#pragma unroll
                    for (int j = 0; j < NB; ++j) {
                        const int row = warp * RW + j * 8 + (lane & 7);
#pragma unroll
                        for (int kp = 0; kp < D / 32; ++kp) {          // two k-steps per ldmatrix.x4
                            const int chunk = kp * 4 + (lane >> 3);    // 16-byte column chunk 0..D/8-1
                            const uint32_t addr = kt + (chunk >> 3) * (P * 128) + row * 128 +
                                                  (((chunk & 7) ^ (row & 7)) << 4);
                            uint32_t b0, b1, b2, b3;
                            ldsm_x4(addr, b0, b1, b2, b3);
                            // split layout: the second half of head_dim in this slot belongs to the group's first query
                            // head only (row 0 of the A fragment); the other heads' second halves follow in their own slots
                            const bool mine = !SPLIT || kp < D / 64 || g == 0;
                            Mma<T>::run(sc[j], mine ? qa[2 * kp][0] : 0u, 0u, mine ? qa[2 * kp][1] : 0u, 0u, b0, b1);
                            Mma<T>::run(sc[j], mine ? qa[2 * kp + 1][0] : 0u, 0u, mine ? qa[2 * kp + 1][1] : 0u, 0u, b2, b3);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * s);
                ++it;
                if constexpr (SPLIT) {
#pragma unroll 1
                    for (int r = 1; r < NREP; ++r) {                    // second K half of query head r of the group
                        s = it % NS; ph = (it / NS) & 1u;
                        if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) { alive = false; break; }
                        if (valid) {
                            const uint32_t kt = smem_u32(ring + s * kTile);
#pragma unroll
                            for (int j = 0; j < NB; ++j) {
                                const int row = warp * RW + j * 8 + (lane & 7);
#pragma unroll
                                for (int kp = D / 64; kp < D / 32; ++kp) {
                                    const int chunk = kp * 4 + (lane >> 3);
                                    const uint32_t addr = kt + (chunk >> 3) * (P * 128) + row * 128 +
                                                          (((chunk & 7) ^ (row & 7)) << 4);
                                    uint32_t b0, b1, b2, b3;
                                    ldsm_x4(addr, b0, b1, b2, b3);
                                    const bool mine = g == r;
                                    Mma<T>::run(sc[j], mine ? qa[2 * kp][0] : 0u, 0u, mine ? qa[2 * kp][1] : 0u, 0u, b0, b1);
                                    Mma<T>::run(sc[j], mine ? qa[2 * kp + 1][0] : 0u, 0u, mine ? qa[2 * kp + 1][1] : 0u, 0u, b2, b3);
                                }
                            }
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty0 + 8 * s);
                        ++it;
                    }
                    if (!alive) break;
                }

                // ---------------- online softmax (row g only) ---------------
                uint32_t pa[NB];                                        // packed probabilities, A-operand order
                if (valid) {
                    const long long n_here = n_keys - (long long)pg * P;   // tokens of this page that exist
                    float mx = -INFINITY;
#pragma unroll
                    for (int j = 0; j < NB; ++j) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int tok = warp * RW + j * 8 + 2 * tq + e;
                            const float v = (tok < n_here) ? sc[j][e] * prm.scale_log2 : -INFINITY;
                            sc[j][e] = v;
                            mx = fmaxf(mx, v);
                        }
                    }
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                    const float m_new = fmaxf(m, mx);
                    const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
                    const float alpha = exp2f(m - m_ref);
                    float psum = 0.f;
#pragma unroll
                    for (int j = 0; j < NB; ++j) {
                        const float p0 = exp2f(sc[j][0] - m_ref), p1 = exp2f(sc[j][1] - m_ref);
                        psum += p0 + p1;
                        pa[j] = Mma<T>::pack(p0, p1);
                    }
                    l = l * alpha + psum;
                    m = m_new;
                    if (alpha != 1.f) {
#pragma unroll
                        for (int n = 0; n < D / 8; ++n) { o[n][0] *= alpha; o[n][1] *= alpha; }
                    }
                }

                // ---------------- O += P V ----------------------------------
                s = it % NS; ph = (it / NS) & 1u;
                if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) { alive = false; break; }
                if (valid) {
                    const uint32_t vt = smem_u32(ring + s * kTile);
                    // Rows of this warp's group past the row's last key were fetched with the group but never
                    // appended: the pool may hold anything there, and 0 x NaN would poison the sum.  Clear them
                    // in shared memory (only the group that holds a sequence's last key ever does this).  The
                    // slot's next user is a tensor copy (async proxy), hence the proxy fence behind the stores.
                    const int first_bad = (int)(n_keys - (long long)pg * P) - warp * RW;   // >= 1: the group was fetched
                    if (first_bad < RW) {
                        constexpr int kChunks = (D / 64) * 8;               // 16-byte pieces of one token row
                        for (int i = lane; i < (RW - first_bad) * kChunks; i += 32) {
                            const int row = warp * RW + first_bad + i / kChunks, c = i % kChunks;
                            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};"
                                         ::"r"(vt + (c >> 3) * (P * 128) + row * 128 + ((c & 7) << 4)), "r"(0u) : "memory");
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                    }
#pragma unroll
                    for (int ks = 0; ks < RW / 16; ++ks) {              // 16 tokens per k-step
                        const int row = warp * RW + ks * 16 + (lane & 15);   // matrices 0/2: tokens 0-7, 1/3: 8-15
#pragma unroll
                        for (int np = 0; np < D / 16; ++np) {           // two n8 blocks of head_dim per ldmatrix
                            const int chunk = np * 2 + (lane >> 4);
                            const uint32_t addr = vt + (chunk >> 3) * (P * 128) + row * 128 +
                                                  (((chunk & 7) ^ (row & 7)) << 4);
                            uint32_t b0, b1, b2, b3;
                            ldsm_x4_t(addr, b0, b1, b2, b3);
                            float c0[4] = {o[2 * np][0], o[2 * np][1], 0.f, 0.f};
                            float c1[4] = {o[2 * np + 1][0], o[2 * np + 1][1], 0.f, 0.f};
                            Mma<T>::run(c0, pa[2 * ks], 0u, pa[2 * ks + 1], 0u, b0, b1);
                            Mma<T>::run(c1, pa[2 * ks], 0u, pa[2 * ks + 1], 0u, b2, b3);
                            o[2 * np][0] = c0[0]; o[2 * np][1] = c0[1];
                            o[2 * np + 1][0] = c1[0]; o[2 * np + 1][1] = c1[1];
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * s);
                ++it;
            }
            if (!alive) break;

            // ---- merge the 8 warps' states, then write out or a partial -----
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            float* mb = merge + (piece & 1) * L::kMergeFloats;
            if (g < NREP) {
                float* dst = mb + (warp * NREP + g) * (D + 2);
                if (tq == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
                for (int n = 0; n < D / 8; ++n)
                    *reinterpret_cast<float2*>(dst + 2 + n * 8 + 2 * tq) = make_float2(o[n][0], o[n][1]);
            }
            if (!consumer_bar()) { alive = false; break; }
            for (int e = tid; e < NREP * D; e += kConsumerWarps * 32) {
                const int r = e / D, d = e - r * D;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, mb[(w * NREP + r) * (D + 2)]);
                float Lsum = 0.f, acc = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) {
                    const float* src = mb + (w * NREP + r) * (D + 2);
                    const float mw = src[0];
                    if (mw != -INFINITY) {
                        const float wgt = exp2f(mw - M);
                        Lsum += src[1] * wgt;
                        acc += src[2 + d] * wgt;
                    }
                }
                const int hq = h * NREP + r;
                if (direct) {
                    const float lse_nat = Lsum > 0.f ? (M + log2f(Lsum)) * kLn2 : -INFINITY;
                    out[((size_t)b * Hq + hq) * D + d] = gated_out<T>(Lsum > 0.f ? acc / Lsum : 0.f,
                                                                      sink_gate(prm.epi, hq, lse_nat), prm.epi.sinks != nullptr);
                    if (d == 0) prm.lse[(size_t)b * Hq + hq] = lse_nat;
                } else {
                    float* dst = prm.ws + (((size_t)u * 2 + ws_slot) * NREP + r) * (D + 2);
                    __stcg(dst + 2 + d, acc);
                    if (d == 0) { __stcg(dst, M); __stcg(dst + 1, Lsum); }
                }
            }
            t = piece_end;
        }
    }
    if (!alive) { if (lane == 0) give_up(); return; }
}

// Second kernel, one CTA per (row b, stored head h) segment.  A segment that unit boundaries cut is
// merged from the partials its pieces left in the workspace; segments inside one unit were written
// by the main kernel.  Launched with programmatic stream serialisation: its CTAs may become resident
// while the main grid is still busy and wait for it in griddepcontrol.wait.  After that it is two
// rounds of loads (the row's tile counts, then all partials at once) and a store.
constexpr int kFinishGroups = 4;                   // thread groups that split a segment's units among them

template <typename T, int D, int NREP>
__global__ void __launch_bounds__(kFinishGroups * NREP * D / 4)
decode_tma_finish_kernel(const Params prm, int G)
{
    constexpr int kVec = NREP * D / 4;                 // threads per group: one float4 of one output row each
    __shared__ float4 s_acc[kFinishGroups][kVec];
    __shared__ float2 s_ml[kFinishGroups][NREP];
    const int b = blockIdx.x / prm.Hkv, h = blockIdx.x % prm.Hkv;
    const int Hq = prm.Hkv * NREP;
    const int grp = threadIdx.x / kVec, v4 = threadIdx.x % kVec;
    const int r = v4 / (D / 4), d4 = (v4 % (D / 4)) * 4;
    T* out = reinterpret_cast<T*>(prm.out);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");   // a following kernel launched the same way may take its seats
    const int4 info = __ldcg(prm.seginfo + blockIdx.x);
    const int u_first = info.x, u_last = info.y, first_slot = info.z & 1;
    if (u_first == u_last) return;                     // inside one unit (written by the main kernel) or no tile
    // group g takes units u_first + g, u_first + g + kFinishGroups, ...: all loads of a thread are independent
    float M = -INFINITY, Lsum = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int c = u_first + grp; c <= u_last; c += kFinishGroups) {
        const float* src = prm.ws + (((size_t)c * 2 + (c == u_first ? first_slot : 0)) * NREP + r) * (D + 2);
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(src));
        const float2 x01 = __ldcg(reinterpret_cast<const float2*>(src + 2 + d4));   // rows are 8-byte aligned
        const float2 x23 = __ldcg(reinterpret_cast<const float2*>(src + 4 + d4));
        if (ml.x == -INFINITY) continue;               // an empty unit's neutral record, or a piece that saw no key: the rest of the record is not defined
        const float Mn = fmaxf(M, ml.x);
        const float a = (M == -INFINITY) ? 0.f : exp2f(M - Mn), w = exp2f(ml.x - Mn);
        Lsum = Lsum * a + ml.y * w;
        acc.x = acc.x * a + x01.x * w; acc.y = acc.y * a + x01.y * w;
        acc.z = acc.z * a + x23.x * w; acc.w = acc.w * a + x23.y * w;
        M = Mn;
    }
    s_acc[grp][v4] = acc;
    if (d4 == 0) s_ml[grp][r] = make_float2(M, Lsum);
    __syncthreads();
    if (grp == 0) {
        float Mt = -INFINITY;
#pragma unroll
        for (int g = 0; g < kFinishGroups; ++g) Mt = fmaxf(Mt, s_ml[g][r].x);
        float Lt = 0.f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int g = 0; g < kFinishGroups; ++g) {
            const float2 ml = s_ml[g][r];
            if (ml.x == -INFINITY) continue;
            const float w = exp2f(ml.x - Mt);
            const float4 x = s_acc[g][v4];
            Lt += ml.y * w;
            o.x += x.x * w; o.y += x.y * w; o.z += x.z * w; o.w += x.w * w;
        }
        const float inv = Lt > 0.f ? 1.f / Lt : 0.f;
        const int hq = h * NREP + r;
        const float lse_nat = Lt > 0.f ? (Mt + log2f(Lt)) * kLn2 : -INFINITY;
        const float gate = sink_gate(prm.epi, hq, lse_nat);
        const bool on = prm.epi.sinks != nullptr;
        T* dst = out + ((size_t)b * Hq + hq) * D + d4;
        dst[0] = gated_out<T>(o.x * inv, gate, on); dst[1] = gated_out<T>(o.y * inv, gate, on);
        dst[2] = gated_out<T>(o.z * inv, gate, on); dst[3] = gated_out<T>(o.w * inv, gate, on);
        if (d4 == 0) prm.lse[(size_t)b * Hq + hq] = lse_nat;
    }
}

// ------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

int sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v > 0 ? v : 148;
    }();
    return n;
}

constexpr size_t kCounterBytes = 16384;            // [0] unit counter (zero between calls)

size_t partial_bytes(int G, int nrep, int D) {
    return ((size_t)kPhases * G * 2 * nrep * (D + 2) * sizeof(float) + 255) / 256 * 256;
}

template <typename T, int D, int P, int NREP, typename PosT, bool SPLIT>
int launch_one(const TileMaps& maps, Params prm, int G, cudaStream_t stream)
{
    using L = Layout<D, P, NREP>;
    auto kern = decode_tma_kernel<T, D, P, NREP, PosT, SPLIT>;
    // per device and idempotent; set on every call so that the library keeps no state
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes) != cudaSuccess)
        return FPKV_ELAUNCH;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(G); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = L::kSmemBytes; cfg.stream = stream;
        cfg.attrs = attr; cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, kern, maps, prm) != cudaSuccess) return FPKV_ELAUNCH;
    }
    // the finish kernel may become resident while the main grid runs; it waits for it on the device
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(prm.B * prm.Hkv); cfg.blockDim = dim3(kFinishGroups * NREP * D / 4); cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, decode_tma_finish_kernel<T, D, NREP>, prm, G) == cudaSuccess ? FPKV_OK
                                                                                                  : FPKV_ELAUNCH;
}

template <typename T, int D, int P, typename PosT>
int launch_nrep(int nrep, const TileMaps& maps, const Params& prm, int G, cudaStream_t s)
{
    switch (nrep) {
        case 1: return launch_one<T, D, P, 1, PosT, false>(maps, prm, G, s);
        case 2: return launch_one<T, D, P, 2, PosT, false>(maps, prm, G, s);
        case 4: return launch_one<T, D, P, 4, PosT, false>(maps, prm, G, s);
        case 8: return launch_one<T, D, P, 8, PosT, false>(maps, prm, G, s);
    }
    return FPKV_ESHAPE;
}

template <typename T, typename PosT>
int launch_split(int nrep, const TileMaps& maps, const Params& prm, int G, cudaStream_t s)
{
    switch (nrep) {
        case 2: return launch_one<T, 128, 128, 2, PosT, true>(maps, prm, G, s);
        case 4: return launch_one<T, 128, 128, 4, PosT, true>(maps, prm, G, s);
    }
    return FPKV_ESHAPE;
}

template <typename T, typename PosT>
int launch_shape(int D, int nrep, bool split, const TileMaps& maps, const Params& prm, int G, cudaStream_t s)
{
    if (split) return launch_split<T, PosT>(nrep, maps, prm, G, s);
    return D == 128 ? launch_nrep<T, 128, 128, PosT>(nrep, maps, prm, G, s)
                    : launch_nrep<T, 64, 128, PosT>(nrep, maps, prm, G, s);
}

}  // namespace

bool decode_tma_supported(const PoolView& pv, int Hq)
{
    if (pv.dtype != FPKV_BF16 && pv.dtype != FPKV_F16) return false;
    if (pv.P != 128 || (pv.D != 64 && pv.D != 128)) return false;
    if (Hq % pv.H) return false;
    const int nrep = Hq / pv.H;
    if (nrep != 1 && nrep != 2 && nrep != 4 && nrep != 8) return false;
    // split layout: a half-plane row must be one 128-byte swizzle row (head_dim 128); groups of 2 or 4 query heads
    if (pv.split_hq && (pv.D != 128 || Hq != pv.split_hq || (nrep != 2 && nrep != 4))) return false;
    // TMA coordinates are 32-bit token rows within one layer's K and V planes
    if ((long long)2 * pv.H * pv.n_pages * pv.P >= (1ll << 31)) return false;
    return encode_fn() != nullptr;
}

size_t decode_tma_workspace_bytes(int Hq, int Hkv, int D)
{
    const int nrep = Hq / Hkv;
    const int G = sm_count() < kMaxGrid ? sm_count() : kMaxGrid;
    return kCounterBytes + partial_bytes(G, nrep, D) + (size_t)kMaxBatchPerLaunch * Hkv * sizeof(int4);
}

int launch_decode_tma(const PoolView& pv, int layer, void* out, float* lse, const void* q,
                      long long q_stride_b, long long q_stride_h, const int64_t* batch_idx,
                      const void* pos, int pos_type, int B, int Hq, float sm_scale,
                      void* workspace, const Epilogue& epi, int32_t* status, cudaStream_t stream, bool after_append)
{
    if (B == 0) return FPKV_OK;
    const int nrep = Hq / pv.H;
    const CUtensorMapDataType dt = pv.dtype == FPKV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    // A tensor of `rows` token rows of `halves` 64-element column groups (row pitch halves * 128 bytes), seen through a
    // box of `box_rows` rows and `box_halves` column groups, 128-byte swizzle.
    auto encode = [&](CUtensorMap* m, void* base, unsigned long long rows, int halves, int box_rows, int box_halves) {
        const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)halves};
        const cuuint64_t strides[2] = {(cuuint64_t)halves * 128, 128};
        const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_halves};
        const cuuint32_t estr[3] = {1, 1, 1};
        return encode_fn()(m, dt, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    const unsigned long long R = (unsigned long long)pv.n_pages * pv.P;
    const int RWh = pv.P / kConsumerWarps;             // rows of one consumer warp
    TileMaps maps;
    memset(&maps, 0, sizeof(maps));
    bool ok;
    if (!pv.split_hq) {
        // one layer's K and V planes as one tensor: a page box, and a box of one warp's rows of one column group
        ok = encode(&maps.kv, pv.plane(layer, 0, 0), 2ull * pv.H * R, pv.D / 64, pv.P, pv.D / 64) &&
             encode(&maps.kv_rows, pv.plane(layer, 0, 0), 2ull * pv.H * R, pv.D / 64, RWh, 1);
    } else {
        ok = encode(&maps.kt, pv.kt_plane(layer, 0), (unsigned long long)pv.H * R, 1, pv.P, 1) &&
             encode(&maps.kt_rows, pv.kt_plane(layer, 0), (unsigned long long)pv.H * R, 1, RWh, 1) &&
             encode(&maps.khw, pv.khw_plane(layer, 0), (unsigned long long)pv.split_hq * R, 1, pv.P, 1) &&
             encode(&maps.khw_rows, pv.khw_plane(layer, 0), (unsigned long long)pv.split_hq * R, 1, RWh, 1) &&
             encode(&maps.v, pv.v_plane(layer, 0), (unsigned long long)pv.H * R, 2, pv.P, 2) &&
             encode(&maps.v_rows, pv.v_plane(layer, 0), (unsigned long long)pv.H * R, 2, RWh, 1);
    }
    if (!ok) return FPKV_ELAUNCH;

    const int G = sm_count() < kMaxGrid ? sm_count() : kMaxGrid;
    const size_t esz = 2;
    for (int b0 = 0; b0 < B; b0 += kMaxBatchPerLaunch) {
        Params prm;
        prm.page_table = pv.page_table; prm.p2l = pv.p2l;
        prm.batch_idx = batch_idx + b0;
        prm.pos = (const char*)pos + (size_t)b0 * (pos_type == FPKV_I32 ? 4 : 8);
        prm.q = (const char*)q + (size_t)b0 * q_stride_b * esz;
        prm.out = (char*)out + (size_t)b0 * Hq * pv.D * esz;
        prm.lse = lse + (size_t)b0 * Hq;
        prm.counters = (int*)workspace;
        prm.ws = (float*)((char*)workspace + kCounterBytes);
        prm.seginfo = (int4*)((char*)workspace + kCounterBytes + partial_bytes(G, nrep, pv.D));
        prm.status = status;
        prm.q_stride_b = q_stride_b; prm.q_stride_h = q_stride_h;
        prm.B = (B - b0 < kMaxBatchPerLaunch) ? B - b0 : kMaxBatchPerLaunch;
        prm.Hkv = pv.H; prm.n_pages = pv.n_pages; prm.max_batch = pv.max_batch;
        prm.after_append = (after_append && b0 == 0) ? 1 : 0;
        prm.rows_per_plane = pv.n_pages * pv.P;
        prm.scale_log2 = sm_scale * kLog2e;
        prm.epi = epi;
        int rc;
        if (pv.dtype == FPKV_BF16)
            rc = pos_type == FPKV_I32 ? launch_shape<__nv_bfloat16, int32_t>(pv.D, nrep, pv.split_hq != 0, maps, prm, G, stream)
                                      : launch_shape<__nv_bfloat16, int64_t>(pv.D, nrep, pv.split_hq != 0, maps, prm, G, stream);
        else
            rc = pos_type == FPKV_I32 ? launch_shape<__half, int32_t>(pv.D, nrep, pv.split_hq != 0, maps, prm, G, stream)
                                      : launch_shape<__half, int64_t>(pv.D, nrep, pv.split_hq != 0, maps, prm, G, stream);
        if (rc != FPKV_OK) return rc;
    }
    return FPKV_OK;
}

}  // namespace fpkv
