// Paged decode attention for 16-bit pools on sm_100a: TMA-staged KV pages,
// mbarrier ring, tensor-core dot products, warp-shuffle online softmax.
//
// The kernel is bound by HBM reads of K and V.  Everything is arranged so that
// every SM streams an equal share of the batch's pages at full rate:
//
//  * Work unit ("tile") = one page of one stored head of one row: a K tile and
//    a V tile of page_size x head_dim elements, each contiguous in the pool
//    (32 KiB at page 128, head_dim 128, 16-bit).  Tiles are numbered row-major
//    over (row b, stored head h, logical page) and the flat range is cut into
//    gridDim.x equal contiguous shares, one persistent CTA per SM.  A share can
//    start and end in the middle of a (b, h) segment; such a piece leaves an
//    unnormalised partial (m, l, acc) in the workspace and takes a ticket; the
//    CTA that takes a segment's last ticket merges the pieces and writes the
//    result (nobody waits).  Segments that lie inside one share are normalised
//    and written directly.  The ticket words must be zero on entry and are
//    left zero, so the workspace is zero-filled once, not per call.
//  * One producer warp walks the share, looks page ids up in the page table
//    (32 tiles per coalesced read, two lookups ahead of use) and issues one
//    TMA tensor copy per K or V tile into a ring of shared-memory slots; the
//    copy lands with the 128-byte swizzle so that ldmatrix reads are free of
//    bank conflicts.  Every copy targets this CTA's own shared memory only.
//  * Eight consumer warps each own page_size/8 token rows of every tile.  The
//    GQA group's query heads are the M rows of mma.sync.m16n8k16 (zero padded
//    to 16), so all query heads of a stored head consume the one staged tile.
//    Scores stay in registers; the row maximum is a two-step quad shuffle;
//    probabilities are repacked in place as the A operand of the P.V product.
//  * Every mbarrier wait is bounded: when the limit is hit the CTA raises
//    FPKV_STATUS_TIMEOUT, all roles leave their loops, the producer drains the
//    copies it has in flight (again bounded) and the kernel returns.
//
// Semantics: the reference's decode mask + FlexAttention call
// (falcon_perception/paged_inference.py:783-826,
//  falcon_perception/paged_attention.py:234-333, falcon_perception/model.py:156-162).

#include <cuda.h>          // CUtensorMap (types only; the encoder is fetched at run time)
#include "common.cuh"

namespace fpkv {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxBatchPerLaunch = 1024;
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
__device__ __forceinline__ void consumer_bar() {           // the 8 consumer warps only
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
}

// ------------------------------------------------------------ shared layout
template <int D, int P, int NREP>
struct Layout {
    static constexpr int kTileBytes = P * D * 2;                       // one K or V tile
    static constexpr int kMergeFloats = kConsumerWarps * NREP * (D + 2);
    static constexpr int kFixedBytes = 2 * kMergeFloats * 4             // double-buffered merge area
                                       + 2 * 16 * 8                     // mbarriers (<= 16 slots)
                                       + 16 * 4 + 64;                   // slot flags, abort flag, pad
    static constexpr int kBatchBytes = (kMaxBatchPerLaunch + 1) * 4 + kMaxBatchPerLaunch * 8;
    static constexpr int kSlotsFit = (kSmemBudget - 1024 - kFixedBytes - kBatchBytes) / kTileBytes;
    static constexpr int kSlots = (kSlotsFit > 12 ? 12 : kSlotsFit) & ~1;   // K and V alternate: even
    static constexpr int kSmemBytes = 1024 + kSlots * kTileBytes + kFixedBytes + kBatchBytes;
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
    float* ws;                 // partials [gridDim.x][2][NREP][D+2]
    int* tickets;              // [gridDim.x] arrival counts of cut segments, indexed by first owner; zero between calls
    int32_t* status;
    long long q_stride_b, q_stride_h;
    int B, Hkv, n_pages, max_batch;
    int row_base_k;            // first pool row (in tokens) of plane (layer, K, head 0), relative to the map
    int rows_per_plane;        // n_pages * P
    float scale_log2;
};

// CTA share [r0, r1) of the flat tile range.
__device__ __forceinline__ long long share_begin(long long T, int c, int G) { return T * c / G; }

// ------------------------------------------------------------------ kernel
template <typename T, int D, int P, int NREP, typename PosT>
__global__ void __launch_bounds__(kThreads, 1)
decode_tma_kernel(const __grid_constant__ CUtensorMap tmap, const Params prm)
{
    using L = Layout<D, P, NREP>;
    constexpr int NS = L::kSlots;
    constexpr int kTile = L::kTileBytes;
    constexpr int RW = P / kConsumerWarps;            // token rows per consumer warp (16 at P=128)
    constexpr int NB = RW / 8;                        // n8 score blocks per warp
    static_assert(RW % 16 == 0, "page_size must be a multiple of 128 rows / 8 warps * 16");
    static_assert(NREP <= 8, "query heads per stored head must fit the lower 8 MMA rows");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    float* merge = reinterpret_cast<float*>(ring + NS * kTile);               // [2][W][NREP][D+2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(merge + 2 * L::kMergeFloats); // full[NS], empty[NS]
    int* slot_valid = reinterpret_cast<int*>(bars + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot_valid + 16);
    int* last_flag = const_cast<int*>(reinterpret_cast<volatile int*>(abort_flag) + 1);
    int* cum = const_cast<int*>(reinterpret_cast<volatile int*>(abort_flag) + 4);   // [B+1] tiles before row b
    long long* slot_of = reinterpret_cast<long long*>(cum + kMaxBatchPerLaunch + 1 + ((kMaxBatchPerLaunch + 1) & 1));

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int B = prm.B, Hkv = prm.Hkv;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + NS);

    // ---- prologue: barriers, per-row page counts, exclusive scan -----------
    if (tid == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, kConsumerWarps); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int b = tid; b < B; b += kThreads) {
        const long long slot = prm.batch_idx[b];
        const long long p = load_pos<PosT>(prm.pos, b);
        int npg = 0;
        if (slot < 0 || slot >= prm.max_batch) raise_status(prm.status, FPKV_STATUS_BAD_SLOT);
        else if (p < 0 || p / P >= prm.n_pages) raise_status(prm.status, FPKV_STATUS_BAD_POS);
        else npg = (int)(p / P) + 1;
        slot_of[b] = (npg > 0) ? slot : 0;
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
        if (lane == 0) cum[0] = 0;
    }
    __syncthreads();
    const long long Ttot = cum[B];
    const int G = gridDim.x, cta = blockIdx.x;
    // rows without any tile (bad slot or position): out = 0, lse = -inf, one CTA per such row
    {
        const int Hq = Hkv * NREP;
        T* out0 = reinterpret_cast<T*>(prm.out);
        for (int b = cta; b < B; b += G) {
            if (cum[b + 1] != cum[b]) continue;
            for (int e = tid; e < Hq * D; e += kThreads) out0[(size_t)b * Hq * D + e] = ElemTraits<T>::from_float(0.f);
            for (int e = tid; e < Hq; e += kThreads) prm.lse[(size_t)b * Hq + e] = -INFINITY;
        }
    }
    const int r0 = (int)share_begin(Ttot, cta, G), r1 = (int)share_begin(Ttot, cta + 1, G);

    // Row that owns flat tile t (cum[b] <= t < cum[b+1]); B >= 1 and t < Ttot.
    auto row_of = [&](int t) {
        int lo = 0, hi = B;                            // invariant: cum[lo] <= t < cum[hi]
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (cum[mid] <= t) lo = mid; else hi = mid; }
        return lo;
    };

    if (warp == kConsumerWarps) {
        // =========================== producer warp ==========================
        // Lane j of lookup round c resolves tile r0 + 32*c + j: pool row of its
        // K tile, or -1 when the page is unmapped.  Page ids are read one round
        // ahead of the inverse-table check, which is read one round ahead of use.
        auto tile_page = [&](int t, long long& pt_index, int& h) -> bool {   // false: t outside the share
            if (t >= r1) return false;
            const int b = row_of(t);
            const int npg = (cum[b + 1] - cum[b]) / Hkv;
            const int rel = t - cum[b];
            h = rel / npg;
            pt_index = slot_of[b] * prm.n_pages + (rel - h * npg);
            return true;
        };
        auto load_page = [&](int t, int& h, long long& slot_row) -> long long {
            long long idx;
            if (!tile_page(t, idx, h)) { slot_row = 0; return -1; }
            slot_row = idx / prm.n_pages * prm.n_pages;
            return prm.page_table[idx];
        };
        int h_c = 0, h_n = 0, h_nn = 0;
        long long sr_c, sr_n, sr_nn;
        long long pg_c = load_page(r0 + lane, h_c, sr_c);
        long long pg_n = load_page(r0 + 32 + lane, h_n, sr_n);
        auto check = [&](long long pg, long long slot_row) -> long long {   // -> inverse-table entry (or -1)
            if (pg < 0) return -1;
            if (pg >= prm.n_pages) { raise_status(prm.status, FPKV_STATUS_BAD_PAGE); return -1; }
            return prm.p2l[slot_row + pg];
        };
        long long inv_c = check(pg_c, sr_c);
        uint32_t it = 0;                               // ring position (one per K or V tile)
        bool ok = true;
        for (int base = r0; base < r1 && ok; base += 32) {
            const long long inv_n = check(pg_n, sr_n);
            const long long pg_nn = load_page(base + 64 + lane, h_nn, sr_nn);
            const int n_here = min(32, r1 - base);
            const int row_k = (inv_c >= 0) ? prm.row_base_k + h_c * prm.rows_per_plane + (int)pg_c * P : -1;
            for (int j = 0; j < n_here; ++j) {
                const int rk = __shfl_sync(0xffffffffu, row_k, j);
                if (lane == 0) {
#pragma unroll
                    for (int kv = 0; kv < 2; ++kv, ++it) {
                        const uint32_t s = it % NS, ph = (it / NS) & 1u;
                        if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag)) { ok = false; break; }
                        slot_valid[s] = rk >= 0;
                        if (rk >= 0) {
                            mbar_arrive_expect_tx(full0 + 8 * s, kTile);
                            tma_load_3d(smem_u32(ring + s * kTile), &tmap, 0,
                                        rk + kv * Hkv * prm.rows_per_plane, 0, full0 + 8 * s);
                        } else {
                            mbar_arrive(full0 + 8 * s);
                        }
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
            }
            pg_c = pg_n; sr_c = sr_n; h_c = h_n; inv_c = inv_n;
            pg_n = pg_nn; sr_n = sr_nn; h_n = h_nn;
        }
        if (lane == 0) {
            if (!ok) {
                if (!*abort_flag) raise_status(prm.status, FPKV_STATUS_TIMEOUT);
                *abort_flag = 1;
                // drain: every copy issued has an expect_tx on its full barrier; wait for each once
                const uint32_t first = it > (uint32_t)NS ? it - NS : 0;
                for (uint32_t i = first; i < it; ++i) {
                    const uint32_t s = i % NS, ph = (i / NS) & 1u;
                    for (uint32_t k = 0; k < kSpinLimit && !mbar_try_wait(full0 + 8 * s, ph); ++k) {}
                }
            }
        }
        return;
    }

    // ============================ consumer warps ============================
    const int g = lane >> 2, tq = lane & 3;            // MMA row group / thread-in-quad
    const T* qbase = reinterpret_cast<const T*>(prm.q);
    T* out = reinterpret_cast<T*>(prm.out);
    uint32_t it = 0;
    int piece = 0;
    bool alive = true;

    for (int t = r0; t < r1; ++piece) {
        // ---- piece = part of one (b, h) segment inside this share ----------
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
            // ---------------- S = Q K^T for this warp's RW tokens -----------
            uint32_t s = it % NS, ph = (it / NS) & 1u;
            if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) { alive = false; break; }
            const bool valid = slot_valid[s] != 0;
            float sc[NB][4];
#pragma unroll
            for (int j = 0; j < NB; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f; }
            if (valid) {
                const uint32_t kt = smem_u32(ring + s * kTile);
#pragma unroll
                for (int j = 0; j < NB; ++j) {
                    const int row = warp * RW + j * 8 + (lane & 7);
#pragma unroll
                    for (int kp = 0; kp < D / 32; ++kp) {              // two k-steps per ldmatrix.x4
                        const int chunk = kp * 4 + (lane >> 3);        // 16-byte column chunk 0..D/8-1
                        const uint32_t addr = kt + (chunk >> 3) * (P * 128) + row * 128 +
                                              (((chunk & 7) ^ (row & 7)) << 4);
                        uint32_t b0, b1, b2, b3;
                        ldsm_x4(addr, b0, b1, b2, b3);
                        Mma<T>::run(sc[j], qa[2 * kp][0], 0u, qa[2 * kp][1], 0u, b0, b1);
                        Mma<T>::run(sc[j], qa[2 * kp + 1][0], 0u, qa[2 * kp + 1][1], 0u, b2, b3);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
            ++it;

            // ---------------- online softmax (row g only) -------------------
            uint32_t pa[NB];                                            // packed probabilities, A-operand order
            if (valid) {
                const long long n_here = n_keys - (long long)pg * P;    // tokens of this page that exist
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

            // ---------------- O += P V --------------------------------------
            s = it % NS; ph = (it / NS) & 1u;
            if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) { alive = false; break; }
            if (valid) {
                const uint32_t vt = smem_u32(ring + s * kTile);
#pragma unroll
                for (int ks = 0; ks < RW / 16; ++ks) {                  // 16 tokens per k-step
                    const int row = warp * RW + ks * 16 + (lane & 15);  // matrices 0/2: tokens 0-7, 1/3: 8-15
#pragma unroll
                    for (int np = 0; np < D / 16; ++np) {               // two n8 blocks of head_dim per ldmatrix
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
        // A warp whose wait ran out still joins the barrier below, so that no
        // consumer is left waiting for it; all of them then leave together.
        if (!alive && lane == 0) {
            if (!*abort_flag) raise_status(prm.status, FPKV_STATUS_TIMEOUT);
            *abort_flag = 1;
        }

        // ---- merge the 8 warps' states, then write out or a partial ---------
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        float* mb = merge + (piece & 1) * L::kMergeFloats;
        if (alive && g < NREP) {
            float* dst = mb + (warp * NREP + g) * (D + 2);
            if (tq == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
            for (int n = 0; n < D / 8; ++n)
                *reinterpret_cast<float2*>(dst + 2 + n * 8 + 2 * tq) = make_float2(o[n][0], o[n][1]);
        }
        consumer_bar();
        if (*abort_flag) break;
        const int Hq = Hkv * NREP;
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
                out[((size_t)b * Hq + hq) * D + d] = ElemTraits<T>::from_float(Lsum > 0.f ? acc / Lsum : 0.f);
                if (d == 0) prm.lse[(size_t)b * Hq + hq] = Lsum > 0.f ? (M + log2f(Lsum)) * kLn2 : -INFINITY;
            } else {
                float* dst = prm.ws + (((size_t)cta * 2 + ws_slot) * NREP + r) * (D + 2);
                __stcg(dst + 2 + d, acc);
                if (d == 0) { __stcg(dst, M); __stcg(dst + 1, Lsum); }
            }
        }
        if (!direct) {
            // Segment cut by share boundaries: publish the partial, take a ticket; the last of the
            // segment's pieces to arrive merges them all.  The ticket word belongs to the share that
            // owns the segment's first tile and goes back to zero for the next call.
            const int c_first = (int)(((long long)(seg0 + 1) * G - 1) / Ttot);
            const int c_last = (int)(((long long)seg1 * G - 1) / Ttot);
            __threadfence();
            consumer_bar();
            if (tid == 0) {
                int expected = 0;
                for (int c = c_first; c <= c_last; ++c)
                    expected += share_begin(Ttot, c, G) != share_begin(Ttot, c + 1, G);
                const int prev = atomicAdd(prm.tickets + c_first, 1);
                *last_flag = (prev + 1 == expected);
                if (prev + 1 == expected) prm.tickets[c_first] = 0;
            }
            consumer_bar();
            if (*last_flag) {
                __threadfence();
                for (int e = tid; e < NREP * D; e += kConsumerWarps * 32) {
                    const int r = e / D, d = e - r * D;
                    float M = -INFINITY;
                    for (int c = c_first; c <= c_last; ++c) {
                        if (share_begin(Ttot, c, G) == share_begin(Ttot, c + 1, G)) continue;   // empty share
                        const int slot = (seg0 <= share_begin(Ttot, c, G)) ? 0 : 1;
                        M = fmaxf(M, __ldcg(prm.ws + (((size_t)c * 2 + slot) * NREP + r) * (D + 2)));
                    }
                    float Lsum = 0.f, acc = 0.f;
                    for (int c = c_first; c <= c_last; ++c) {
                        if (share_begin(Ttot, c, G) == share_begin(Ttot, c + 1, G)) continue;
                        const int slot = (seg0 <= share_begin(Ttot, c, G)) ? 0 : 1;
                        const float* src = prm.ws + (((size_t)c * 2 + slot) * NREP + r) * (D + 2);
                        const float mc = __ldcg(src);
                        if (mc != -INFINITY) {
                            const float wgt = exp2f(mc - M);
                            Lsum += __ldcg(src + 1) * wgt;
                            acc += __ldcg(src + 2 + d) * wgt;
                        }
                    }
                    const int hq = h * NREP + r;
                    out[((size_t)b * Hq + hq) * D + d] = ElemTraits<T>::from_float(Lsum > 0.f ? acc / Lsum : 0.f);
                    if (d == 0) prm.lse[(size_t)b * Hq + hq] = Lsum > 0.f ? (M + log2f(Lsum)) * kLn2 : -INFINITY;
                }
            }
        }
        t = piece_end;
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

constexpr size_t kTicketBytes = 1024;              // one int per share (<= 256 SMs)

template <typename T, int D, int P, int NREP, typename PosT>
int launch_one(const CUtensorMap& map, Params prm, int G, cudaStream_t stream)
{
    using L = Layout<D, P, NREP>;
    auto kern = decode_tma_kernel<T, D, P, NREP, PosT>;
    // per device and idempotent; set on every call so that the library keeps no state
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes) != cudaSuccess)
        return FPKV_ELAUNCH;
    kern<<<G, kThreads, L::kSmemBytes, stream>>>(map, prm);
    return cudaGetLastError() == cudaSuccess ? FPKV_OK : FPKV_ELAUNCH;
}

template <typename T, int D, int P, typename PosT>
int launch_nrep(int nrep, const CUtensorMap& map, const Params& prm, int G, cudaStream_t s)
{
    switch (nrep) {
        case 1: return launch_one<T, D, P, 1, PosT>(map, prm, G, s);
        case 2: return launch_one<T, D, P, 2, PosT>(map, prm, G, s);
        case 4: return launch_one<T, D, P, 4, PosT>(map, prm, G, s);
        case 8: return launch_one<T, D, P, 8, PosT>(map, prm, G, s);
    }
    return FPKV_ESHAPE;
}

template <typename T, typename PosT>
int launch_shape(int D, int nrep, const CUtensorMap& map, const Params& prm, int G, cudaStream_t s)
{
    return D == 128 ? launch_nrep<T, 128, 128, PosT>(nrep, map, prm, G, s)
                    : launch_nrep<T, 64, 128, PosT>(nrep, map, prm, G, s);
}

}  // namespace

bool decode_tma_supported(const PoolView& pv, int Hq)
{
    if (pv.dtype != FPKV_BF16 && pv.dtype != FPKV_F16) return false;
    if (pv.P != 128 || (pv.D != 64 && pv.D != 128)) return false;
    if (Hq % pv.H) return false;
    const int nrep = Hq / pv.H;
    if (nrep != 1 && nrep != 2 && nrep != 4 && nrep != 8) return false;
    // TMA coordinates are 32-bit token rows within one layer's K and V planes
    if ((long long)2 * pv.H * pv.n_pages * pv.P >= (1ll << 31)) return false;
    return encode_fn() != nullptr;
}

size_t decode_tma_workspace_bytes(int Hq, int Hkv, int D)
{
    const int nrep = Hq / Hkv;
    return kTicketBytes + (size_t)sm_count() * 2 * nrep * (D + 2) * sizeof(float);
}

int launch_decode_tma(const PoolView& pv, int layer, void* out, float* lse, const void* q,
                      long long q_stride_b, long long q_stride_h, const int64_t* batch_idx,
                      const void* pos, int pos_type, int B, int Hq, float sm_scale,
                      void* workspace, int32_t* status, cudaStream_t stream)
{
    if (B == 0) return FPKV_OK;
    const int nrep = Hq / pv.H;
    // One layer's K and V planes as a 3-D tensor: (64 elements = 128 bytes, token rows, head_dim/64).
    CUtensorMap map;
    const cuuint64_t dims[3] = {64, (cuuint64_t)2 * pv.H * pv.n_pages * pv.P, (cuuint64_t)(pv.D / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)pv.D * 2, 128};
    const cuuint32_t box[3] = {64, (cuuint32_t)pv.P, (cuuint32_t)(pv.D / 64)};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapDataType dt = pv.dtype == FPKV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (encode_fn()(&map, dt, 3, pv.plane(layer, 0, 0), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return FPKV_ELAUNCH;

    const int G = sm_count() < 256 ? sm_count() : 256;
    const size_t esz = 2;
    for (int b0 = 0; b0 < B; b0 += kMaxBatchPerLaunch) {
        Params prm;
        prm.page_table = pv.page_table; prm.p2l = pv.p2l;
        prm.batch_idx = batch_idx + b0;
        prm.pos = (const char*)pos + (size_t)b0 * (pos_type == FPKV_I32 ? 4 : 8);
        prm.q = (const char*)q + (size_t)b0 * q_stride_b * esz;
        prm.out = (char*)out + (size_t)b0 * Hq * pv.D * esz;
        prm.lse = lse + (size_t)b0 * Hq;
        prm.tickets = (int*)workspace;
        prm.ws = (float*)((char*)workspace + kTicketBytes);
        prm.status = status;
        prm.q_stride_b = q_stride_b; prm.q_stride_h = q_stride_h;
        prm.B = (B - b0 < kMaxBatchPerLaunch) ? B - b0 : kMaxBatchPerLaunch;
        prm.Hkv = pv.H; prm.n_pages = pv.n_pages; prm.max_batch = pv.max_batch;
        prm.row_base_k = 0; prm.rows_per_plane = pv.n_pages * pv.P;
        prm.scale_log2 = sm_scale * kLog2e;
        int rc;
        if (pv.dtype == FPKV_BF16)
            rc = pos_type == FPKV_I32 ? launch_shape<__nv_bfloat16, int32_t>(pv.D, nrep, map, prm, G, stream)
                                      : launch_shape<__nv_bfloat16, int64_t>(pv.D, nrep, map, prm, G, stream);
        else
            rc = pos_type == FPKV_I32 ? launch_shape<__half, int32_t>(pv.D, nrep, map, prm, G, stream)
                                      : launch_shape<__half, int64_t>(pv.D, nrep, map, prm, G, stream);
        if (rc != FPKV_OK) return rc;
    }
    return FPKV_OK;
}

}  // namespace fpkv
