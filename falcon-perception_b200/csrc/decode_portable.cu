// Portable paged decode attention (CUDA cores): any pool dtype (fp32, bf16,
// fp16), head_dim 64 or 128, any page size.  It is the path for shapes the
// TMA + tensor-core kernel does not take (fp32 pools, small pages, wide GQA
// groups) and the on-device cross-check for that kernel; it is not tuned.
//
// Grid (B * Hq, S): CTA (row, split) walks the split's share of the row's
// pages.  Each warp keeps an online-softmax state over the tokens it visits;
// a lane owns head_dim/32 consecutive elements of q, of the K row and of the
// output accumulator, so a token costs one coalesced K row read, a 5-step
// shuffle reduction and one coalesced V row read.  Warps merge through shared
// memory and the CTA writes one partial (m, l, acc[head_dim]) per split; a
// second kernel merges the splits.
//
// The same kernel serves packed prefill rows for shapes the tensor-core prefill
// kernel does not take: a row is then a packed token, its number of visible
// keys comes from the caller's extent array instead of input_pos + 1, and with
// one split per row the CTA writes the normalised result itself.
//
// Visible key set of row b (slot s = batch_idx[b], p = input_pos[b]): logical
// positions 0..p whose page id PT[s, j / P] is mapped and maps back
// (P2L[s, page] >= 0) -- the reference's decode mask after conversion to
// physical pages (falcon_perception/paged_inference.py:797-826,
// falcon_perception/paged_attention.py:267-333).

#include "common.cuh"

namespace fpkv {

constexpr int kPortableWarps = 4;
constexpr int kPortableMaxSplits = 32;

__host__ __device__ inline int portable_splits(int B, int Hq) {
    int s = (4 * 148) / (B * Hq > 0 ? B * Hq : 1);
    if (s < 1) s = 1;
    if (s > kPortableMaxSplits) s = kPortableMaxSplits;
    return s;
}

// Where row (b, hq) of the result goes: element strides of out and lse over rows and heads.
struct OutLayout { long long out_row, out_head, lse_row, lse_head; };
// Split pool layout (common.cuh): first K halves per KV head, second K halves per query head, V per KV head.
// kt == nullptr: the uniform layout.
struct SplitPtrs { const char* kt; const char* khw; const char* v; size_t half_plane_bytes; };
static inline SplitPtrs split_ptrs(const PoolView& pv, int layer) {
    if (!pv.split_hq) return SplitPtrs{nullptr, nullptr, nullptr, 0};
    return SplitPtrs{pv.kt_plane(layer, 0), pv.khw_plane(layer, 0), pv.v_plane(layer, 0), pv.half_plane_bytes()};
}

template <typename T, int D, typename PosT, bool DIRECT>
__global__ void __launch_bounds__(kPortableWarps * 32)
decode_portable_kernel(const char* __restrict__ pool_layer, size_t plane_bytes, int H,
                       const int64_t* __restrict__ page_table, const int64_t* __restrict__ p2l,
                       int n_pages, int max_batch, int P,
                       const T* __restrict__ q, long long q_stride_b, long long q_stride_h,
                       const int64_t* __restrict__ batch_idx, const PosT* __restrict__ pos,
                       const int32_t* __restrict__ extent,
                       int Hq, float scale_log2, float* __restrict__ ws, T* __restrict__ out, float* __restrict__ lse,
                       OutLayout lay, Epilogue epi, int32_t* status, SplitPtrs sp)
{
    constexpr int E = D / 32;                     // elements per lane
    const int row = blockIdx.x;                   // b * Hq + hq
    const int b = row / Hq, hq = row % Hq;
    const int S = gridDim.y, split = blockIdx.y;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int n_rep = Hq / H;
    const int h = hq / n_rep;

    __shared__ float sm_m[kPortableWarps], sm_l[kPortableWarps];
    __shared__ float sm_acc[kPortableWarps][D];

    const long long slot = batch_idx[b];
    // visible keys: 0..pos for a decode row, 0..extent-1 for a packed prefill token (0 for pads)
    const long long want = extent != nullptr ? (slot > 0 ? (long long)extent[b] : 0) : (long long)pos[b] + 1;
    int n_pg = 0;
    long long n_keys = 0;
    if (slot < 0 || slot >= max_batch) {
        if (threadIdx.x == 0 && split == 0) raise_status(status, FPKV_STATUS_BAD_SLOT);
    } else if (want < (extent != nullptr ? 0 : 1) || (want + P - 1) / P > n_pages) {
        if (threadIdx.x == 0 && split == 0) raise_status(status, FPKV_STATUS_BAD_POS);
    } else {
        n_keys = want;
        n_pg = (int)((n_keys + P - 1) / P);
    }
    const int pg0 = (int)((long long)n_pg * split / S);
    const int pg1 = (int)((long long)n_pg * (split + 1) / S);

    float qv[E];
    {
        const T* qp = q + b * q_stride_b + hq * q_stride_h + lane * E;
#pragma unroll
        for (int e = 0; e < E; ++e) qv[e] = ElemTraits<T>::to_float(qp[e]) * scale_log2;
    }
    float m = -INFINITY, l = 0.f, acc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = 0.f;

    const T* Kp = reinterpret_cast<const T*>(pool_layer + (size_t)h * plane_bytes);
    const T* Vp = reinterpret_cast<const T*>(pool_layer + ((size_t)H + h) * plane_bytes);
    int k_row = D;                                // elements between consecutive tokens in the K array this lane reads
    if (sp.kt != nullptr) {                       // a lane's E elements lie in one half of the head
        k_row = D / 2;
        Kp = lane * E < D / 2 ? reinterpret_cast<const T*>(sp.kt + (size_t)h * sp.half_plane_bytes)
                              : reinterpret_cast<const T*>(sp.khw + (size_t)hq * sp.half_plane_bytes) - D / 2;
        Vp = reinterpret_cast<const T*>(sp.v + (size_t)h * plane_bytes);
    }

    for (int pg = pg0; pg < pg1; ++pg) {
        const long long page = page_table[slot * n_pages + pg];
        if (page < 0) continue;
        if (page >= n_pages) { if (threadIdx.x == 0) raise_status(status, FPKV_STATUS_BAD_PAGE); continue; }
        if (p2l[slot * n_pages + page] < 0) continue;
        long long n_here = n_keys - (long long)pg * P;
        if (n_here > P) n_here = P;
        for (int t = warp; t < n_here; t += kPortableWarps) {
            const size_t off = ((size_t)page * P + t) * D + lane * E;
            const size_t koff = ((size_t)page * P + t) * k_row + lane * E;
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < E; ++e) s += qv[e] * ElemTraits<T>::to_float(Kp[koff + e]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            const float m_new = fmaxf(m, s);
            const float alpha = exp2f(m - m_new);          // m = -inf -> 0
            const float pr = exp2f(s - m_new);
            l = l * alpha + pr;
#pragma unroll
            for (int e = 0; e < E; ++e) acc[e] = acc[e] * alpha + pr * ElemTraits<T>::to_float(Vp[off + e]);
            m = m_new;
        }
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int e = 0; e < E; ++e) sm_acc[warp][lane * E + e] = acc[e];
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kPortableWarps; ++w) M = fmaxf(M, sm_m[w]);
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < kPortableWarps; ++w)
        if (sm_m[w] != -INFINITY) L += sm_l[w] * exp2f(sm_m[w] - M);
    float* dst = DIRECT ? nullptr : ws + ((size_t)row * S + split) * (D + 2);
    const float lse_nat = L > 0.f ? (M + log2f(L)) * kLn2 : -INFINITY;
    const float gate = DIRECT ? sink_gate(epi, hq, lse_nat) : 1.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kPortableWarps; ++w)
            if (sm_m[w] != -INFINITY) o += sm_acc[w][d] * exp2f(sm_m[w] - M);
        if (DIRECT) out[b * lay.out_row + hq * lay.out_head + d] = gated_out<T>(L > 0.f ? o / L : 0.f, gate, epi.sinks != nullptr);
        else dst[2 + d] = o;
    }
    if (threadIdx.x == 0) {
        if (DIRECT) lse[b * lay.lse_row + hq * lay.lse_head] = lse_nat;
        else { dst[0] = M; dst[1] = L; }
    }
}

// Merge S partials of each (b, hq) row: out = sum_s acc_s 2^(m_s - M) / L.
template <typename T, int D>
__global__ void __launch_bounds__(D)
decode_portable_merge_kernel(const float* __restrict__ ws, int S, T* __restrict__ out, float* __restrict__ lse,
                             int Hq, Epilogue epi)
{
    const int row = blockIdx.x, d = threadIdx.x;
    const float* src = ws + (size_t)row * S * (D + 2);
    float M = -INFINITY;
    for (int s = 0; s < S; ++s) M = fmaxf(M, src[s * (D + 2)]);
    float L = 0.f, o = 0.f;
    for (int s = 0; s < S; ++s) {
        const float ms = src[s * (D + 2)];
        if (ms == -INFINITY) continue;
        const float w = exp2f(ms - M);
        L += src[s * (D + 2) + 1] * w;
        o += src[s * (D + 2) + 2 + d] * w;
    }
    const float lse_nat = L > 0.f ? (M + log2f(L)) * kLn2 : -INFINITY;
    out[(size_t)row * D + d] = gated_out<T>(L > 0.f ? o / L : 0.f, sink_gate(epi, row % Hq, lse_nat), epi.sinks != nullptr);
    if (d == 0) lse[row] = lse_nat;
}

size_t decode_portable_workspace_bytes(int B, int Hq, int D) {
    return (size_t)B * Hq * portable_splits(B, Hq) * (D + 2) * sizeof(float);
}

template <typename T, int D, typename PosT>
static int launch_typed(const PoolView& pv, int layer, void* out, float* lse, const void* q,
                        long long q_stride_b, long long q_stride_h, const int64_t* batch_idx,
                        const void* pos, int B, int Hq, float sm_scale, void* workspace,
                        const Epilogue& epi, int32_t* status, cudaStream_t stream)
{
    const int S = portable_splits(B, Hq);
    dim3 grid(B * Hq, S);
    decode_portable_kernel<T, D, PosT, false><<<grid, kPortableWarps * 32, 0, stream>>>(
        pv.plane(layer, 0, 0), pv.plane_bytes(), pv.H, pv.page_table, pv.p2l, pv.n_pages, pv.max_batch, pv.P,
        (const T*)q, q_stride_b, q_stride_h, batch_idx, (const PosT*)pos, nullptr, Hq, sm_scale * kLog2e,
        (float*)workspace, nullptr, nullptr, OutLayout{0, 0, 0, 0}, Epilogue{nullptr, 0, 0}, status, split_ptrs(pv, layer));
    if (cudaGetLastError() != cudaSuccess) return FPKV_ELAUNCH;
    decode_portable_merge_kernel<T, D><<<B * Hq, D, 0, stream>>>((const float*)workspace, S, (T*)out, lse, Hq, epi);
    return cudaGetLastError() == cudaSuccess ? FPKV_OK : FPKV_ELAUNCH;
}

template <typename T, int D>
static int launch_pos(const PoolView& pv, int layer, void* out, float* lse, const void* q, long long qsb,
                      long long qsh, const int64_t* bi, const void* pos, int pos_type, int B, int Hq,
                      float sc, void* ws, const Epilogue& epi, int32_t* st, cudaStream_t s)
{
    return pos_type == FPKV_I32
        ? launch_typed<T, D, int32_t>(pv, layer, out, lse, q, qsb, qsh, bi, pos, B, Hq, sc, ws, epi, st, s)
        : launch_typed<T, D, int64_t>(pv, layer, out, lse, q, qsb, qsh, bi, pos, B, Hq, sc, ws, epi, st, s);
}

int launch_decode_portable(const PoolView& pv, int layer, void* out, float* lse, const void* q,
                           long long qsb, long long qsh, const int64_t* bi, const void* pos, int pos_type,
                           int B, int Hq, float sc, void* ws, const Epilogue& epi, int32_t* st, cudaStream_t s)
{
    if (B == 0) return FPKV_OK;
#define FPKV_DISPATCH(T)                                                                              \
    return pv.D == 64 ? launch_pos<T, 64>(pv, layer, out, lse, q, qsb, qsh, bi, pos, pos_type, B, Hq, sc, ws, epi, st, s) \
                      : launch_pos<T, 128>(pv, layer, out, lse, q, qsb, qsh, bi, pos, pos_type, B, Hq, sc, ws, epi, st, s)
    switch (pv.dtype) {
        case FPKV_F32:  FPKV_DISPATCH(float);
        case FPKV_BF16: FPKV_DISPATCH(__nv_bfloat16);
        case FPKV_F16:  FPKV_DISPATCH(__half);
    }
#undef FPKV_DISPATCH
    return FPKV_EDTYPE;
}

// Packed prefill rows through the same kernel: one CTA per (token, query head), one split, direct output
// to out (Hq, L, D) / lse (Hq, L).
template <typename T, int D>
static int launch_prefill_typed(const PoolView& pv, int layer, void* out, float* lse, const void* q, long long qsh,
                                long long qst, const int64_t* bi, const int32_t* extent, int L, int Hq, float sc,
                                const Epilogue& epi, int32_t* st, cudaStream_t s)
{
    const OutLayout lay = epi.token_major ? OutLayout{(long long)Hq * D, (long long)D, 1, (long long)L}
                                          : OutLayout{(long long)D, (long long)L * D, 1, (long long)L};
    for (int t0 = 0; t0 < L; t0 += 32768) {            // grid.x = rows * heads stays far below its limit
        const int n = L - t0 < 32768 ? L - t0 : 32768;
        dim3 grid(n * Hq, 1);
        decode_portable_kernel<T, D, int32_t, true><<<grid, kPortableWarps * 32, 0, s>>>(
            pv.plane(layer, 0, 0), pv.plane_bytes(), pv.H, pv.page_table, pv.p2l, pv.n_pages, pv.max_batch, pv.P,
            (const T*)q + (long long)t0 * qst, qst, qsh, bi + t0, nullptr, extent + t0, Hq, sc * kLog2e, nullptr,
            (T*)out + (long long)t0 * lay.out_row, lse + t0, lay, epi, st, split_ptrs(pv, layer));
        if (cudaGetLastError() != cudaSuccess) return FPKV_ELAUNCH;
    }
    return FPKV_OK;
}

int launch_prefill_portable(const PoolView& pv, int layer, void* out, float* lse, const void* q, long long qsh,
                            long long qst, const int64_t* bi, const int32_t* extent, int L, int Hq, float sc,
                            const Epilogue& epi, int32_t* st, cudaStream_t s)
{
    if (L == 0) return FPKV_OK;
#define FPKV_DISPATCH(T)                                                                                   \
    return pv.D == 64 ? launch_prefill_typed<T, 64>(pv, layer, out, lse, q, qsh, qst, bi, extent, L, Hq, sc, epi, st, s) \
                      : launch_prefill_typed<T, 128>(pv, layer, out, lse, q, qsh, qst, bi, extent, L, Hq, sc, epi, st, s)
    switch (pv.dtype) {
        case FPKV_F32:  FPKV_DISPATCH(float);
        case FPKV_BF16: FPKV_DISPATCH(__nv_bfloat16);
        case FPKV_F16:  FPKV_DISPATCH(__half);
    }
#undef FPKV_DISPATCH
    return FPKV_EDTYPE;
}

}  // namespace fpkv
