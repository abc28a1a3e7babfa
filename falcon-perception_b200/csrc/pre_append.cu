// Per-head RMS norm, rotary embedding and K/V append in one pass over the QKV
// projection: what Attention._pre_attention does behind the projection
// (falcon_perception/model.py:107-120, falcon_perception/rope.py:30-104)
// followed by insert_kv (model.py:150-155), without the intermediate tensors
// (normalised q/k, GQA-expanded k/v, rotated q/k, permuted copies) and the
// separate append.
//
// Eight lanes handle one head row of one token: a query head (normalise, rotate,
// write to the query output), a stored key head (normalise, rotate, write into
// the page pool) or a stored value head (copy into the pool); a warp has four
// rows in flight.  A lane holds D / 8 consecutive elements (16-byte accesses),
// i.e. whole rotation pairs (x[2i], x[2i+1]).
//
// Arithmetic follows the reference step by step so that results agree to the
// last bit wherever the order of the sum of squares does not matter: fp32
// throughout, x * rsqrt(mean(x^2) + eps) rounded to the storage type, then
// each half of the head rotated in fp32 (products and sums rounded separately,
// no fused multiply-add) and rounded again.  The first half uses the 1-D table
// freqs_cis[t, i], the second half the 2-D table freqs_cis_2d[t, head, i] of
// the QUERY head when one is given, and is left as normalised otherwise.
//
// Pool layouts: with n_heads == n_q_heads the pool holds the reference's
// expanded heads (stored head h = key head h / n_rep rotated with query head
// h's 2-D table); with n_heads == n_kv_heads it holds each key head once,
// rotated with the table of the first query head of its group, which equals the
// reference whenever the 2-D frequencies agree within a group or no 2-D table is
// in use.  The split layout (common.cuh) stores the first half of each key head once and the second half per query
// head with that head's table: exactly the reference's content in fewer bytes.
// HBM/latency-bound byte work: no shared memory, no tensor cores.

#include "common.cuh"

namespace fpkv {
namespace {

struct PreAppendParams {
    char* pool_layer; size_t plane_bytes; int H_out;
    int split;                          // split layout: keys per query head (shared first half stored once), values per KV head
    char* kt_base; char* khw_base; char* v_base; size_t half_plane_bytes;
    const int64_t* page_table; int n_pages, max_batch, P;
    const char* qkv; long long qkv_row_bytes;
    int Hq, Hkv;
    const float2* freqs; const float2* freqs2d;
    const int64_t* batch_idx; const void* pos;
    int n_tok; int decode_mode;
    char* q_out; long long q_head_bytes, q_tok_bytes;
    float eps; int32_t* status;
};

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __attribute__((unused)) __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Rounding to the storage type goes through the conversion unit, which is as narrow as the special-function unit
// (16 results per clock per SM); for bf16 a pair is rounded by one packed conversion and unpacked with shifts.
template <typename T> __device__ __forceinline__ void round_pair(float a, float b, float& ra, float& rb, T& ta, T& tb) {
    ta = from_f32<T>(a); tb = from_f32<T>(b); ra = to_f32<T>(ta); rb = to_f32<T>(tb);
}
template <> __device__ __forceinline__ void round_pair<__nv_bfloat16>(float a, float b, float& ra, float& rb,
                                                                      __nv_bfloat16& ta, __nv_bfloat16& tb) {
    uint32_t w;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(b), "f"(a));          // first source lands in the upper half
    ra = __uint_as_float(w << 16); rb = __uint_as_float(w & 0xffff0000u);
    const uint16_t lo = (uint16_t)(w & 0xffffu), hi = (uint16_t)(w >> 16);
    ta = *reinterpret_cast<const __nv_bfloat16*>(&lo); tb = *reinterpret_cast<const __nv_bfloat16*>(&hi);
}

template <typename T, int E> struct alignas(16) Row { T v[E]; };   // E elements of one lane, moved as 16-byte vectors

#ifndef FPKV_LANES_PER_ROW
#define FPKV_LANES_PER_ROW 8
#endif
constexpr int kLanesPerRow = FPKV_LANES_PER_ROW;        // lanes that share one head row
constexpr int kRowsPerWarp = 32 / kLanesPerRow;

template <typename T, int D, typename PosT>
__global__ void __launch_bounds__(256)
pre_append_kernel(const PreAppendParams prm)
{
    constexpr int E = D / kLanesPerRow;                    // elements per lane: 8 or 16, whole rotation pairs
    using RowT = Row<T, E>;
    const int lane = threadIdx.x % 32;
    const int sub = lane % kLanesPerRow;                   // position of the lane within its row
    const int HK = prm.split ? prm.Hq : prm.H_out, HV = prm.split ? prm.Hkv : prm.H_out;   // key rows and value rows per token
    const int items = prm.Hq + HK + HV;                    // per token: query heads, stored key heads, stored value heads
    const unsigned total = (unsigned)prm.n_tok * (unsigned)items;      // the launcher keeps this below 2^31: 32-bit index math
    const int n_rep = prm.Hq / prm.Hkv;
    const bool expanded = prm.split || prm.H_out == prm.Hq;       // one key row per query head, each with its own 2-D table
    const PosT* pos = static_cast<const PosT*>(prm.pos);
    const unsigned rows_per_pass = gridDim.x * blockDim.x / kLanesPerRow;
    // whole warps stay in the loop together (shuffles below): rows past the end are computed on row 0 and dropped
    const unsigned padded = (total + kRowsPerWarp - 1u) / kRowsPerWarp * kRowsPerWarp;
    for (unsigned w0 = (blockIdx.x * blockDim.x + threadIdx.x) / kLanesPerRow; w0 < padded; w0 += rows_per_pass) {
        const bool live = w0 < total;
        const unsigned w = live ? w0 : 0u;
        const int t = (int)(w / (unsigned)items);
        const int item = (int)(w - (unsigned)t * (unsigned)items);
        const int kind = item < prm.Hq ? 0 : (item < prm.Hq + HK ? 1 : 2);   // 0 query, 1 key, 2 value
        const int ho = kind == 0 ? item : (kind == 1 ? item - prm.Hq : item - prm.Hq - HK);
        // source head inside the token's QKV row, and the query head whose 2-D table applies
        int src_head, table_head;
        if (kind == 0) { src_head = ho; table_head = ho; }
        else {
            const int kvh = (kind == 1 ? expanded : (expanded && !prm.split)) ? ho / n_rep : ho;
            src_head = (kind == 1 ? prm.Hq : prm.Hq + prm.Hkv) + kvh;
            table_head = expanded ? ho : ho * n_rep;
        }
        // destination
        char* dst = nullptr;
        bool store = live;
        if (kind == 0) {
            dst = prm.q_out + ho * prm.q_head_bytes + t * prm.q_tok_bytes;
        } else {
            const bool reporter = live && sub == 0 && item == prm.Hq;
            const long long slot = prm.batch_idx[t];
            const long long p = (long long)pos[t];
            if (slot < 0 || slot >= prm.max_batch) { if (reporter) raise_status(prm.status, FPKV_STATUS_BAD_SLOT); store = false; }
            else if (p < 0 || p / prm.P >= prm.n_pages) { if (reporter) raise_status(prm.status, FPKV_STATUS_BAD_POS); store = false; }
            else {
                long long page = prm.page_table[slot * prm.n_pages + p / prm.P];
                if (page < 0) {                            // decode: the reference clamps to the reserved page; packed: caller error
                    if (!prm.decode_mode && reporter) raise_status(prm.status, FPKV_STATUS_BAD_PAGE);
                    page = 0;
                } else if (page >= prm.n_pages) {
                    if (reporter) raise_status(prm.status, FPKV_STATUS_BAD_PAGE);
                    store = false; page = 0;
                }
                const long long addr = page * prm.P + p % prm.P;
                if (!prm.split) {
                    dst = prm.pool_layer + ((size_t)(kind - 1) * prm.H_out + ho) * prm.plane_bytes + (size_t)addr * D * sizeof(T);
                } else if (kind == 2) {
                    dst = prm.v_base + (size_t)ho * prm.plane_bytes + (size_t)addr * D * sizeof(T);
                } else if (sub * E < D / 2) {              // first half of the key row: once per KV head, from the group's first query head
                    if (ho % n_rep != 0) store = false;
                    dst = prm.kt_base + (size_t)(ho / n_rep) * prm.half_plane_bytes + (size_t)addr * (D / 2) * sizeof(T);
                } else {                                   // second half: per query head; `dst` is biased so that the lane offset below fits
                    dst = prm.khw_base + (size_t)ho * prm.half_plane_bytes + (size_t)addr * (D / 2) * sizeof(T) - (size_t)(D / 2) * sizeof(T);
                }
            }
        }
        const RowT in = *reinterpret_cast<const RowT*>(prm.qkv + t * prm.qkv_row_bytes + ((size_t)src_head * D + sub * E) * sizeof(T));
        RowT out;
        if (kind == 2) {
            out = in;
        }
        // the norm's sum runs over the eight lanes of a row; value rows take part with a sum nobody uses
        float x[E];
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) { x[e] = to_f32<T>(in.v[e]); ss = __fadd_rn(ss, __fmul_rn(x[e], x[e])); }
#pragma unroll
        for (int o = kLanesPerRow / 2; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
        if (kind != 2) {
            const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)D), prm.eps)));
#pragma unroll
            for (int e = 0; e < E; e += 2) {               // the norm's output is rounded to the storage type
                T ta, tb;
                round_pair<T>(__fmul_rn(x[e], r), __fmul_rn(x[e + 1], r), x[e], x[e + 1], ta, tb);
                out.v[e] = ta; out.v[e + 1] = tb;          // what stays when the half is not rotated
            }
            const int i0 = sub * (E / 2);                  // first pair of this lane; a lane's pairs lie in one half of the head
            const float2* table = nullptr;
            if (i0 < D / 4) table = prm.freqs + (size_t)t * (D / 4) + i0;
            else if (prm.freqs2d != nullptr) table = prm.freqs2d + ((size_t)t * prm.Hq + table_head) * (D / 4) + (i0 - D / 4);
#pragma unroll
            for (int pr = 0; pr < E / 2; ++pr) {
                const float a = x[2 * pr], b = x[2 * pr + 1];
                if (table != nullptr) {
                    const float2 cs = table[pr];
                    float ra, rb;
                    round_pair<T>(__fsub_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y)),
                                  __fadd_rn(__fmul_rn(a, cs.y), __fmul_rn(b, cs.x)), ra, rb, out.v[2 * pr], out.v[2 * pr + 1]);
                }
            }
        }
        if (store) *reinterpret_cast<RowT*>(dst + (size_t)sub * E * sizeof(T)) = out;
    }
}

template <typename T, int D>
int launch_typed(const PreAppendParams& prm, int pos_type, cudaStream_t stream)
{
    const long long rows = (long long)prm.n_tok * (prm.split ? 2 * prm.Hq + prm.Hkv : prm.Hq + 2 * prm.H_out);
    const int rows_per_block = 256 / kLanesPerRow;
    long long blocks = (rows + rows_per_block - 1) / rows_per_block;
    if (blocks > 148 * 8) blocks = 148 * 8;               // grid-stride beyond eight CTAs per SM
    if (pos_type == FPKV_I32) pre_append_kernel<T, D, int32_t><<<(unsigned)blocks, 256, 0, stream>>>(prm);
    else pre_append_kernel<T, D, int64_t><<<(unsigned)blocks, 256, 0, stream>>>(prm);
    return cudaGetLastError() == cudaSuccess ? FPKV_OK : FPKV_ELAUNCH;
}

}  // namespace

int launch_pre_append(const PoolView& pv, int layer, const void* qkv, long long qkv_stride_t, int Hq, int Hkv,
                      const float* freqs_cis, const float* freqs_cis_2d, const int64_t* batch_idx, const void* pos,
                      int pos_type, int n_tok, bool decode_mode, void* q_out, long long q_stride_h,
                      long long q_stride_t, float eps, int32_t* status, cudaStream_t stream)
{
    if (n_tok == 0) return FPKV_OK;
    if ((long long)n_tok * (2 * Hq + 2 * pv.H) >= (1ll << 31) - 4) return FPKV_ESHAPE;
    PreAppendParams prm;
    prm.pool_layer = pv.plane(layer, 0, 0); prm.plane_bytes = pv.plane_bytes(); prm.H_out = pv.H;
    prm.split = pv.split_hq ? 1 : 0;
    prm.kt_base = prm.khw_base = prm.v_base = nullptr; prm.half_plane_bytes = pv.half_plane_bytes();
    if (pv.split_hq) { prm.kt_base = pv.kt_plane(layer, 0); prm.khw_base = pv.khw_plane(layer, 0); prm.v_base = pv.v_plane(layer, 0); }
    prm.page_table = pv.page_table; prm.n_pages = pv.n_pages; prm.max_batch = pv.max_batch; prm.P = pv.P;
    prm.qkv = static_cast<const char*>(qkv); prm.qkv_row_bytes = qkv_stride_t * pv.esize;
    prm.Hq = Hq; prm.Hkv = Hkv;
    prm.freqs = reinterpret_cast<const float2*>(freqs_cis); prm.freqs2d = reinterpret_cast<const float2*>(freqs_cis_2d);
    prm.batch_idx = batch_idx; prm.pos = pos; prm.n_tok = n_tok; prm.decode_mode = decode_mode ? 1 : 0;
    prm.q_out = static_cast<char*>(q_out); prm.q_head_bytes = q_stride_h * pv.esize; prm.q_tok_bytes = q_stride_t * pv.esize;
    prm.eps = eps; prm.status = status;
    if (pv.D == 128) {
        if (pv.dtype == FPKV_BF16) return launch_typed<__nv_bfloat16, 128>(prm, pos_type, stream);
        if (pv.dtype == FPKV_F16) return launch_typed<__half, 128>(prm, pos_type, stream);
        return launch_typed<float, 128>(prm, pos_type, stream);
    }
    if (pv.D == 64) {
        if (pv.dtype == FPKV_BF16) return launch_typed<__nv_bfloat16, 64>(prm, pos_type, stream);
        if (pv.dtype == FPKV_F16) return launch_typed<__half, 64>(prm, pos_type, stream);
        return launch_typed<float, 64>(prm, pos_type, stream);
    }
    return FPKV_ESHAPE;
}

}  // namespace fpkv
