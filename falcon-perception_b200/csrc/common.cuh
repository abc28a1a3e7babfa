// Shared device/host helpers for the fpkv kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/fpkv.h"

namespace fpkv {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Host-side view of one call's pool arguments after validation.
//
// Two pool layouts.  Uniform (split_hq == 0): the reference's (L, 2, 1, H, rows, D), K planes of all heads, then V
// planes.  Split (split_hq = number of query heads): per layer
//     K first halves   [H ][rows][D/2]   one per KV head: the half that carries the 1-D rotary embedding
//     K second halves  [Hq][rows][D/2]   one per QUERY head: the half that carries the per-query-head 2-D embedding
//     V                [H ][rows][D]     one per KV head
// which holds exactly what the reference's GQA-expanded cache holds (its copies of a KV head differ only in the
// second half of K) in (3 H + Hq) D / 2 instead of 2 Hq D elements per token.
struct PoolView {
    char* base;                       // start of the pool
    const int64_t* page_table;
    const int64_t* p2l;
    int num_layers, H, n_pages, P, D, max_batch, dtype, esize;
    int split_hq;                     // 0: uniform layout; otherwise the split layout for this many query heads
    __host__ __device__ size_t rows() const { return (size_t)n_pages * P; }
    // bytes between consecutive (layer, k|v, head) planes of the uniform layout
    __host__ __device__ size_t plane_bytes() const { return rows() * D * esize; }
    __host__ __device__ size_t half_plane_bytes() const { return rows() * (D / 2) * esize; }
    __host__ __device__ size_t layer_bytes() const {
        return split_hq ? (size_t)(3 * H + split_hq) * half_plane_bytes() : (size_t)2 * H * plane_bytes();
    }
    __host__ __device__ char* layer_base(int layer) const { return base + (size_t)layer * layer_bytes(); }
    __host__ __device__ char* plane(int layer, int kv, int h) const {          // uniform layout
        return base + ((size_t)(layer * 2 + kv) * H + h) * plane_bytes();
    }
    // split layout
    __host__ __device__ char* kt_plane(int layer, int hkv) const { return layer_base(layer) + (size_t)hkv * half_plane_bytes(); }
    __host__ __device__ char* khw_plane(int layer, int hq) const { return layer_base(layer) + (size_t)(H + hq) * half_plane_bytes(); }
    __host__ __device__ char* v_plane(int layer, int hkv) const {
        return layer_base(layer) + (size_t)(H + split_hq) * half_plane_bytes() + (size_t)hkv * plane_bytes();
    }
};

__device__ __forceinline__ void raise_status(int32_t* status, uint32_t bits) {
    if (status != nullptr) atomicOr(reinterpret_cast<unsigned int*>(status), bits);
}

template <typename PosT>
__device__ __forceinline__ long long load_pos(const void* p, int i) {
    return (long long)reinterpret_cast<const PosT*>(p)[i];
}

template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> {
    static __device__ __forceinline__ float to_float(float x) { return x; }
    static __device__ __forceinline__ float from_float(float x) { return x; }
};
template <> struct ElemTraits<__nv_bfloat16> {
    static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};
template <> struct ElemTraits<__half> {
    static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
};

// Optional epilogue of the attention kernels: the sink gate of the reference's _post_attention
// (falcon_perception/model.py:122-128), out * sigmoid(lse - sinks[head]), and for prefill the
// (L, heads * head_dim) output layout its output projection reads.  The gate is applied to the
// already rounded output and rounded again, as the reference's two-step computation does.
struct Epilogue {
    const void* sinks;      // device (n_q_heads) or nullptr: no gate
    int sinks_dtype;        // fpkv_dtype
    int token_major;        // prefill only: out as (1, L, n_q_heads, head_dim)
};
__device__ __forceinline__ float sink_gate(const Epilogue& e, int hq, float lse_natural) {
    if (e.sinks == nullptr) return 1.f;
    float sk;
    if (e.sinks_dtype == FPKV_F32) sk = reinterpret_cast<const float*>(e.sinks)[hq];
    else if (e.sinks_dtype == FPKV_BF16) sk = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(e.sinks)[hq]);
    else sk = __half2float(reinterpret_cast<const __half*>(e.sinks)[hq]);
    return 1.f / (1.f + __expf(sk - lse_natural));          // lse = -inf -> 0
}
template <typename T>
__device__ __forceinline__ T gated_out(float o, float gate, bool on) {
    const T r = ElemTraits<T>::from_float(o);
    return on ? ElemTraits<T>::from_float(ElemTraits<T>::to_float(r) * gate) : r;
}

// ---- launchers implemented in the .cu files (host side, internal) ----------
int launch_append(const PoolView& pv, int layer, const int64_t* batch_idx, const void* pos, int pos_type,
                  const void* k, long long k_stride_tok, long long k_stride_h,
                  const void* v, long long v_stride_tok, long long v_stride_h,
                  int n_tok, bool decode_mode, int32_t* status, cudaStream_t stream);

int launch_pre_append(const PoolView& pv, int layer, const void* qkv, long long qkv_stride_t, int Hq, int Hkv,
                      const float* freqs_cis, const float* freqs_cis_2d, const int64_t* batch_idx, const void* pos,
                      int pos_type, int n_tok, bool decode_mode, void* q_out, long long q_stride_h,
                      long long q_stride_t, float eps, int32_t* status, cudaStream_t stream);
int launch_gather(const PoolView& pv, int layer, int slot, int n_tokens, void* k_out, void* v_out,
                  int32_t* status, cudaStream_t stream);

size_t decode_portable_workspace_bytes(int B, int Hq, int D);
int launch_decode_portable(const PoolView& pv, int layer, void* out, float* lse, const void* q,
                           long long q_stride_b, long long q_stride_h, const int64_t* batch_idx,
                           const void* pos, int pos_type, int B, int Hq, float sm_scale,
                           void* workspace, const Epilogue& epi, int32_t* status, cudaStream_t stream);

bool decode_tma_supported(const PoolView& pv, int Hq);
size_t decode_tma_workspace_bytes(int Hq, int Hkv, int D);
int launch_decode_tma(const PoolView& pv, int layer, void* out, float* lse, const void* q,
                      long long q_stride_b, long long q_stride_h, const int64_t* batch_idx,
                      const void* pos, int pos_type, int B, int Hq, float sm_scale,
                      void* workspace, const Epilogue& epi, int32_t* status, cudaStream_t stream, bool after_append);

int launch_prefill_portable(const PoolView& pv, int layer, void* out, float* lse, const void* q, long long q_stride_h,
                            long long q_stride_t, const int64_t* batch_idx, const int32_t* extent, int L, int Hq,
                            float sm_scale, const Epilogue& epi, int32_t* status, cudaStream_t stream);
int launch_alloc_step(int64_t* page_table, int64_t* p2l, int n_pages, int max_batch, int32_t* free_pages,
                      int32_t* free_slots, int32_t* counts, const int32_t* ops, int n_ops, int32_t* status,
                      cudaStream_t stream);
int decode_attn_checked(const fpkv_pool* pool, int32_t layer, void* out, float* lse, const void* q,
                        int64_t q_stride_b, int64_t q_stride_h, const int64_t* batch_idx, const void* input_pos,
                        int32_t pos_type, int32_t B, int32_t n_q_heads, float sm_scale, void* workspace,
                        size_t workspace_bytes, int32_t flags, const fpkv_epilogue* epilogue, int32_t* status,
                        void* stream, bool clear_counters);
bool prefill_tc_supported(const PoolView& pv, int Hq);
int launch_prefill_tc(const PoolView& pv, int layer, void* out, float* lse, const void* q, long long q_stride_h,
                      long long q_stride_t, const int64_t* batch_idx, const int32_t* extent, int L, int Hq,
                      float sm_scale, const Epilogue& epi, int32_t* status, cudaStream_t stream);

}  // namespace fpkv
