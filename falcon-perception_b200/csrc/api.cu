// extern "C" boundary of libfpkv.so: argument validation, then the launchers.
// Declarations and the reference code each entry point replaces: include/fpkv.h.

#include "common.cuh"

using namespace fpkv;

namespace {

constexpr size_t kCounterBytes = 16384;  // head of the decode workspace: counters of the TMA kernel

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int esize_of(int dtype) {
    switch (dtype) {
        case FPKV_F32: return 4;
        case FPKV_BF16: case FPKV_F16: return 2;
    }
    return 0;
}

// Validate the pool descriptor and build the internal view.
int make_view(const fpkv_pool* pool, int layer, PoolView* pv) {
    if (pool == nullptr || pool->data == nullptr || pool->page_table == nullptr ||
        pool->physical_to_logical == nullptr)
        return FPKV_EINVAL;
    const int es = esize_of(pool->dtype);
    if (es == 0) return FPKV_EDTYPE;
    if (pool->num_layers <= 0 || pool->n_heads <= 0 || pool->n_pages <= 0 || pool->max_batch_size <= 0)
        return FPKV_EINVAL;
    if (layer < 0 || layer >= pool->num_layers) return FPKV_EINVAL;
    if (pool->head_dim != 64 && pool->head_dim != 128) return FPKV_ESHAPE;
    if (pool->page_size <= 0 || pool->page_size % 16 != 0) return FPKV_ESHAPE;
    if (!aligned16(pool->data)) return FPKV_EALIGN;
    pv->base = static_cast<char*>(pool->data);
    pv->page_table = pool->page_table;
    pv->p2l = pool->physical_to_logical;
    pv->num_layers = pool->num_layers; pv->H = pool->n_heads; pv->n_pages = pool->n_pages;
    pv->P = pool->page_size; pv->D = pool->head_dim; pv->max_batch = pool->max_batch_size;
    pv->dtype = pool->dtype; pv->esize = es;
    pv->split_hq = pool->split_q_heads;
    if (pv->split_hq < 0 || (pv->split_hq > 0 && (pv->split_hq % pv->H != 0 || pv->split_hq == pv->H))) return FPKV_ESHAPE;
    return FPKV_OK;
}

int check_rows(const void* p, long long s0, long long s1, int esize) {
    if (p == nullptr) return FPKV_EINVAL;
    if (!aligned16(p) || (s0 * esize) % 16 != 0 || (s1 * esize) % 16 != 0) return FPKV_EALIGN;
    return FPKV_OK;
}

// The optional epilogue descriptor of the attention entry points.
int make_epilogue(const fpkv_epilogue* e, int n_q_heads, Epilogue* out) {
    out->sinks = nullptr; out->sinks_dtype = FPKV_F32; out->token_major = 0;
    if (e == nullptr) return FPKV_OK;
    if (e->sinks != nullptr && esize_of(e->sinks_dtype) == 0) return FPKV_EDTYPE;
    // the kernels read sinks[hq] with 2- or 4-byte loads for hq < n_q_heads
    if (e->sinks != nullptr && (n_q_heads <= 0 || reinterpret_cast<uintptr_t>(e->sinks) % esize_of(e->sinks_dtype)))
        return FPKV_EALIGN;
    out->sinks = e->sinks; out->sinks_dtype = e->sinks_dtype; out->token_major = e->token_major != 0;
    return FPKV_OK;
}

int check_arch() {
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return FPKV_EARCH;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return FPKV_EARCH;
    return major == 10 ? FPKV_OK : FPKV_EARCH;
}

}  // namespace

namespace fpkv {

// fpkv_decode_attn behind its argument checks; `clear_counters` zeroes the work counters at the head of the
// workspace on the stream first (for a workspace whose previous contents are not known to be clean), after
// every check has passed, so that a refused call enqueues nothing.
int decode_attn_checked(const fpkv_pool* pool, int32_t layer, void* out, float* lse, const void* q,
                        int64_t q_stride_b, int64_t q_stride_h, const int64_t* batch_idx, const void* input_pos,
                        int32_t pos_type, int32_t B, int32_t n_q_heads, float sm_scale, void* workspace,
                        size_t workspace_bytes, int32_t flags, const fpkv_epilogue* epilogue, int32_t* status,
                        void* stream, bool clear_counters)
{
    PoolView pv;
    int rc = make_view(pool, layer, &pv);
    if (rc) return rc;
    Epilogue epi;
    if ((rc = make_epilogue(epilogue, n_q_heads, &epi))) return rc;
    if (B < 0 || n_q_heads <= 0 || (pos_type != FPKV_I32 && pos_type != FPKV_I64)) return FPKV_EINVAL;
    if (n_q_heads % pv.H) return FPKV_ESHAPE;
    if (pv.split_hq && n_q_heads != pv.split_hq) return FPKV_ESHAPE;      // a split pool serves exactly its query heads
    if (B == 0) return FPKV_OK;
    if (out == nullptr || lse == nullptr || batch_idx == nullptr || input_pos == nullptr || workspace == nullptr)
        return FPKV_EINVAL;
    if ((rc = check_rows(q, q_stride_b, q_stride_h, pv.esize))) return rc;
    if (!aligned16(out) || !aligned16(workspace)) return FPKV_EALIGN;
    const int which = flags & 3;
    const bool tma_ok = decode_tma_supported(pv, n_q_heads);
    if (which == FPKV_DECODE_TMA && !tma_ok) return FPKV_ESHAPE;
    const bool use_tma = which == FPKV_DECODE_TMA || (which == FPKV_DECODE_AUTO && tma_ok);
    // both kernels leave the counter words at the head of the workspace alone or at zero
    const size_t need = use_tma ? decode_tma_workspace_bytes(n_q_heads, pv.H, pv.D)
                                : decode_portable_workspace_bytes(B, n_q_heads, pv.D) + kCounterBytes;
    if (workspace_bytes < need) return FPKV_EWORKSPACE;
    if ((rc = check_arch())) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (clear_counters && cudaMemsetAsync(workspace, 0, 1024, s) != cudaSuccess) return FPKV_ELAUNCH;
    return use_tma ? launch_decode_tma(pv, layer, out, lse, q, q_stride_b, q_stride_h, batch_idx, input_pos,
                                       pos_type, B, n_q_heads, sm_scale, workspace, epi, status, s,
                                       (flags & FPKV_DECODE_AFTER_APPEND) != 0)
                   : launch_decode_portable(pv, layer, out, lse, q, q_stride_b, q_stride_h, batch_idx,
                                            input_pos, pos_type, B, n_q_heads, sm_scale,
                                            static_cast<char*>(workspace) + kCounterBytes, epi, status, s);
}

}  // namespace fpkv

extern "C" {

int fpkv_version(void) { return 200; }

// The hash of the sources this library was compiled from (the build script passes it in); the marker
// prefix lets the build script find it in the file without loading the library.
#ifndef FPKV_SRC_HASH
#define FPKV_SRC_HASH "0000000000000000"
#endif
static const char kBuildId[] = "fpkv-build-id:" FPKV_SRC_HASH;
const char* fpkv_build_id(void) { return kBuildId + 14; }

const char* fpkv_strerror(int code) {
    switch (code) {
        case FPKV_OK: return "ok";
        case FPKV_EINVAL: return "invalid argument (null pointer, negative size or bad enum)";
        case FPKV_ESHAPE: return "unsupported shape (head_dim, page_size or head ratio)";
        case FPKV_EALIGN: return "pointer or stride is not 16-byte aligned";
        case FPKV_EARCH: return "device is not sm_100";
        case FPKV_ELAUNCH: return "CUDA error at kernel launch";
        case FPKV_EWORKSPACE: return "workspace too small";
        case FPKV_EDTYPE: return "dtype not supported by this entry point";
        case FPKV_ESTATIC: return "request needs more scratch than the library's built-in static array holds";
    }
    return "unknown fpkv error code";
}

int fpkv_append_decode(const fpkv_pool* pool, int32_t layer, const int64_t* batch_idx, const void* input_pos,
                       int32_t pos_type, const void* k, int64_t k_stride_b, int64_t k_stride_h,
                       const void* v, int64_t v_stride_b, int64_t v_stride_h, int32_t B, int32_t* status,
                       void* stream)
{
    PoolView pv;
    int rc = make_view(pool, layer, &pv);
    if (rc) return rc;
    if (B < 0 || (pos_type != FPKV_I32 && pos_type != FPKV_I64)) return FPKV_EINVAL;
    if (B == 0) return FPKV_OK;
    if (batch_idx == nullptr || input_pos == nullptr) return FPKV_EINVAL;
    if ((rc = check_rows(k, k_stride_b, k_stride_h, pv.esize))) return rc;
    if ((rc = check_rows(v, v_stride_b, v_stride_h, pv.esize))) return rc;
    if ((rc = check_arch())) return rc;
    return launch_append(pv, layer, batch_idx, input_pos, pos_type, k, k_stride_b, k_stride_h, v, v_stride_b,
                         v_stride_h, B, /*decode_mode=*/true, status, static_cast<cudaStream_t>(stream));
}

int fpkv_append_packed(const fpkv_pool* pool, int32_t layer, const int64_t* batch_idx, const void* input_pos,
                       int32_t pos_type, const void* k, int64_t k_stride_h, int64_t k_stride_t,
                       const void* v, int64_t v_stride_h, int64_t v_stride_t, int32_t L, int32_t* status,
                       void* stream)
{
    PoolView pv;
    int rc = make_view(pool, layer, &pv);
    if (rc) return rc;
    if (L < 0 || (pos_type != FPKV_I32 && pos_type != FPKV_I64)) return FPKV_EINVAL;
    if (L == 0) return FPKV_OK;
    if (batch_idx == nullptr || input_pos == nullptr) return FPKV_EINVAL;
    if ((rc = check_rows(k, k_stride_h, k_stride_t, pv.esize))) return rc;
    if ((rc = check_rows(v, v_stride_h, v_stride_t, pv.esize))) return rc;
    if ((rc = check_arch())) return rc;
    return launch_append(pv, layer, batch_idx, input_pos, pos_type, k, k_stride_t, k_stride_h, v, v_stride_t,
                         v_stride_h, L, /*decode_mode=*/false, status, static_cast<cudaStream_t>(stream));
}

int fpkv_pre_append(const fpkv_pool* pool, int32_t layer, const void* qkv, int64_t qkv_stride_t, int32_t n_q_heads,
                    int32_t n_kv_heads, const float* freqs_cis, const float* freqs_cis_2d, const int64_t* batch_idx,
                    const void* input_pos, int32_t pos_type, int32_t n_tok, int32_t decode_mode, void* q_out,
                    int64_t q_stride_h, int64_t q_stride_t, float eps, int32_t* status, void* stream)
{
    PoolView pv;
    int rc = make_view(pool, layer, &pv);
    if (rc) return rc;
    if (n_tok < 0 || (pos_type != FPKV_I32 && pos_type != FPKV_I64) || n_q_heads <= 0 || n_kv_heads <= 0) return FPKV_EINVAL;
    if (n_q_heads % n_kv_heads) return FPKV_ESHAPE;
    if (pv.split_hq ? (pv.split_hq != n_q_heads || pv.H != n_kv_heads)
                    : (pv.H != n_q_heads && pv.H != n_kv_heads)) return FPKV_ESHAPE;     // expanded, compact or split pool
    if (pv.D != 64 && pv.D != 128) return FPKV_ESHAPE;
    if (qkv_stride_t < (int64_t)(n_q_heads + 2 * n_kv_heads) * pv.D) return FPKV_ESHAPE;
    if (!(eps >= 0.f)) return FPKV_EINVAL;
    if (n_tok == 0) return FPKV_OK;
    if (qkv == nullptr || freqs_cis == nullptr || batch_idx == nullptr || input_pos == nullptr || q_out == nullptr)
        return FPKV_EINVAL;
    if ((rc = check_rows(qkv, qkv_stride_t, qkv_stride_t, pv.esize))) return rc;
    if ((rc = check_rows(q_out, q_stride_h, q_stride_t, pv.esize))) return rc;
    if ((reinterpret_cast<uintptr_t>(freqs_cis) & 7u) || (reinterpret_cast<uintptr_t>(freqs_cis_2d) & 7u)) return FPKV_EALIGN;
    if ((rc = check_arch())) return rc;
    return launch_pre_append(pv, layer, qkv, qkv_stride_t, n_q_heads, n_kv_heads, freqs_cis, freqs_cis_2d, batch_idx,
                             input_pos, pos_type, n_tok, decode_mode != 0, q_out, q_stride_h, q_stride_t, eps, status,
                             static_cast<cudaStream_t>(stream));
}

int fpkv_gather(const fpkv_pool* pool, int32_t layer, int32_t slot, int32_t n_tokens, void* k_out, void* v_out,
                int32_t* status, void* stream)
{
    PoolView pv;
    int rc = make_view(pool, layer, &pv);
    if (rc) return rc;
    if (n_tokens < 0 || slot < 0 || slot >= pv.max_batch) return FPKV_EINVAL;
    if ((long long)n_tokens > (long long)pv.n_pages * pv.P) return FPKV_EINVAL;
    if (n_tokens == 0) return FPKV_OK;
    if (k_out == nullptr || v_out == nullptr) return FPKV_EINVAL;
    if (!aligned16(k_out) || !aligned16(v_out)) return FPKV_EALIGN;
    if ((rc = check_arch())) return rc;
    return launch_gather(pv, layer, slot, n_tokens, k_out, v_out, status, static_cast<cudaStream_t>(stream));
}

int fpkv_decode_workspace_bytes(const fpkv_pool* pool, int32_t B, int32_t n_q_heads, int32_t flags, size_t* bytes)
{
    PoolView pv;
    int rc = make_view(pool, 0, &pv);
    if (rc) return rc;
    if (bytes == nullptr || B < 0 || n_q_heads <= 0) return FPKV_EINVAL;
    if (n_q_heads % pv.H) return FPKV_ESHAPE;
    // sized for the kernel that `flags` selects, exactly as fpkv_decode_attn checks it
    const int which = flags & 3;
    const bool tma_ok = decode_tma_supported(pv, n_q_heads);
    if (which == FPKV_DECODE_TMA && !tma_ok) return FPKV_ESHAPE;
    const bool use_tma = which == FPKV_DECODE_TMA || (which == FPKV_DECODE_AUTO && tma_ok);
    *bytes = (use_tma ? decode_tma_workspace_bytes(n_q_heads, pv.H, pv.D)
                      : decode_portable_workspace_bytes(B, n_q_heads, pv.D) + kCounterBytes) + 256;
    return FPKV_OK;
}

int fpkv_decode_attn(const fpkv_pool* pool, int32_t layer, void* out, float* lse, const void* q,
                     int64_t q_stride_b, int64_t q_stride_h, const int64_t* batch_idx, const void* input_pos,
                     int32_t pos_type, int32_t B, int32_t n_q_heads, float sm_scale, void* workspace,
                     size_t workspace_bytes, int32_t flags, const fpkv_epilogue* epilogue, int32_t* status,
                     void* stream)
{
    return fpkv::decode_attn_checked(pool, layer, out, lse, q, q_stride_b, q_stride_h, batch_idx, input_pos, pos_type, B,
                                     n_q_heads, sm_scale, workspace, workspace_bytes, flags, epilogue, status, stream,
                                     /*clear_counters=*/false);
}

int fpkv_alloc_step(const fpkv_pool* pool, const fpkv_alloc_state* state, const int32_t* ops, int32_t n_ops,
                    int32_t* status, void* stream)
{
    // only the tables matter here: any page size or head_dim is fine
    if (pool == nullptr || pool->page_table == nullptr || pool->physical_to_logical == nullptr) return FPKV_EINVAL;
    if (state == nullptr || state->free_pages == nullptr || state->free_slots == nullptr || state->counts == nullptr)
        return FPKV_EINVAL;
    if (pool->n_pages <= 0 || pool->max_batch_size <= 0 || n_ops < 0) return FPKV_EINVAL;
    if (n_ops == 0) return FPKV_OK;
    if (ops == nullptr) return FPKV_EINVAL;
    if (!aligned16(ops)) return FPKV_EALIGN;
    const int rc = check_arch();
    if (rc) return rc;
    return launch_alloc_step(const_cast<int64_t*>(pool->page_table), const_cast<int64_t*>(pool->physical_to_logical),
                             pool->n_pages, pool->max_batch_size, state->free_pages, state->free_slots, state->counts,
                             ops, n_ops, status, static_cast<cudaStream_t>(stream));
}

int fpkv_prefill_attn(const fpkv_pool* pool, int32_t layer, void* out, float* lse, const void* q,
                      int64_t q_stride_h, int64_t q_stride_t, const int64_t* batch_idx, const int32_t* extent,
                      int32_t L, int32_t n_q_heads, float sm_scale, int32_t flags, const fpkv_epilogue* epilogue,
                      int32_t* status, void* stream)
{
    PoolView pv;
    int rc = make_view(pool, layer, &pv);
    if (rc) return rc;
    Epilogue epi;
    if ((rc = make_epilogue(epilogue, n_q_heads, &epi))) return rc;
    if (L < 0 || n_q_heads <= 0) return FPKV_EINVAL;
    if (n_q_heads % pv.H) return FPKV_ESHAPE;
    if (pv.split_hq && n_q_heads != pv.split_hq) return FPKV_ESHAPE;
    if (L == 0) return FPKV_OK;
    if (out == nullptr || lse == nullptr || batch_idx == nullptr || extent == nullptr) return FPKV_EINVAL;
    if ((rc = check_rows(q, q_stride_h, q_stride_t, pv.esize))) return rc;
    if (!aligned16(out)) return FPKV_EALIGN;
    const int which = flags & 3;
    const bool tc_ok = prefill_tc_supported(pv, n_q_heads);
    if (which == FPKV_PREFILL_TC && !tc_ok) return FPKV_ESHAPE;
    if ((rc = check_arch())) return rc;
    if (which == FPKV_PREFILL_TC || (which == FPKV_PREFILL_AUTO && tc_ok))
        return launch_prefill_tc(pv, layer, out, lse, q, q_stride_h, q_stride_t, batch_idx, extent, L, n_q_heads,
                                 sm_scale, epi, status, static_cast<cudaStream_t>(stream));
    return launch_prefill_portable(pv, layer, out, lse, q, q_stride_h, q_stride_t, batch_idx, extent, L, n_q_heads,
                                   sm_scale, epi, status, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
