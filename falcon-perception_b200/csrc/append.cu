// K/V append through the page table, and the gather that reads it back.
//
// One launch writes K and V of every new token: thread -> one 16-byte piece
// of one (token, head) row; blockIdx.y selects K or V.  The page-table lookup
// is done in the kernel, so nothing but the caller's index tensors is read
// beforehand.  HBM-bound byte movement; no shared memory is needed because
// every row piece is read once and written once.
//
// Semantics follow the reference's PagedKVCache.assign
// (falcon_perception/paged_attention.py:212-230, decode: a negative page id
// is clamped to reserved page 0) and assign_prefill_no_paging (:387-391).

#include "common.cuh"

namespace fpkv {

template <typename PosT>
__global__ void __launch_bounds__(256)
append_kernel(char* __restrict__ pool_layer,           // plane(layer, 0, 0)
              size_t plane_bytes, int H,
              const int64_t* __restrict__ page_table, int n_pages, int max_batch, int P,
              const int64_t* __restrict__ batch_idx, const PosT* __restrict__ pos,
              const char* __restrict__ k, long long k_tok_bytes, long long k_head_bytes,
              const char* __restrict__ v, long long v_tok_bytes, long long v_head_bytes,
              int n_tok, int vec_per_row, bool decode_mode, int32_t* status)
{
    // Launched with programmatic stream serialisation: the grid may become resident while the
    // preceding kernel drains; nothing is read or written before that kernel is complete.  A kernel
    // launched the same way behind this one may start its own set-up now.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const long long total = (long long)n_tok * H * vec_per_row;
    const int kv = blockIdx.y;
    const char* src = kv ? v : k;
    const long long tok_bytes = kv ? v_tok_bytes : k_tok_bytes;
    const long long head_bytes = kv ? v_head_bytes : k_head_bytes;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % vec_per_row);
        const long long r = i / vec_per_row;
        const int h = (int)(r % H);
        const int t = (int)(r / H);
        const long long slot = batch_idx[t];
        const long long p = (long long)pos[t];
        if (slot < 0 || slot >= max_batch) { if (c == 0 && h == 0) raise_status(status, FPKV_STATUS_BAD_SLOT); continue; }
        if (p < 0 || p / P >= n_pages)     { if (c == 0 && h == 0) raise_status(status, FPKV_STATUS_BAD_POS); continue; }
        long long page = page_table[slot * n_pages + p / P];
        if (page < 0) {
            // decode: the reference clamps to the reserved page; packed: caller error, same landing place
            if (!decode_mode && c == 0 && h == 0) raise_status(status, FPKV_STATUS_BAD_PAGE);
            page = 0;
        } else if (page >= n_pages) {
            if (c == 0 && h == 0) raise_status(status, FPKV_STATUS_BAD_PAGE);
            continue;
        }
        const long long addr = page * P + p % P;
        const uint4 val = *reinterpret_cast<const uint4*>(src + t * tok_bytes + h * head_bytes + (long long)c * 16);
        char* dst = pool_layer + ((size_t)kv * H + h) * plane_bytes + ((size_t)addr * vec_per_row + c) * 16;
        *reinterpret_cast<uint4*>(dst) = val;
    }
}

// Split layout: k and v arrive with the query head count (the reference's expanded tensors).  The first
// half of K and all of V are taken from the first head of each group and stored once per KV head; the
// second half of K is stored for every query head.
template <typename PosT>
__global__ void __launch_bounds__(256)
append_split_kernel(PoolView pv, int layer, const int64_t* __restrict__ batch_idx, const PosT* __restrict__ pos,
                    const char* __restrict__ k, long long k_tok_bytes, long long k_head_bytes,
                    const char* __restrict__ v, long long v_tok_bytes, long long v_head_bytes,
                    int n_tok, int vec_per_row, bool decode_mode, int32_t* status)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int Hq = pv.split_hq, n_rep = Hq / pv.H, half = vec_per_row / 2;
    const long long total = (long long)n_tok * Hq * vec_per_row;
    const int kv = blockIdx.y;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % vec_per_row);
        const long long r = i / vec_per_row;
        const int hq = (int)(r % Hq);
        const int t = (int)(r / Hq);
        const bool first = hq % n_rep == 0;
        if (kv ? !first : (c < half && !first)) continue;       // shared parts come from the group's first head only
        const long long slot = batch_idx[t];
        const long long p = (long long)pos[t];
        if (slot < 0 || slot >= pv.max_batch) { if (c == 0 && hq == 0) raise_status(status, FPKV_STATUS_BAD_SLOT); continue; }
        if (p < 0 || p / pv.P >= pv.n_pages)  { if (c == 0 && hq == 0) raise_status(status, FPKV_STATUS_BAD_POS); continue; }
        long long page = pv.page_table[slot * pv.n_pages + p / pv.P];
        if (page < 0) {
            if (!decode_mode && c == 0 && hq == 0) raise_status(status, FPKV_STATUS_BAD_PAGE);
            page = 0;
        } else if (page >= pv.n_pages) {
            if (c == 0 && hq == 0) raise_status(status, FPKV_STATUS_BAD_PAGE);
            continue;
        }
        const size_t addr = (size_t)(page * pv.P + p % pv.P);
        char* dst;
        if (kv) {
            dst = pv.v_plane(layer, hq / n_rep) + (addr * vec_per_row + c) * 16;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(v + t * v_tok_bytes + hq * v_head_bytes + (long long)c * 16);
        } else {
            dst = (c < half ? pv.kt_plane(layer, hq / n_rep) + (addr * half + c) * 16
                            : pv.khw_plane(layer, hq) + (addr * half + (c - half)) * 16);
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(k + t * k_tok_bytes + hq * k_head_bytes + (long long)c * 16);
        }
    }
}

int launch_append(const PoolView& pv, int layer, const int64_t* batch_idx, const void* pos, int pos_type,
                  const void* k, long long k_stride_tok, long long k_stride_h,
                  const void* v, long long v_stride_tok, long long v_stride_h,
                  int n_tok, bool decode_mode, int32_t* status, cudaStream_t stream)
{
    if (n_tok == 0) return FPKV_OK;
    const int vec_per_row = pv.D * pv.esize / 16;
    const long long total = (long long)n_tok * (pv.split_hq ? pv.split_hq : pv.H) * vec_per_row;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;           // grid-stride beyond 16 CTAs per SM
    dim3 grid((unsigned)blocks, 2);
    char* pool_layer = pv.plane(layer, 0, 0);
    const long long es = pv.esize;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t err;
    if (pv.split_hq) {
        const long long es2 = pv.esize;
        if (pos_type == FPKV_I32)
            err = cudaLaunchKernelEx(&cfg, append_split_kernel<int32_t>, pv, layer, batch_idx, (const int32_t*)pos,
                (const char*)k, k_stride_tok * es2, k_stride_h * es2, (const char*)v, v_stride_tok * es2, v_stride_h * es2,
                n_tok, vec_per_row, decode_mode, status);
        else
            err = cudaLaunchKernelEx(&cfg, append_split_kernel<int64_t>, pv, layer, batch_idx, (const int64_t*)pos,
                (const char*)k, k_stride_tok * es2, k_stride_h * es2, (const char*)v, v_stride_tok * es2, v_stride_h * es2,
                n_tok, vec_per_row, decode_mode, status);
        if (err != cudaSuccess) return FPKV_ELAUNCH;
        return cudaGetLastError() == cudaSuccess ? FPKV_OK : FPKV_ELAUNCH;
    }
    if (pos_type == FPKV_I32)
        err = cudaLaunchKernelEx(&cfg, append_kernel<int32_t>, pool_layer, pv.plane_bytes(), pv.H, pv.page_table,
            pv.n_pages, pv.max_batch, pv.P, batch_idx, (const int32_t*)pos,
            (const char*)k, k_stride_tok * es, k_stride_h * es, (const char*)v, v_stride_tok * es, v_stride_h * es,
            n_tok, vec_per_row, decode_mode, status);
    else
        err = cudaLaunchKernelEx(&cfg, append_kernel<int64_t>, pool_layer, pv.plane_bytes(), pv.H, pv.page_table,
            pv.n_pages, pv.max_batch, pv.P, batch_idx, (const int64_t*)pos,
            (const char*)k, k_stride_tok * es, k_stride_h * es, (const char*)v, v_stride_tok * es, v_stride_h * es,
            n_tok, vec_per_row, decode_mode, status);
    if (err != cudaSuccess) return FPKV_ELAUNCH;
    return cudaGetLastError() == cudaSuccess ? FPKV_OK : FPKV_ELAUNCH;
}

// Gather logical tokens [0, n_tokens) of one slot into (H, n_tokens, D).
__global__ void __launch_bounds__(256)
gather_kernel(const char* __restrict__ pool_layer, size_t plane_bytes, int H,
              const int64_t* __restrict__ page_table, const int64_t* __restrict__ p2l,
              int n_pages, int P, int slot, int n_tokens, int vec_per_row,
              char* __restrict__ k_out, char* __restrict__ v_out, int32_t* status)
{
    const long long total = (long long)n_tokens * H * vec_per_row;
    const int kv = blockIdx.y;
    char* dst_base = kv ? v_out : k_out;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % vec_per_row);
        const long long r = i / vec_per_row;
        const int t = (int)(r % n_tokens);
        const int h = (int)(r / n_tokens);
        uint4 val = make_uint4(0, 0, 0, 0);
        const long long page = page_table[(long long)slot * n_pages + t / P];
        if (page >= n_pages) {
            if (c == 0 && h == 0) raise_status(status, FPKV_STATUS_BAD_PAGE);
        } else if (page >= 0 && p2l[(long long)slot * n_pages + page] >= 0) {
            const long long addr = page * P + t % P;
            val = *reinterpret_cast<const uint4*>(pool_layer + ((size_t)kv * H + h) * plane_bytes +
                                                  ((size_t)addr * vec_per_row + c) * 16);
        }
        *reinterpret_cast<uint4*>(dst_base + (((size_t)h * n_tokens + t) * vec_per_row + c) * 16) = val;
    }
}

// Split layout: K comes back per QUERY head (Hq, n_tokens, D), put together from the shared first half and the
// head's own second half, i.e. as the reference's expanded cache holds it; V per KV head (H, n_tokens, D).
__global__ void __launch_bounds__(256)
gather_split_kernel(PoolView pv, int layer, int slot, int n_tokens, int vec_per_row,
                    char* __restrict__ k_out, char* __restrict__ v_out, int32_t* status)
{
    const int kv = blockIdx.y, Hq = pv.split_hq, n_rep = Hq / pv.H, half = vec_per_row / 2;
    const int heads = kv ? pv.H : Hq;
    const long long total = (long long)n_tokens * heads * vec_per_row;
    char* dst_base = kv ? v_out : k_out;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % vec_per_row);
        const long long r = i / vec_per_row;
        const int t = (int)(r % n_tokens);
        const int h = (int)(r / n_tokens);
        uint4 val = make_uint4(0, 0, 0, 0);
        const long long page = pv.page_table[(long long)slot * pv.n_pages + t / pv.P];
        if (page >= pv.n_pages) {
            if (c == 0 && h == 0) raise_status(status, FPKV_STATUS_BAD_PAGE);
        } else if (page >= 0 && pv.p2l[(long long)slot * pv.n_pages + page] >= 0) {
            const size_t addr = (size_t)(page * pv.P + t % pv.P);
            const char* src = kv ? pv.v_plane(layer, h) + (addr * vec_per_row + c) * 16
                                 : (c < half ? pv.kt_plane(layer, h / n_rep) + (addr * half + c) * 16
                                             : pv.khw_plane(layer, h) + (addr * half + (c - half)) * 16);
            val = *reinterpret_cast<const uint4*>(src);
        }
        *reinterpret_cast<uint4*>(dst_base + (((size_t)h * n_tokens + t) * vec_per_row + c) * 16) = val;
    }
}

int launch_gather(const PoolView& pv, int layer, int slot, int n_tokens, void* k_out, void* v_out,
                  int32_t* status, cudaStream_t stream)
{
    if (n_tokens == 0) return FPKV_OK;
    const int vec_per_row = pv.D * pv.esize / 16;
    const long long total = (long long)n_tokens * (pv.split_hq ? pv.split_hq : pv.H) * vec_per_row;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    dim3 grid((unsigned)blocks, 2);
    if (pv.split_hq) {
        gather_split_kernel<<<grid, 256, 0, stream>>>(pv, layer, slot, n_tokens, vec_per_row, (char*)k_out, (char*)v_out, status);
        return cudaGetLastError() == cudaSuccess ? FPKV_OK : FPKV_ELAUNCH;
    }
    gather_kernel<<<grid, 256, 0, stream>>>(pv.plane(layer, 0, 0), pv.plane_bytes(), pv.H, pv.page_table, pv.p2l,
                                            pv.n_pages, pv.P, slot, n_tokens, vec_per_row,
                                            (char*)k_out, (char*)v_out, status);
    return cudaGetLastError() == cudaSuccess ? FPKV_OK : FPKV_ELAUNCH;
}

}  // namespace fpkv
