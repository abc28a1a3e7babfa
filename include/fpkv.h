/*
 * fpkv.h - C ABI of libfpkv.so: the paged KV-cache hot path of
 * Falcon-Perception (page pool, page table, K/V append, paged decode and
 * prefill attention) as CUDA kernels for sm_100a.
 *
 * The reference project is pure Python and has no FFI of its own; the
 * boundary it offers is two Python call sites.  Every entry point below names
 * the reference code it replaces (path:line within the reference project).
 *
 * Conventions
 *  - Every pointer marked "device" is device memory owned by the caller (in
 *    practice a torch tensor's data_ptr()).  Except where an entry point's
 *    comment says otherwise, the library never allocates, frees or keeps
 *    device memory and holds no mutable global state, so calls on different
 *    streams are independent.
 *  - `stream` is a cudaStream_t passed as void*.  Kernels are enqueued on it
 *    and the call returns without synchronising, so every entry point may be
 *    captured in a CUDA graph unless its comment says otherwise.
 *  - Return value: 0 (FPKV_OK) or a negative FPKV_E* code; fpkv_strerror()
 *    gives the text.  Arguments are validated on the host before any launch.
 *  - `status`, where present, is an optional device int32 word (may be NULL).
 *    Kernels OR FPKV_STATUS_* bits into it when they meet an out-of-range
 *    slot / position / page id or when a bounded wait runs out; they never
 *    trap and never spin without a limit.  The caller zeroes and reads it.
 *  - Strides are in ELEMENTS.  The last (head_dim) dimension is contiguous
 *    and every row starts on a 16-byte boundary.
 */
#ifndef FPKV_H_
#define FPKV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FPKV_API __attribute__((visibility("default")))
#else
#define FPKV_API
#endif

#define FPKV_OK          0
#define FPKV_EINVAL     -1   /* NULL pointer, negative size, bad enum          */
#define FPKV_ESHAPE     -2   /* unsupported head_dim / page_size / head ratio  */
#define FPKV_EALIGN     -3   /* pointer or stride not 16-byte aligned          */
#define FPKV_EARCH      -4   /* device is not sm_100                           */
#define FPKV_ELAUNCH    -5   /* CUDA reported an error at launch               */
#define FPKV_EWORKSPACE -6   /* workspace too small                            */
#define FPKV_EDTYPE     -7   /* dtype not supported by this entry point        */

#define FPKV_STATUS_BAD_SLOT   1u   /* batch_idx outside [0, max_batch_size)   */
#define FPKV_STATUS_BAD_POS    2u   /* position outside the page table         */
#define FPKV_STATUS_BAD_PAGE   4u   /* page id outside [0, n_pages)            */
#define FPKV_STATUS_TIMEOUT    8u   /* a bounded on-chip wait ran out          */
#define FPKV_STATUS_OPEN_SPAN 16u   /* set by the host-side mask builder, not by a
                                       kernel: an image span was not closed inside
                                       its sequence and was cut at the sequence's end */

typedef enum { FPKV_F32 = 0, FPKV_BF16 = 1, FPKV_F16 = 2 } fpkv_dtype;
typedef enum { FPKV_I32 = 0, FPKV_I64 = 1 } fpkv_itype;

/*
 * The page pool and its tables: the state of the reference's PagedKVCache
 * (falcon_perception/paged_attention.py:39-74).
 *   data                 device, (num_layers, 2, 1, n_heads, n_pages*page_size,
 *                        head_dim) contiguous, i.e. `kv_cache` (:72-74);
 *                        n_heads is the number of heads STORED (the KV heads).
 *                        The reference creates it zero-filled (:74).  Here it
 *                        may hold anything, NaN and Inf bit patterns included,
 *                        in rows that were never appended: the attention
 *                        kernels read whole tiles but clear the value rows
 *                        beyond a sequence's last visible key on chip, so
 *                        garbage never reaches a result.  Reserved page 0
 *                        (rows [0, page_size) of every plane) is the landing
 *                        place of padding rows and is never read.
 *                        SPLIT LAYOUT (split_q_heads = the model's query head
 *                        count, a multiple of n_heads greater than it): the
 *                        reference expands K and V to the query heads before
 *                        caching (model.py:114-115), and its copies of a KV head
 *                        differ only in the second half of K, which carries the
 *                        per-query-head 2-D rotary embedding (rope.py:59-104).
 *                        The split pool stores exactly that content once: per
 *                        layer, contiguous,
 *                          K first halves  [n_heads]      [rows][head_dim/2]
 *                          K second halves [split_q_heads][rows][head_dim/2]
 *                          V               [n_heads]      [rows][head_dim]
 *                        with rows = n_pages*page_size, i.e. (3*n_heads +
 *                        split_q_heads)*head_dim/2 elements per token instead of
 *                        the reference's 2*split_q_heads*head_dim.  Append entry
 *                        points then take K and V with split_q_heads heads (the
 *                        reference's expanded tensors; the first head of each
 *                        group supplies the shared parts), fpkv_pre_append writes
 *                        the layout directly, the attention entry points are
 *                        called with n_q_heads = split_q_heads.
 *   page_table           device int64 (max_batch_size, n_pages)   (:58-59)
 *   physical_to_logical  device int64 (max_batch_size, n_pages)   (:70)
 */
typedef struct fpkv_pool {
    void*          data;
    const int64_t* page_table;
    const int64_t* physical_to_logical;
    int32_t num_layers;
    int32_t n_heads;
    int32_t n_pages;
    int32_t page_size;
    int32_t head_dim;
    int32_t max_batch_size;
    int32_t dtype;              /* fpkv_dtype */
    int32_t split_q_heads;      /* 0: the layout above; > 0: the split layout below */
} fpkv_pool;

/*
 * Optional epilogue of the attention entry points (pass NULL for none): what
 * the reference does right after attention in Attention._post_attention
 * (falcon_perception/model.py:122-128), folded into the kernels' output stage.
 *   sinks        device (n_q_heads) of `sinks_dtype`, or NULL.  When given,
 *                out is written as round(round(out) * sigmoid(lse - sinks[h])),
 *                the reference's two-step value; lse is returned ungated.
 *   token_major  prefill only: write out as (1, L, n_q_heads, head_dim), the
 *                layout the output projection reads after the reference's
 *                permute(0, 2, 1, 3).flatten(2), instead of (1, n_q_heads, L,
 *                head_dim).  (For decode the two layouts are the same memory.)
 */
typedef struct fpkv_epilogue {
    const void* sinks;
    int32_t sinks_dtype;        /* fpkv_dtype */
    int32_t token_major;
} fpkv_epilogue;

/* Library version (major*10000 + minor*100 + patch). */
FPKV_API int fpkv_version(void);

/* Hash of the sources the library was built from (16 hex digits): the build
 * script compiles it in, the Python loader compares it with the tree and
 * refuses a library built from something else. */
FPKV_API const char* fpkv_build_id(void);

/* Text for a return code; never NULL. */
FPKV_API const char* fpkv_strerror(int code);

/*
 * The allocator's free lists on the device: the reference's `free_pages` and
 * `free_batch_idx` Python lists (paged_attention.py:62-68) as stacks with the
 * same order (element 0 at the bottom, the list's last element on top).
 *   free_pages  device int32 (n_pages);         counts[0] entries are valid
 *   free_slots  device int32 (max_batch_size);  counts[1] entries are valid
 *   counts      device int32 [2]
 * The caller fills them once (the constructor state is free_pages =
 * [n_pages-1 .. 1], free_slots = [max_batch_size-1 .. 1]) and again whenever
 * it reorders its own copy of the lists by hand.
 */
typedef struct fpkv_alloc_state {
    int32_t* free_pages;
    int32_t* free_slots;
    int32_t* counts;
} fpkv_alloc_state;

/*
 * Apply one scheduling step's allocator calls on the device, in order, with
 * one launch: free stacks, page_table and physical_to_logical.  Replaces the
 * device side of PagedKVCache.allocate, reserve and erase
 * (paged_attention.py:102-109, 145-158, 166-182), which issue a few tensor
 * operations and one host-to-device tensor per call and rewrite whole table
 * rows; here a call is one 16-byte record and an erase touches only the
 * entries the slot owns.  The host keeps its own copy of the lists (it needs
 * them for can_reserve and the RuntimeError of an over-reserve); this entry
 * point WRITES pool->page_table and pool->physical_to_logical.
 * ops: device int32 [n_ops][4], 16-byte aligned, each {kind, slot, a, b}:
 *   kind 0  allocate  pop the slot stack; the popped slot must be `slot`
 *   kind 1  reserve   take the top b pages, in list order, as logical pages
 *                     a .. a+b-1 of `slot` (free_pages[-b:] of :147-158)
 *   kind 2  erase     push the slot's pages (logical 0 .. a-1) back reversed,
 *                     set those entries of both tables to -1, push the slot
 *   kind 3  map       page_table[slot, a] = b; physical_to_logical[slot, b] = a
 *                     (for callers that keep their own free lists)
 *   kind 4  clear     both table rows of `slot` to -1 in full
 * Slot 0 and page 0 are reserved and never edited; records naming them, ids
 * out of range, a pop that does not give `slot`, or a reserve beyond the
 * stack are skipped and raise FPKV_STATUS_BAD_SLOT / _BAD_PAGE.
 */
FPKV_API int fpkv_alloc_step(const fpkv_pool* pool, const fpkv_alloc_state* state,
                             const int32_t* ops, int32_t n_ops, int32_t* status, void* stream);

/*
 * Decode append: one new K/V row per sequence, written through the page
 * table.  Replaces PagedKVCache.assign (paged_attention.py:184-232):
 *   page = max(page_table[batch_idx[b], input_pos[b] / page_size], 0)
 *   pool[layer, 0|1, 0, h, page*page_size + input_pos[b] % page_size, :] = k|v[b, h, 0, :]
 * batch_idx  device int64 (B);  input_pos device (B) of `pos_type`.
 * k, v       device (B, n_heads, 1, head_dim) of the pool's dtype with
 *            element strides k_stride_b / k_stride_h (resp. v_*).
 */
FPKV_API int fpkv_append_decode(const fpkv_pool* pool, int32_t layer,
                       const int64_t* batch_idx, const void* input_pos, int32_t pos_type,
                       const void* k, int64_t k_stride_b, int64_t k_stride_h,
                       const void* v, int64_t v_stride_b, int64_t v_stride_h,
                       int32_t B, int32_t* status, void* stream);

/*
 * Packed prefill append: L tokens of one packed row, each with its own slot
 * and position.  Replaces PagedKVCache.assign_prefill_no_paging
 * (paged_attention.py:364-393).  A negative page id is a caller error there
 * (the engine reserves first, paged_inference.py:1198-1204); here such a row
 * goes to reserved page 0 and FPKV_STATUS_BAD_PAGE is raised.
 * batch_idx, input_pos  device (L) (the reference's (1,L) tensors).
 * k, v                  device (1, n_heads, L, head_dim); strides over the
 *                       head and token dimensions.
 */
FPKV_API int fpkv_append_packed(const fpkv_pool* pool, int32_t layer,
                       const int64_t* batch_idx, const void* input_pos, int32_t pos_type,
                       const void* k, int64_t k_stride_h, int64_t k_stride_t,
                       const void* v, int64_t v_stride_h, int64_t v_stride_t,
                       int32_t L, int32_t* status, void* stream);

/*
 * Norm + rotary embedding + append in one pass over the QKV projection.
 * Replaces the part of Attention._pre_attention behind the projection
 * (falcon_perception/model.py:107-120: split, per-head RMS norm of q and k,
 * repeat_kv, apply_3d_rotary_emb of falcon_perception/rope.py:87-104, permutes)
 * together with the insert_kv that follows it (model.py:150-155).
 *   qkv          device (n_tok) rows of (n_q_heads + 2*n_kv_heads)*head_dim
 *                elements of the pool's dtype, [q | k | v], row stride
 *                qkv_stride_t elements (the (B,S,.) projection output flattened)
 *   freqs_cis    device float (n_tok, head_dim/4, 2): cos, sin of the 1-D table
 *                already indexed by position (complex64 viewed as real)
 *   freqs_cis_2d device float (n_tok, n_q_heads, head_dim/4, 2), or NULL when no
 *                token carries a 2-D position (the second half of every head is
 *                then only normalised)
 *   batch_idx, input_pos   slot and position of every token (as the two appends)
 *   decode_mode  1: a negative page id is clamped to page 0 (fpkv_append_decode),
 *                0: it is reported (fpkv_append_packed)
 *   q_out        device: normalised, rotated queries, element (h, t, d) at
 *                h*q_stride_h + t*q_stride_t + d
 *   eps          the norm's epsilon (the reference leaves it at fp32 epsilon)
 * The pool holds either n_q_heads heads (the reference's expanded layout: stored
 * head h is key head h / n_rep rotated with query head h's 2-D table) or
 * n_kv_heads heads (each key head once, rotated with the 2-D table of the first
 * query head of its group: identical to the reference when the 2-D frequencies
 * agree within a group or freqs_cis_2d is NULL).
 */
FPKV_API int fpkv_pre_append(const fpkv_pool* pool, int32_t layer,
                    const void* qkv, int64_t qkv_stride_t, int32_t n_q_heads, int32_t n_kv_heads,
                    const float* freqs_cis, const float* freqs_cis_2d,
                    const int64_t* batch_idx, const void* input_pos, int32_t pos_type,
                    int32_t n_tok, int32_t decode_mode,
                    void* q_out, int64_t q_stride_h, int64_t q_stride_t,
                    float eps, int32_t* status, void* stream);

/*
 * Gather: read logical positions [0, n_tokens) of one slot back through the
 * page table into contiguous (n_heads, n_tokens, head_dim) buffers.  The
 * inverse of the two appends; what the reference's attention kernels do
 * implicitly through kv_indices (paged_attention.py:267-301).  Positions whose
 * page is unmapped read as zeros.
 */
FPKV_API int fpkv_gather(const fpkv_pool* pool, int32_t layer, int32_t slot, int32_t n_tokens,
                void* k_out, void* v_out, int32_t* status, void* stream);

/*
 * Paged decode attention: one query token per row against logical keys
 * 0..input_pos[b] of slot batch_idx[b].  Replaces, for S_q == 1, the decode
 * mask pipeline plus FlexAttention call of the reference:
 * PagedInferenceEngine.get_decoding_block_mask (paged_inference.py:783-826),
 * PagedKVCache.convert_logical_block_mask / get_mask_mod
 * (paged_attention.py:234-333) and compiled_flex_attn_decode
 * (attention.py:17, called at model.py:156-162).
 *   score = (q . k) * sm_scale, softmax in fp32,
 *   out (B, n_q_heads, 1, head_dim) contiguous, dtype of q,
 *   lse (B, n_q_heads, 1) fp32, natural log; a row with no visible key
 *   (slot 0, unmapped pages) gives out = 0, lse = -inf.
 * Query head hq reads stored head hq / (n_q_heads / pool->n_heads).
 * q: device (B, n_q_heads, 1, head_dim) with element strides q_stride_b/_h.
 * workspace: device, at least fpkv_decode_workspace_bytes() bytes, 16-byte
 * aligned.  Its first 16 KiB hold work counters that must be ZERO on
 * entry; every call that completes leaves them zero, so zero-fill the
 * workspace once when it is allocated (and again after a call that raised
 * FPKV_STATUS_TIMEOUT).  The rest needs no initialisation.  Two calls that
 * share a workspace must not overlap on the device.
 * flags: FPKV_DECODE_AUTO picks the TMA + tensor-core kernel when the shape is
 * in its range (16-bit pool, page_size 128, head_dim 64/128, 1/2/4/8 query
 * heads per stored head) and the portable CUDA-core kernel otherwise;
 * FPKV_DECODE_PORTABLE / FPKV_DECODE_TMA force one (the latter returns
 * FPKV_ESHAPE outside its range).
 */
#define FPKV_DECODE_AUTO     0
#define FPKV_DECODE_PORTABLE 1
#define FPKV_DECODE_TMA      2
/* OR into flags when the call directly follows fpkv_append_decode of the same
 * step on the same stream, with nothing enqueued in between: the attention
 * kernel then starts its set-up (index reads, page-table walk) while the
 * append is still running and waits for it only before the first pool read.
 * Never set it after anything else: the kernel would read batch_idx,
 * input_pos and q before the preceding work is known to be complete. */
#define FPKV_DECODE_AFTER_APPEND 4
/*
 * Bytes of scratch fpkv_decode_attn needs for a batch of B rows with n_q_heads
 * query heads when called with the same kernel choice in `flags` (an upper
 * bound that does not depend on the context lengths; the TMA kernel's need
 * does not depend on B either).  FPKV_ESHAPE when FPKV_DECODE_TMA is forced
 * outside its range.
 */
FPKV_API int fpkv_decode_workspace_bytes(const fpkv_pool* pool, int32_t B, int32_t n_q_heads,
                                int32_t flags, size_t* bytes);

FPKV_API int fpkv_decode_attn(const fpkv_pool* pool, int32_t layer,
                     void* out, float* lse,
                     const void* q, int64_t q_stride_b, int64_t q_stride_h,
                     const int64_t* batch_idx, const void* input_pos, int32_t pos_type,
                     int32_t B, int32_t n_q_heads, float sm_scale,
                     void* workspace, size_t workspace_bytes, int32_t flags,
                     const fpkv_epilogue* epilogue, int32_t* status, void* stream);

/*
 * Paged prefill / chunked-prefill attention over a packed row of L query
 * tokens.  Replaces create_prefill_blockmask + compiled_flex_attn_prefill
 * (paged_attention.py:343-362, attention.py:18,75-96, called at
 * model.py:156-162); unlike the reference, which attends over the fresh k, v,
 * keys and values are read from the pool through the page table, so it also
 * serves a chunk of a prompt whose earlier tokens are already cached.
 *
 * The reference's mask -- query t sees key u of the same sequence iff u <= t
 * or both lie in the same image span -- always selects a prefix of the
 * sequence, because a span is a contiguous run containing t.  The caller
 * passes that prefix length per token:
 *   extent[t] = input_pos[t] + 1              for a token outside image spans,
 *   extent[t] = (position of the span's end)  for a token inside one,
 *   extent[t] = 0                             for a pad token (batch_idx 0).
 * Keys 0 .. extent[t]-1 of slot batch_idx[t] must already be in the pool.
 * Every aligned group of 128 packed tokens may hold tokens of one slot only
 * (plus pads), which the reference's packing guarantees
 * (paged_inference.py:634-672); other rows raise FPKV_STATUS_BAD_SLOT.
 *
 * q    device (1, n_q_heads, L, head_dim), element strides q_stride_h / _t
 * out  device (1, n_q_heads, L, head_dim) contiguous, 16-byte aligned, dtype
 *      of q
 * lse  device (1, n_q_heads, L) fp32 natural log; rows without a visible key
 *      give out = 0, lse = -inf.
 * flags: FPKV_PREFILL_AUTO runs the tcgen05 tensor-core kernel for 16-bit
 * pools with page_size 128 and head_dim 128 or 64 (a split pool: head_dim
 * 128) and a portable CUDA-core kernel (any pool dtype, head_dim 64/128,
 * any page size; not tuned) otherwise;
 * FPKV_PREFILL_PORTABLE / FPKV_PREFILL_TC force one (the latter returns
 * FPKV_ESHAPE outside its range).  Needs no workspace.
 */
#define FPKV_PREFILL_AUTO     0
#define FPKV_PREFILL_PORTABLE 1
#define FPKV_PREFILL_TC       2
FPKV_API int fpkv_prefill_attn(const fpkv_pool* pool, int32_t layer,
                               void* out, float* lse,
                               const void* q, int64_t q_stride_h, int64_t q_stride_t,
                               const int64_t* batch_idx, const int32_t* extent,
                               int32_t L, int32_t n_q_heads, float sm_scale, int32_t flags,
                               const fpkv_epilogue* epilogue, int32_t* status, void* stream);

/*
 * fpkv_decode_attn without the workspace argument, for callers that cannot
 * allocate device memory.  It has no counterpart in the reference.
 *
 * Who needs it: an engine that gave all free HBM to its page pool at start-up
 * and so has nothing to cudaMalloc from later; a decode loop that must not
 * call cudaMalloc because that call synchronises the whole device; a host that
 * runs this library under its own memory manager and allows no allocation in
 * plugin code.  The scratch is a fixed array of FPKV_STATIC_SCRATCH_BYTES
 * inside the library image: every GPU that loads libfpkv.so holds it until
 * the process exits.  The call itself allocates and frees nothing.
 *
 * Arguments, results and error codes are those of fpkv_decode_attn with the
 * TMA + tensor-core kernel forced (16-bit pool, page_size 128, head_dim
 * 64/128, 1/2/4/8 query heads per stored head; FPKV_ESHAPE otherwise).
 * A head layout whose scratch need exceeds FPKV_STATIC_SCRATCH_BYTES is
 * refused with FPKV_ESTATIC (at head_dim 128: more than 4 query heads per
 * stored head).  There is no FPKV_DECODE_AFTER_APPEND mode.
 *
 * The first call on each GPU looks up the array's device address (with that
 * GPU current) and keeps it; make that first call before any stream capture.
 * All calls on a GPU share the one array, which keeps the last call's
 * contents; the words that must be zero are cleared at the head of each call.
 * Calls that overlap on the same GPU race on it: issue them in order.
 */
#define FPKV_STATIC_SCRATCH_BYTES (4u << 20)
#define FPKV_ESTATIC    -8   /* needs more scratch than the built-in array has */
FPKV_API int fpkv_decode_attn_static(const fpkv_pool* pool, int32_t layer,
                                     void* out, float* lse,
                                     const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                     const int64_t* batch_idx, const void* input_pos, int32_t pos_type,
                                     int32_t B, int32_t n_q_heads, float sm_scale,
                                     int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* FPKV_H_ */
