"""CPU restatement of Falcon-Perception's paged KV-cache hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file.
It is the checker that the parity tests, the smoke entry and the benchmark's
CPU-baseline leg run beside the CUDA path; it is never the thing shipped and
never a fallback.

What it restates (paths are relative to the reference project root):

* page pool / page table / free lists / capacity bookkeeping
      falcon_perception/paged_attention.py:39-74   (constructor state)
      falcon_perception/paged_attention.py:95-182  (can_reserve, allocate,
                                                    reserve, erase)
* decode K/V append             falcon_perception/paged_attention.py:184-232
* packed prefill K/V append     falcon_perception/paged_attention.py:364-393
* decode attention semantics    falcon_perception/paged_inference.py:783-826
                                falcon_perception/paged_attention.py:234-333
                                falcon_perception/model.py:150-162
* prefill mask                  falcon_perception/attention.py:75-96
                                falcon_perception/paged_attention.py:343-362
* sink gate after attention     falcon_perception/model.py:122-128

The attention arithmetic itself lives in a third-party dependency of the
reference, torch 2.11.0 FlexAttention (torch/nn/attention/flex_attention.py),
which is not part of the reference tree.  Its published behaviour is restated
here: scores = q.k / sqrt(head_dim), softmax in fp32 over the allowed keys,
out = P.V returned in q's dtype, lse = natural-log-sum-exp of the scaled
scores in fp32, and a row with no allowed key gives out = 0, lse = -inf.

Parity pin: the reference ships no tests or golden vectors for this path.
The oracle is pinned instead against outputs of the reference itself, run on
CPU in the build container and committed under tests/golden/ together with
the generating script (tests/golden/make_golden.py); tests/test_oracle_golden.py
replays them.

One deliberate difference from the reference: the pool stores the real KV
heads (n_kv_heads) instead of the reference's GQA-expanded copies
(falcon_perception/model.py:74-83,114-115).  Reference head h*n_rep + r is a
copy of KV head h, and query head hq reads KV head hq // n_rep.
"""

from __future__ import annotations

import math

import numpy as np
import torch


def _ceil_div(a: int, b: int) -> int:
    return -(-int(a) // int(b))


class OraclePagedKVCache:
    """Page pool, page table and free-list allocator (host restatement).

    State after construction follows paged_attention.py:39-74: slot 0 and
    page 0 are reserved, row 0 of the page table is all zeros, every other
    table entry is -1, the free lists hold the remaining ids in descending
    order so that ``pop()`` hands out the smallest id first.
    """

    def __init__(self, n_pages, page_size, max_batch_size, n_heads, head_dim,
                 num_layers, dtype=torch.float32):
        self.n_pages = int(n_pages)
        self.page_size = int(page_size)
        self.max_batch_size = int(max_batch_size)
        self.dtype = dtype
        self.page_table = np.full((max_batch_size, n_pages), -1, dtype=np.int64)
        self.page_table[0, :] = 0
        self.physical_to_logical = np.full((max_batch_size, n_pages), -1, dtype=np.int64)
        self.page_table_cpu = [[] for _ in range(max_batch_size)]
        self.capacity = [0] * max_batch_size
        self.free_pages = list(range(n_pages - 1, 0, -1))
        self.free_batch_idx = list(range(max_batch_size - 1, 0, -1))
        self.kv_shape = (num_layers, 2, 1, n_heads, n_pages * page_size, head_dim)
        self.kv_cache = torch.zeros(self.kv_shape, dtype=dtype)

    # -- allocator (paged_attention.py:95-182) ------------------------------
    @property
    def num_free_pages(self) -> int:
        return len(self.free_pages)

    def can_reserve(self, size, batch_idx_int=None) -> bool:
        if batch_idx_int is None:
            return self.num_free_pages * self.page_size >= size and len(self.free_batch_idx) > 0
        return self.reserve(batch_idx_int, size, dry_run=True)

    def allocate(self) -> int:
        slot = self.free_batch_idx.pop()
        self.capacity[slot] = 0
        self.page_table[slot, :] = -1
        self.physical_to_logical[slot, :] = -1
        return slot

    def reserve(self, slot, seq_len, dry_run=False) -> bool:
        have = self.capacity[slot]
        if seq_len <= have:
            return True
        need = _ceil_div(seq_len - have, self.page_size)
        fits = need <= self.num_free_pages
        if dry_run:
            return fits
        if not fits:
            raise RuntimeError(
                f"Cannot reserve {need} pages for a sequence of length {seq_len} "
                f"in batch {slot}. Only {self.num_free_pages} pages available. "
                f"Current capacity is {have} tokens.")
        first = have // self.page_size
        taken = self.free_pages[len(self.free_pages) - need:]
        del self.free_pages[len(self.free_pages) - need:]
        for i, page in enumerate(taken):
            self.page_table[slot, first + i] = page
            self.physical_to_logical[slot, page] = first + i
        self.page_table_cpu[slot] = self.page_table_cpu[slot] + taken
        self.capacity[slot] = have + need * self.page_size
        return True

    def erase(self, slot) -> None:
        self.free_batch_idx.append(slot)
        self.free_pages.extend(self.page_table_cpu[slot][::-1])
        self.page_table_cpu[slot] = []
        self.page_table[slot, :] = -1
        self.physical_to_logical[slot, :] = -1
        self.capacity[slot] = 0

    # -- K/V append ---------------------------------------------------------
    def append_decode(self, layer, batch_idx, input_pos, k, v):
        """One new token per row (paged_attention.py:212-230).

        batch_idx (B,), input_pos (B,1) or (B,), k/v (B,H,1,D).  A negative
        page id is redirected to reserved page 0 (the clamp at :222).
        """
        bidx = np.asarray(batch_idx, dtype=np.int64).reshape(-1)
        pos = np.asarray(input_pos, dtype=np.int64).reshape(-1)
        P = self.page_size
        page = np.maximum(self.page_table[bidx, pos // P], 0)
        addr = torch.from_numpy(page * P + pos % P)
        # (B,H,1,D) -> (H,B,D); rows land at pool[layer, kv, 0, h, addr[b], :]
        self.kv_cache[layer, 0, 0][:, addr, :] = k[:, :, 0, :].transpose(0, 1).to(self.dtype)
        self.kv_cache[layer, 1, 0][:, addr, :] = v[:, :, 0, :].transpose(0, 1).to(self.dtype)

    def append_packed(self, layer, batch_idx, input_pos, k, v):
        """Packed prefill row (paged_attention.py:387-391): batch_idx and
        input_pos are (1,L) per-token, k/v are (1,H,L,D); no clamp."""
        bidx = np.asarray(batch_idx, dtype=np.int64).reshape(-1)
        pos = np.asarray(input_pos, dtype=np.int64).reshape(-1)
        P = self.page_size
        addr = torch.from_numpy(self.page_table[bidx, pos // P] * P + pos % P)
        self.kv_cache[layer, 0, 0][:, addr, :] = k[0].to(self.dtype)
        self.kv_cache[layer, 1, 0][:, addr, :] = v[0].to(self.dtype)

    # -- gather (the inverse of append; used by attention and by tests) -----
    def key_addresses(self, slot, n_tokens):
        """Physical token addresses of logical positions [0, n_tokens) of a
        slot, and a validity flag per position (paged_attention.py:303-311:
        a key is visible only if its page maps back to a logical block)."""
        P = self.page_size
        j = np.arange(n_tokens, dtype=np.int64)
        page = self.page_table[slot, j // P]
        safe = np.maximum(page, 0)
        valid = (page >= 0) & (self.physical_to_logical[slot, safe] >= 0)
        return safe * P + j % P, valid


def decode_attention(cache: OraclePagedKVCache, layer, q, batch_idx, input_pos,
                     sm_scale=None):
    """Paged decode attention for q (B,Hq,1,D): row b of slot s = batch_idx[b]
    at position p = input_pos[b] sees logical keys 0..p of that slot
    (paged_inference.py:797-826 builds exactly this set; the conversion to
    physical pages is paged_attention.py:267-333).  Returns out (B,Hq,1,D) in
    q's dtype and lse (B,Hq,1) fp32."""
    B, Hq, S, D = q.shape
    assert S == 1
    Hkv = cache.kv_shape[3]
    n_rep = Hq // Hkv
    scale = (1.0 / math.sqrt(D)) if sm_scale is None else float(sm_scale)
    bidx = np.asarray(batch_idx, dtype=np.int64).reshape(-1)
    pos = np.asarray(input_pos, dtype=np.int64).reshape(-1)
    out = torch.zeros((B, Hq, 1, D), dtype=torch.float32)
    lse = torch.full((B, Hq, 1), float("-inf"), dtype=torch.float32)
    K_pool = cache.kv_cache[layer, 0, 0]
    V_pool = cache.kv_cache[layer, 1, 0]
    for b in range(B):
        addr, valid = cache.key_addresses(int(bidx[b]), int(pos[b]) + 1)
        addr = torch.from_numpy(addr[valid])
        if addr.numel() == 0:
            continue
        Kb = K_pool[:, addr, :].float()                     # (Hkv, n, D)
        Vb = V_pool[:, addr, :].float()
        qb = q[b, :, 0, :].float().view(Hkv, n_rep, D)      # (Hkv, n_rep, D)
        s = torch.matmul(qb, Kb.transpose(1, 2)) * scale    # (Hkv, n_rep, n)
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l.unsqueeze(-1))
        out[b, :, 0, :] = torch.matmul(p, Vb).reshape(Hq, D)
        lse[b, :, 0] = l.reshape(Hq)
    return out.to(q.dtype), lse


def image_span_ids(input_ids, soi_id, eoi_id):
    """Per-token image index of a packed row (attention.py:79-88): tokens from
    an image-start token (inclusive) to the matching end-of-image token
    (exclusive) carry the running count of image starts; every other token
    carries 0."""
    ids = np.asarray(input_ids, dtype=np.int64).reshape(-1)
    n_soi = np.cumsum(ids == soi_id)
    n_eoi = np.cumsum(ids == eoi_id)
    inside = (n_soi - n_eoi) > 0
    return (n_soi * inside).astype(np.int64)


def prefill_allowed(doc_id, img_id):
    """Dense (L,L) boolean mask of the packed prefill row
    (paged_attention.py:343-362): query t may see key u iff both are in the
    same image span, or u <= t within the same document."""
    doc = np.asarray(doc_id, dtype=np.int64).reshape(-1)
    img = np.asarray(img_id, dtype=np.int64).reshape(-1)
    L = doc.shape[0]
    t = np.arange(L)
    same_img = (img[:, None] > 0) & (img[:, None] == img[None, :])
    causal_doc = (t[:, None] >= t[None, :]) & (doc[:, None] == doc[None, :])
    return same_img | causal_doc


def _masked_attention(q, k, v, allowed, scale):
    """q (Hq,Lq,D), k/v (Hkv,Lk,D) fp32, allowed (Lq,Lk) bool."""
    Hq, Lq, D = q.shape
    Hkv = k.shape[0]
    n_rep = Hq // Hkv
    qg = q.reshape(Hkv, n_rep * Lq, D)
    s = torch.matmul(qg, k.transpose(1, 2)).view(Hkv, n_rep, Lq, -1) * scale
    s = s.masked_fill(~allowed.view(1, 1, Lq, -1), float("-inf"))
    l = torch.logsumexp(s, dim=-1)                      # (Hkv, n_rep, Lq)
    p = torch.exp(s - torch.where(torch.isinf(l), torch.zeros_like(l), l).unsqueeze(-1))
    p = torch.where(torch.isinf(l).unsqueeze(-1), torch.zeros_like(p), p)
    o = torch.matmul(p.view(Hkv, n_rep * Lq, -1), v).view(Hq, Lq, D)
    return o, l.reshape(Hq, Lq)


def prefill_attention(q, k, v, doc_id, img_id, sm_scale=None):
    """Unpaged prefill attention over the fresh packed row (model.py:150-162
    with the mask of paged_attention.py:343-362).  q (1,Hq,L,D); k,v
    (1,Hkv,L,D).  Returns out (1,Hq,L,D) in q's dtype, lse (1,Hq,L) fp32."""
    _, Hq, L, D = q.shape
    scale = (1.0 / math.sqrt(D)) if sm_scale is None else float(sm_scale)
    allowed = torch.from_numpy(prefill_allowed(doc_id, img_id))
    o, l = _masked_attention(q[0].float(), k[0].float(), v[0].float(), allowed, scale)
    return o.unsqueeze(0).to(q.dtype), l.unsqueeze(0)


def paged_prefill_attention(cache: OraclePagedKVCache, layer, q, slot, q_pos,
                            kv_len, img_id_seq, sm_scale=None):
    """Chunked prefill through the page table (no counterpart in the
    reference, which never chunks; its result must equal the matching rows of
    the unchunked prefill_attention).  q (Hq,Lq,D) are the queries of ONE
    sequence at absolute positions q_pos (Lq,); keys are logical positions
    [0, kv_len) of ``slot`` read from pages; img_id_seq (kv_len,) is that
    sequence's per-position image index."""
    Hq, Lq, D = q.shape
    scale = (1.0 / math.sqrt(D)) if sm_scale is None else float(sm_scale)
    addr, valid = cache.key_addresses(int(slot), int(kv_len))
    addr_t = torch.from_numpy(addr)
    K = cache.kv_cache[layer, 0, 0][:, addr_t, :].float()
    V = cache.kv_cache[layer, 1, 0][:, addr_t, :].float()
    qp = np.asarray(q_pos, dtype=np.int64).reshape(-1)
    img = np.asarray(img_id_seq, dtype=np.int64).reshape(-1)
    u = np.arange(kv_len)
    same_img = (img[qp][:, None] > 0) & (img[qp][:, None] == img[None, :])
    allowed = (same_img | (u[None, :] <= qp[:, None])) & valid[None, :]
    o, l = _masked_attention(q.float(), K, V, torch.from_numpy(allowed), scale)
    return o.to(q.dtype), l


def post_attention_gate(out, lse, sinks):
    """The sink gate and layout change right after attention
    (falcon_perception/model.py:122-128): out (B,Hq,S,D) in the model dtype,
    lse (B,Hq,S) fp32, sinks (Hq,).  scale = sigmoid(lse - sinks[h]); the
    product is formed in fp32 from the rounded output and rounded back to the
    output dtype; the result is laid out (B, S, Hq*D) for the output
    projection.  (The projection itself is a library GEMM and not restated.)"""
    scale = torch.sigmoid(lse - sinks.float().view(1, -1, 1))
    gated = (out.float() * scale.unsqueeze(-1)).to(out.dtype)
    return gated.permute(0, 2, 1, 3).contiguous().flatten(2)


def _rms_norm_rows(x):
    """F.rms_norm(x, (D,)) without weight and with eps left at its default
    (falcon_perception/model.py:112-113): computed in fp32 as
    x * rsqrt(mean(x^2) + eps), eps = machine epsilon of fp32 (the arithmetic
    type, also for 16-bit inputs), and rounded back to x's dtype."""
    x32 = x.float()
    eps = torch.finfo(torch.float32).eps
    return (x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def _rotate_pairs(x, cos, sin):
    """Adjacent pairs (x[2i], x[2i+1]) rotated by (cos, sin)[i], in fp32."""
    x32 = x.float()
    even, odd = x32[..., 0::2], x32[..., 1::2]
    out = torch.empty_like(x32)
    out[..., 0::2] = even * cos - odd * sin
    out[..., 1::2] = even * sin + odd * cos
    return out


def pre_attention_tail(qkv, n_q_heads, n_kv_heads, head_dim, freqs_cis, freqs_cis_2d=None):
    """What Attention._pre_attention does to the QKV projection before the
    cache and the attention kernel see it (falcon_perception/model.py:107-120):
    split, per-head RMS norm of q and k, GQA expansion of k and v to the query
    head count (repeat_interleave), rotary embedding, (B,S,H,D) -> (B,H,S,D).
    Rotary embedding (falcon_perception/rope.py:30-104): the first half of the
    head dimension is rotated pairwise by freqs_cis[b, s, i] (1-D, complex64,
    shape (B,S,D/4)); the second half by freqs_cis_2d[b, s, h, i] (per QUERY
    head, shape (B,S,Hq,D/4)) when it is given, and left alone otherwise.  Each
    half is rotated in fp32 and rounded to the input dtype.
    qkv (B,S,(Hq+2*Hkv)*D).  Returns xq, xk, xv as (B,Hq,S,D)."""
    B, S, _ = qkv.shape
    D, Hq, Hkv = head_dim, n_q_heads, n_kv_heads
    xq, xk, xv = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    xq = _rms_norm_rows(xq.reshape(B, S, Hq, D))
    xk = _rms_norm_rows(xk.reshape(B, S, Hkv, D))
    xv = xv.reshape(B, S, Hkv, D)
    n_rep = Hq // Hkv
    xk = xk.repeat_interleave(n_rep, dim=2)
    xv = xv.repeat_interleave(n_rep, dim=2)
    fc = freqs_cis.reshape(B, S, 1, D // 4)
    outs = []
    for x in (xq, xk):
        t = _rotate_pairs(x[..., :D // 2], fc.real, fc.imag).to(x.dtype)
        hw = x[..., D // 2:]
        if freqs_cis_2d is not None:
            hw = _rotate_pairs(hw, freqs_cis_2d.real, freqs_cis_2d.imag).to(x.dtype)
        outs.append(torch.cat([t, hw], dim=-1))
    return outs[0].permute(0, 2, 1, 3), outs[1].permute(0, 2, 1, 3), xv.permute(0, 2, 1, 3)
