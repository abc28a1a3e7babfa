"""GPU: the split pool layout -- first half of K and V once per KV head, second half of K once per query head.

The reference expands K and V to the query heads before caching (falcon_perception/model.py:114-115) and rotates
the second half of every expanded key copy with its own query head's 2-D table (rope.py:59-104), so its copies of
a KV head differ there and only there.  The split layout stores exactly that content; these tests hold it against
the reference's expanded cache (golden vectors of Attention._pre_attention with distinct per-head 2-D
frequencies, and the oracle run with the query head count) bit for bit, and the attention over it against the
oracle's attention over the expanded cache."""

import numpy as np
import pytest
import torch

import workloads as wl
from fpkv import _lib
from fpkv.paged_attention import PagedKVCache, paged_attention
from oracle import paged_kv_oracle as orc
from helpers import assert_attention_close
from test_oracle_golden import pre_attention_case
from test_pre_append_gpu import close_to_ulp

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["pre_attention_bf16_2d", "pre_attention_bf16_text", "pre_attention_f32"])
def test_fused_pre_append_writes_the_reference_expanded_content(name):
    """Packed prefill form on a split pool: every query head's key, put together from the shared first half and
    its own second half, is the reference's rotated key of that head (the golden file of the 2-D case has distinct
    frequencies inside a group); V is the projection's value row, once per KV head."""
    qkv, fc, fc2, g, (B, S, Hq, Hkv, D) = pre_attention_case(name)
    dtype = qkv.dtype
    L = B * S
    qkv, fc = qkv.reshape(1, L, -1), fc.reshape(1, L, -1)
    fc2 = fc2.reshape(1, L, Hq, -1) if fc2 is not None else None
    gq = torch.from_numpy(g["xq"]).permute(1, 0, 2, 3).reshape(1, Hq, L, D)
    gk = torch.from_numpy(g["xk"]).permute(1, 0, 2, 3).reshape(1, Hq, L, D)
    P = 16
    cache = PagedKVCache(32, P, 8, Hkv, D, 2, dtype, "cuda", split_q_heads=Hq)
    # the layout's size: (3 Hkv + Hq) D / 2 elements per token and layer instead of the expanded 2 Hq D
    assert cache.kv_cache.shape == (2, 32 * P * (3 * Hkv + Hq) * D // 2)
    n0 = L // 2
    s0, s1 = cache.allocate(), cache.allocate()
    cache.reserve(s0, None, n0 + 3); cache.reserve(s1, None, L - n0 + 20)
    bidx = torch.tensor([[s0] * n0 + [s1] * (L - n0)])
    ipos = torch.tensor([list(range(3, 3 + n0)) + list(range(20, 20 + L - n0))])
    xq = cache.pre_attention_append(1, qkv.cuda(), Hq, Hkv, fc.cuda(), fc2.cuda() if fc2 is not None else None,
                                    bidx.cuda(), ipos.cuda())
    cache.check_status()
    ok, info = close_to_ulp(xq, gq, dtype)
    assert ok, ("xq", info)
    v_in = qkv[..., (Hq + Hkv) * D:].reshape(1, L, Hkv, D).permute(0, 2, 1, 3)
    for t, (s, p) in enumerate(zip(bidx.reshape(-1).tolist(), ipos.reshape(-1).tolist())):
        k, v = cache.gather(1, s, p + 1)
        assert tuple(k.shape) == (Hq, p + 1, D) and tuple(v.shape) == (Hkv, p + 1, D)
        ok, info = close_to_ulp(k[:, p], gk[0, :, t], dtype)
        assert ok, ("k", t, info)
        assert torch.equal(v[:, p].cpu(), v_in[0, :, t]), ("v", t)
    assert not cache.kv_cache[0].any()                     # the other layer is untouched
    if fc2 is not None and Hq != Hkv:                       # the case really has different copies inside a group
        assert not torch.equal(gk[0, 0, :, D // 2:], gk[0, 1, :, D // 2:])


def _expanded_inputs(seed, lens, Hq, Hkv, D, dtype, scale=1.0):
    """K as the reference caches it: Hq heads whose first halves agree within a group and whose second halves
    do not; V as Hq identical copies per group."""
    g = torch.Generator().manual_seed(seed)
    n_rep = Hq // Hkv

    def make(n_tok):
        kt = (torch.randn(n_tok, Hkv, D // 2, generator=g) * scale).repeat_interleave(n_rep, 1)
        khw = torch.randn(n_tok, Hq, D // 2, generator=g) * scale
        k = torch.cat([kt, khw], -1).to(dtype)
        v = (torch.randn(n_tok, Hkv, D, generator=g) * scale).repeat_interleave(n_rep, 1).to(dtype)
        return k, v
    hist = [make(n) for n in lens]
    new = make(len(lens))
    q = (torch.randn(len(lens), Hq, 1, D, generator=g) * scale).to(dtype)
    return hist, new, q


@pytest.mark.parametrize("dtype,D,Hq,Hkv", [(torch.bfloat16, 128, 16, 8), (torch.bfloat16, 128, 8, 2), (torch.float16, 128, 4, 2),
                                            (torch.float16, 64, 4, 2), (torch.float32, 64, 4, 2)])
def test_split_pool_holds_the_expanded_cache_and_attends_like_it(dtype, D, Hq, Hkv):
    P, n_pages = 128, 40
    lens = [1, 127, 128, 300, 515, 700]
    n_rep = Hq // Hkv
    hist, (k_new, v_new), q = _expanded_inputs(17, lens, Hq, Hkv, D, dtype)
    c = PagedKVCache(n_pages, P, 8, Hkv, D, 1, dtype, "cuda", split_q_heads=Hq)
    o = orc.OraclePagedKVCache(n_pages, P, 8, Hq, D, 1, dtype)                  # the reference's expanded layout
    perm = (np.random.default_rng(3).permutation(n_pages - 1) + 1).tolist()
    c.free_pages = list(perm); o.free_pages = list(perm)
    slots = []
    for n, (kh, vh) in zip(lens, hist):
        s = c.allocate(); assert o.allocate() == s; slots.append(s)
        c.reserve(s, None, n + 1); o.reserve(s, n + 1)
        kk, vv = kh.permute(1, 0, 2).unsqueeze(0), vh.permute(1, 0, 2).unsqueeze(0)      # (1, Hq, n, D)
        ip, bi = torch.arange(n).view(1, n), torch.full((1, n), s)
        c.insert_kv(0, kk.cuda(), vv.cuda(), input_pos=ip.cuda(), batch_idx=bi.cuda())
        o.append_packed(0, bi, ip, kk, vv)
    bidx = torch.tensor(slots); pos = torch.tensor(lens, dtype=torch.int32)
    kd, vd = k_new.unsqueeze(2), v_new.unsqueeze(2)                             # (B, Hq, 1, D)
    c.insert_kv(0, kd.cuda(), vd.cuda(), input_pos=pos.cuda().view(-1, 1), batch_idx=bidx.cuda())
    o.append_decode(0, bidx, pos, kd, vd)
    # the three regions hold the expanded cache's content, bit for bit (reserved page 0 aside)
    ok_, ov_ = o.kv_cache[0, 0, 0], o.kv_cache[0, 1, 0]                         # (Hq, rows, D)
    assert torch.equal(c.k_first(0)[:, P:].cpu(), ok_[::n_rep, P:, :D // 2])
    assert torch.equal(c.k_second(0)[:, P:].cpu(), ok_[:, P:, D // 2:])
    assert torch.equal(c.v_plane(0)[:, P:].cpu(), ov_[::n_rep, P:])
    gk, gv = c.gather(0, slots[3], lens[3] + 1)
    addr = torch.from_numpy(o.key_addresses(slots[3], lens[3] + 1)[0])
    assert torch.equal(gk.cpu(), ok_[:, addr]) and torch.equal(gv.cpu(), ov_[::n_rep][:, addr])
    # decode attention over the split pool = the oracle's attention over the expanded cache
    ref_out, ref_lse = orc.decode_attention(o, 0, q.float(), bidx, pos)
    kernels = [_lib.DECODE_PORTABLE] + ([_lib.DECODE_AUTO] if dtype != torch.float32 else [])
    if dtype != torch.float32 and D == 128:
        kernels.append(_lib.DECODE_TMA)             # asked for by name: an unsupported shape would be refused, not rerouted
    for kern in kernels:
        c.decode_kernel = kern
        out, lse = paged_attention(q.cuda(), c, 0, bidx.cuda(), pos.cuda())
        assert_attention_close(out, lse, ref_out, ref_lse, f"split decode, kernel {kern}")
    c.check_status()


@pytest.mark.parametrize("Hq,Hkv", [(8, 4), (8, 2), (6, 2)])
@pytest.mark.parametrize("kernel", [_lib.PREFILL_PORTABLE, _lib.PREFILL_AUTO, _lib.PREFILL_TC])
def test_split_pool_prefill(kernel, Hq, Hkv):
    """Packed prefill with an image span over a split pool against the oracle's attention over the expanded K, V."""
    T = wl.image_text_tokens
    D = 128
    n_rep = Hq // Hkv
    case = wl.make_prefill_case(81, [T(3, 150, 40), T(0, 0, 200)], Hq=Hq, Hkv=Hkv, D=D, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(5)
    L = case.L
    kt = torch.randn(1, Hkv, L, D // 2, generator=g).repeat_interleave(n_rep, 1)
    k = torch.cat([kt, torch.randn(1, Hq, L, D // 2, generator=g)], -1).bfloat16()
    v = torch.randn(1, Hkv, L, D, generator=g).repeat_interleave(n_rep, 1).bfloat16()
    c = PagedKVCache(8, 128, 4, Hkv, D, 1, torch.bfloat16, "cuda", split_q_heads=Hq)
    c.prefill_kernel = kernel
    slots = []
    for toks in case.seq_tokens:
        s = c.allocate(); slots.append(s); c.reserve(s, None, len(toks))
    bidx, ipos = case.batch_idx_for(slots).cuda(), case.input_pos.cuda()
    mask = c.create_prefill_blockmask(bidx, case.input_ids.cuda(), wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    c.insert_kv(0, k.cuda(), v.cuda(), input_pos=ipos, batch_idx=bidx)
    out, lse = paged_attention(case.q.bfloat16().cuda(), c, 0, bidx, ipos, mask)
    img = orc.image_span_ids(case.input_ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    ref_out, ref_lse = orc.prefill_attention(case.q.bfloat16().float(), k.float(), v.float(), bidx.cpu(), img)   # Hq "KV" heads: n_rep 1
    live = case.seq_index.view(-1) > 0
    assert_attention_close(out[0][:, live], lse[0][:, live], torch.as_tensor(ref_out)[0][:, live],
                           torch.as_tensor(ref_lse)[0][:, live], f"split prefill, kernel {kernel}")
    c.check_status()


@pytest.mark.parametrize("Hq,Hkv", [(16, 8), (8, 2)])
def test_split_pool_long_contexts_on_the_tiled_decode_kernel(Hq, Hkv):
    """Contexts of many pages (several work units per sequence, partial last groups) on the TMA decode kernel over a
    split pool, against the oracle's attention over the reference's expanded cache."""
    P, D, dtype = 128, 128, torch.bfloat16
    lens = [4097, 2500, 1023, 3333, 640, 2049, 129, 3967]
    n_pages = sum((n + 1 + P - 1) // P for n in lens) + 3
    hist, (k_new, v_new), q = _expanded_inputs(29, lens, Hq, Hkv, D, dtype)
    c = PagedKVCache(n_pages, P, len(lens) + 1, Hkv, D, 1, dtype, "cuda", split_q_heads=Hq)
    o = orc.OraclePagedKVCache(n_pages, P, len(lens) + 1, Hq, D, 1, dtype)
    perm = (np.random.default_rng(5).permutation(n_pages - 1) + 1).tolist()
    c.free_pages = list(perm); o.free_pages = list(perm)
    slots = []
    for n, (kh, vh) in zip(lens, hist):
        s = c.allocate(); assert o.allocate() == s; slots.append(s)
        c.reserve(s, None, n + 1); o.reserve(s, n + 1)
        kk, vv = kh.permute(1, 0, 2).unsqueeze(0), vh.permute(1, 0, 2).unsqueeze(0)
        ip, bi = torch.arange(n).view(1, n), torch.full((1, n), s)
        c.insert_kv(0, kk.cuda(), vv.cuda(), input_pos=ip.cuda(), batch_idx=bi.cuda())
        o.append_packed(0, bi, ip, kk, vv)
    bidx = torch.tensor(slots); pos = torch.tensor(lens, dtype=torch.int32)
    kd, vd = k_new.unsqueeze(2), v_new.unsqueeze(2)
    c.insert_kv(0, kd.cuda(), vd.cuda(), input_pos=pos.cuda().view(-1, 1), batch_idx=bidx.cuda())
    o.append_decode(0, bidx, pos, kd, vd)
    ref_out, ref_lse = orc.decode_attention(o, 0, q.float(), bidx, pos)
    c.decode_kernel = _lib.DECODE_TMA
    out, lse = paged_attention(q.cuda(), c, 0, bidx.cuda(), pos.cuda())
    assert_attention_close(out, lse, ref_out, ref_lse, "split decode, long contexts")
    c.check_status()


def test_split_pool_argument_errors():
    c = PagedKVCache(8, 128, 4, 4, 128, 1, torch.bfloat16, "cuda", split_q_heads=8)
    q4 = torch.zeros(2, 4, 1, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(AssertionError, match="exactly split_q_heads"):
        c.decode_attention(0, q4, torch.tensor([1, 2], device="cuda"), torch.zeros(2, dtype=torch.int32, device="cuda"))
    k4 = torch.zeros(2, 4, 1, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(AssertionError, match="number of heads must match"):     # insert_kv wants the expanded heads
        c.insert_kv(0, k4, k4, input_pos=torch.zeros(2, 1, dtype=torch.int32, device="cuda"),
                    batch_idx=torch.tensor([1, 2], device="cuda"))
    with pytest.raises(AssertionError):
        PagedKVCache(8, 128, 4, 4, 128, 1, torch.bfloat16, "cpu", split_q_heads=6)
