"""GPU: size-independent properties of paged attention at the benchmark's sizes.

Attention is linear in the values and its log-sum-exp does not depend on them; the order of the rows of a decode batch
does not matter.  Values are small dyadic numbers, so that the sum of two value fills is exact in 16 bits and the
only differences left are the kernels' own roundings of the outputs."""

import numpy as np
import pytest
import torch

from fpkv import _lib
import workloads as wl
from fpkv.paged_attention import PagedKVCache, paged_attention

pytestmark = pytest.mark.gpu


def dyadic(shape, gen, device):
    """Multiples of 1/16 in [-1/2, 1/2]: sums of two of them are exact in bf16 and fp16."""
    return (torch.randint(-8, 9, shape, generator=gen, device=device).float() / 16).bfloat16()


def close_in_output_ulps(a, b, what, ulps=3, scale=None):
    """|a - b| within `ulps` bf16 units of `scale` (default: the larger of the two; for a sum of two rounded results
    the roundings are relative to the summands, so the caller passes their magnitudes)."""
    a, b = a.float(), b.float()
    ref = torch.maximum(a.abs(), b.abs()) if scale is None else scale.float()
    tol = ulps * 2.0 ** -8 * ref.clamp_min(2.0 ** -6)
    bad = (a - b).abs() > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} elements differ by more than {ulps} bf16 ulps, worst {(a - b).abs().max().item()}"


@pytest.mark.parametrize("kernel", [_lib.DECODE_TMA, _lib.DECODE_PORTABLE])
def test_decode_is_linear_in_the_values_and_blind_to_row_order(kernel):
    """Config 2's batch (64 sequences of 1K-8K tokens, 16 / 8 heads, head_dim 128) on a pool of the pages in use."""
    dev = torch.device("cuda")
    B, Hq, Hkv, D, P, n_pages = 64, 16, 8, 128, 128, 4096
    rng = np.random.default_rng(77)
    lens = rng.integers(1024, 8193, size=B).tolist()
    c = PagedKVCache(n_pages, P, B + 1, Hkv, D, 1, torch.bfloat16, dev)
    c.decode_kernel = kernel
    c.free_pages = (rng.permutation(n_pages - 1) + 1).tolist()
    slots = []
    for n in lens:
        s = c.allocate(); slots.append(s); c.reserve(s, None, n + 1)
    g = torch.Generator(device=dev).manual_seed(5)
    pool = c.kv_cache.view(2, Hkv, n_pages, P, D)
    pool[0].copy_((torch.randn((Hkv, n_pages, P, D), device=dev, generator=g) * D ** -0.5).bfloat16())
    va, vb = dyadic((Hkv, n_pages, P, D), g, dev), dyadic((Hkv, n_pages, P, D), g, dev)
    q = torch.randn((B, Hq, 1, D), device=dev, generator=g).bfloat16()
    bidx = torch.tensor(slots, device=dev); pos = torch.tensor(lens, dtype=torch.int32, device=dev)
    outs = []
    for v in (va, vb, (va.float() + vb.float()).bfloat16()):
        pool[1].copy_(v)
        outs.append(paged_attention(q, c, 0, bidx, pos))
    (oa, la), (ob, lb), (oab, lab) = outs
    assert torch.equal(la, lb) and torch.equal(la, lab), "the log-sum-exp depends on the values"
    close_in_output_ulps(oa.float() + ob.float(), oab, "decode: out(Va) + out(Vb) against out(Va + Vb)",
                         scale=oa.float().abs() + ob.float().abs())
    perm = torch.from_numpy(rng.permutation(B)).to(dev)
    op, lp = paged_attention(q[perm].contiguous(), c, 0, bidx[perm].contiguous(), pos[perm].contiguous())
    close_in_output_ulps(op, oab[perm], "decode: batch rows in another order", ulps=2)
    assert (lp - lab[perm]).abs().max().item() < 1e-4
    c.check_status()


@pytest.mark.parametrize("kernel", [_lib.PREFILL_TC, _lib.PREFILL_PORTABLE])
def test_prefill_is_linear_in_the_values(kernel):
    """Config 3's packed row (8 x (1024 image + 64 text) tokens, image-prefix mask)."""
    dev = torch.device("cuda")
    case = wl.config3_prefill_case()
    c = PagedKVCache(96, 128, 12, case.Hkv, case.D, 1, torch.bfloat16, dev)
    c.prefill_kernel = kernel
    slots = []
    for toks in case.seq_tokens:
        s = c.allocate(); slots.append(s); c.reserve(s, None, len(toks))
    bidx, ipos = case.batch_idx_for(slots).to(dev), case.input_pos.to(dev)
    mask = c.create_prefill_blockmask(bidx, case.input_ids.to(dev), wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    g = torch.Generator(device=dev).manual_seed(6)
    q, k = case.q.bfloat16().to(dev), case.k.bfloat16().to(dev)
    va, vb = dyadic(tuple(case.v.shape), g, dev), dyadic(tuple(case.v.shape), g, dev)
    outs = []
    for v in (va, vb, (va.float() + vb.float()).bfloat16()):
        c.insert_kv(0, k, v, input_pos=ipos, batch_idx=bidx)
        outs.append(paged_attention(q, c, 0, bidx, ipos, mask))
    (oa, la), (ob, lb), (oab, lab) = outs
    assert torch.equal(la, lb) and torch.equal(la, lab), "the log-sum-exp depends on the values"
    close_in_output_ulps(oa.float() + ob.float(), oab, "prefill: out(Va) + out(Vb) against out(Va + Vb)",
                         scale=oa.float().abs() + ob.float().abs())
    c.check_status()


def test_split_pool_equals_uniform_pool_when_the_copies_agree():
    """Config 2's batch: a split pool whose per-query-head second halves are copies of the KV head's second half holds
    the same cache as the uniform pool, and decode attention over the two gives the same rows."""
    dev = torch.device("cuda")
    B, Hq, Hkv, D, P, n_pages = 64, 16, 8, 128, 128, 4096
    n_rep = Hq // Hkv
    rng = np.random.default_rng(78)
    lens = rng.integers(1024, 8193, size=B).tolist()
    perm = (rng.permutation(n_pages - 1) + 1).tolist()
    caches = []
    for split in (None, Hq):
        c = PagedKVCache(n_pages, P, B + 1, Hkv, D, 1, torch.bfloat16, dev, split_q_heads=split)
        c.decode_kernel = _lib.DECODE_TMA
        c.free_pages = list(perm)
        slots = []
        for n in lens:
            s = c.allocate(); slots.append(s); c.reserve(s, None, n + 1)
        caches.append((c, slots))
    (u, slots), (s, slots_s) = caches
    assert slots == slots_s and u.page_table_cpu[slots[0]] == s.page_table_cpu[slots[0]]
    g = torch.Generator(device=dev).manual_seed(9)
    k = (torch.randn((Hkv, n_pages * P, D), device=dev, generator=g) * D ** -0.5).bfloat16()
    v = (torch.randn((Hkv, n_pages * P, D), device=dev, generator=g) * D ** -0.5).bfloat16()
    pool = u.kv_cache.view(2, Hkv, n_pages * P, D)
    pool[0].copy_(k); pool[1].copy_(v)
    s.k_first(0).copy_(k[:, :, :D // 2])
    s.k_second(0).copy_(k[:, :, D // 2:].repeat_interleave(n_rep, 0))
    s.v_plane(0).copy_(v)
    del k, v
    q = torch.randn((B, Hq, 1, D), device=dev, generator=g).bfloat16()
    bidx = torch.tensor(slots, device=dev); pos = torch.tensor(lens, dtype=torch.int32, device=dev)
    ou, lu = paged_attention(q, u, 0, bidx, pos)
    os_, ls = paged_attention(q, s, 0, bidx, pos)
    close_in_output_ulps(os_, ou, "split pool against uniform pool", ulps=2)
    assert (ls - lu).abs().max().item() < 1e-4
    u.check_status(); s.check_status()
