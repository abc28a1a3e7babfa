"""GPU: the fused norm + rotary embedding + append step (fpkv_pre_append) against the oracle's
pre_attention_tail (pinned to the reference's Attention._pre_attention by the golden files) followed by the
oracle's append.  The step is floating-point work: results may differ from the reference where the order
of the fp32 sum of squares matters, by at most one unit in the last place of the storage type on a small
fraction of the elements; values (V) are copied and must be bit-exact."""

import numpy as np
import pytest
import torch

import workloads as wl
from fpkv.paged_attention import PagedKVCache
from oracle import paged_kv_oracle as orc
from test_oracle_golden import pre_attention_case

pytestmark = pytest.mark.gpu


def close_to_ulp(got, ref, dtype):
    """16-bit storage: all elements within one unit in the last place and at least 99 % identical (the fp32
    differences almost always vanish in the rounding).  fp32 storage: nothing hides the order of the sum of
    squares; absolute error below 2e-6 on values of order one (a few fp32 ulps through norm and rotation; a
    rotated pair may cancel to a small value, so the bound is absolute)."""
    got, ref = got.float().cpu(), ref.float().cpu()
    same = (got == ref).float().mean().item()
    rel = ((got - ref).abs() / ref.abs().clamp_min(1e-3)).max().item()
    if dtype == torch.float32:
        err = (got - ref).abs().max().item()
        return err <= 2e-6, (same, err)
    ulp = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}[dtype]
    return same >= 0.99 and rel <= 1.01 * ulp, (same, rel)


def run_case(name, expanded, packed):
    qkv, fc, fc2, g, (B, S, Hq, Hkv, D) = pre_attention_case(name)
    dtype = qkv.dtype
    if packed:                                             # one packed row: the engine's prefill form
        qkv, fc = qkv.reshape(1, B * S, -1), fc.reshape(1, B * S, -1)
        fc2 = fc2.reshape(1, B * S, Hq, -1) if fc2 is not None else None
        gq = torch.from_numpy(g["xq"]).permute(1, 0, 2, 3).reshape(1, Hq, B * S, D)
        gk = torch.from_numpy(g["xk"]).permute(1, 0, 2, 3).reshape(1, Hq, B * S, D)
        B, S = 1, B * S
    else:
        gq, gk = torch.from_numpy(g["xq"]), torch.from_numpy(g["xk"])
    if not packed and S != 1:
        pytest.skip("a decode step has one token per row")
    H = Hq if expanded else Hkv
    P = 16
    cache = PagedKVCache(32, P, 8, H, D, 2, dtype, "cuda")
    if packed:                                             # two sequences side by side in the packed row
        n0 = S // 2
        s0, s1 = cache.allocate(), cache.allocate()
        cache.reserve(s0, None, n0 + 3); cache.reserve(s1, None, S - n0 + 20)
        bidx = torch.tensor([[s0] * n0 + [s1] * (S - n0)])
        ipos = torch.tensor([list(range(3, 3 + n0)) + list(range(20, 20 + S - n0))])
    else:
        slots = [cache.allocate() for _ in range(B)]
        lens = [5 + 7 * i for i in range(B)]
        for s, n in zip(slots, lens):
            cache.reserve(s, None, n + 1)
        bidx = torch.tensor(slots)
        ipos = torch.tensor(lens, dtype=torch.int32).view(B, 1)
    xq = cache.pre_attention_append(1, qkv.cuda(), Hq, Hkv, fc.cuda(), fc2.cuda() if fc2 is not None else None,
                                    bidx.cuda(), ipos.cuda())
    cache.check_status()
    # queries: against the reference's own output
    ok, info = close_to_ulp(xq, gq, dtype)
    assert ok, ("xq", info)
    # keys and values: read back through the page table, against the reference's rotated keys
    n_rep = Hq // Hkv
    ref_k = gk if expanded else gk[:, ::n_rep]            # compact pool: the first query head's copy of each group
    v_in = qkv[..., (Hq + Hkv) * D:].reshape(B, S, Hkv, D)
    ref_v = (v_in.repeat_interleave(n_rep, 2) if expanded else v_in).permute(0, 2, 1, 3)
    flat_slot, flat_pos = bidx.reshape(-1).tolist(), ipos.reshape(-1).tolist()
    for t, (s, p) in enumerate(zip(flat_slot, flat_pos)):
        k, v = cache.gather(1, s, p + 1)
        b_, s_ = (0, t) if packed else (t, 0)
        ok, info = close_to_ulp(k[:, p], ref_k[b_, :, s_], dtype)
        assert ok, ("k", t, info)
        assert torch.equal(v[:, p].cpu(), ref_v[b_, :, s_]), ("v", t)
    # nothing else was written: layer 0 untouched
    assert not cache.kv_cache[0].any()
    return cache


@pytest.mark.parametrize("name", list(wl.PRE_ATTENTION_CASES))
@pytest.mark.parametrize("expanded", [True, False])
def test_packed_prefill_form(name, expanded):
    seed, B, S, Hq, Hkv, D, with_2d, dtype = wl.PRE_ATTENTION_CASES[name]
    if not expanded and with_2d and Hq != Hkv:
        # the compact pool keeps the first query head's rotation of each group: compare exactly that
        pass
    run_case(name, expanded, packed=True)


@pytest.mark.parametrize("expanded", [True, False])
def test_decode_form(expanded):
    run_case("pre_attention_bf16_text", expanded, packed=False)


def test_same_as_separate_calls_then_attention():
    """The fused step followed by decode attention equals norm + rotary in torch, insert_kv and attention."""
    name = "pre_attention_bf16_text"
    qkv, fc, fc2, g, (B, S, Hq, Hkv, D) = pre_attention_case(name)
    a = PagedKVCache(16, 128, 8, Hkv, D, 1, qkv.dtype, "cuda")
    b = PagedKVCache(16, 128, 8, Hkv, D, 1, qkv.dtype, "cuda")
    slots = [a.allocate() for _ in range(B)]
    for _ in range(B):
        b.allocate()
    for s in slots:
        a.reserve(s, None, 1); b.reserve(s, None, 1)
    bidx = torch.tensor(slots, device="cuda"); ipos = torch.zeros(B, 1, dtype=torch.int32, device="cuda")
    xq = a.pre_attention_append(0, qkv.cuda(), Hq, Hkv, fc.cuda(), None, bidx, ipos)
    oq, ok_, ov = orc.pre_attention_tail(qkv, Hq, Hkv, D, fc, None)
    n_rep = Hq // Hkv
    b.insert_kv(0, ok_[:, ::n_rep].contiguous().cuda(), ov[:, ::n_rep].contiguous().cuda(), input_pos=ipos, batch_idx=bidx)
    out_a, lse_a = a.decode_attention(0, xq, bidx, ipos.view(-1))
    out_b, lse_b = b.decode_attention(0, oq.contiguous().cuda(), bidx, ipos.view(-1))
    # one key per row: the output is that key's value
    assert torch.equal(out_a, out_b) or (out_a.float() - out_b.float()).abs().max().item() < 1e-2
    assert (lse_a - lse_b).abs().max().item() < 2e-2


def test_argument_errors():
    from fpkv import _lib
    cache = PagedKVCache(8, 16, 4, 4, 128, 1, torch.bfloat16, "cuda")
    qkv = torch.zeros(1, 1, (8 + 2 * 4) * 128, dtype=torch.bfloat16, device="cuda")
    fc = torch.ones(1, 1, 32, dtype=torch.complex64, device="cuda")
    with pytest.raises(AssertionError):                   # pool holds neither head count
        cache.pre_attention_append(0, qkv, 16, 2, fc, None, torch.tensor([1], device="cuda"),
                                   torch.zeros(1, 1, dtype=torch.int32, device="cuda"))
    with pytest.raises(AssertionError):                   # width does not match the head counts
        cache.pre_attention_append(0, qkv[..., :-128], 8, 4, fc, None, torch.tensor([1], device="cuda"),
                                   torch.zeros(1, 1, dtype=torch.int32, device="cuda"))
