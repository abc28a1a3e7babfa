"""GPU: K/V append and gather through the C ABI, bit-exact against the oracle
and against pool digests recorded from the reference."""

import hashlib

import numpy as np
import pytest
import torch

import workloads as wl
from fpkv.paged_attention import PagedKVCache
from oracle import paged_kv_oracle as orc
from helpers import golden, oracle_from_case, product_from_case
from test_oracle_golden import DECODE_CASES, PREFILL_CASES

pytestmark = pytest.mark.gpu


def digest(pool_l, P):
    return hashlib.sha256(pool_l[:, :, :, P:, :].contiguous().cpu().numpy().tobytes()).hexdigest()


@pytest.mark.parametrize("name", sorted(DECODE_CASES))
def test_append_matches_reference_digest(name):
    """fp32 pool: packed history append + decode append land exactly where the
    reference put them (page 0, where pad rows collide, is excluded)."""
    make, pads = DECODE_CASES[name]
    case = make()
    case.dtype = torch.float32
    for lst in (case.k_hist, case.v_hist):
        lst[:] = [t.float() for t in lst]
    case.k_new, case.v_new, case.q = case.k_new.float(), case.v_new.float(), case.q.float()
    c, slots, *_ = product_from_case(case, pad_rows=pads)
    g = golden(name)
    assert slots == g["slots"].tolist()
    assert np.array_equal(c.page_table.cpu().numpy(), g["page_table"])
    assert digest(c.kv_cache[0], case.P) == str(g["pool_sha256"])
    c.check_status()


@pytest.mark.parametrize("name", sorted(DECODE_CASES))
def test_append_bit_exact_native_dtype(name):
    make, pads = DECODE_CASES[name]
    case = make()
    c, slots, bidx, pos, k, v, q = product_from_case(case, pad_rows=pads)
    o, *_ = oracle_from_case(case, pad_rows=pads)
    P = case.P
    assert torch.equal(c.kv_cache[0][:, :, :, P:, :].cpu(), o.kv_cache[0][:, :, :, P:, :])
    # gather reads back exactly what was appended, in logical order
    for s, L, kh, vh in zip(slots, case.lens, case.k_hist, case.v_hist):
        gk, gv = c.gather(0, s, L + 1)
        i = slots.index(s)
        assert torch.equal(gk[:, :L].cpu(), kh[0]) and torch.equal(gv[:, :L].cpu(), vh[0])
        assert torch.equal(gk[:, L].cpu(), case.k_new[i, :, 0]) and torch.equal(gv[:, L].cpu(), case.v_new[i, :, 0])
    c.check_status()


@pytest.mark.parametrize("name", sorted(PREFILL_CASES))
def test_packed_append_matches_reference(name):
    make, n_pages, mb = PREFILL_CASES[name]
    case = make()
    g = golden(name)
    c = PagedKVCache(n_pages, case.P, mb, case.Hkv, case.D, 1, torch.float32, "cuda")
    slots = []
    for toks in case.seq_tokens:
        s = c.allocate(); slots.append(s); c.reserve(s, None, len(toks))
    bidx = case.batch_idx_for(slots).cuda()
    k, v = case.k.float().cuda(), case.v.float().cuda()
    rk, rv = c.insert_kv(0, k, v, input_pos=case.input_pos.cuda(), batch_idx=bidx)
    assert rk is k and rv is v                   # prefill attends over the fresh tensors
    assert digest(c.kv_cache[0], case.P) == str(g["pool_sha256"])
    c.check_status()


def test_strided_views_need_no_copy():
    """The model hands (B,S,H,D)->(B,H,S,D) permuted views; rows are read in place."""
    torch.manual_seed(0)
    B, H, D, P = 5, 4, 128, 16
    c = PagedKVCache(32, P, 8, H, D, 2, torch.bfloat16, "cuda")
    o = orc.OraclePagedKVCache(32, P, 8, H, D, 2, torch.bfloat16)
    slots = []
    for _ in range(B):
        s = c.allocate(); o.allocate(); c.reserve(s, None, 40); o.reserve(s, 40); slots.append(s)
    bidx = torch.tensor(slots, device="cuda"); pos = torch.tensor([0, 15, 16, 17, 39], dtype=torch.int32, device="cuda")
    # k and v as the model makes them: slices of one fused qkv projection output
    qkv = torch.randn(B, 1, 4 * H * D, device="cuda").to(torch.bfloat16)
    k = qkv[..., 2 * H * D:3 * H * D].view(B, 1, H, D).permute(0, 2, 1, 3)
    v = qkv[..., 3 * H * D:].view(B, 1, H, D).permute(0, 2, 1, 3)
    assert not k.is_contiguous() and not v.is_contiguous()
    K, V = c.insert_kv(1, k, v, input_pos=pos.view(B, 1), batch_idx=bidx)
    assert K.data_ptr() == c.kv_cache[1, 0].data_ptr() and tuple(K.shape) == (1, H, 32 * P, D)
    o.append_decode(1, bidx.cpu(), pos.cpu(), k.cpu(), v.cpu())
    assert torch.equal(c.kv_cache.cpu(), o.kv_cache)
    # packed, int64 positions, permuted (1,L,H,D) source
    L = 37
    kp = torch.randn(1, L, H, D, device="cuda").to(torch.bfloat16).permute(0, 2, 1, 3)
    vp = torch.randn(1, L, H, D, device="cuda").to(torch.bfloat16).permute(0, 2, 1, 3)
    ip = torch.arange(L, device="cuda").view(1, L); bi = torch.full((1, L), slots[2], device="cuda")
    c.insert_kv(0, kp, vp, input_pos=ip, batch_idx=bi)
    o.append_packed(0, bi.cpu(), ip.cpu(), kp.cpu(), vp.cpu())
    assert torch.equal(c.kv_cache.cpu(), o.kv_cache)
    c.check_status()


def test_unmapped_and_bad_indices_raise_status_not_faults():
    c = PagedKVCache(8, 16, 4, 2, 64, 1, torch.float32, "cuda")
    s = c.allocate(); c.reserve(s, None, 16)
    k = torch.ones(2, 2, 1, 64, device="cuda")
    # decode: a position past the reserved pages has page id -1 -> reserved page 0, as in the reference
    c.insert_kv(0, k, k, input_pos=torch.tensor([[3], [20]], dtype=torch.int32, device="cuda"),
                batch_idx=torch.tensor([s, s], device="cuda"))
    assert c.kv_cache[0, 0, 0, :, 16 * c.page_table_cpu[s][0] + 3].eq(1).all()
    assert c.kv_cache[0, 0, 0, :, 4].eq(1).all()          # 20 % 16 inside page 0
    c.check_status()
    # slot out of range: skipped and reported
    c.insert_kv(0, k, k, input_pos=torch.tensor([[3], [3]], dtype=torch.int32, device="cuda"),
                batch_idx=torch.tensor([s, 99], device="cuda"))
    with pytest.raises(RuntimeError, match="bad slot"):
        c.check_status()
    c.insert_kv(0, k, k, input_pos=torch.tensor([[3], [100000]], dtype=torch.int32, device="cuda"),
                batch_idx=torch.tensor([s, s], device="cuda"))
    with pytest.raises(RuntimeError, match="bad position"):
        c.check_status()
    # packed: an unmapped page is a caller error
    kp = torch.ones(1, 2, 2, 64, device="cuda")
    c.insert_kv(0, kp, kp, input_pos=torch.tensor([[1, 40]], device="cuda"), batch_idx=torch.tensor([[s, s]], device="cuda"))
    with pytest.raises(RuntimeError, match="bad page"):
        c.check_status()


def test_full_size_round_trip():
    """Config-2 sized batch (64 rows, 8 heads, head_dim 128, bf16) over a large
    permuted pool: append then gather returns the appended rows."""
    case = wl.config2_case(n_pages=8192, with_history=False)
    c = PagedKVCache(case.n_pages, case.P, case.max_batch_size, case.Hkv, case.D, 1, torch.bfloat16, "cuda")
    c.free_pages = list(case.free_pages)
    slots = []
    for L in case.lens:
        s = c.allocate(); c.reserve(s, None, L + 1); slots.append(s)
    bidx = torch.tensor(slots, device="cuda"); pos = torch.tensor(case.lens, dtype=torch.int32, device="cuda")
    k, v = case.k_new.cuda(), case.v_new.cuda()
    c.insert_kv(0, k, v, input_pos=pos.view(-1, 1), batch_idx=bidx)
    for i in (0, 17, 63):
        gk, gv = c.gather(0, slots[i], case.lens[i] + 1)
        assert torch.equal(gk[:, -1], k[i, :, 0]) and torch.equal(gv[:, -1], v[i, :, 0])
        assert gk[:, :-1].abs().max().item() == 0          # untouched history is still zero
    assert int(c.kv_cache.ne(0).any(-1).sum().item()) == 2 * 8 * 64   # exactly B rows per head and K/V written
    c.check_status()
