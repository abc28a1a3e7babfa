"""GPU: paged decode attention through the C ABI against the golden vectors
(reference, fp32) and the CPU oracle, for both kernels."""

import numpy as np
import pytest
import torch

from fpkv import _lib
import workloads as wl
from fpkv.paged_attention import PagedKVCache, paged_attention
from oracle import paged_kv_oracle as orc
from helpers import assert_attention_close, golden, oracle_from_case, product_from_case
from test_oracle_golden import DECODE_CASES

pytestmark = pytest.mark.gpu

KERNELS = {"portable": _lib.DECODE_PORTABLE, "tma": _lib.DECODE_TMA}


def tma_takes(case):
    return case.dtype in (torch.bfloat16, torch.float16) and case.P == 128 and case.Hq // case.Hkv in (1, 2, 4, 8)


@pytest.mark.parametrize("kernel", sorted(KERNELS))
@pytest.mark.parametrize("name", sorted(DECODE_CASES))
def test_decode_against_reference_golden(name, kernel):
    make, pads = DECODE_CASES[name]
    case = make()
    if kernel == "tma" and not tma_takes(case):
        pytest.skip("shape outside the TMA kernel's range (served by the portable kernel)")
    g = golden(name)
    c, slots, bidx, pos, k, v, q = product_from_case(case, pad_rows=pads)
    c.decode_kernel = KERNELS[kernel]
    out, lse = paged_attention(q, c, 0, bidx, pos)
    assert out.dtype == q.dtype and lse.dtype == torch.float32
    assert tuple(out.shape) == tuple(q.shape) and tuple(lse.shape) == tuple(q.shape[:3])
    assert_attention_close(out, lse, g["out"], g["lse"], f"{name}/{kernel}")
    c.check_status()


def test_config1_fp32_auto_kernel():
    """The CPU-runnable configuration, fp32 end to end."""
    case = wl.config1_case()
    g = golden("decode_cfg1")
    c, slots, bidx, pos, k, v, q = product_from_case(case)
    out, lse = paged_attention(q, c, 0, bidx, pos)
    assert (out.cpu() - torch.from_numpy(g["out"])).abs().max().item() < 1e-4
    assert (lse.cpu() - torch.from_numpy(g["lse"])).abs().max().item() < 1e-4


def _random_case(seed, **kw):
    d = dict(B=9, Hq=16, Hkv=8, D=128, P=128, n_pages=96, max_batch_size=12, len_lo=1, len_hi=1100,
             dtype=torch.bfloat16, value_scale=1.0)
    d.update(kw)
    return wl.make_decode_case(seed, **d)


@pytest.mark.parametrize("kernel", sorted(KERNELS))
@pytest.mark.parametrize("kw", [
    dict(),                                                        # GQA 2:1, D=128 (the headline layout)
    dict(value_scale=128 ** -0.5),                                 # config-2 value scaling (near-uniform softmax)
    dict(D=64, Hq=8, Hkv=8),                                       # MHA, D=64
    dict(Hq=32, Hkv=8, dtype=torch.float16),                       # GQA 4:1 fp16
    dict(Hq=16, Hkv=2, D=64),                                      # GQA 8:1
    dict(lens=[127, 128, 129, 255, 256, 257, 0, 1, 1023]),         # page boundaries
    dict(B=1, lens=[700]),                                         # single row
], ids=["gqa2", "scaled", "mha64", "gqa4f16", "gqa8", "edges", "one"])
def test_decode_against_oracle(kw, kernel):
    case = _random_case(4242, **kw)
    c, slots, bidx, pos, k, v, q = product_from_case(case, pad_rows=1)
    c.decode_kernel = KERNELS[kernel]
    o, _, obidx, opos, ok, ov, oq = oracle_from_case(case, pad_rows=1)
    ref_out, ref_lse = orc.decode_attention(o, 0, oq.float(), obidx, opos)
    out, lse = c.decode_attention(0, q, bidx, pos)
    assert_attention_close(out, lse, ref_out, ref_lse, f"{kw}/{kernel}")
    # scratch contents must not matter: poison the workspace (NaN bit patterns) past its 16 KiB header
    # (whose counter words every call leaves at zero) and rerun
    assert int(c._workspace[:1024].max().item()) == 0
    c._workspace[16384:].fill_(255)
    out2, lse2 = c.decode_attention(0, q, bidx, pos)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)
    # the padding row (slot 0) sees nothing
    assert out[-1].abs().max().item() == 0 and torch.isneginf(lse[-1]).all()
    c.check_status()


@pytest.mark.parametrize("kernel", sorted(KERNELS))
def test_one_hot_key_returns_its_value_row(kernel):
    """A key that matches q with a huge score: the answer is that row of V."""
    case = _random_case(77, B=4, lens=[300, 513, 128, 90])
    hot = [17, 400, 127, 0]
    for i, t in enumerate(hot):
        kh = case.k_hist[i]
        kh[0, :, t, :] = 0
        for h in range(case.Hkv):
            # both query heads of the group point at +e0; the hot key has a large e0 component
            kh[0, h, t, 0] = 200.0
        case.q[i, :, 0, :] = 0
        case.q[i, :, 0, 0] = 8.0
    c, slots, bidx, pos, k, v, q = product_from_case(case)
    c.decode_kernel = KERNELS[kernel]
    out, lse = c.decode_attention(0, q, bidx, pos)
    for i, t in enumerate(hot):
        want = case.v_hist[i][0, :, t, :].repeat_interleave(2, 0).float()
        assert (out[i, :, 0].float().cpu() - want).abs().max().item() <= 2e-2
        assert abs(lse[i, 0, 0].item() - 8.0 * 200.0 / 128 ** 0.5) < 0.2


def test_multi_layer_and_reused_pages():
    """Layers are independent planes; pages freed by one sequence and reused by
    another (non-contiguous tables) read correctly."""
    torch.manual_seed(3)
    H, Hq, D, P, NL = 8, 16, 128, 128, 3
    c = PagedKVCache(40, P, 6, H, D, NL, torch.bfloat16, "cuda")
    o = orc.OraclePagedKVCache(40, P, 6, H, D, NL, torch.bfloat16)

    def admit(L, layer):
        s = c.allocate(); assert o.allocate() == s
        c.reserve(s, None, L + 1); o.reserve(s, L + 1)
        kh, vh = torch.randn(1, H, L, D).bfloat16(), torch.randn(1, H, L, D).bfloat16()
        ip, bi = torch.arange(L).view(1, L), torch.full((1, L), s)
        c.insert_kv(layer, kh.cuda(), vh.cuda(), input_pos=ip.cuda(), batch_idx=bi.cuda())
        o.append_packed(layer, bi, ip, kh, vh)
        return s
    a = admit(700, 1); b = admit(300, 1); d = admit(500, 1)
    c.erase(b); o.erase(b); c.erase(a); o.erase(a)
    e = admit(900, 1)                                  # takes a's and b's pages back, out of order
    assert c.page_table_cpu[e] == o.page_table_cpu[e] and sorted(c.page_table_cpu[e]) != c.page_table_cpu[e]
    lens = {d: 500, e: 900}
    bidx = torch.tensor([e, d]); pos = torch.tensor([lens[e], lens[d]], dtype=torch.int32)
    k, v, q = (torch.randn(2, n, 1, D).bfloat16() for n in (H, H, Hq))
    c.insert_kv(1, k.cuda(), v.cuda(), input_pos=pos.cuda().view(2, 1), batch_idx=bidx.cuda())
    o.append_decode(1, bidx, pos, k, v)
    ref_out, ref_lse = orc.decode_attention(o, 1, q.float(), bidx, pos)
    for kern in KERNELS.values():
        c.decode_kernel = kern
        out, lse = c.decode_attention(1, q.cuda(), bidx.cuda(), pos.cuda())
        assert_attention_close(out, lse, ref_out, ref_lse, "reused pages")
    assert c.kv_cache[0].abs().max().item() == 0 and c.kv_cache[2].abs().max().item() == 0
    c.check_status()


def test_config2_full_size_every_row_against_the_oracle():
    """BASELINE config 2 at full size: batch 64, context 1K-8K, page ids permuted over the 65 536-page pool
    (32 GiB).  The context K/V is written through the packed append on the device and through the oracle's
    append on the host (its pool holds only the pages in use; it runs its own allocator, so its page ids
    differ and only the logical content is shared), then one decode step: every row of both kernels against
    the oracle's attention, the appended pool read back bit for bit, and a rerun bitwise equal."""
    case = wl.config2_case(with_history=False)
    assert case.n_pages == 65536 and case.B == 64
    c = PagedKVCache(case.n_pages, case.P, case.max_batch_size, case.Hkv, case.D, 1, torch.bfloat16, "cuda")
    c.free_pages = list(case.free_pages)
    used = sum((L + 1 + case.P - 1) // case.P for L in case.lens)
    o = orc.OraclePagedKVCache(used + 1, case.P, case.max_batch_size, case.Hkv, case.D, 1, torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(5)
    slots = []
    for L in case.lens:
        s = c.allocate(); assert o.allocate() == s; slots.append(s)
        c.reserve(s, None, L + 1); o.reserve(s, L + 1)
        kh = (torch.randn((1, case.Hkv, L, case.D), device="cuda", generator=g) * case.D ** -0.5).bfloat16()
        vh = (torch.randn((1, case.Hkv, L, case.D), device="cuda", generator=g) * case.D ** -0.5).bfloat16()
        ip, bi = torch.arange(L, device="cuda").view(1, L), torch.full((1, L), s, device="cuda")
        c.insert_kv(0, kh, vh, input_pos=ip, batch_idx=bi)
        o.append_packed(0, bi.cpu(), ip.cpu(), kh.cpu(), vh.cpu())
    # scattered over the whole pool, not a compact prefix of it
    pages = [p for s in slots for p in c.page_table_cpu[s]]
    assert len(pages) == used and max(pages) > 60000 and min(pages) < 5000
    bidx = torch.tensor(slots); pos = torch.tensor(case.lens, dtype=torch.int32)
    k, v, q = case.k_new.cuda(), case.v_new.cuda(), case.q.cuda()
    c.insert_kv(0, k, v, input_pos=pos.cuda().view(-1, 1), batch_idx=bidx.cuda())
    o.append_decode(0, bidx, pos, case.k_new, case.v_new)
    ref_out, ref_lse = orc.decode_attention(o, 0, case.q.float(), bidx, pos)
    for name, kern in KERNELS.items():
        c.decode_kernel = kern
        out, lse = c.decode_attention(0, q, bidx.cuda(), pos.cuda())
        assert_attention_close(out, lse, ref_out, ref_lse, f"config 2, all 64 rows, {name}")
        out2, lse2 = c.decode_attention(0, q, bidx.cuda(), pos.cuda())
        assert torch.equal(out, out2) and torch.equal(lse, lse2), name
    # the pool, read back through the page table, holds exactly what the oracle's pool holds
    for i in (0, 17, 40, 63):
        gk, gv = c.gather(0, slots[i], case.lens[i] + 1)
        addr, valid = o.key_addresses(slots[i], case.lens[i] + 1)
        assert valid.all()
        assert torch.equal(gk.cpu(), o.kv_cache[0, 0, 0][:, torch.from_numpy(addr)])
        assert torch.equal(gv.cpu(), o.kv_cache[0, 1, 0][:, torch.from_numpy(addr)])
    c.check_status()


def test_rows_never_appended_may_hold_anything():
    """The pool a caller hands over through the C ABI need not be zero-filled: rows behind a sequence's last
    key (the tail of its last page, fetched with the page) may hold NaN or Inf bit patterns without reaching
    any result."""
    case = _random_case(626, B=7, lens=[1, 15, 16, 17, 130, 255, 300], n_pages=40, max_batch_size=9)
    o, _, obidx, opos, ok, ov, oq = oracle_from_case(case)
    ref_out, ref_lse = orc.decode_attention(o, 0, oq.float(), obidx, opos)
    from fpkv.paged_attention import PagedKVCache as Cache
    c = Cache(case.n_pages, case.P, case.max_batch_size, case.Hkv, case.D, 1, case.dtype, "cuda")
    c.kv_cache.view(torch.int16).fill_(-1)                       # 0xFFFF: a NaN in bf16 and fp16
    c.free_pages = list(case.free_pages)
    slots = []
    for L, kh, vh in zip(case.lens, case.k_hist, case.v_hist):
        s = c.allocate(); slots.append(s); c.reserve(s, None, L + 1)
        c.insert_kv(0, kh.cuda(), vh.cuda(), input_pos=torch.arange(L, device="cuda").view(1, L),
                    batch_idx=torch.full((1, L), s, device="cuda"))
    bidx = torch.tensor(slots, device="cuda"); pos = torch.tensor(case.lens, dtype=torch.int32, device="cuda")
    c.insert_kv(0, case.k_new.cuda(), case.v_new.cuda(), input_pos=pos.view(-1, 1), batch_idx=bidx)
    for name, kern in KERNELS.items():
        c.decode_kernel = kern
        out, lse = c.decode_attention(0, case.q.cuda(), bidx, pos)
        assert torch.isfinite(out.float()).all(), name
        assert_attention_close(out, lse, ref_out, ref_lse, f"NaN-filled pool, {name}")
    c.check_status()


def test_decode_step_equals_separate_calls():
    """The fused step (append, then attention whose set-up overlaps the append)
    gives bit-identical results to insert_kv + paged_attention, step after step."""
    case = _random_case(515, B=12, lens=[5, 127, 128, 300, 511, 640, 900, 1023, 64, 33, 700, 256], n_pages=160,
                        max_batch_size=14)
    ca, slots, bidx, pos, k, v, q = product_from_case(case)
    cb, *_ = product_from_case(case)
    o, _, obidx, opos, ok, ov, oq = oracle_from_case(case)
    g = torch.Generator().manual_seed(1)
    for step in range(1, 6):
        kn, vn, qn = (torch.randn(12, n, 1, 128, generator=g).bfloat16() for n in (8, 8, 16))
        p = pos + step
        for s_ in slots:
            ca.reserve(s_, None, 1100); cb.reserve(s_, None, 1100)
        ca.insert_kv(0, kn.cuda(), vn.cuda(), input_pos=p.view(-1, 1), batch_idx=bidx)
        out_a, lse_a = paged_attention(qn.cuda(), ca, 0, bidx, p)
        out_b, lse_b = cb.decode_step(0, qn.cuda(), kn.cuda(), vn.cuda(), bidx, p)
        assert torch.equal(out_a, out_b) and torch.equal(lse_a, lse_b)
        assert torch.equal(ca.kv_cache, cb.kv_cache)
        for s_ in slots:
            o.reserve(s_, 1100)
        o.append_decode(0, obidx, p.cpu(), kn, vn)
        ref_out, ref_lse = orc.decode_attention(o, 0, qn.float(), obidx, p.cpu())
        assert_attention_close(out_b, lse_b, ref_out, ref_lse, f"step {step}")
    ca.check_status(); cb.check_status()


def test_batch_larger_than_one_launch():
    """More rows than one launch of the TMA kernel takes (512): the call is split into launches that share the
    workspace; short contexts, so that the oracle stays quick."""
    case = wl.make_decode_case(909, B=700, Hq=16, Hkv=8, D=128, P=128, n_pages=1500, max_batch_size=702,
                               len_lo=1, len_hi=200, dtype=torch.bfloat16)
    c, slots, bidx, pos, k, v, q = product_from_case(case)
    o, _, obidx, opos, ok, ov, oq = oracle_from_case(case)
    ref_out, ref_lse = orc.decode_attention(o, 0, oq.float(), obidx, opos)
    for kern in KERNELS.values():
        c.decode_kernel = kern
        out, lse = c.decode_attention(0, q, bidx, pos)
        assert_attention_close(out, lse, ref_out, ref_lse, f"B=700 kernel {kern}")
    out2, lse2 = c.decode_step(0, q, k, v, bidx, pos)            # fused path over several launches
    c.decode_kernel = _lib.DECODE_TMA
    out3, lse3 = c.decode_attention(0, q, bidx, pos)
    assert_attention_close(out2, lse2, ref_out, ref_lse, "B=700 fused")
    assert torch.equal(out3, c.decode_attention(0, q, bidx, pos)[0])
    c.check_status()


@pytest.mark.parametrize("B,hi", [(2, 300), (8, 700), (12, 1400), (24, 1000), (30, 1200), (36, 1100), (44, 1300), (60, 900)])
def test_work_unit_schedule_across_batch_sizes(B, hi):
    """Total tile counts from below the number of SMs to many per SM: phases of the unit schedule that are
    shorter than the grid leave units without tiles, which nobody may read.  The workspace is poisoned, the
    portable kernel is the cross-check."""
    case = wl.make_decode_case(1234 + B, B=B, Hq=16, Hkv=8, D=128, P=128, n_pages=B * 12 + 2, max_batch_size=B + 1,
                               len_lo=hi // 2, len_hi=hi, dtype=torch.bfloat16)
    c, slots, bidx, pos, k, v, q = product_from_case(case)
    c.decode_kernel = _lib.DECODE_PORTABLE
    out_p, lse_p = c.decode_attention(0, q, bidx, pos)
    c.decode_kernel = _lib.DECODE_TMA
    c._workspace[16384:].fill_(255)                      # NaN bit patterns in every partial and table of the scratch
    out_t, lse_t = c.decode_attention(0, q, bidx, pos)
    assert_attention_close(out_t, lse_t, out_p.float().cpu(), lse_p.cpu(), f"B={B}")
    c.check_status()
