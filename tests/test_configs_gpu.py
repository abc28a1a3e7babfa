"""GPU: the larger BASELINE configurations as parity cases.

config 3  chunked multimodal prefill (8 x [1024 image + 64 text], 512-row query chunks, K/V written to
          pages first) while 56 other sequences decode in the same step -- full size, against the oracle.
config 4  long-context decode under fragmentation: every 64 of 512 steps a quarter of the sequences finish,
          are erased, and new ones are admitted into the freed pages -- the full schedule at full context
          lengths (16K-32K) with the oracle running beside it, plus a reduced-size variant with every step
          compared.
config 5  one GPU's share of the 28-layer stack: 64 sequences, 61 GB pool, two layers against the oracle.
"""

import numpy as np
import pytest
import torch

from fpkv import _lib
import workloads as wl
from fpkv.attention import PrefillMask
from fpkv.paged_attention import PagedKVCache, paged_attention
from oracle import paged_kv_oracle as orc
from helpers import assert_attention_close

pytestmark = pytest.mark.gpu


def test_config3_chunked_prefill_with_decoders_in_the_same_step():
    pre = wl.config3_prefill_case(n_seq=8)
    dec = wl.make_decode_case(3003, B=56, Hq=16, Hkv=8, D=128, P=128, n_pages=4096, max_batch_size=66,
                              len_lo=1024, len_hi=8192, dtype=torch.bfloat16, value_scale=128 ** -0.5,
                              with_history=False)
    n_pages = 4096
    c = PagedKVCache(n_pages, 128, 66, 8, 128, 1, torch.bfloat16, "cuda")
    o = orc.OraclePagedKVCache(n_pages, 128, 66, 8, 128, 1, torch.bfloat16)
    c.free_pages = list(dec.free_pages); o.free_pages = list(dec.free_pages)
    # 56 decoding sequences with context already in pages (same random context on both sides)
    g = torch.Generator().manual_seed(11)
    dslots = []
    for L in dec.lens:
        s = c.allocate(); assert o.allocate() == s; dslots.append(s)
        c.reserve(s, None, L + 1); o.reserve(s, L + 1)
        kh = (torch.randn(1, 8, L, 128, generator=g) * 128 ** -0.5).bfloat16()
        vh = (torch.randn(1, 8, L, 128, generator=g) * 128 ** -0.5).bfloat16()
        ip, bi = torch.arange(L).view(1, L), torch.full((1, L), s)
        c.insert_kv(0, kh.cuda(), vh.cuda(), input_pos=ip.cuda(), batch_idx=bi.cuda())
        o.append_packed(0, bi, ip, kh, vh)
    # 8 new prompts admitted in this step
    pslots = []
    for toks in pre.seq_tokens:
        s = c.allocate(); assert o.allocate() == s; pslots.append(s)
        c.reserve(s, None, len(toks)); o.reserve(s, len(toks))
    assert c.page_table_cpu == o.page_table_cpu and c.free_pages == o.free_pages

    # ---- the step: packed append of the prompts' K/V, prefill attention in 512-row chunks, decode step ----
    bidx = pre.batch_idx_for(pslots).cuda(); ipos = pre.input_pos.cuda()
    q, k, v = pre.q.cuda(), pre.k.cuda(), pre.v.cuda()
    mask = c.create_prefill_blockmask(bidx, pre.input_ids.cuda(), wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    c.insert_kv(0, k, v, input_pos=ipos, batch_idx=bidx)
    ext = mask.extent(ipos)
    out = torch.zeros_like(q); lse = torch.full((1, 16, pre.L), float("-inf"), device="cuda")
    for off, toks in zip(pre.offsets, pre.seq_tokens):
        for c0 in range(0, len(toks), 512):
            c1 = min(len(toks), c0 + 512)
            sl = slice(off + c0, off + c1)
            m = PrefillMask(mask.doc_id[sl], mask.img_id[sl]); m._extent = ext[sl].contiguous()
            oc, lc = c.prefill_attention(0, q[:, :, sl], bidx[:, sl], ipos[:, sl], m)
            out[:, :, sl] = oc; lse[:, :, sl] = lc
    dbi = torch.tensor(dslots); dpos = torch.tensor(dec.lens, dtype=torch.int32)
    dout, dlse = c.decode_step(0, dec.q.cuda(), dec.k_new.cuda(), dec.v_new.cuda(), dbi.cuda(), dpos.cuda())

    # ---- oracle: the reference never mixes the two; its prefill and decode results are computed apart ----
    o.append_packed(0, bidx.cpu(), ipos.cpu(), pre.k, pre.v)
    o.append_decode(0, dbi, dpos, dec.k_new, dec.v_new)
    assert torch.equal(c.kv_cache[..., 128:, :].cpu(), o.kv_cache[..., 128:, :])          # bit-exact pool
    img = orc.image_span_ids(pre.input_ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    ref_out, ref_lse = orc.prefill_attention(pre.q.float(), pre.k.float(), pre.v.float(), bidx.cpu(), img)
    live = pre.seq_index.view(-1) > 0
    assert_attention_close(out[0][:, live], lse[0][:, live], ref_out[0][:, live], ref_lse[0][:, live], "cfg3 prefill")
    rd_out, rd_lse = orc.decode_attention(o, 0, dec.q.float(), dbi, dpos)
    assert_attention_close(dout, dlse, rd_out, rd_lse, "cfg3 decode")
    c.check_status()


def _churn(c, o, rng, P, lens, slots, step, new_len, frac, D=128, H=8):
    """Seeded choice of sequences finish; new ones of new_len tokens take over the freed pages."""
    B = len(slots)
    gone = rng.permutation(B)[:max(1, B // frac)].tolist()
    for i in gone:
        c.erase(slots[i])
        if o is not None:
            o.erase(slots[i])
    g = torch.Generator().manual_seed(1000 + step)
    for i in gone:
        s = c.allocate(); c.reserve(s, None, new_len + 1)
        if o is not None:
            assert o.allocate() == s; o.reserve(s, new_len + 1)
        kh = torch.randn(1, H, new_len, D, generator=g).bfloat16(); vh = torch.randn(1, H, new_len, D, generator=g).bfloat16()
        ip, bi = torch.arange(new_len).view(1, -1), torch.full((1, new_len), s)
        c.insert_kv(0, kh.cuda(), vh.cuda(), input_pos=ip.cuda(), batch_idx=bi.cuda())
        if o is not None:
            o.append_packed(0, bi, ip, kh, vh)
        slots[i], lens[i] = s, new_len
    return gone


def test_config4_churn_reduced_size_against_oracle():
    P, B, n_pages = 128, 8, 160
    rng = np.random.default_rng(4004)
    c = PagedKVCache(n_pages, P, B + 1, 8, 128, 1, torch.bfloat16, "cuda")
    o = orc.OraclePagedKVCache(n_pages, P, B + 1, 8, 128, 1, torch.bfloat16)
    perm = (rng.permutation(n_pages - 1) + 1).tolist()
    c.free_pages = list(perm); o.free_pages = list(perm)
    lens = rng.integers(1024, 2049, size=B).tolist()
    slots = []
    g = torch.Generator().manual_seed(7)
    for L in lens:
        s = c.allocate(); assert o.allocate() == s; slots.append(s)
        c.reserve(s, None, L + 1); o.reserve(s, L + 1)
        kh, vh = torch.randn(1, 8, L, 128, generator=g).bfloat16(), torch.randn(1, 8, L, 128, generator=g).bfloat16()
        ip, bi = torch.arange(L).view(1, L), torch.full((1, L), s)
        c.insert_kv(0, kh.cuda(), vh.cuda(), input_pos=ip.cuda(), batch_idx=bi.cuda()); o.append_packed(0, bi, ip, kh, vh)
    for step in range(16):
        if step and step % 4 == 0:
            _churn(c, o, rng, P, lens, slots, step, new_len=200, frac=4)
            assert c.page_table_cpu == o.page_table_cpu and c.free_pages == o.free_pages
        for i, s in enumerate(slots):                     # grow by a page when the next token needs one
            c.reserve(s, None, lens[i] + 1); o.reserve(s, lens[i] + 1)
        bi = torch.tensor(slots); pos = torch.tensor(lens, dtype=torch.int32)
        kn, vn, qn = (torch.randn(B, n, 1, 128, generator=g).bfloat16() for n in (8, 8, 16))
        out, lse = c.decode_step(0, qn.cuda(), kn.cuda(), vn.cuda(), bi.cuda(), pos.cuda())
        o.append_decode(0, bi, pos, kn, vn)
        ref_out, ref_lse = orc.decode_attention(o, 0, qn.float(), bi, pos)
        assert_attention_close(out, lse, ref_out, ref_lse, f"churn step {step}")
        lens = [L + 1 for L in lens]
    assert torch.equal(c.kv_cache[..., P:, :].cpu(), o.kv_cache[..., P:, :])
    assert torch.equal(c.page_table.cpu(), torch.from_numpy(o.page_table))
    assert torch.equal(c.physical_to_logical.cpu(), torch.from_numpy(o.physical_to_logical))
    c.check_status()


def test_config4_full_schedule_against_the_oracle():
    """BASELINE config 4 as written: batch 32, context 16K-32K, 512 decode steps; every 64 steps a seeded
    quarter of the sequences finishes and is erased and new 2048-token sequences are admitted (packed
    append) into the freed pages.  The oracle runs the whole schedule beside the product on its own
    full-size pool (every append, every allocator call); attention is compared on all rows at the first
    and last step, at the first step after each admission and in the middle of each period, and at the end
    both page tables and the whole pool are compared bit for bit."""
    P, B, n_pages, H, D = 128, 32, 10240, 8, 128
    rng = np.random.default_rng(4004)
    c = PagedKVCache(n_pages, P, B + 1, H, D, 1, torch.bfloat16, "cuda")
    o = orc.OraclePagedKVCache(n_pages, P, B + 1, H, D, 1, torch.bfloat16)
    perm = (rng.permutation(n_pages - 1) + 1).tolist()
    c.free_pages = list(perm); o.free_pages = list(perm)
    lens = rng.integers(16384, 32769, size=B).tolist()
    slots = []
    for L in lens:
        s = c.allocate(); assert o.allocate() == s; slots.append(s)
        c.reserve(s, None, L + 1); o.reserve(s, L + 1)
    # the initial contexts: random values in every page, the same bytes on both sides
    c.kv_cache.normal_(0, D ** -0.5)
    o.kv_cache.copy_(c.kv_cache.cpu())
    g = torch.Generator(device="cuda").manual_seed(3)
    checked = 0
    for step in range(512):
        if step and step % 64 == 0:
            gone = rng.permutation(B)[:B // 4].tolist()
            for i in gone:
                c.erase(slots[i]); o.erase(slots[i])
            for i in gone:
                s = c.allocate(); assert o.allocate() == s
                c.reserve(s, None, 2048 + 1); o.reserve(s, 2048 + 1)
                kh = (torch.randn((1, H, 2048, D), device="cuda", generator=g) * D ** -0.5).bfloat16()
                vh = (torch.randn((1, H, 2048, D), device="cuda", generator=g) * D ** -0.5).bfloat16()
                ip, bi = torch.arange(2048, device="cuda").view(1, -1), torch.full((1, 2048), s, device="cuda")
                c.insert_kv(0, kh, vh, input_pos=ip, batch_idx=bi)
                o.append_packed(0, bi.cpu(), ip.cpu(), kh.cpu(), vh.cpu())
                slots[i], lens[i] = s, 2048
            assert c.page_table_cpu == o.page_table_cpu and c.free_pages == o.free_pages
            for i in gone:                               # freed pages are reused and the new tables are scattered
                pages = c.page_table_cpu[slots[i]]
                assert len(pages) == 17 and max(pages) - min(pages) > 17
        for i, s in enumerate(slots):                     # grow by a page when the next token needs one
            c.reserve(s, None, lens[i] + 1); o.reserve(s, lens[i] + 1)
        bi = torch.tensor(slots); pos = torch.tensor(lens, dtype=torch.int32)
        kn, vn, qn = ((torch.randn((B, n, 1, D), device="cuda", generator=g) * D ** -0.5).bfloat16() for n in (H, H, 16))
        out, lse = c.decode_step(0, qn, kn, vn, bi.cuda(), pos.cuda())
        o.append_decode(0, bi, pos, kn.cpu(), vn.cpu())
        if step in (0, 511) or step % 64 in (0, 32):
            ref_out, ref_lse = orc.decode_attention(o, 0, qn.cpu().float(), bi, pos)
            assert_attention_close(out, lse, ref_out, ref_lse, f"config 4, step {step}")
            checked += 1
        lens = [L + 1 for L in lens]
    assert checked == 17
    assert torch.equal(c.page_table.cpu(), torch.from_numpy(o.page_table))
    assert torch.equal(c.physical_to_logical.cpu(), torch.from_numpy(o.physical_to_logical))
    assert torch.equal(c.kv_cache[..., P:, :].cpu(), o.kv_cache[..., P:, :])
    c.check_status()


def test_config5_one_gpu_share_of_the_stack_against_the_oracle():
    """BASELINE config 5, one GPU's share: 64 sequences with context 2K-8K in a 28-layer pool (61 GB); one
    decode step appends and attends in every layer.  Two layers hold real contexts (written through the
    packed append on both sides) and are compared with the oracle on every row; the layers in between must
    come out holding nothing but their own appended rows, i.e. the layer planes are independent."""
    NL, B, H, Hq, D, P, n_pages = 28, 64, 8, 16, 128, 128, 4352
    case = wl.make_decode_case(5005, B=B, Hq=Hq, Hkv=H, D=D, P=P, n_pages=n_pages, max_batch_size=B + 1,
                               len_lo=2048, len_hi=8192, dtype=torch.bfloat16, value_scale=D ** -0.5, with_history=False)
    c = PagedKVCache(n_pages, P, B + 1, H, D, NL, torch.bfloat16, "cuda")
    c.free_pages = list(case.free_pages)
    used = sum((L + 1 + P - 1) // P for L in case.lens)
    full_layers = (5, 27)
    oracles = {l: orc.OraclePagedKVCache(used + 1, P, B + 1, H, D, 1, torch.bfloat16) for l in full_layers}
    g = torch.Generator(device="cuda").manual_seed(55)
    slots = []
    for L in case.lens:
        s = c.allocate(); slots.append(s); c.reserve(s, None, L + 1)
        ip, bi = torch.arange(L, device="cuda").view(1, L), torch.full((1, L), s, device="cuda")
        for l in full_layers:
            o = oracles[l]
            assert o.allocate() == s; o.reserve(s, L + 1)
            kh = (torch.randn((1, H, L, D), device="cuda", generator=g) * D ** -0.5).bfloat16()
            vh = (torch.randn((1, H, L, D), device="cuda", generator=g) * D ** -0.5).bfloat16()
            c.insert_kv(l, kh, vh, input_pos=ip, batch_idx=bi)
            o.append_packed(0, bi.cpu(), ip.cpu(), kh.cpu(), vh.cpu())
    bidx = torch.tensor(slots); pos = torch.tensor(case.lens, dtype=torch.int32)
    outs = {}
    step_in = {}
    for l in range(NL):                                   # the decode step of the whole stack, layer after layer
        kn, vn, qn = ((torch.randn((B, n, 1, D), device="cuda", generator=g) * D ** -0.5).bfloat16() for n in (H, H, Hq))
        outs[l] = c.decode_step(l, qn, kn, vn, bidx.cuda(), pos.cuda())
        step_in[l] = (kn, vn, qn)
    for l in full_layers:
        kn, vn, qn = step_in[l]
        oracles[l].append_decode(0, bidx, pos, kn.cpu(), vn.cpu())
        ref_out, ref_lse = orc.decode_attention(oracles[l], 0, qn.cpu().float(), bidx, pos)
        assert_attention_close(outs[l][0], outs[l][1], ref_out, ref_lse, f"config 5, layer {l}, all 64 rows")
    for l in (0, 4, 6, 26):                               # neighbours of the full layers: only this step's rows
        kn, vn, qn = step_in[l]
        plane = c.kv_cache[l][..., P:, :]
        assert int((plane != 0).sum().item()) == int((kn != 0).sum().item()) + int((vn != 0).sum().item())
        out, lse = outs[l]                                # one non-zero key per row: out is its value, among zeros
        assert torch.isfinite(lse).all()
    c.check_status()
