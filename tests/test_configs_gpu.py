"""GPU: the larger BASELINE configurations as parity cases.

config 3  chunked multimodal prefill (8 x [1024 image + 64 text], 512-row query chunks, K/V written to
          pages first) while 56 other sequences decode in the same step -- full size, against the oracle.
config 4  long-context decode under fragmentation: every few steps a quarter of the sequences finish, are
          erased, and new ones are admitted into the freed pages -- oracle parity at a reduced size, and at
          full context lengths (16K-32K) the properties that do not need a CPU pass: allocator state equal
          to the oracle's, both kernels agreeing, reruns bitwise equal.
"""

import numpy as np
import pytest
import torch

from fpkv import _lib, workloads as wl
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


def test_config4_full_context_lengths_properties():
    """batch 32, context 16K-32K, 2048-token admissions into freed pages; 24 steps with churn every 8."""
    P, B, n_pages = 128, 32, 10240
    rng = np.random.default_rng(4004)
    c = PagedKVCache(n_pages, P, B + 1, 8, 128, 1, torch.bfloat16, "cuda")
    o = orc.OraclePagedKVCache(n_pages, P, B + 1, 1, 8, 1, torch.bfloat16)       # allocator only (tiny pool)
    perm = (rng.permutation(n_pages - 1) + 1).tolist()
    c.free_pages = list(perm); o.free_pages = list(perm)
    lens = rng.integers(16384, 32769, size=B).tolist()
    slots = []
    for L in lens:
        s = c.allocate(); assert o.allocate() == s; slots.append(s)
        c.reserve(s, None, L + 64); o.reserve(s, L + 64)
    c.kv_cache.normal_(0, 128 ** -0.5)                       # every reserved page holds plausible values
    g = torch.Generator(device="cuda").manual_seed(3)
    for step in range(24):
        if step and step % 8 == 0:
            gone = rng.permutation(B)[:B // 4].tolist()
            for i in gone:
                c.erase(slots[i]); o.erase(slots[i])
            for i in gone:
                s = c.allocate(); assert o.allocate() == s
                c.reserve(s, None, 2048 + 64); o.reserve(s, 2048 + 64)
                slots[i], lens[i] = s, 2048
            assert c.page_table_cpu == o.page_table_cpu and c.free_pages == o.free_pages
            for i in gone:                               # freed pages are reused and the new tables are scattered
                pages = c.page_table_cpu[slots[i]]
                assert len(pages) == 17 and max(pages) - min(pages) > 17
        bi = torch.tensor(slots, device="cuda"); pos = torch.tensor(lens, dtype=torch.int32, device="cuda")
        kn, vn, qn = ((torch.randn(B, n, 1, 128, device="cuda", generator=g) * 128 ** -0.5).bfloat16() for n in (8, 8, 16))
        c.decode_kernel = _lib.DECODE_TMA
        out, lse = c.decode_step(0, qn, kn, vn, bi, pos)
        if step % 8 == 7 or step == 8:
            out2, lse2 = c.decode_attention(0, qn, bi, pos)
            assert torch.equal(out, out2) and torch.equal(lse, lse2)                      # rerun is bitwise equal
            c.decode_kernel = _lib.DECODE_PORTABLE
            outp, lsep = c.decode_attention(0, qn, bi, pos)
            assert_attention_close(out, lse, outp.float().cpu(), lsep.cpu(), f"tma vs portable, step {step}")
            gk, gv = c.gather(0, slots[0], lens[0] + 1)                                   # appended row is where it belongs
            assert torch.equal(gk[:, -1], kn[0, :, 0]) and torch.equal(gv[:, -1], vn[0, :, 0])
        lens = [L + 1 for L in lens]
    assert torch.equal(c.page_table.cpu(), torch.from_numpy(o.page_table))
    c.check_status()
