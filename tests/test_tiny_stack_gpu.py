"""GPU: a tiny decoder stack driven the way the reference engine drives the
path -- packed prefill of several prompts (one with an image span), then decode
steps with page growth across page boundaries, every layer calling insert_kv +
attention with the sink gate -- against the same stack computed densely in
fp32 without any cache.  This exercises the flow, not one kernel: allocator,
packed append, prefill attention with the token-major gated output, the fused
decode step, several layers sharing one pool."""

import math

import pytest
import torch
import torch.nn.functional as F

import workloads as wl
from fpkv.paged_attention import PagedKVCache
from oracle import paged_kv_oracle as orc

pytestmark = pytest.mark.gpu

NL, DIM, HQ, HKV, D, FFN, VOCAB, P = 2, 256, 4, 2, 128, 512, 64, 128


def make_weights(gen):
    w = lambda *s: (torch.randn(s, generator=gen) * 0.06).bfloat16()
    return dict(emb=w(VOCAB, DIM), head=w(DIM, VOCAB),
                layers=[dict(qkv=w(DIM, (HQ + 2 * HKV) * D), wo=w(HQ * D, DIM), up=w(DIM, 2 * FFN), down=w(FFN, DIM),
                             sinks=(torch.randn(HQ, generator=gen)).bfloat16()) for _ in range(NL)])


def split_qkv(qkv, T):
    q = qkv[:, :HQ * D].view(T, HQ, D)
    k = qkv[:, HQ * D:(HQ + HKV) * D].view(T, HKV, D)
    v = qkv[:, (HQ + HKV) * D:].view(T, HKV, D)
    return q, k, v


def ffn(x, lw):
    gu = F.rms_norm(x, (DIM,)) @ lw["up"]
    return x + (F.relu(gu[:, :FFN]).square() * gu[:, FFN:]) @ lw["down"]


def dense_reference(W, tokens, img):
    """fp32 forward of ONE sequence without a cache: hidden state of every position.  Mask as the
    reference's: causal, plus bidirectional inside an image span."""
    Wf = lambda t: t.float()
    T = len(tokens)
    x = Wf(W["emb"])[torch.tensor(tokens)]
    allowed = torch.from_numpy(orc.prefill_allowed([1] * T, img))
    for lw in W["layers"]:
        qkv = F.rms_norm(x, (DIM,)) @ Wf(lw["qkv"])
        q, k, v = split_qkv(qkv, T)
        # the cache holds 16-bit K/V and the kernels read 16-bit q: round like the product does
        q, k, v = (t.bfloat16().float() for t in (q, k, v))
        kq = k.repeat_interleave(HQ // HKV, 1); vq = v.repeat_interleave(HQ // HKV, 1)
        s = torch.einsum("thd,uhd->htu", q, kq) / math.sqrt(D)
        s = s.masked_fill(~allowed.unsqueeze(0), float("-inf"))
        lse = torch.logsumexp(s, -1)                                        # (HQ, T)
        o = torch.einsum("htu,uhd->thd", torch.softmax(s, -1), vq)          # (T, HQ, D)
        o = o.bfloat16().float() * torch.sigmoid(lse.t() - Wf(lw["sinks"]).view(1, HQ)).unsqueeze(-1)
        x = x + o.bfloat16().float().reshape(T, HQ * D) @ Wf(lw["wo"])
        x = ffn(x, {k_: Wf(v_) for k_, v_ in lw.items()})
    return x


def test_prefill_then_decode_matches_dense_recomputation():
    gen = torch.Generator().manual_seed(2024)
    W = make_weights(gen)
    Wd = dict(emb=W["emb"].cuda(), head=W["head"].cuda(), layers=[{k: v.cuda() for k, v in lw.items()} for lw in W["layers"]])
    ids = lambda n: torch.randint(10, VOCAB, (n,), generator=gen).tolist()      # ids >= 10: never a special token
    prompts = [ids(100), ids(3) + [wl.IMG_CLS_ID] + ids(149) + [wl.END_OF_IMG_ID] + ids(40), ids(250)]
    n_new = 12                                       # decode steps; prompt 2 crosses a page boundary at 256
    cache = PagedKVCache(16, P, 5, HKV, D, NL, torch.bfloat16, "cuda")

    # ---- prefill: pack with 128-alignment as the reference engine does (paged_inference.py:637-678) ----
    case = wl.make_prefill_case(0, prompts, Hq=HQ, Hkv=HKV, D=D, P=P, dtype=torch.bfloat16)
    slots = []
    for p in prompts:
        s = cache.allocate(); slots.append(s); cache.reserve(s, None, len(p))
    bidx, ipos, tok = case.batch_idx_for(slots).cuda(), case.input_pos.cuda(), case.input_ids.cuda()
    L = case.L
    mask = cache.create_prefill_blockmask(bidx, tok, wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    x = Wd["emb"][tok.view(-1)]
    for li, lw in enumerate(Wd["layers"]):
        q, k, v = split_qkv(F.rms_norm(x, (DIM,)) @ lw["qkv"], L)
        cache.insert_kv(li, k.permute(1, 0, 2).unsqueeze(0), v.permute(1, 0, 2).unsqueeze(0), input_pos=ipos, batch_idx=bidx)
        o, _ = cache.prefill_attention(li, q.permute(1, 0, 2).unsqueeze(0), bidx, ipos, mask, sinks=lw["sinks"],
                                       token_major=True)
        x = ffn(x + o.view(L, HQ * D) @ lw["wo"], lw)
    hidden = {i: [x[case.offsets[i]:case.offsets[i] + len(p)].float().cpu()] for i, p in enumerate(prompts)}
    seqs = [list(p) for p in prompts]
    last = torch.stack([x[case.offsets[i] + len(p) - 1] for i, p in enumerate(prompts)])

    # ---- decode: greedy, one fused step per layer, pages reserved as sequences grow ----
    for step in range(n_new):
        nxt = (last.float() @ Wd["head"].float()).argmax(-1).tolist()
        for i, t in enumerate(nxt):
            seqs[i].append(int(t))
            cache.reserve(slots[i], None, len(seqs[i]))
        B = len(seqs)
        bi = torch.tensor(slots, device="cuda"); pos = torch.tensor([len(s) - 1 for s in seqs], dtype=torch.int32, device="cuda")
        x = Wd["emb"][torch.tensor(nxt, device="cuda")]
        for li, lw in enumerate(Wd["layers"]):
            q, k, v = split_qkv(F.rms_norm(x, (DIM,)) @ lw["qkv"], B)
            o, _ = cache.decode_step(li, q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), bi, pos, sinks=lw["sinks"])
            x = ffn(x + o.view(B, HQ * D) @ lw["wo"], lw)
        for i in range(B):
            hidden[i].append(x[i:i + 1].float().cpu())
        last = x
    cache.check_status()
    assert len(cache.page_table_cpu[slots[2]]) == 3          # 250 + 12 tokens crossed into a third page

    # ---- the same sequences, dense, no cache ----
    for i, toks in enumerate(seqs):
        # spans come from the prompt only: a generated token is decoded causally whatever its id
        n_p = len(prompts[i])
        img = list(orc.image_span_ids(toks[:n_p], wl.IMG_CLS_ID, wl.END_OF_IMG_ID)) + [0] * (len(toks) - n_p)
        ref = dense_reference(W, toks, img)                   # hidden of every consumed position
        got = torch.cat(hidden[i])
        assert got.shape == ref.shape
        cos = F.cosine_similarity(got, ref, dim=-1)
        rel = (got - ref).norm(dim=-1) / ref.norm(dim=-1)
        assert cos.min().item() > 0.999 and rel.max().item() < 0.05, (i, cos.min().item(), rel.max().item())


def rope_table(positions, D):
    """1-D rotary table of the given positions, (len, D/4) complex64, theta 10000 over the first half of head_dim."""
    freqs = 1.0 / (10000.0 ** (torch.arange(0, D // 2, 2).float() / (D // 2)))
    ang = torch.outer(torch.as_tensor(positions).float(), freqs)
    return torch.polar(torch.ones_like(ang), ang)


def test_flow_with_fused_norm_rotary_append():
    """The same flow with the front of the call site folded in: the projection output goes through
    pre_attention_append (norm, rotary embedding, append in one kernel) in the prefill and in every decode step,
    against dense recomputation built on the oracle's pre_attention_tail."""
    gen = torch.Generator().manual_seed(77)
    W = make_weights(gen)
    Wd = dict(emb=W["emb"].cuda(), head=W["head"].cuda(), layers=[{k: v.cuda() for k, v in lw.items()} for lw in W["layers"]])
    ids = lambda n: torch.randint(10, VOCAB, (n,), generator=gen).tolist()
    prompts = [ids(120), ids(250)]
    n_new = 10
    cache = PagedKVCache(16, P, 4, HKV, D, NL, torch.bfloat16, "cuda")
    case = wl.make_prefill_case(0, prompts, Hq=HQ, Hkv=HKV, D=D, P=P, dtype=torch.bfloat16)
    slots = []
    for p in prompts:
        s = cache.allocate(); slots.append(s); cache.reserve(s, None, len(p))
    bidx, ipos, tok = case.batch_idx_for(slots).cuda(), case.input_pos.cuda(), case.input_ids.cuda()
    L = case.L
    mask = cache.create_prefill_blockmask(bidx, tok, wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    fc = rope_table(case.input_pos.view(-1), D).view(1, L, D // 4).cuda()
    x = Wd["emb"][tok.view(-1)]
    for li, lw in enumerate(Wd["layers"]):
        qkv = (F.rms_norm(x, (DIM,)) @ lw["qkv"]).view(1, L, -1)
        xq = cache.pre_attention_append(li, qkv, HQ, HKV, fc, None, bidx, ipos)
        o, _ = cache.prefill_attention(li, xq, bidx, ipos, mask, sinks=lw["sinks"], token_major=True)
        x = ffn(x + o.view(L, HQ * D) @ lw["wo"], lw)
    hidden = {i: [x[case.offsets[i]:case.offsets[i] + len(p)].float().cpu()] for i, p in enumerate(prompts)}
    seqs = [list(p) for p in prompts]
    last = torch.stack([x[case.offsets[i] + len(p) - 1] for i, p in enumerate(prompts)])
    for step in range(n_new):
        nxt = (last.float() @ Wd["head"].float()).argmax(-1).tolist()
        for i, t in enumerate(nxt):
            seqs[i].append(int(t)); cache.reserve(slots[i], None, len(seqs[i]))
        B = len(seqs)
        bi = torch.tensor(slots, device="cuda")
        pos = torch.tensor([len(s) - 1 for s in seqs], dtype=torch.int32, device="cuda")
        fcd = rope_table(pos.cpu(), D).view(B, 1, D // 4).cuda()
        x = Wd["emb"][torch.tensor(nxt, device="cuda")]
        for li, lw in enumerate(Wd["layers"]):
            qkv = (F.rms_norm(x, (DIM,)) @ lw["qkv"]).view(B, 1, -1)
            xq = cache.pre_attention_append(li, qkv, HQ, HKV, fcd, None, bi, pos.view(B, 1))
            o, _ = cache.decode_attention(li, xq, bi, pos, sinks=lw["sinks"])
            x = ffn(x + o.view(B, HQ * D) @ lw["wo"], lw)
        for i in range(B):
            hidden[i].append(x[i:i + 1].float().cpu())
        last = x
    cache.check_status()

    # dense recomputation: the oracle's norm + rotary on the whole sequence, causal attention, no cache
    for i, toks in enumerate(seqs):
        T = len(toks)
        Wf = lambda t: t.float()
        xr = Wf(W["emb"])[torch.tensor(toks)]
        allowed = torch.from_numpy(orc.prefill_allowed([1] * T, [0] * T))
        fcr = rope_table(range(T), D).view(1, T, D // 4)
        for lw in W["layers"]:
            qkv = (F.rms_norm(xr, (DIM,)) @ Wf(lw["qkv"])).bfloat16().view(1, T, -1)     # the product's projection is bf16
            q, k, v = orc.pre_attention_tail(qkv, HQ, HKV, D, fcr, None)                  # (1, HQ, T, D), expanded
            q, k, v = q[0].float(), k[0].float(), v[0].float()
            s = torch.einsum("htd,hud->htu", q, k) / math.sqrt(D)
            s = s.masked_fill(~allowed.unsqueeze(0), float("-inf"))
            lse = torch.logsumexp(s, -1)
            o = torch.einsum("htu,hud->thd", torch.softmax(s, -1), v)
            o = o.bfloat16().float() * torch.sigmoid(lse.t() - Wf(lw["sinks"]).view(1, HQ)).unsqueeze(-1)
            xr = xr + o.bfloat16().float().reshape(T, HQ * D) @ Wf(lw["wo"])
            xr = ffn(xr, {k_: Wf(v_) for k_, v_ in lw.items()})
        got = torch.cat(hidden[i])
        assert got.shape == xr.shape
        cos = F.cosine_similarity(got, xr, dim=-1)
        rel = (got - xr).norm(dim=-1) / xr.norm(dim=-1)
        assert cos.min().item() > 0.999 and rel.max().item() < 0.05, (i, cos.min().item(), rel.max().item())
