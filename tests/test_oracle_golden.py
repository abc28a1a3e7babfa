"""CPU: the oracle against the golden vectors recorded from the reference."""

import hashlib
import json
import os

import numpy as np
import pytest
import torch

import workloads as wl
from oracle import paged_kv_oracle as orc
from helpers import GOLDEN, golden, oracle_from_case

DECODE_CASES = {
    "decode_cfg1": (lambda: wl.config1_case(), 0),
    "decode_bf16_d128": (lambda: wl.make_decode_case(2101, B=6, Hq=16, Hkv=8, D=128, P=128, n_pages=48,
                                                     max_batch_size=8, len_lo=1, len_hi=700,
                                                     dtype=torch.bfloat16, value_scale=1.0), 2),
    "decode_bf16_scaled": (lambda: wl.make_decode_case(2102, B=5, Hq=16, Hkv=8, D=128, P=128, n_pages=48,
                                                       max_batch_size=8, len_lo=100, len_hi=900,
                                                       dtype=torch.bfloat16, value_scale=128 ** -0.5), 0),
    "decode_p16_edges": (lambda: wl.make_decode_case(2103, B=7, Hq=8, Hkv=2, D=64, P=16, n_pages=40,
                                                     max_batch_size=9, len_lo=0, len_hi=0, dtype=torch.float32,
                                                     lens=[0, 1, 15, 16, 17, 31, 64]), 1),
    "decode_mha_fp16": (lambda: wl.make_decode_case(2104, B=3, Hq=4, Hkv=4, D=64, P=32, n_pages=40,
                                                    max_batch_size=5, len_lo=5, len_hi=300,
                                                    dtype=torch.float16), 0),
}

T = wl.image_text_tokens
PREFILL_CASES = {
    "prefill_mixed_d64": (lambda: wl.make_prefill_case(
        3101, [T(3, 100, 20), T(0, 0, 50), T(5, 200, 30) + T(2, 37, 9), T(0, 128, 0)],
        Hq=4, Hkv=2, D=64, P=128, dtype=torch.bfloat16), 16, 6),
    "prefill_img_d128": (lambda: wl.make_prefill_case(
        3102, [T(0, 256, 31), T(7, 130, 100)], Hq=4, Hkv=2, D=128, P=128, dtype=torch.bfloat16,
        value_scale=1.0), 12, 4),
}


def pool_digest(pool_l, P):
    return hashlib.sha256(pool_l[:, :, :, P:, :].contiguous().numpy().tobytes()).hexdigest()


def snapshot(c):
    return dict(free_pages=list(c.free_pages), free_batch_idx=list(c.free_batch_idx), capacity=list(c.capacity),
                page_table_cpu=[list(r) for r in c.page_table_cpu],
                page_table=np.asarray(c.page_table).astype(int).tolist(),
                physical_to_logical=np.asarray(c.physical_to_logical).astype(int).tolist())


def test_allocator_traces_match_reference():
    traces = json.load(open(os.path.join(GOLDEN, "allocator_traces.json")))
    assert len(traces) >= 4
    for tr in traces:
        n_pages, P, mb = tr["ctor"]
        o = orc.OraclePagedKVCache(n_pages, P, mb, 1, 8, 1, torch.float32)
        for step in tr["steps"]:
            op = step["op"]
            if op == "init":
                pass
            elif op[0] == "allocate":
                assert o.allocate() == step["result"]
            elif op[0] == "reserve":
                if step["error"] is not None:
                    with pytest.raises(RuntimeError) as e:
                        o.reserve(op[1], op[2])
                    assert str(e.value) == step["error"]
                else:
                    assert o.reserve(op[1], op[2]) == step["result"]
            elif op[0] == "can_reserve":
                assert bool(o.can_reserve(op[1], op[2])) == step["result"]
            elif op[0] == "erase":
                o.erase(op[1])
            assert snapshot(o) == step["state"], op


def test_known_answers_small_pool():
    """Hand-checkable allocator answers (12 pages of 4 tokens, 4 slots)."""
    o = orc.OraclePagedKVCache(12, 4, 4, 1, 8, 1, torch.float32)
    assert o.free_pages == list(range(11, 0, -1)) and o.free_batch_idx == [3, 2, 1]
    assert (o.page_table[0] == 0).all() and (o.page_table[1:] == -1).all()
    a = o.allocate(); assert a == 1
    o.reserve(a, 9)
    assert o.page_table_cpu[a] == [3, 2, 1] and o.capacity[a] == 12 and o.free_pages == list(range(11, 3, -1))
    b = o.allocate(); o.reserve(b, 5); assert b == 2 and o.page_table_cpu[b] == [5, 4]
    o.reserve(a, 13)
    assert o.page_table_cpu[a] == [3, 2, 1, 6]
    assert o.physical_to_logical[a].tolist() == [-1, 2, 1, 0, -1, -1, 3, -1, -1, -1, -1, -1]
    assert not o.can_reserve(21) and o.can_reserve(20)
    o.erase(a)
    assert o.free_pages == [11, 10, 9, 8, 7, 6, 1, 2, 3] and o.free_batch_idx == [3, 1]
    d = o.allocate(); o.reserve(d, 6); assert d == 1 and o.page_table_cpu[d] == [2, 3]
    with pytest.raises(RuntimeError, match="Cannot reserve 248 pages"):
        o.reserve(d, 1000)


@pytest.mark.parametrize("name", sorted(DECODE_CASES))
def test_decode_matches_reference(name):
    make, pads = DECODE_CASES[name]
    case = make()
    g = golden(name)
    o, slots, bidx, pos, k, v, q = oracle_from_case(case, dtype=torch.float32, pad_rows=pads)
    assert slots == g["slots"].tolist()
    assert np.array_equal(o.page_table, g["page_table"])
    assert pool_digest(o.kv_cache[0], case.P) == str(g["pool_sha256"])
    out, lse = orc.decode_attention(o, 0, q.float(), bidx, pos)
    assert np.abs(out.numpy() - g["out"]).max() < 2e-5
    fin = np.isfinite(g["lse"])
    assert np.array_equal(fin, np.isfinite(lse.numpy()))
    assert np.abs(lse.numpy()[fin] - g["lse"][fin]).max() < 2e-5
    if pads:   # padding rows (slot 0): nothing visible
        assert np.all(g["out"][case.B:] == 0) and np.all(np.isneginf(g["lse"][case.B:]))


@pytest.mark.parametrize("name", sorted(PREFILL_CASES))
def test_prefill_matches_reference(name):
    make, n_pages, mb = PREFILL_CASES[name]
    case = make()
    g = golden(name)
    o = orc.OraclePagedKVCache(n_pages, case.P, mb, case.Hkv, case.D, 1, torch.float32)
    slots = []
    for toks in case.seq_tokens:
        s = o.allocate(); slots.append(s); o.reserve(s, len(toks))
    assert slots == g["slots"].tolist()
    bidx = case.batch_idx_for(slots)
    q, k, v = case.q.float(), case.k.float(), case.v.float()
    o.append_packed(0, bidx, case.input_pos, k, v)
    assert pool_digest(o.kv_cache[0], case.P) == str(g["pool_sha256"])
    img = orc.image_span_ids(case.input_ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    assert np.array_equal(img, g["img_id"])
    out, lse = orc.prefill_attention(q, k, v, bidx, img)
    live = (case.seq_index.view(-1) > 0).numpy()
    assert np.abs(out.numpy() - g["out"])[0][:, live].max() < 2e-5
    assert np.abs(lse.numpy() - g["lse"])[0][:, live].max() < 2e-5
    # chunked evaluation through the pages gives the same rows
    s, off, L = slots[0], case.offsets[0], len(case.seq_tokens[0])
    for c0 in range(0, L, 50):
        c1 = min(L, c0 + 50)
        po, pl = orc.paged_prefill_attention(o, 0, q[0, :, off + c0:off + c1], s, np.arange(c0, c1), L,
                                             img[off:off + L])
        assert np.abs(po.numpy() - g["out"][0][:, off + c0:off + c1]).max() < 2e-5
        assert np.abs(pl.numpy() - g["lse"][0][:, off + c0:off + c1]).max() < 2e-5


def test_sink_gate_matches_reference():
    """Attention._post_attention with an identity projection, recorded from the reference."""
    rng = np.random.default_rng(4101)
    B, Hq, S, D = 3, 8, 5, 64
    out = torch.from_numpy(rng.standard_normal((B, Hq, S, D), dtype=np.float32)).bfloat16()
    lse = torch.from_numpy(rng.standard_normal((B, Hq, S), dtype=np.float32) * 3)
    lse[0, 1, 2] = float("-inf")
    sinks = torch.from_numpy(rng.standard_normal(Hq, dtype=np.float32)).bfloat16()
    got = orc.post_attention_gate(out, lse, sinks)
    assert np.array_equal(got.float().numpy(), golden("post_attention")["gated"])


def pre_attention_case(name):
    """Inputs of one fused norm + rotary case: the projection from the seed, the rotary tables and the
    reference's outputs from the golden file."""
    seed, B, S, Hq, Hkv, D, with_2d, dtype = wl.PRE_ATTENTION_CASES[name]
    g = golden(name)
    qkv = wl.pre_attention_qkv(np.random.default_rng(seed), B, S, Hq, Hkv, D, dtype)
    fc = torch.view_as_complex(torch.from_numpy(g["freqs_cis"]).contiguous())
    fc2 = torch.view_as_complex(torch.from_numpy(g["freqs_cis_2d"]).contiguous()) if with_2d else None
    return qkv, fc, fc2, g, (B, S, Hq, Hkv, D)


@pytest.mark.parametrize("name", list(wl.PRE_ATTENTION_CASES))
def test_pre_attention_tail_matches_reference(name):
    """Attention._pre_attention behind the QKV projection (norm, GQA expansion, 1-D and 2-D rotary embedding),
    recorded from the reference: the oracle's restatement is bit-identical."""
    qkv, fc, fc2, g, (B, S, Hq, Hkv, D) = pre_attention_case(name)
    xq, xk, xv = orc.pre_attention_tail(qkv, Hq, Hkv, D, fc, fc2)
    assert np.array_equal(xq.float().numpy(), g["xq"]) and np.array_equal(xk.float().numpy(), g["xk"])
    # values pass through untouched, expanded to the query head count
    v_in = qkv[..., (Hq + Hkv) * D:].reshape(B, S, Hkv, D).repeat_interleave(Hq // Hkv, 2).permute(0, 2, 1, 3)
    assert torch.equal(xv, v_in)
