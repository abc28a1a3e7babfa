"""Generate the golden vectors under tests/golden/ by running the reference.

Run from the repository root, in a container that has the reference checkout:

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py [/path/to/reference]

(default: $FALCON_PERCEPTION_SRC, else a `reference` checkout beside this repository)

The reference (tiiuae/Falcon-Perception) is imported read-only and driven on
the CPU in fp32 through its own code: ``PagedKVCache`` for the allocator and
the two append paths, ``PagedInferenceEngine.get_decoding_block_mask`` +
``convert_logical_block_mask`` + ``compiled_flex_attn_decode`` for decode
attention, ``create_prefill_blockmask`` + ``compiled_flex_attn_prefill`` for
prefill attention.  TORCHDYNAMO_DISABLE=1 makes its torch.compile handles run
eagerly (Inductor cannot build CPU code in the build container).

Every vector is also compared with the CPU oracle (oracle/paged_kv_oracle.py)
before it is written, so a golden file on disk means "reference and oracle
agreed on this case".  The reference caches GQA-expanded heads; it is fed
``repeat_interleave(n_rep)`` copies of the real KV heads and its pool is
compared head-group-wise.

Inputs are never stored: tests rebuild them from the seeds in
tests/workloads.py.  Only outputs (attention out / lse, table snapshots, pool
digests) are written, so the files stay small.
"""

import hashlib
import json
import os
import sys
import types
import warnings

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
warnings.filterwarnings("ignore")

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FALCON_PERCEPTION_SRC", os.path.join(os.path.dirname(ROOT), "reference"))
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(ROOT, "falcon-perception_b200"))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

# the engine module pulls in post-processing that needs pycocotools (absent)
_stub = types.ModuleType("pycocotools"); _stub.mask = types.ModuleType("pycocotools.mask")
sys.modules.setdefault("pycocotools", _stub); sys.modules.setdefault("pycocotools.mask", _stub.mask)

from falcon_perception.paged_attention import PagedKVCache as RefCache      # noqa: E402
from falcon_perception.attention import (compiled_flex_attn_decode,          # noqa: E402
                                         compiled_flex_attn_prefill)
from torch.nn.attention.flex_attention import AuxRequest                     # noqa: E402

from oracle import paged_kv_oracle as orc                                    # noqa: E402
import workloads as wl                                             # noqa: E402

OUT = os.path.join(ROOT, "tests", "golden")


def pool_digest(pool_l, P):
    """sha256 of one layer's (2,1,H,n_tok,D) pool without reserved page 0."""
    return hashlib.sha256(pool_l[:, :, :, P:, :].contiguous().numpy().tobytes()).hexdigest()


def snapshot(c):
    pt = c.page_table.numpy() if torch.is_tensor(c.page_table) else c.page_table
    p2l = c.physical_to_logical.numpy() if torch.is_tensor(c.physical_to_logical) else c.physical_to_logical
    return dict(free_pages=list(map(int, c.free_pages)), free_batch_idx=list(map(int, c.free_batch_idx)),
                capacity=list(map(int, c.capacity)),
                page_table_cpu=[list(map(int, r)) for r in c.page_table_cpu],
                page_table=pt.astype(int).tolist(), physical_to_logical=p2l.astype(int).tolist())


# --------------------------------------------------------------------------
# 1. allocator traces
# --------------------------------------------------------------------------
def allocator_traces():
    traces = []

    def run(ctor, ops):
        n_pages, P, mb = ctor
        ref = RefCache(n_pages, P, mb, 1, 8, 1, torch.float32, "cpu")
        o = orc.OraclePagedKVCache(n_pages, P, mb, 1, 8, 1, torch.float32)
        rec = [dict(op="init", state=snapshot(ref))]
        assert snapshot(ref) == snapshot(o)
        for op in ops:
            kind = op[0]
            res = err = None
            try:
                if kind == "allocate":
                    res = ref.allocate(); assert o.allocate() == res
                elif kind == "reserve":
                    _, slot, n = op
                    res = ref.reserve(slot, torch.tensor([slot]), n)
                    assert o.reserve(slot, n) == res
                elif kind == "can_reserve":
                    _, n, slot = op
                    res = bool(ref.can_reserve(n, slot)); assert bool(o.can_reserve(n, slot)) == res
                elif kind == "erase":
                    ref.erase(op[1]); o.erase(op[1])
            except RuntimeError as e:
                err = str(e)
                try:
                    o.reserve(op[1], op[2]); raise AssertionError("oracle did not raise")
                except RuntimeError as e2:
                    assert str(e2) == err, (str(e2), err)
            st = snapshot(ref)
            assert st == snapshot(o), (op, st, snapshot(o))
            rec.append(dict(op=list(op), result=res, error=err, state=st))
        traces.append(dict(ctor=list(ctor), steps=rec))

    # hand-written known-answer sequence
    run((12, 4, 4), [("allocate",), ("reserve", 1, 9), ("allocate",), ("reserve", 2, 5),
                     ("reserve", 1, 13), ("can_reserve", 21, None), ("can_reserve", 20, None),
                     ("can_reserve", 30, 2), ("can_reserve", 9, 2), ("erase", 1), ("allocate",),
                     ("reserve", 1, 6), ("reserve", 1, 1000), ("reserve", 1, 6), ("erase", 2), ("erase", 1)])
    # seeded random churn
    for seed, ctor in [(11, (24, 4, 6)), (12, (40, 16, 5)), (13, (17, 128, 9))]:
        rng = np.random.default_rng(seed)
        n_pages, P, mb = ctor
        live, ops, cap = [], [], {}
        # mirror of slot ids the reference will hand out: replay on a scratch oracle
        scratch = orc.OraclePagedKVCache(n_pages, P, mb, 1, 8, 1, torch.float32)
        for _ in range(60):
            r = rng.random()
            if (r < 0.3 and scratch.free_batch_idx) or not live:
                if not scratch.free_batch_idx:
                    continue
                s = scratch.allocate(); live.append(s); ops.append(("allocate",))
                n = int(rng.integers(1, 3 * P))
                ops.append(("can_reserve", n, s))
                if scratch.can_reserve(n, s):
                    scratch.reserve(s, n)
                ops.append(("reserve", s, n))
            elif r < 0.7:
                s = live[int(rng.integers(len(live)))]
                n = scratch.capacity[s] + int(rng.integers(0, 2 * P))
                ops.append(("can_reserve", n, s))
                if scratch.can_reserve(n, s):
                    scratch.reserve(s, n)
                ops.append(("reserve", s, n))
            elif r < 0.8:
                ops.append(("can_reserve", int(rng.integers(1, n_pages * P)), None))
            else:
                s = live.pop(int(rng.integers(len(live))))
                scratch.erase(s); ops.append(("erase", s))
        run(ctor, ops)
    with open(os.path.join(OUT, "allocator_traces.json"), "w") as f:
        json.dump(traces, f, separators=(",", ":"))
    print("allocator traces:", len(traces), "traces,", sum(len(t["steps"]) for t in traces), "steps")


# --------------------------------------------------------------------------
# 2. decode cases
# --------------------------------------------------------------------------
def _engine_decode_mask(ref, block_mask, bidx, pos):
    """The reference engine's own slice of the logical causal block mask
    (PagedInferenceEngine.get_decoding_block_mask), called unbound."""
    from falcon_perception.paged_inference import PagedInferenceEngine
    fake = types.SimpleNamespace(block_mask=block_mask)
    m = PagedInferenceEngine.get_decoding_block_mask(fake, bidx, pos)
    return ref.convert_logical_block_mask(m, bidx)


def run_decode_case(case: wl.DecodeCase, pad_rows=0, max_len=None):
    """Drive reference and oracle through: reserve -> packed append of the
    history -> decode append -> decode attention.  ``pad_rows`` extra rows with
    slot 0 / position 0 are appended to the decode batch (CUDA-graph padding
    in the reference engine)."""
    n_rep = case.Hq // case.Hkv
    f32 = torch.float32
    ref = RefCache(case.n_pages, case.P, case.max_batch_size, case.Hq, case.D, 1, f32, "cpu")
    o = orc.OraclePagedKVCache(case.n_pages, case.P, case.max_batch_size, case.Hkv, case.D, 1, f32)
    ref.free_pages = list(case.free_pages); o.free_pages = list(case.free_pages)
    slots = []
    for L, kh, vh in zip(case.lens, case.k_hist, case.v_hist):
        s = ref.allocate(); assert o.allocate() == s; slots.append(s)
        ref.reserve(s, torch.tensor([s]), L + 1); o.reserve(s, L + 1)
        if L > 0:
            ipos = torch.arange(L).view(1, L); bid = torch.full((1, L), s)
            ref.insert_kv(0, kh.float().repeat_interleave(n_rep, 1), vh.float().repeat_interleave(n_rep, 1),
                          input_pos=ipos, batch_idx=bid)
            o.append_packed(0, bid, ipos, kh.float(), vh.float())
    B = case.B + pad_rows
    bidx = torch.tensor(slots + [0] * pad_rows, dtype=torch.int64)
    pos = torch.tensor(list(case.lens) + [0] * pad_rows, dtype=torch.int32)

    def padded(x):
        return torch.cat([x.float(), torch.zeros((pad_rows,) + tuple(x.shape[1:]))]) if pad_rows else x.float()
    k, v, q = padded(case.k_new), padded(case.v_new), padded(case.q)
    K, V = ref.insert_kv(0, k.repeat_interleave(n_rep, 1), v.repeat_interleave(n_rep, 1),
                         input_pos=pos.view(B, 1), batch_idx=bidx)
    o.append_decode(0, bidx, pos, k, v)
    # pool parity, head-group-wise, page 0 excluded
    for r in range(n_rep):
        assert torch.equal(ref.kv_cache[0][:, :, r::n_rep, case.P:, :], o.kv_cache[0][:, :, :, case.P:, :])
    assert snapshot(ref) == snapshot(o)
    max_len = max_len or (max(case.lens) // case.P + 1) * case.P
    bm = ref.create_causal_blockmask(B=case.max_batch_size, L=max_len)
    pm = _engine_decode_mask(ref, bm, bidx, pos)
    out, aux = compiled_flex_attn_decode(q, K, V, block_mask=pm, return_aux=AuxRequest(lse=True))
    lse = aux.lse
    o_out, o_lse = orc.decode_attention(o, 0, q, bidx, pos)
    err_o = (out - o_out).abs().max().item()
    fin = torch.isfinite(lse)
    assert torch.equal(fin, torch.isfinite(o_lse))
    err_l = (lse[fin] - o_lse[fin]).abs().max().item() if fin.any() else 0.0
    assert err_o < 2e-5 and err_l < 2e-5, (err_o, err_l)
    return dict(out=out.numpy(), lse=lse.numpy(), slots=np.array(slots),
                page_table=ref.page_table.numpy(), pool_sha256=np.array(pool_digest(o.kv_cache[0], case.P)),
                oracle_err=np.array([err_o, err_l]))


def decode_goldens():
    cases = {
        "decode_cfg1": (wl.config1_case(), 0),
        # bf16-rounded inputs, reference run in fp32 (the tolerance target of the bf16 kernels)
        "decode_bf16_d128": (wl.make_decode_case(2101, B=6, Hq=16, Hkv=8, D=128, P=128, n_pages=48,
                                                 max_batch_size=8, len_lo=1, len_hi=700,
                                                 dtype=torch.bfloat16, value_scale=1.0), 2),
        "decode_bf16_scaled": (wl.make_decode_case(2102, B=5, Hq=16, Hkv=8, D=128, P=128, n_pages=48,
                                                   max_batch_size=8, len_lo=100, len_hi=900,
                                                   dtype=torch.bfloat16, value_scale=128 ** -0.5), 0),
        # page-boundary lengths with a small page
        "decode_p16_edges": (wl.make_decode_case(2103, B=7, Hq=8, Hkv=2, D=64, P=16, n_pages=40,
                                                 max_batch_size=9, len_lo=0, len_hi=0, dtype=torch.float32,
                                                 lens=[0, 1, 15, 16, 17, 31, 64]), 1),
        "decode_mha_fp16": (wl.make_decode_case(2104, B=3, Hq=4, Hkv=4, D=64, P=32, n_pages=40,
                                                max_batch_size=5, len_lo=5, len_hi=300,
                                                dtype=torch.float16), 0),
    }
    for name, (case, pads) in cases.items():
        g = run_decode_case(case, pad_rows=pads)
        np.savez_compressed(os.path.join(OUT, name + ".npz"), **g)
        print(name, "lens", case.lens, "oracle-vs-reference err", g["oracle_err"])


# --------------------------------------------------------------------------
# 3. prefill cases
# --------------------------------------------------------------------------
def run_prefill_case(case: wl.PrefillCase, n_pages, max_batch_size):
    n_rep = case.Hq // case.Hkv
    f32 = torch.float32
    ref = RefCache(n_pages, case.P, max_batch_size, case.Hq, case.D, 1, f32, "cpu")
    o = orc.OraclePagedKVCache(n_pages, case.P, max_batch_size, case.Hkv, case.D, 1, f32)
    slots = []
    for toks in case.seq_tokens:
        s = ref.allocate(); assert o.allocate() == s; slots.append(s)
        ref.reserve(s, torch.tensor([s]), len(toks)); o.reserve(s, len(toks))
    bidx = case.batch_idx_for(slots)
    mask = ref.create_prefill_blockmask(bidx, case.input_ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    q, k, v = case.q.float(), case.k.float(), case.v.float()
    K, V = ref.insert_kv(0, k.repeat_interleave(n_rep, 1), v.repeat_interleave(n_rep, 1),
                         input_pos=case.input_pos, batch_idx=bidx)
    o.append_packed(0, bidx, case.input_pos, k, v)
    for r in range(n_rep):
        assert torch.equal(ref.kv_cache[0][:, :, r::n_rep, case.P:, :], o.kv_cache[0][:, :, :, case.P:, :])
    out, aux = compiled_flex_attn_prefill(q, K, V, block_mask=mask, return_aux=AuxRequest(lse=True),
                                          kernel_options={"FORCE_USE_FLEX_ATTENTION": True})
    img = orc.image_span_ids(case.input_ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    o_out, o_lse = orc.prefill_attention(q, k, v, bidx, img)
    live = (case.seq_index.view(-1) > 0)
    err_o = (out - o_out)[0, :, live].abs().max().item()
    err_l = (aux.lse - o_lse)[0, :, live].abs().max().item()
    assert err_o < 2e-5 and err_l < 2e-5, (err_o, err_l)
    # chunked, paged evaluation must give the same rows
    for i, (s, toks) in enumerate(zip(slots, case.seq_tokens)):
        off, L = case.offsets[i], len(toks)
        img_seq = img[off:off + L]
        for c0 in range(0, L, 96):
            c1 = min(L, c0 + 96)
            po, pl = orc.paged_prefill_attention(o, 0, q[0, :, off + c0:off + c1], s, np.arange(c0, c1), L, img_seq)
            assert (po - out[0, :, off + c0:off + c1]).abs().max().item() < 2e-5
            assert (pl - aux.lse[0, :, off + c0:off + c1]).abs().max().item() < 2e-5
    out = out * live.view(1, 1, -1, 1)          # pad rows are never consumed: store zeros there
    lse = aux.lse * live.view(1, 1, -1)
    return dict(out=out.numpy(), lse=lse.numpy(), slots=np.array(slots), img_id=img,
                pool_sha256=np.array(pool_digest(o.kv_cache[0], case.P)), oracle_err=np.array([err_o, err_l]))


def prefill_goldens():
    T = wl.image_text_tokens
    cases = {
        # text only, image in the middle with registers, two images in one sequence, short tail
        "prefill_mixed_d64": (wl.make_prefill_case(3101, [T(3, 100, 20), T(0, 0, 50), T(5, 200, 30) + T(2, 37, 9),
                                                          T(0, 128, 0)],
                                                   Hq=4, Hkv=2, D=64, P=128, dtype=torch.bfloat16), 16, 6),
        "prefill_img_d128": (wl.make_prefill_case(3102, [T(0, 256, 31), T(7, 130, 100)],
                                                  Hq=4, Hkv=2, D=128, P=128, dtype=torch.bfloat16,
                                                  value_scale=1.0), 12, 4),
    }
    for name, (case, n_pages, mb) in cases.items():
        g = run_prefill_case(case, n_pages, mb)
        np.savez_compressed(os.path.join(OUT, name + ".npz"), **g)
        print(name, "L", case.L, "oracle-vs-reference err", g["oracle_err"])


# --------------------------------------------------------------------------
# 4. the sink gate after attention (Attention._post_attention, model.py:122-128)
# --------------------------------------------------------------------------
def post_attention_golden():
    from falcon_perception.model import Attention
    rng = np.random.default_rng(4101)
    B, Hq, S, D = 3, 8, 5, 64
    out = torch.from_numpy(rng.standard_normal((B, Hq, S, D), dtype=np.float32)).bfloat16()
    lse = torch.from_numpy(rng.standard_normal((B, Hq, S), dtype=np.float32) * 3)
    lse[0, 1, 2] = float("-inf")                      # a row that saw no key
    sinks = torch.from_numpy(rng.standard_normal(Hq, dtype=np.float32)).bfloat16()
    fake = types.SimpleNamespace(sinks=sinks, wo=lambda x: x)       # identity projection: the gate and layout only
    ref = Attention._post_attention(fake, out, lse)
    mine = orc.post_attention_gate(out, lse, sinks)
    assert torch.equal(ref, mine)
    np.savez_compressed(os.path.join(OUT, "post_attention.npz"), gated=ref.float().numpy())
    print("post_attention: oracle equals reference bit for bit,", tuple(ref.shape))


# --------------------------------------------------------------------------
# 5. norm, GQA expansion and rotary embedding in front of the cache (Attention._pre_attention, model.py:105-120)
# --------------------------------------------------------------------------
def pre_attention_inputs(seed, B, S, Hq, Hkv, D, with_2d, dtype):
    """Seeded inputs of one case (the tests rebuild the projection from the seed and read the rotary tables from the file)."""
    from falcon_perception.rope import precompute_freqs_cis, apply_golden_freqs_cis_to_visual_pos
    rng = np.random.default_rng(seed)
    qkv = wl.pre_attention_qkv(rng, B, S, Hq, Hkv, D, dtype)
    pos = torch.from_numpy(rng.integers(0, 4096, (B, S)))
    freqs_cis = precompute_freqs_cis(D // 2, 4096)[pos]                         # (B, S, D/4) complex64
    freqs_2d = None
    if with_2d:
        freqs_hFP = torch.from_numpy(rng.standard_normal((Hq, D // 4, 2), dtype=np.float32) * 3)
        pos_hw = torch.from_numpy(rng.uniform(-1, 1, (B, S, 2)).astype(np.float32))
        pos_hw[:, ::3] = 0                                                       # text tokens: identity rotation
        freqs_2d = apply_golden_freqs_cis_to_visual_pos(freqs_hFP, pos_hw)       # (B, S, Hq, D/4) complex64
    return qkv, freqs_cis, freqs_2d


def pre_attention_goldens():
    from falcon_perception.model import Attention
    for name, (seed, B, S, Hq, Hkv, D, with_2d, dtype) in wl.PRE_ATTENTION_CASES.items():
        qkv, fc, fc2 = pre_attention_inputs(seed, B, S, Hq, Hkv, D, with_2d, dtype)
        fake = types.SimpleNamespace(wqkv=lambda x: qkv, q_dim=Hq * D, kv_dim=Hkv * D, head_dim=D, n_rep=Hq // Hkv)
        x = torch.zeros(B, S, 16, dtype=dtype)                                   # the projection is injected: x is unused
        rq, rk, rv = Attention._pre_attention(fake, x, fc, fc2)
        mq, mk, mv = orc.pre_attention_tail(qkv, Hq, Hkv, D, fc, fc2)
        assert torch.equal(rq, mq) and torch.equal(rk, mk) and torch.equal(rv, mv), name
        np.savez_compressed(os.path.join(OUT, name + ".npz"), xq=rq.float().numpy(), xk=rk.float().numpy(),
                            freqs_cis=torch.view_as_real(fc).numpy(),
                            freqs_cis_2d=torch.view_as_real(fc2).numpy() if fc2 is not None else np.zeros(0, np.float32))
        print(name + ": oracle equals reference bit for bit,", tuple(rq.shape), tuple(rk.shape))


if __name__ == "__main__":
    torch.manual_seed(0)
    pre_attention_goldens()
    post_attention_golden()
    allocator_traces()
    decode_goldens()
    prefill_goldens()
