"""GPU: the reference's own model and call site with this package's cache dropped in.

A small random-init ``FalconPerception`` (the reference's class, imported from its
installed copy) runs the same packed prompts -- two sequences, one with an image
span and 2-D rotary positions -- and then greedy decode steps through

  (i)  the reference's ``PagedKVCache`` + its mask pipeline + FlexAttention, and
  (ii) ``fpkv.PagedKVCache`` behind the reference's ``Attention.forward``, re-routed
       by ``fpkv.engine_glue.install_attention`` (both the plain and the fused form),
       with ``SlotState`` supplying the decode step's inputs.

Logits must agree within the 16-bit tolerance at every step and the greedy token
must be the same wherever the reference's own top-2 margin exceeds that tolerance.
The reference is not part of this repository: the test is skipped when it is not
installed under baseline/_ref (or named by FALCON_PERCEPTION_SRC).

The reference's FlexAttention handles are ``torch.compile`` objects; the test swaps
in the uncompiled functions (same arithmetic, no minutes-long kernel generation)
unless FPKV_DROPIN_COMPILED=1 asks for the stock compiled path.
"""

import os
import sys
import types

import pytest
import torch

from fpkv.engine_glue import SlotState, decoding_block_mask, install_attention
from fpkv.paged_attention import PagedKVCache

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOI, EOI, IMG, TXT = 3, 4, 5, 6


def _reference_root():
    for cand in (os.path.join(ROOT, "baseline", "_ref"), os.environ.get("FALCON_PERCEPTION_SRC", "")):
        if cand and os.path.isdir(os.path.join(cand, "falcon_perception")):
            return cand
    return None


@pytest.fixture(scope="module")
def ref():
    root = _reference_root()
    if root is None:
        pytest.skip("the reference project is not installed under baseline/_ref")
    if root not in sys.path:
        sys.path.insert(0, root)
    stub = types.ModuleType("pycocotools"); stub.mask = types.ModuleType("pycocotools.mask")   # post-processing only
    sys.modules.setdefault("pycocotools", stub); sys.modules.setdefault("pycocotools.mask", stub.mask)
    import falcon_perception.attention as ref_attention
    import falcon_perception.model as ref_model
    import falcon_perception.paged_attention as ref_paged
    from falcon_perception.paged_inference import PagedInferenceEngine
    if os.environ.get("FPKV_DROPIN_COMPILED") != "1":
        from torch.nn.attention.flex_attention import create_block_mask, flex_attention
        ref_model.compiled_flex_attn_decode = flex_attention
        ref_model.compiled_flex_attn_prefill = flex_attention
        ref_attention._compiled_create_block_mask = create_block_mask
    return types.SimpleNamespace(model=ref_model, paged=ref_paged, engine=PagedInferenceEngine)


def build_model(ref, dtype, golden_per_query_head):
    from falcon_perception import ModelArgs
    args = ModelArgs(max_seq_len=1024, dim=256, n_layers=2, n_heads=4, head_dim=128, n_kv_heads=2, vocab_size=512,
                     ffn_dim=512, perception_heads=False, do_segmentation=False)
    torch.manual_seed(1234)
    m = ref.model.FalconPerception(args)
    with torch.no_grad():
        for layer in m.layers.values():
            layer.attention.sinks.copy_(torch.randn(args.n_heads))
        g = torch.randn(args.n_heads, args.head_dim // 4, 2) * 0.3
        if not golden_per_query_head:                         # the same 2-D frequencies within a GQA group
            g = g[:: args.n_heads // args.n_kv_heads].repeat_interleave(args.n_heads // args.n_kv_heads, 0)
        m.freqs_cis_golden.copy_(g)
    return m.to(device="cuda", dtype=dtype).eval(), args


def packed_prompts():
    """Two prompts packed with 128-alignment as the engine packs them (paged_inference.py:634-678):
    text + a 12 x 10 patch image + text, and plain text."""
    gen = torch.Generator().manual_seed(7)
    a_ids = [TXT] * 5 + [SOI] + [IMG] * 119 + [EOI] + [TXT] * 30
    b_ids = torch.randint(6, 500, (70,), generator=gen).tolist()
    hw = torch.zeros(len(a_ids), 2)
    hw[6:6 + 119] = torch.stack([torch.arange(1, 120) // 10, torch.arange(1, 120) % 10], 1).float()
    seqs = [(a_ids, hw), (b_ids, torch.zeros(len(b_ids), 2))]
    ids, pos, doc, rhw, offsets, off = [], [], [], [], [], 0
    for i, (t, h) in enumerate(seqs):
        gap = (-len(t)) % 128
        ids += t + [0] * gap; pos += list(range(len(t))) + [0] * gap; doc += [i + 1] * len(t) + [0] * gap
        rhw.append(torch.cat([h, torch.zeros(gap, 2)])); offsets.append(off); off += len(t) + gap
    return (torch.tensor(ids).view(1, -1), torch.tensor(pos).view(1, -1), torch.tensor(doc).view(1, -1),
            torch.cat(rhw).view(1, -1, 2), offsets, [len(t) for t, _ in seqs])


def run_reference(ref, model, args, dtype, n_steps):
    ids, pos, doc, rhw, offsets, lens = (x.cuda() if torch.is_tensor(x) else x for x in packed_prompts())
    cache = ref.paged.PagedKVCache(16, 128, 4, args.n_heads, args.head_dim, args.n_layers, dtype, "cuda")
    slots = [cache.allocate() for _ in lens]
    for s, n in zip(slots, lens):
        cache.reserve(s, torch.tensor([s], device="cuda"), n + n_steps + 1)
    bidx = torch.tensor([0] + slots, device="cuda")[doc]
    mask = cache.create_prefill_blockmask(bidx, ids, SOI, EOI)
    with torch.inference_mode():
        logits, _ = model.forward(ids, mask, cache, rope_pos_t=pos, rope_pos_hw=rhw, input_pos=pos, batch_idx=bidx,
                                  flex_attn_kernel_options={"FORCE_USE_FLEX_ATTENTION": True})
        last = torch.tensor([o + n - 1 for o, n in zip(offsets, lens)], device="cuda")
        out = [logits[0, last].float()]
        engine = types.SimpleNamespace(block_mask=cache.create_causal_blockmask(B=4, L=1024))
        sl = torch.tensor(slots, device="cuda")
        cur = torch.tensor(lens, dtype=torch.int32, device="cuda")
        for _ in range(n_steps):
            tok = out[-1].argmax(-1)
            m = ref.engine.get_decoding_block_mask(engine, sl, cur)
            m = cache.convert_logical_block_mask(m, sl)
            lg, _ = model.forward(tok.view(-1, 1), m, cache, rope_pos_t=cur.long().view(-1, 1), input_pos=cur.view(-1, 1),
                                  batch_idx=sl, flex_attn_kernel_options={})
            out.append(lg[:, 0].float())
            cur = cur + 1
    return out


def run_fpkv(ref, model, args, dtype, n_steps, stored_heads, forced_tokens, split_q_heads=None):
    ids, pos, doc, rhw, offsets, lens = (x.cuda() if torch.is_tensor(x) else x for x in packed_prompts())
    cache = PagedKVCache(16, 128, 4, stored_heads, args.head_dim, args.n_layers, dtype, "cuda", split_q_heads=split_q_heads)
    slots = [cache.allocate() for _ in lens]
    for s, n in zip(slots, lens):
        cache.reserve(s, None, n + n_steps + 1)
    bidx = torch.tensor([0] + slots, device="cuda")[doc]
    mask = cache.create_prefill_blockmask(bidx, ids, SOI, EOI)
    state = SlotState(4, "cuda")
    with torch.inference_mode():
        logits, _ = model.forward(ids, mask, cache, rope_pos_t=pos, rope_pos_hw=rhw, input_pos=pos, batch_idx=bidx,
                                  flex_attn_kernel_options={"FORCE_USE_FLEX_ATTENTION": True})
        last = torch.tensor([o + n - 1 for o, n in zip(offsets, lens)], device="cuda")
        out = [logits[0, last].float()]
        for s, n, t in zip(slots, lens, forced_tokens[0].tolist()):
            state.begin(s, n, n, t)                           # position of the next token, rope position, first sampled token
        block_mask = cache.create_causal_blockmask(B=4, L=1024)
        for step in range(n_steps):
            B = state.stage(slots)                            # the step's one upload
            sl, cur, rope, tok = state.step_inputs(B)
            m = cache.convert_logical_block_mask(decoding_block_mask(block_mask, sl, cur), sl)
            lg, _ = model.forward(tok.view(-1, 1), m, cache, rope_pos_t=rope.view(-1, 1), input_pos=cur.view(-1, 1),
                                  batch_idx=sl, flex_attn_kernel_options={})
            out.append(lg[:, 0].float())
            # the reference's greedy choice is fed to both runs, so that a near-tie cannot send them down different paths
            state.advance(B, forced_tokens[step + 1] if step + 1 < len(forced_tokens) else lg[:, 0].argmax(-1))
    cache.check_status()
    return out


@pytest.mark.parametrize("dtype,golden_per_head,stored,fused,tol", [
    (torch.bfloat16, False, "kv", True, 6e-2),       # compact pool, every step fused: the fast kernels
    (torch.bfloat16, False, "kv", False, 6e-2),      # compact pool, the reference's own pre/post attention around the calls
    (torch.bfloat16, True, "q", True, 6e-2),         # per-query-head 2-D frequencies: the reference's expanded layout
    (torch.bfloat16, True, "split", True, 6e-2),     # the same frequencies on the split pool (5/8 of the expanded bytes), fused
    (torch.bfloat16, True, "split", False, 6e-2),    # ... and with the reference's own pre/post attention around the calls
    (torch.float32, True, "split", False, 2e-3),
    (torch.float32, True, "q", False, 2e-3),         # fp32 end to end (portable kernels): tight
    (torch.float32, False, "kv", True, 2e-3),
])
def test_reference_model_with_fpkv_cache(ref, dtype, golden_per_head, stored, fused, tol):
    n_steps = 6
    model, args = build_model(ref, dtype, golden_per_head)
    want = run_reference(ref, model, args, dtype, n_steps)
    forced = [w.argmax(-1) for w in want]
    original = install_attention(ref.model.Attention, fused=fused)
    try:
        got = run_fpkv(ref, model, args, dtype, n_steps, args.n_heads if stored == "q" else args.n_kv_heads, forced,
                       split_q_heads=args.n_heads if stored == "split" else None)
    finally:
        ref.model.Attention.forward = original
    same, decided = 0, 0
    for step, (w, g) in enumerate(zip(want, got)):
        scale = w.abs().max().item()
        err = (w - g).abs().max().item()
        assert err <= tol * max(scale, 1.0), f"step {step}: logits differ by {err} (scale {scale})"
        top2 = w.topk(2, -1).values
        clear = (top2[:, 0] - top2[:, 1]) > 4 * err           # rows whose greedy token does not hang on the rounding
        decided += int(clear.sum())
        same += int((w.argmax(-1) == g.argmax(-1))[clear].sum())
        assert torch.equal(w.argmax(-1)[clear], g.argmax(-1)[clear]), f"step {step}: greedy token differs"
    assert decided >= n_steps and same == decided
