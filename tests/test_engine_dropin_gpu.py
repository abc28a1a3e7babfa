"""GPU: the reference's own inference engine, end to end, on this package's cache.

``PagedInferenceEngine.generate`` of the reference (scheduler with admission and a waiting queue, packed prefill with
an image span, decode steps with page growth, CUDA-graph capture of the decode forward, ``paged_inference.py:289-1374``)
runs a small random-init ``FalconPerception`` over four pre-tokenised requests, once with the reference's
``PagedKVCache`` + FlexAttention and once per configuration with ``fpkv.PagedKVCache`` put in its place:

  * ``falcon_perception.paged_inference.PagedKVCache`` replaced by a factory for ``fpkv.PagedKVCache`` (the reference's
    expanded head layout, or the split layout with the KV heads),
  * ``Attention.forward`` re-routed by ``fpkv.engine_glue.install_attention``,
  * ``get_decoding_block_mask`` replaced by the three-line form of ``fpkv.engine_glue.decoding_block_mask``.

Nothing else of the engine is touched.  Every request must come back with exactly the reference's tokens (in bf16: up
to a step where the reference's own logits hold a tie that rounding decides).  Requests:
one with an image span (2-D rotary positions, image-prefix mask), one that crosses a page boundary while decoding,
and one more than there are slots, so that it is admitted while others decode.  The reference is not part of this
repository: the test is skipped when it is not installed under baseline/_ref (or named by FALCON_PERCEPTION_SRC).
"""

import os
import sys
import types

import pytest
import torch

from fpkv.engine_glue import decoding_block_mask, install_attention, install_engine
from fpkv.paged_attention import PagedKVCache
from test_dropin_gpu import _reference_root

pytestmark = pytest.mark.gpu
SOI, EOI, IMG = 3, 4, 5


class FakeTokenizer:
    """The attributes the engine and ``ModelArgs.update`` read; requests arrive tokenised."""
    padding_side = "right"
    pad_token_id, eos_token_id, bos_id = 0, 1, None
    start_of_image_token_id, image_cls_token_id, end_of_image_token_id, image_token_id = 2, SOI, EOI, IMG
    image_row_sep_token_id = 7
    image_reg_1_token_id, image_reg_2_token_id, image_reg_3_token_id, image_reg_4_token_id = 8, 9, 10, 11
    seg_token_id, coord_token_id, size_token_id = 12, 13, 14


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
    import falcon_perception.paged_inference as ref_engine
    # the uncompiled FlexAttention functions: same arithmetic, no minutes-long kernel generation
    from torch.nn.attention.flex_attention import create_block_mask, flex_attention
    ref_model.compiled_flex_attn_decode = flex_attention
    ref_model.compiled_flex_attn_prefill = flex_attention
    ref_attention._compiled_create_block_mask = create_block_mask
    return types.SimpleNamespace(model=ref_model, engine=ref_engine)


def build_model(ref, dtype, head_dim=128):
    from falcon_perception import ModelArgs
    args = ModelArgs(max_seq_len=1024, dim=256, n_layers=2, n_heads=4, head_dim=head_dim, n_kv_heads=2, vocab_size=512,
                     ffn_dim=512, perception_heads=False, do_segmentation=False)
    args.update(FakeTokenizer())
    torch.manual_seed(1234)
    m = ref.model.FalconPerception(args)
    with torch.no_grad():
        for layer in m.layers.values():
            layer.attention.sinks.copy_(torch.randn(args.n_heads))
        m.freqs_cis_golden.copy_(torch.randn(args.n_heads, args.head_dim // 4, 2) * 0.3)   # one 2-D table row per query head
    return m.to(device="cuda", dtype=dtype).eval(), args


def make_requests(ref):
    gen = torch.Generator().manual_seed(11)
    a = [30] * 5 + [SOI] + [IMG] * 119 + [EOI] + [31] * 30           # text, a 12 x 10 patch image, text
    hw = torch.zeros(len(a), 2)
    hw[6:6 + 119] = torch.stack([torch.arange(1, 120) // 10, torch.arange(1, 120) % 10], 1).float()
    specs = [(a, hw)]
    for n in (70, 250, 33):                                          # 250 + 12 new tokens crosses a page boundary
        specs.append((torch.randint(20, 500, (n,), generator=gen).tolist(), torch.zeros(n, 2)))
    requests = []
    for i, (ids, rhw) in enumerate(specs):
        s = ref.engine.Sequence(text="", image=None, request_idx=i, task="detection")
        s.input_ids = torch.tensor(ids, dtype=torch.int64)           # set: the engine skips its tokeniser
        s.rope_pos_t = torch.arange(len(ids), dtype=torch.long)
        s.rope_pos_hw = rhw
        requests.append(s)
    return requests


def generate(ref, model, args, cache, graphs, batched_setup=False):
    eng_mod = ref.engine
    saved = (eng_mod.PagedKVCache, eng_mod.PagedInferenceEngine.get_decoding_block_mask, ref.model.Attention.forward)
    restore = None
    try:
        if cache != "reference":
            def fpkv_cache(**kw):
                if cache == "split":                                 # KV heads stored once, second K halves per query head
                    kw = dict(kw, n_heads=args.n_kv_heads, split_q_heads=args.n_heads)
                return PagedKVCache(**kw)
            if batched_setup:                                        # all substitutions at once, decode set-up batched too
                restore = install_engine(eng_mod, ref.model.Attention, fused=True, cache_factory=fpkv_cache)
            else:
                eng_mod.PagedKVCache = fpkv_cache
                eng_mod.PagedInferenceEngine.get_decoding_block_mask = \
                    lambda self, batch_idx, input_pos: decoding_block_mask(self.block_mask, batch_idx, input_pos)
                install_attention(ref.model.Attention, fused=True)
        engine = eng_mod.PagedInferenceEngine(model, FakeTokenizer(), None, max_batch_size=4, max_seq_length=1024,
                                              n_pages=24, seed=0, enable_hr_cache=False, capture_cudagraph=graphs,
                                              max_decode_steps_between_prefills=3)
        done = engine.generate(make_requests(ref),
                               sampling_params=eng_mod.SamplingParams(max_new_tokens=12, stop_token_ids=[1]))
        if cache != "reference":
            engine.paged_kv_cache.check_status()
            assert engine.paged_kv_cache.num_free_pages == 23 and len(engine.paged_kv_cache.free_batch_idx) == 3
        return [(s.output_ids.tolist(), s.output_probs.tolist()) for s in done]
    finally:
        if restore is not None:
            restore()
        else:
            eng_mod.PagedKVCache, eng_mod.PagedInferenceEngine.get_decoding_block_mask, ref.model.Attention.forward = saved


def same_tokens(want, got, what, tie):
    """Every request's tokens equal the reference's.  With tie > 0 (16-bit models) a request may part ways at a step
    where the two runs' chosen tokens have the same probability within `tie` (a tie in the reference's own logits that
    rounding decides); what follows such a step is no longer comparable."""
    parted = 0
    for r, ((w, wp), (g, gp)) in enumerate(zip(want, got)):
        assert len(w) == len(g), f"{what}: request {r} has {len(g)} tokens, the reference {len(w)}"
        for i, (a, b) in enumerate(zip(w, g)):
            if a != b:
                assert tie > 0 and abs(wp[i] - gp[i]) <= tie * max(wp[i], gp[i]), \
                    f"{what}: request {r} step {i}: token {b} (p = {gp[i]:.4f}) against the reference's {a} (p = {wp[i]:.4f})"
                parted += 1
                break
    return parted


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reference_engine_generates_the_same_tokens_on_the_fpkv_cache(ref, dtype):
    model, args = build_model(ref, dtype)
    tie = 0.0 if dtype == torch.float32 else 0.05
    # (the uncompiled FlexAttention cannot be captured in a CUDA graph; the reference side runs its decode eagerly)
    want = generate(ref, model, args, "reference", graphs=False)
    assert len(want) == 4 and all(len(t) == 12 for t, _ in want)
    parted = 0
    for cache in ("expanded", "split"):
        for graphs in (False, True):
            got = generate(ref, model, args, cache, graphs)
            parted += same_tokens(want, got, f"{cache} pool, {'CUDA graphs' if graphs else 'eager decode'}", tie)
    # the engine's own decode step with its per-request copies batched (install_engine), graphs on
    got = generate(ref, model, args, "split", graphs=True, batched_setup=True)
    parted += same_tokens(want, got, "batched decode set-up", tie)
    assert parted <= 4, f"{parted} of 20 request runs parted from the reference at a tie: too many to be chance"


def test_reference_engine_with_head_dim_64_on_the_expanded_pool(ref):
    """The smaller released variants have head_dim 64: their exact layout is the reference's own (one stored head per
    query head), served by the same tiled kernels (single-head items in prefill, n_rep = 1 in decode)."""
    model, args = build_model(ref, torch.bfloat16, head_dim=64)
    want = generate(ref, model, args, "reference", graphs=False)
    got = generate(ref, model, args, "expanded", graphs=True, batched_setup=True)
    assert same_tokens(want, got, "head_dim 64, expanded pool", 0.05) <= 1
