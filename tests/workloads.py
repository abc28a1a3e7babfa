"""Seeded synthetic inputs for the paged KV-cache path.

The reference project measures on model checkpoints and datasets that are
fetched from the network; none of that is used here.  These generators build
inputs with the same shapes, dtypes and value distributions from a seed, on
the CPU, with numpy's PCG64 stream so that the same seed gives the same bytes
on every machine.  Both the tests and the benchmark draw from here.

Draw order for a decode case (fixed; golden files depend on it):
  lens -> page permutation -> per sequence (k_hist, v_hist) -> k_new, v_new, q.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

# Synthetic token ids for packed prefill rows.  The reference's tokenizer
# supplies the real ids (falcon_perception/paged_inference.py:694-699); only
# their roles matter to the mask.
PAD_ID, IMG_CLS_ID, END_OF_IMG_ID, IMG_PATCH_ID, TEXT_ID = 0, 3, 4, 5, 6


def _normal(rng, shape, scale, dtype):
    x = rng.standard_normal(shape, dtype=np.float32)
    if scale != 1.0:
        x *= np.float32(scale)
    return torch.from_numpy(x).to(dtype)


@dataclass
class DecodeCase:
    """One decode step over B sequences with existing context in pages."""
    B: int
    Hq: int
    Hkv: int
    D: int
    P: int
    n_pages: int
    max_batch_size: int
    dtype: torch.dtype
    lens: list                      # context length of each sequence BEFORE the new token
    free_pages: list                # shuffled free list handed to the cache before reserving
    k_hist: list = field(default_factory=list)   # per sequence (1,Hkv,L,D)
    v_hist: list = field(default_factory=list)
    k_new: torch.Tensor = None      # (B,Hkv,1,D)
    v_new: torch.Tensor = None
    q: torch.Tensor = None          # (B,Hq,1,D)


def make_decode_case(seed, B, Hq, Hkv, D, P, n_pages, max_batch_size, len_lo,
                     len_hi, dtype=torch.float32, value_scale=1.0,
                     lens=None, with_history=True) -> DecodeCase:
    rng = np.random.default_rng(seed)
    drawn = rng.integers(len_lo, len_hi + 1, size=B).tolist()
    lens = drawn if lens is None else list(lens)
    free_pages = (rng.permutation(n_pages - 1) + 1).tolist()
    case = DecodeCase(B, Hq, Hkv, D, P, n_pages, max_batch_size, dtype, lens, free_pages)
    if with_history:
        for L in lens:
            case.k_hist.append(_normal(rng, (1, Hkv, L, D), value_scale, dtype))
            case.v_hist.append(_normal(rng, (1, Hkv, L, D), value_scale, dtype))
    case.k_new = _normal(rng, (B, Hkv, 1, D), value_scale, dtype)
    case.v_new = _normal(rng, (B, Hkv, 1, D), value_scale, dtype)
    case.q = _normal(rng, (B, Hq, 1, D), value_scale, dtype)
    return case


def config1_case() -> DecodeCase:
    """The CPU-runnable fp32 case: batch 4, 16/8 heads, head_dim 64, page 128,
    64-page pool, context uniform in [64,512], values N(0,1)."""
    return make_decode_case(1001, B=4, Hq=16, Hkv=8, D=64, P=128, n_pages=64,
                            max_batch_size=8, len_lo=64, len_hi=512,
                            dtype=torch.float32)


def config2_case(B=64, n_pages=65536, len_lo=1024, len_hi=8192, with_history=False,
                 seed=2002) -> DecodeCase:
    """bf16 decode: batch 64, 16/8 heads, head_dim 128, page 128, context
    uniform in [1024,8192], page ids permuted over a 64K-page pool, values
    N(0,1)/sqrt(head_dim).  ``with_history=False`` leaves the (large) context
    K/V to the caller, e.g. generated directly on the device."""
    return make_decode_case(seed, B=B, Hq=16, Hkv=8, D=128, P=128, n_pages=n_pages,
                            max_batch_size=B + 1, len_lo=len_lo, len_hi=len_hi,
                            dtype=torch.bfloat16, value_scale=128 ** -0.5,
                            with_history=with_history)


@dataclass
class PrefillCase:
    """One packed prefill row: every sequence starts on a multiple of
    ``align`` tokens; the gap is filled with pad tokens that carry slot 0 and
    position 0 (falcon_perception/paged_inference.py:637-678)."""
    Hq: int
    Hkv: int
    D: int
    P: int
    dtype: torch.dtype
    seq_tokens: list                # per sequence: list of token ids
    offsets: list                   # start of each sequence in the packed row
    input_ids: torch.Tensor = None  # (1,L) int64
    input_pos: torch.Tensor = None  # (1,L) int64
    seq_index: torch.Tensor = None  # (1,L) int64: 1-based sequence number, 0 for pads
    q: torch.Tensor = None          # (1,Hq,L,D)
    k: torch.Tensor = None          # (1,Hkv,L,D)
    v: torch.Tensor = None

    @property
    def L(self):
        return int(self.input_ids.shape[1])

    def batch_idx_for(self, slots):
        """(1,L) int64 slot id per token given the slot of each sequence."""
        lut = torch.tensor([0] + list(slots), dtype=torch.int64)
        return lut[self.seq_index]


def image_text_tokens(n_lead_text, n_image, n_text, registers=0):
    """<text>*n_lead, <cls> reg*registers <img>*(n_image-1-registers) <eoi>,
    <text>*n_text: the image span is n_image tokens, CLS inclusive, EOI
    exclusive (falcon_perception/data.py:513-522 lays real ones out this way
    with four register tokens)."""
    toks = [TEXT_ID] * n_lead_text
    if n_image > 0:
        toks += [IMG_CLS_ID] + [IMG_PATCH_ID] * (n_image - 1) + [END_OF_IMG_ID]
    toks += [TEXT_ID] * n_text
    return toks


def make_prefill_case(seed, seq_tokens, Hq, Hkv, D, P=128, align=128,
                      dtype=torch.float32, value_scale=1.0) -> PrefillCase:
    rng = np.random.default_rng(seed)
    ids, pos, sidx, offsets, off = [], [], [], [], 0
    for i, toks in enumerate(seq_tokens):
        L = len(toks)
        gap = (-L) % align
        offsets.append(off)
        ids += list(toks) + [PAD_ID] * gap
        pos += list(range(L)) + [0] * gap
        sidx += [i + 1] * L + [0] * gap
        off += L + gap
    case = PrefillCase(Hq, Hkv, D, P, dtype, [list(t) for t in seq_tokens], offsets)
    case.input_ids = torch.tensor(ids, dtype=torch.int64).view(1, -1)
    case.input_pos = torch.tensor(pos, dtype=torch.int64).view(1, -1)
    case.seq_index = torch.tensor(sidx, dtype=torch.int64).view(1, -1)
    Ltot = off
    case.q = _normal(rng, (1, Hq, Ltot, D), value_scale, dtype)
    case.k = _normal(rng, (1, Hkv, Ltot, D), value_scale, dtype)
    case.v = _normal(rng, (1, Hkv, Ltot, D), value_scale, dtype)
    return case


def config3_prefill_case(n_seq=8, seed=3003) -> PrefillCase:
    """bf16 multimodal prefill: each sequence is a 1024-token image block
    (CLS + 1023 patches = the 32x32 grid) followed by end-of-image and 63 text
    tokens (1088 tokens, packed to 1152)."""
    toks = image_text_tokens(0, 1024, 63)
    return make_prefill_case(seed, [toks] * n_seq, Hq=16, Hkv=8, D=128, P=128,
                             dtype=torch.bfloat16, value_scale=128 ** -0.5)


# Cases of the fused "norm + rotary embedding + append" step.  name: (seed, B, S, Hq, Hkv, D, with_2d, dtype).
# The rotary tables of a case are stored with its golden file; the projection is rebuilt from the seed.
PRE_ATTENTION_CASES = {
    "pre_attention_bf16_2d": (5101, 2, 7, 8, 4, 128, True, torch.bfloat16),
    "pre_attention_bf16_text": (5102, 5, 1, 8, 4, 128, False, torch.bfloat16),
    "pre_attention_f16_d64": (5103, 1, 9, 4, 4, 64, True, torch.float16),
    "pre_attention_f32": (5104, 2, 3, 4, 2, 64, True, torch.float32),
}


def pre_attention_qkv(rng, B, S, Hq, Hkv, D, dtype):
    """The QKV projection output of a case: the first draw of its generator."""
    return torch.from_numpy(rng.standard_normal((B, S, (Hq + 2 * Hkv) * D), dtype=np.float32) * 1.7).to(dtype)
