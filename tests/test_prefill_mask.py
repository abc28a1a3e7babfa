"""CPU: the prefix-extent form of the prefill mask is the reference's mask.

The kernels never see image ids: they get one number per packed token, the
length of the visible prefix of its own sequence.  This checks, on the dense
(L, L) mask the oracle builds from the reference's rule, that the two agree."""

import numpy as np
import torch

from fpkv import workloads as wl
from fpkv.attention import image_span_ids, prefill_extents
from oracle import paged_kv_oracle as orc

T = wl.image_text_tokens


def _check(seq_tokens):
    case = wl.make_prefill_case(1, seq_tokens, Hq=2, Hkv=1, D=64)
    slots = list(range(1, len(seq_tokens) + 1))
    doc = case.batch_idx_for(slots).view(-1)
    img = image_span_ids(case.input_ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    assert np.array_equal(img.numpy(), orc.image_span_ids(case.input_ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID))
    ext = prefill_extents(doc.to(torch.int32), img, case.input_pos.view(-1)).numpy()
    allowed = orc.prefill_allowed(doc.numpy(), img.numpy())
    pos = case.input_pos.view(-1).numpy()
    L = case.L
    for t in range(L):
        if doc[t] == 0:
            assert ext[t] == 0
            continue
        same_doc = (doc.numpy() == int(doc[t]))
        want = allowed[t] & same_doc                     # visible keys of row t, as packed indices
        got = same_doc & (pos < ext[t])
        assert np.array_equal(want, got), t
        assert (allowed[t] & ~same_doc).sum() == 0       # nothing outside the own sequence is ever visible
    return ext


def test_extent_equals_reference_mask():
    _check([T(3, 100, 20), T(0, 0, 50), T(5, 200, 30) + T(2, 37, 9), T(0, 128, 0)])
    _check([T(0, 1024, 63)] * 2)
    ext = _check([T(2, 5, 3)])
    # <t><t> <cls><p><p><p><p> <eoi> <t><t><t>: span = positions 2..6, so rows 2..6 all see 7 keys
    assert ext[:11].tolist() == [1, 2, 7, 7, 7, 7, 7, 8, 9, 10, 11]
