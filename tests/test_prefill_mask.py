"""CPU: the prefix-extent form of the prefill mask is the reference's mask.

The kernels never see image ids: they get one number per packed token, the
length of the visible prefix of its own sequence.  This checks, on the dense
(L, L) mask the oracle builds from the reference's rule, that the two agree."""

import numpy as np
import torch

import workloads as wl
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


def test_unclosed_span_is_cut_at_the_sequence_end_and_reported():
    """A span without its end-of-image token runs on, by the reference's rule, into the sequences packed
    behind it (tokens of different sequences would see each other).  Here it ends with its own sequence and
    the caller is told through the status word."""
    open_span = [wl.TEXT_ID] * 3 + [wl.IMG_CLS_ID] + [wl.IMG_PATCH_ID] * 6          # no end-of-image token
    case = wl.make_prefill_case(2, [open_span, T(2, 5, 3), T(0, 0, 40)], Hq=2, Hkv=1, D=64)
    doc = case.batch_idx_for([1, 2, 3]).view(-1).to(torch.int32)
    img = image_span_ids(case.input_ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    # the reference's rule really crosses the boundary: the open span reaches the second sequence's first tokens
    allowed = orc.prefill_allowed(doc.numpy(), img.numpy())
    first_of_second = int((doc == 2).nonzero()[0])
    assert allowed[3, first_of_second] and doc[3] == 1
    status = torch.zeros(1, dtype=torch.int32)
    ext = prefill_extents(doc, img, case.input_pos.view(-1), status)
    assert int(status) == 16
    # sequence 1: rows 0..2 causal, rows 3..9 (the span) see the whole sequence, nothing beyond it
    assert ext[:10].tolist() == [1, 2, 3, 10, 10, 10, 10, 10, 10, 10]
    # By the reference's cumulative counts the damage is not local: one missing end token leaves every later
    # token of the packed row "inside an image" (the second sequence's own end token only brings the count
    # back to one).  Each run of equal image number is cut at the end of its own sequence.
    second = ext[first_of_second:first_of_second + 11].tolist()
    assert second == [2, 2] + [11] * 9
    third = (doc == 3).nonzero().view(-1)
    assert ext[third].tolist() == [40] * 40
    assert (ext[doc == 0] == 0).all()
    # closed spans raise nothing
    status.zero_()
    case2 = wl.make_prefill_case(3, [T(2, 5, 3), T(1, 9, 2)], Hq=2, Hkv=1, D=64)
    prefill_extents(case2.batch_idx_for([1, 2]).view(-1).to(torch.int32),
                    image_span_ids(case2.input_ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID), case2.input_pos.view(-1), status)
    assert int(status) == 0
