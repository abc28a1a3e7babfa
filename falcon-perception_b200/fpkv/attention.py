"""Mask descriptors for the paged attention kernels.

The reference builds FlexAttention ``BlockMask`` objects (sparsity metadata
plus a ``mask_mod`` closure, ``falcon_perception/attention.py:22-102``) and
converts them to physical page ids every decode step
(``falcon_perception/paged_attention.py:234-301``).  The kernels here derive
the same visibility rule from the index tensors themselves, so a mask is just
a small record of those tensors.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor


@dataclass
class CausalDecodeMask:
    """Logical causal mask over ``B`` slots and ``L`` positions with
    ``page_size`` blocks: what ``create_causal_blockmask`` returns.  Row b at
    position p sees keys 0..p of its own slot."""
    B: int
    L: int
    page_size: int

    @property
    def BLOCK_SIZE(self):
        return (self.page_size, self.page_size)

    @property
    def seq_lengths(self):
        return (self.L, self.L)

    def for_step(self, batch_idx: Tensor, input_pos: Tensor) -> "DecodeStepMask":
        """The slice the reference engine takes each decode step
        (``paged_inference.py:783-826``)."""
        return DecodeStepMask(batch_idx, input_pos, self.page_size)


@dataclass
class DecodeStepMask:
    """Decode-step mask: slot and position of every row of the batch."""
    batch_idx: Tensor
    input_pos: Tensor
    page_size: int


@dataclass
class PrefillMask:
    """Packed-row prefill mask (``paged_attention.py:343-362``): query t sees
    key u iff both lie in the same image span (``img_id`` equal and non-zero)
    or u <= t within the same document (``doc_id`` equal)."""
    doc_id: Tensor      # (L,) int32 slot of each token, 0 for pads
    img_id: Tensor      # (L,) int32 running image number, 0 outside image spans
    BLOCK_SIZE: int = 128
    _extent: Tensor | None = None     # filled on first use, shared by all layers of the step

    @property
    def L(self):
        return int(self.doc_id.shape[0])

    def extent(self, input_pos: Tensor, status: Tensor | None = None) -> Tensor:
        """Visible-prefix length of every packed token (int32, (L,)): the
        whole mask in one number per row.  A query sees keys u <= pos of its
        own sequence, plus every key of its own image span; a span is a
        contiguous run that contains the query, so the union is the prefix
        [0, extent) with extent = pos + 1 outside spans and the span's end
        inside one.  Pads (slot 0) get 0.  ``status`` (device int32 word) gets
        STATUS_OPEN_SPAN when a span had to be cut at its sequence's end."""
        if self._extent is None:
            self._extent = prefill_extents(self.doc_id, self.img_id, input_pos.reshape(-1), status)
        return self._extent


STATUS_OPEN_SPAN = 16


def image_span_ids(input_ids: Tensor, soi_id: int, eoi_id: int) -> Tensor:
    """Per-token image number of a (1,L) or (L,) id row: tokens from an
    image-start token (inclusive) to the next end-of-image token (exclusive)
    carry the running count of image starts, all others 0
    (``falcon_perception/attention.py:79-88``).  Integer prefix sums on the
    tensor's own device."""
    ids = input_ids.reshape(-1)
    n_soi = torch.cumsum(ids == soi_id, dim=0)
    n_eoi = torch.cumsum(ids == eoi_id, dim=0)
    inside = (n_soi - n_eoi) > 0
    return (n_soi * inside).to(torch.int32)


def prefill_extents(doc_id: Tensor, img_id: Tensor, input_pos: Tensor, status: Tensor | None = None) -> Tensor:
    """extent[t] for a packed row (see ``PrefillMask.extent``).  Index
    arithmetic on the tensors' device, no host synchronisation: the end of
    token t's image span is the last packed index that carries the same image
    number, found with one scatter-max over the row.

    A span that is not closed by an end-of-image token inside its own sequence
    runs on, by the reference's rule (``falcon_perception/attention.py:79-88``:
    the counts are cumulative over the whole packed row), into the pads and
    the sequences packed behind it, and the reference then lets tokens of
    different sequences see each other.  Keys of another sequence are not
    reachable through one slot's pages, and the engine never builds such a
    prompt, so here the span is cut at the end of its own sequence and
    ``STATUS_OPEN_SPAN`` is OR-ed into ``status`` (when given) so that the
    caller hears about it from ``check_status``."""
    L = doc_id.shape[0]
    idx = torch.arange(L, device=doc_id.device, dtype=torch.int64)
    img = img_id.to(torch.int64)
    last = torch.zeros(L + 1, dtype=torch.int64, device=doc_id.device).scatter_reduce_(0, img, idx, "amax")
    # last packed index of the run of equal slot ids that token t belongs to (a sequence is one such run)
    run_ends = torch.ones(L, dtype=torch.bool, device=doc_id.device)
    run_ends[:-1] = doc_id[1:] != doc_id[:-1]
    seq_last = torch.where(run_ends, idx, torch.full_like(idx, L)).flip(0).cummin(0).values.flip(0)
    span_last = last[img]
    crosses = (img > 0) & (doc_id > 0) & (span_last > seq_last)
    if status is not None:
        status.bitwise_or_((crosses.any() * STATUS_OPEN_SPAN).to(status.dtype))
    pos = input_pos.to(torch.int64)
    ext = torch.where(img > 0, pos + (torch.minimum(span_last, seq_last) - idx) + 1, pos + 1)
    return torch.where(doc_id > 0, ext, torch.zeros_like(ext)).to(torch.int32)
