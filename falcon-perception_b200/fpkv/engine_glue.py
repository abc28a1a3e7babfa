"""Engine-side glue for an engine built like the reference's PagedInferenceEngine.

The reference engine prepares every decode step on the host and the device in
many small pieces (``falcon_perception/paged_inference.py``): it slices a
FlexAttention ``BlockMask`` and converts it to physical pages (``:783-826``,
``:847-848``), copies slot ids and positions through two pinned buffers, then
issues one tiny device copy per sequence for the rope position, the last token
and the box values (``:966-1003``); prefill and decode are separate steps
(``:1244-1286``) and a prompt is always prefilled whole (``:1162-1204``).  With
the kernels of this package none of the mask work is needed, and the rest
shrinks to:

* ``install_attention`` -- the attention call site of the reference model
  (``model.py:139-164``) routed through ``fpkv.PagedKVCache``;
* ``decoding_block_mask`` -- what ``get_decoding_block_mask`` becomes;
* ``install_decode_setup`` -- the reference engine's own decode step with its
  per-request device copies batched (``:966-1003``), and ``install_engine``,
  which applies all the substitutions to an engine module at once;
* ``SlotState`` -- per-slot position / rope position / last token kept on the
  device (the reference's ``_input_pos`` and ``_rope_pos_t``, ``:346-352``, plus
  the last token), advanced by one batched device update after sampling, so
  that a decode step uploads ONE thing: the list of slots in the batch;
* ``MixedStepPlanner`` -- admission, growth, preemption (the reference's rules,
  ``:1148-1242``) producing steps that mix prefill chunks of newly admitted
  prompts with decode rows of the running sequences, and ``pack_prefill_rows``
  which lays such chunks out as the reference packs a prefill row (``:634-678``).

Host logic only; the K/V path is the CUDA library behind ``PagedKVCache``.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import Tensor

from .attention import CausalDecodeMask, DecodeStepMask, PrefillMask
from .paged_attention import PagedKVCache


# ------------------------------------------------------------ attention call
def decoding_block_mask(block_mask: CausalDecodeMask, batch_idx: Tensor, input_pos: Tensor) -> DecodeStepMask:
    """Replacement body of ``PagedInferenceEngine.get_decoding_block_mask``
    (``paged_inference.py:783-826``): the step's mask is the slot and position
    of every row; the kernels walk the page table themselves."""
    assert batch_idx.ndim == 1, "batch_idx must be 1D"
    assert input_pos.ndim == 1, "input_pos must be 1D"
    return block_mask.for_step(batch_idx, input_pos)


def fpkv_attention_forward(self, x, attention_masks, kv_cache, freqs_cis, freqs_cis_2d=None, input_pos=None,
                           batch_idx=None, flex_attn_kernel_options=None, *, fused: bool = True):
    """``Attention.forward`` of the reference model (``model.py:139-164``) on an
    ``fpkv.PagedKVCache``.  ``self`` is the reference's Attention module (its
    ``wqkv``, ``wo``, ``sinks``, ``n_rep``, ``head_dim``, ``layer_id`` are used).

    fused=True: per-head norm, rotary embedding and the K/V append run as one
    kernel behind the QKV projection, the sink gate and the (B,S,H*D) layout
    come out of the attention kernel, and ``wo`` consumes that directly.
    fused=False: the reference's own ``_pre_attention`` / ``_post_attention``
    around ``insert_kv`` and the paged attention entry (K/V heads sliced back
    to one copy per group when the pool stores the KV heads; a split pool takes
    the expanded K and V as they are)."""
    del flex_attn_kernel_options
    B, S, _ = x.shape
    n_q, n_kv, D = self.n_kv_heads * self.n_rep, self.n_kv_heads, self.head_dim
    decode = S == 1
    if fused:
        qkv = self.wqkv(F.rms_norm(x, (x.size(-1),)))
        xq = kv_cache.pre_attention_append(self.layer_id, qkv, n_q, n_kv, freqs_cis, freqs_cis_2d, batch_idx, input_pos)
        if decode:
            out, _ = kv_cache.decode_attention(self.layer_id, xq, batch_idx, input_pos.reshape(-1), sinks=self.sinks)
        else:
            out, _ = kv_cache.prefill_attention(self.layer_id, xq, batch_idx, input_pos, attention_masks,
                                                sinks=self.sinks, token_major=True)
        return self.wo(out.reshape(B, S, n_q * D))
    xq, xk, xv = self._pre_attention(x, freqs_cis, freqs_cis_2d)
    if kv_cache.n_heads == n_kv and self.n_rep > 1 and not kv_cache.split_q_heads:   # each KV head stored once: drop the copies
        xk, xv = xk[:, ::self.n_rep], xv[:, ::self.n_rep]
    if decode:
        out, lse = kv_cache.decode_step(self.layer_id, xq, xk, xv, batch_idx, input_pos)
    else:
        kv_cache.insert_kv(self.layer_id, xk, xv, input_pos=input_pos, batch_idx=batch_idx)
        out, lse = kv_cache.prefill_attention(self.layer_id, xq, batch_idx, input_pos, attention_masks)
    return self._post_attention(out, lse)


def install_attention(attention_cls, fused: bool = True):
    """Route ``attention_cls.forward`` (the reference's ``falcon_perception.model.Attention``)
    through this package whenever the cache it is given is an ``fpkv.PagedKVCache``;
    any other cache goes to the original method.  Returns the original method."""
    original = attention_cls.forward

    def forward(self, x, attention_masks, kv_cache, freqs_cis, freqs_cis_2d=None, input_pos=None, batch_idx=None,
                flex_attn_kernel_options=None):
        if isinstance(kv_cache, PagedKVCache):
            return fpkv_attention_forward(self, x, attention_masks, kv_cache, freqs_cis, freqs_cis_2d, input_pos,
                                          batch_idx, flex_attn_kernel_options, fused=fused)
        return original(self, x, attention_masks, kv_cache, freqs_cis, freqs_cis_2d, input_pos, batch_idx,
                        flex_attn_kernel_options)
    attention_cls.forward = forward
    return original


# ------------------------------------------------- decode step set-up, batched
def batched_decode_forward(self, sequences):
    """``PagedInferenceEngine._decode_forward`` (``paged_inference.py:954-1031``)
    with the graph's inputs filled by a handful of batched operations instead of
    four small device copies per request (rope position, last token and the two
    box values, ``:986-1003``) and three element-wise writes into pinned memory
    per request (``:970-975``).  Same buffers, same graph, same results; the
    eager path (no captured graph) is the reference's own."""
    if not self.cudagraph_captured:
        return self._fpkv_original_decode_forward(sequences)
    B = len(sequences)
    graph_bs = next(x for x in self._graph_bs if x >= B)
    graph = self._graphs[graph_bs]
    gv = self._graph_vars
    slots = [seq.batch_idx for seq in sequences]
    # host: slots and positions of the batch, written into the pinned staging buffers in one go each
    self._decode_gv_bidx_pinned.zero_()
    slots_t = torch.tensor(slots, dtype=torch.int64)
    self._decode_bidx_pinned[:B] = slots_t
    self._decode_gv_bidx_pinned[:B] = slots_t
    self._decode_pos_pinned[:B] = torch.tensor([seq.total_length - 1 for seq in sequences], dtype=torch.int32)
    # device: positions by slot, then rope positions, last tokens and box values of the whole batch at once
    self._decode_bidx_gpu[:B].copy_(self._decode_bidx_pinned[:B], non_blocking=True)
    self._decode_pos_gpu[:B].copy_(self._decode_pos_pinned[:B], non_blocking=True)
    self._input_pos.scatter_(0, self._decode_bidx_gpu[:B], self._decode_pos_gpu[:B])
    self._rope_pos_t.scatter_(0, self._decode_bidx_gpu[:B],
                              torch.stack([seq.pos_t for seq in sequences]).to(self._rope_pos_t.dtype))
    gv["input_ids"][:B].copy_(torch.stack([seq.last_token_id for seq in sequences]))
    gv["input_ids"][B:].zero_()
    gv["batch_idx"].copy_(self._decode_gv_bidx_pinned, non_blocking=True)
    gv["coord_xy"].zero_()
    gv["size_hw"].zero_()
    boxed = [i for i, seq in enumerate(sequences) if seq.current_bbox_xy is not None]
    if boxed:
        rows = slice(0, B) if len(boxed) == B else torch.tensor(boxed, device=gv["coord_xy"].device)
        gv["coord_xy"][rows] = torch.stack([sequences[i].current_bbox_xy for i in boxed]).to(gv["coord_xy"].dtype)
        gv["size_hw"][rows] = torch.stack([sequences[i].current_bbox_hw for i in boxed]).to(gv["size_hw"].dtype)
    graph.replay()
    return gv["logits_out"][:B], gv["h_out"][:B]


def install_decode_setup(engine_cls):
    """Replace ``engine_cls._decode_forward`` (the reference's
    ``PagedInferenceEngine``) by ``batched_decode_forward``.  Returns the
    original method."""
    original = engine_cls._decode_forward
    engine_cls._fpkv_original_decode_forward = original
    engine_cls._decode_forward = batched_decode_forward
    return original


def install_engine(engine_module, attention_cls, fused: bool = True, cache_factory=None):
    """Everything an engine built like the reference's needs to run on this
    package, in one call: ``engine_module.PagedKVCache`` (the name the engine
    constructs its cache through, ``paged_inference.py:27,321``) becomes
    ``cache_factory`` (default: ``fpkv.PagedKVCache`` with the arguments the
    engine passes), ``get_decoding_block_mask`` becomes ``decoding_block_mask``,
    ``Attention.forward`` goes through ``install_attention`` and the decode
    step's set-up through ``install_decode_setup``.  Returns a function that
    puts everything back."""
    engine_cls = engine_module.PagedInferenceEngine
    saved = (engine_module.PagedKVCache, engine_cls.get_decoding_block_mask, engine_cls._decode_forward, attention_cls.forward)
    engine_module.PagedKVCache = cache_factory or PagedKVCache
    engine_cls.get_decoding_block_mask = \
        lambda self, batch_idx, input_pos: decoding_block_mask(self.block_mask, batch_idx, input_pos)
    install_attention(attention_cls, fused=fused)
    install_decode_setup(engine_cls)

    def restore():
        engine_module.PagedKVCache, engine_cls.get_decoding_block_mask, engine_cls._decode_forward, attention_cls.forward = saved
    return restore


# ------------------------------------------------------- per-slot step state
class SlotState:
    """Position, rope position and last token of every slot, on the device.

    The reference keeps ``_input_pos`` / ``_rope_pos_t`` per slot on the device
    (``paged_inference.py:346-352``) but refreshes them, and the graph's token
    and slot buffers, with one small copy per sequence and step (``:966-1003``).
    Here the state advances on the device (``advance``, one batched update after
    sampling), so the only thing a decode step uploads is the list of slots in
    its batch, padded with slot 0 up to the graph bucket, through one pinned
    buffer and one copy.  Values of newly prefilled sequences ride in the same
    upload (``begin``)."""

    def __init__(self, max_batch_size: int, device):
        self.max_batch_size = max_batch_size
        self.device = torch.device(device)
        self.input_pos = torch.zeros(max_batch_size, dtype=torch.int32, device=device)
        self.rope_pos_t = torch.zeros(max_batch_size, dtype=torch.int64, device=device)
        self.last_token = torch.zeros(max_batch_size, dtype=torch.int64, device=device)
        # the step's batch: slots padded with 0; a fixed device address, so that a captured graph can read it
        self.batch_idx = torch.zeros(max_batch_size, dtype=torch.int64, device=device)
        # one upload row: [slots of the batch | slots being (re)started | their position, rope position, token]
        self._row = 5 * max_batch_size
        pin = self.device.type == "cuda"
        self._host = [torch.zeros(self._row, dtype=torch.int64, pin_memory=pin) for _ in range(2)]
        self._dev = torch.zeros(self._row, dtype=torch.int64, device=device)
        self._done = [None, None]
        self._turn = 0
        self._started = []                                  # (slot, position, rope position, last token)

    def begin(self, slot: int, input_pos: int, rope_pos_t: int, last_token: int):
        """A sequence enters decoding (after its prefill) or its slot is reset (all zeros): recorded on
        the host, uploaded with the next ``stage``."""
        assert 0 < slot < self.max_batch_size
        self._started.append((slot, input_pos, rope_pos_t, last_token))

    def stage(self, slots, bucket: int | None = None) -> int:
        """Upload the step's batch (one copy).  ``slots``: the slot of every sequence of the decode batch;
        ``bucket``: padded batch size (CUDA-graph bucket), rows beyond the batch are slot 0 as in the
        reference (``:970-990``).  Returns the padded batch size; ``batch_idx[:bucket]`` then holds it."""
        n = len(slots)
        bucket = n if bucket is None else bucket
        M = self.max_batch_size
        assert n <= bucket <= M and len(self._started) <= M
        t = self._turn
        self._turn ^= 1
        if self._done[t] is not None:
            self._done[t].synchronize()                     # the copy that last read this pinned buffer
        h = self._host[t].numpy()
        h[:bucket] = 0
        h[:n] = slots
        k = len(self._started)
        h[M:2 * M] = 0                                      # slot 0: a write to the reserved slot's entry, harmless
        for j, col in enumerate(zip(*self._started) if k else ()):
            h[(1 + j) * M:(1 + j) * M + k] = col
        self._started = []
        if self.device.type == "cuda":
            self._dev.copy_(self._host[t], non_blocking=True)
            if self._done[t] is None:
                self._done[t] = torch.cuda.Event()
            self._done[t].record(torch.cuda.current_stream(self.device))
        else:
            self._dev.copy_(self._host[t])
        d = self._dev
        self.batch_idx[:bucket].copy_(d[:bucket])
        if k:
            sl = d[M:M + k]
            self.input_pos.index_copy_(0, sl, d[2 * M:2 * M + k].to(torch.int32))
            self.rope_pos_t.index_copy_(0, sl, d[3 * M:3 * M + k])
            self.last_token.index_copy_(0, sl, d[4 * M:4 * M + k])
        return bucket

    def step_inputs(self, bucket: int):
        """Device tensors of the staged step (gathers by slot; capturable in a CUDA graph):
        batch_idx (bucket,), input_pos (bucket,) int32, rope_pos_t (bucket,) int64, input_ids (bucket,)."""
        bi = self.batch_idx[:bucket]
        return bi, self.input_pos[bi], self.rope_pos_t[bi], self.last_token[bi]

    def advance(self, bucket: int, next_token: Tensor):
        """After sampling: every live row of the batch moves on by one token.  Device work only, no
        host value involved; padding rows (slot 0) stay at zero."""
        bi = self.batch_idx[:bucket]
        live = bi > 0
        self.input_pos.index_add_(0, bi, live.to(torch.int32))
        self.rope_pos_t.index_add_(0, bi, live.to(torch.int64))
        self.last_token.index_copy_(0, bi, torch.where(live, next_token.reshape(-1)[:bucket], torch.zeros_like(bi)))


# ------------------------------------------------------------- step planning
@dataclass
class PrefillChunk:
    """Tokens [start, end) of a sequence enter the model in this step."""
    seq: object
    start: int
    end: int


@dataclass
class StepPlan:
    prefill: list = field(default_factory=list)             # PrefillChunk, in admission order
    decode: list = field(default_factory=list)              # sequences that decode one token
    admitted: list = field(default_factory=list)            # sequences that got a slot in this step
    preempted: list = field(default_factory=list)           # sequences sent back to the waiting queue

    @property
    def kind(self) -> str:
        return {(False, False): "idle", (True, False): "prefill", (False, True): "decode",
                (True, True): "mixed"}[(bool(self.prefill), bool(self.decode))]


class MixedStepPlanner:
    """Scheduling around the cache, with the reference's rules and one change.

    Same as the reference (``paged_inference.py:1148-1242``): a waiting
    sequence is admitted while a slot is free and ``can_reserve(total_length)``
    holds, and gets pages for its whole present length; a running sequence
    grows by ``reserve`` when its next token needs a page; when the pool is
    exhausted the most recently admitted running sequence is preempted (erased,
    back to the front of the waiting queue).  Different: admission does not
    stop the decoders.  A step carries the next chunk of every prompt that is
    being prefilled (at most ``chunk_tokens`` tokens each, ``prefill_token_budget``
    in total) AND one decode row per running sequence; the attention kernels
    serve both from the same pages.  A chunk never ends inside an image span
    (its tokens see each other in both directions, so they enter together): it
    is extended to the span's end, given by ``seq.image_spans`` (a list of
    (start, end) token ranges; absent = none).

    A sequence needs ``total_length`` and a writable ``batch_idx``; the planner
    keeps its own progress record per sequence."""

    def __init__(self, cache: PagedKVCache, chunk_tokens: int = 512, prefill_token_budget: int = 8192):
        self.cache = cache
        self.chunk_tokens = int(chunk_tokens)
        self.prefill_token_budget = int(prefill_token_budget)
        self.waiting: deque = deque()
        self.prefilling: list = []
        self.running: deque = deque()
        self._done_tokens: dict[int, int] = {}               # id(seq) -> tokens already through the model

    def add(self, seq):
        self.waiting.append(seq)

    def _chunk_end(self, seq, start: int, budget: int) -> int:
        end = min(seq.total_length, start + min(self.chunk_tokens, budget))
        for s0, s1 in getattr(seq, "image_spans", ()) or ():
            if s0 < end < s1:                               # the chunk would cut this span
                end = s1
        return min(end, seq.total_length)

    def plan(self) -> StepPlan:
        c = self.cache
        plan = StepPlan()
        # ---- decoders: grow, or preempt the newest when the pool is exhausted (:1206-1242) ----
        batch = []
        while self.running:
            seq = self.running.popleft()
            if c.capacity[seq.batch_idx] >= seq.total_length:
                batch.append(seq)
            elif c.can_reserve(seq.total_length, batch_idx_int=seq.batch_idx):
                c.reserve(seq.batch_idx, None, seq.total_length)
                batch.append(seq)
            else:
                self.running.appendleft(seq)
                newest = self.running.pop()
                self.waiting.appendleft(newest)
                c.erase(newest.batch_idx)
                self._done_tokens.pop(id(newest), None)
                plan.preempted.append(newest)
        self.running = deque(batch)
        plan.decode = list(batch)
        # ---- admission (:1162-1204), without waiting for the decoders to pause ----
        while self.waiting and len(c.free_batch_idx) > 0:
            seq = self.waiting[0]
            if not c.can_reserve(seq.total_length):
                break
            self.waiting.popleft()
            seq.batch_idx = c.allocate()
            c.reserve(seq.batch_idx, None, seq.total_length)
            self._done_tokens[id(seq)] = 0
            self.prefilling.append(seq)
            plan.admitted.append(seq)
        # ---- the next chunk of every prompt in flight, oldest first, within the token budget ----
        budget = self.prefill_token_budget
        for seq in self.prefilling:
            if budget <= 0:
                break
            start = self._done_tokens[id(seq)]
            end = self._chunk_end(seq, start, budget)
            plan.prefill.append(PrefillChunk(seq, start, end))
            budget -= end - start
        return plan

    def commit(self, plan: StepPlan):
        """The step ran: chunks are through the model, finished prompts join the decoders."""
        for ch in plan.prefill:
            self._done_tokens[id(ch.seq)] = ch.end
        still = []
        for seq in self.prefilling:
            if self._done_tokens[id(seq)] >= seq.total_length:
                self._done_tokens.pop(id(seq))
                self.running.append(seq)
            else:
                still.append(seq)
        self.prefilling = still

    def finish(self, seq):
        """A running sequence is complete: its slot and pages go back (:1099-1121)."""
        self.running.remove(seq)
        self.cache.erase(seq.batch_idx)


def pack_prefill_rows(chunks, token_ids, pad_id: int = 0, align: int = 128, device=None):
    """One packed row for a step's prefill chunks, laid out as the reference packs a prefill
    (``paged_inference.py:634-678``): every chunk starts on a multiple of ``align`` rows, the gap holds pad
    tokens that carry slot 0 and position 0, positions are the tokens' positions in their sequence (a
    chunk of a longer prompt starts at its ``start``).  ``token_ids(seq)`` gives a sequence's token ids
    (1-D tensor or list).  Returns input_ids, input_pos, batch_idx as (1, L) int64 tensors, the packed
    offset of every chunk, and the packed index of the last token of every chunk that ends its prompt."""
    ids, pos, bidx, offsets, last = [], [], [], [], {}
    off = 0
    for ch in chunks:
        n = ch.end - ch.start
        gap = (-n) % align
        t = torch.as_tensor(token_ids(ch.seq), dtype=torch.int64)[ch.start:ch.end]
        ids.append(F.pad(t, (0, gap), value=pad_id))
        pos.append(F.pad(torch.arange(ch.start, ch.end, dtype=torch.int64), (0, gap), value=0))
        bidx.append(F.pad(torch.full((n,), ch.seq.batch_idx, dtype=torch.int64), (0, gap), value=0))
        offsets.append(off)
        if ch.end >= ch.seq.total_length:
            last[id(ch.seq)] = off + n - 1
        off += n + gap
    cat = lambda xs: torch.cat(xs).unsqueeze(0) if xs else torch.zeros((1, 0), dtype=torch.int64)
    out = [cat(ids), cat(pos), cat(bidx)]
    if device is not None:
        out = [x.pin_memory().to(device, non_blocking=True) if torch.device(device).type == "cuda" else x for x in out]
    return out[0], out[1], out[2], offsets, last


def chunk_prefill_mask(cache: PagedKVCache, chunks, batch_idx: Tensor, input_ids: Tensor, image_spans_of, soi_id: int,
                       eoi_id: int) -> PrefillMask:
    """The prefill mask of a packed row of chunks.  For whole prompts this is
    ``cache.create_prefill_blockmask`` (``paged_attention.py:343-362``).  A chunk that starts inside
    a prompt cannot be told apart from a fresh prompt by its token ids alone only when an image span were
    cut, which the planner never does; so the mask is built from the ids as for whole prompts."""
    del chunks, image_spans_of
    return cache.create_prefill_blockmask(batch_idx, input_ids, soi_id, eoi_id)
