"""Paged KV cache and paged attention on B200, behind the reference's API.

``PagedKVCache`` keeps the constructor, attributes and methods of the
reference class (``falcon_perception/paged_attention.py:27-393``): page pool,
per-slot page table and its inverse, host mirrors, LIFO free lists,
``allocate / reserve / can_reserve / erase``, ``insert_kv`` with its decode
and packed-prefill forms, and the mask builders.  The bookkeeping is host
Python exactly as there; every byte of K/V moves through the CUDA kernels in
libfpkv.so (append, gather, paged attention).  There is no PyTorch or CPU
fallback for those: a CPU cache can be built (to exercise the allocator), but
its data-path methods raise.

Differences a caller has to know about:
  * ``n_heads`` is the number of heads STORED.  Pass the model's KV heads and
    skip the reference's ``repeat_kv`` expansion (``model.py:114-115``);
    attention maps query head hq to stored head hq // (Hq // n_heads).
  * the mask builders return light records (``fpkv.attention``) instead of
    FlexAttention ``BlockMask`` objects;
  * attention is ``paged_attention(...)`` below instead of a ``flex_attention``
    call on the whole pool.
"""

from __future__ import annotations

import ctypes
import math

import torch
from torch import Tensor

from . import _lib
from .attention import CausalDecodeMask, DecodeStepMask, PrefillMask, image_span_ids
from .kv_cache import KVCacheBase

_DTYPES = {torch.float32: _lib.FPKV_F32, torch.bfloat16: _lib.FPKV_BF16, torch.float16: _lib.FPKV_F16}


def _cdiv(a: int, b: int) -> int:
    return int((a + b - 1) // b)


def _pos_type(t: Tensor) -> int:
    if t.dtype == torch.int32:
        return _lib.FPKV_I32
    if t.dtype == torch.int64:
        return _lib.FPKV_I64
    raise AssertionError("input_pos must be int32 or int64")


def _epilogue(sinks: Tensor | None, token_major: bool = False):
    """fpkv_epilogue for a call, or None: the sink gate of the reference's
    ``_post_attention`` (``model.py:122-128``) and the token-major prefill layout."""
    if sinks is None and not token_major:
        return None
    if sinks is not None:
        assert sinks.is_cuda and sinks.is_contiguous() and sinks.dtype in _DTYPES
    return _lib.FpkvEpilogue(sinks.data_ptr() if sinks is not None else None,
                             _DTYPES[sinks.dtype] if sinks is not None else 0, int(token_major))


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class PagedKVCache(KVCacheBase):
    """Page pool + page table + free lists; see the module docstring."""

    def __init__(self, n_pages: int, page_size: int, max_batch_size: int, n_heads: int, head_dim: int,
                 num_layers: int, dtype: torch.dtype, device: str | torch.device = "cuda",
                 split_q_heads: int | None = None):
        """``split_q_heads`` (the model's query head count, with ``n_heads`` the KV
        heads) selects the split layout: the first half of every key head (1-D
        rotary embedding, the same for all query heads of a group) and V are
        stored once per KV head, the second half of K (per-query-head 2-D rotary
        embedding, ``falcon_perception/rope.py:59-104``) once per query head.  That
        is exactly the content of the reference's expanded cache in
        (3*n_heads + split_q_heads)/(4*split_q_heads) of its bytes (5/8 at two
        query heads per KV head).  ``insert_kv`` then takes the reference's
        expanded K and V (``split_q_heads`` heads), ``pre_attention_append`` writes
        the layout directly, attention is called with ``split_q_heads`` query heads.
        ``kv_cache`` is then a (num_layers, elements) tensor; ``k_first``, ``k_second``
        and ``v_plane`` give views of a layer's three regions."""
        assert dtype in _DTYPES, "dtype must be float32, bfloat16 or float16"
        self.split_q_heads = int(split_q_heads) if split_q_heads else 0
        if self.split_q_heads:
            assert self.split_q_heads % n_heads == 0 and self.split_q_heads > n_heads, \
                "split_q_heads must be a multiple of n_heads (the KV heads) and larger"
        self.n_pages = n_pages
        self.page_size = page_size
        self.max_batch_size = max_batch_size
        self.n_heads = n_heads
        self.head_dim = head_dim
        self.num_layers = num_layers
        self.dtype = dtype
        self.device = device
        self._dev = torch.device(device)

        # [slot, logical page] -> physical page; page 0 and slot 0 are reserved (no-op targets)
        self._page_table = torch.full((max_batch_size, n_pages), -1, dtype=torch.int64, device=device)
        self._page_table[0, :] = 0
        self.page_table_cpu = [[] for _ in range(max_batch_size)]
        self.capacity = [0 for _ in range(max_batch_size)]
        self._free_pages = list(reversed(range(1, n_pages)))
        self._free_batch_idx = list(reversed(range(1, max_batch_size)))
        # [slot, physical page] -> logical page
        self._physical_to_logical = torch.full((max_batch_size, n_pages), -1, dtype=torch.int64, device=device)

        if self.split_q_heads:
            rows = n_pages * page_size
            self.kv_shape = (num_layers, rows * (3 * n_heads + self.split_q_heads) * (head_dim // 2))
        else:
            self.kv_shape = (num_layers, 2, 1, n_heads, n_pages * page_size, head_dim)
        self.kv_cache = torch.zeros(self.kv_shape, dtype=dtype, device=device)

        self._pool = _lib.FpkvPool(self.kv_cache.data_ptr(), self._page_table.data_ptr(),
                                   self._physical_to_logical.data_ptr(), num_layers, n_heads, n_pages,
                                   page_size, head_dim, max_batch_size, _DTYPES[dtype], self.split_q_heads)
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        self._workspace = None
        self.decode_kernel = _lib.DECODE_AUTO       # DECODE_PORTABLE / DECODE_TMA force one kernel
        self.prefill_kernel = _lib.PREFILL_AUTO     # PREFILL_PORTABLE / PREFILL_TC force one kernel

        # On a CUDA cache the free lists also live on the device (stacks in list order) and allocate /
        # reserve / erase queue one record each; one kernel launch applies the queue, in order, before the
        # tables are next used (by a kernel of this class or through the attributes).  The lists above stay
        # the host's mirror: can_reserve and the error of an over-reserve need them without a device read.
        self._pending = []
        if self._dev.type == "cuda":
            self._free_pages_dev = torch.zeros(n_pages, dtype=torch.int32, device=device)
            self._free_slots_dev = torch.zeros(max_batch_size, dtype=torch.int32, device=device)
            self._alloc_counts = torch.zeros(2, dtype=torch.int32, device=device)
            self._alloc = _lib.FpkvAllocState(self._free_pages_dev.data_ptr(), self._free_slots_dev.data_ptr(),
                                              self._alloc_counts.data_ptr())
            # two pinned staging buffers, used in turn, so that a flush allocates nothing and never rewrites
            # host memory that an earlier, still running copy reads
            self._ops_cap = 1024
            self._ops_host = [torch.empty((self._ops_cap, 4), dtype=torch.int32).pin_memory() for _ in range(2)]
            self._ops_done = [None, None]
            self._ops_dev = torch.empty((self._ops_cap, 4), dtype=torch.int32, device=device)
            self._ops_turn = 0
            self._upload_lists()

    # ------------------------------------------------------- split-layout views
    def _split_regions(self, layer_id: int):
        assert self.split_q_heads, "the pool does not use the split layout"
        rows, half = self.n_pages * self.page_size, self.head_dim // 2
        flat = self.kv_cache[layer_id]
        a, b = self.n_heads * rows * half, (self.n_heads + self.split_q_heads) * rows * half
        return (flat[:a].view(self.n_heads, rows, half), flat[a:b].view(self.split_q_heads, rows, half),
                flat[b:].view(self.n_heads, rows, self.head_dim))

    def k_first(self, layer_id: int) -> Tensor:
        """(n_heads, n_pages*page_size, head_dim/2): first half of K, one per KV head."""
        return self._split_regions(layer_id)[0]

    def k_second(self, layer_id: int) -> Tensor:
        """(split_q_heads, n_pages*page_size, head_dim/2): second half of K, one per query head."""
        return self._split_regions(layer_id)[1]

    def v_plane(self, layer_id: int) -> Tensor:
        """(n_heads, n_pages*page_size, head_dim): V, one per KV head."""
        return self._split_regions(layer_id)[2]

    # ------------------------------------------------------------------ tables
    @property
    def page_table(self) -> Tensor:
        """int64 (max_batch_size, n_pages): [slot, logical page] -> physical page."""
        self._flush_tables()
        return self._page_table

    @property
    def physical_to_logical(self) -> Tensor:
        """int64 (max_batch_size, n_pages): [slot, physical page] -> logical page."""
        self._flush_tables()
        return self._physical_to_logical

    @property
    def free_pages(self) -> list:
        """Free physical pages, a LIFO list as in the reference (``free_pages[-n:]`` are taken next).
        Assign a new list to reorder it (tests shuffle it); do not edit the returned list in place, the
        device copy would not follow."""
        return self._free_pages

    @free_pages.setter
    def free_pages(self, pages):
        self._flush_tables()                        # records queued so far were made against the old order
        self._free_pages = list(pages)
        self._upload_lists()

    @property
    def free_batch_idx(self) -> list:
        """Free slots, a LIFO list as in the reference; assign to reorder, do not edit in place."""
        return self._free_batch_idx

    @free_batch_idx.setter
    def free_batch_idx(self, slots):
        self._flush_tables()
        self._free_batch_idx = list(slots)
        self._upload_lists()

    def flush_tables(self):
        """Apply the queued allocator calls now (one copy from a preallocated pinned buffer, one kernel
        launch; nothing is allocated).  Every data-path method and the table attributes do this on their
        own; call it yourself before a region that must not touch the tables (CUDA-graph capture,
        ``decode_attention_noalloc``)."""
        self._flush_tables()

    def _upload_lists(self):
        """The host lists copied whole to the device stacks: at start-up and after the lists were
        reordered by hand (nothing is queued at either time)."""
        if self._dev.type != "cuda":
            return
        assert not self._pending
        fp = torch.tensor(self._free_pages, dtype=torch.int32)
        fs = torch.tensor(self._free_batch_idx, dtype=torch.int32)
        assert fp.numel() <= self.n_pages and fs.numel() <= self.max_batch_size, "a free list is longer than the pool"
        self._free_pages_dev[:fp.numel()].copy_(fp)
        self._free_slots_dev[:fs.numel()].copy_(fs)
        self._alloc_counts.copy_(torch.tensor([fp.numel(), fs.numel()], dtype=torch.int32))

    def _flush_tables(self):
        if self._dev.type != "cuda":
            return
        n = len(self._pending)
        if n == 0:
            return
        if n > self._ops_cap:                       # a step with more calls than ever before: grow (allocates)
            torch.cuda.current_stream(self._dev).synchronize()
            self._ops_cap = max(n, 2 * self._ops_cap)
            self._ops_host = [torch.empty((self._ops_cap, 4), dtype=torch.int32).pin_memory() for _ in range(2)]
            self._ops_done = [None, None]
            self._ops_dev = torch.empty((self._ops_cap, 4), dtype=torch.int32, device=self._dev)
        t = self._ops_turn
        self._ops_turn ^= 1
        if self._ops_done[t] is not None:
            self._ops_done[t].synchronize()         # the copy that last read this buffer (two flushes ago)
        host = self._ops_host[t]
        host.numpy()[:n] = self._pending
        self._pending = []
        self._ops_dev[:n].copy_(host[:n], non_blocking=True)
        if self._ops_done[t] is None:
            self._ops_done[t] = torch.cuda.Event()
        self._ops_done[t].record(torch.cuda.current_stream(self._dev))
        _lib.check(_lib.lib.fpkv_alloc_step(ctypes.byref(self._pool), ctypes.byref(self._alloc),
                                            self._ops_dev.data_ptr(), n, self._status_ptr(), _stream(self._dev)),
                   "fpkv_alloc_step")

    # ------------------------------------------------------------------ helpers
    def _require_cuda(self, *tensors, flush: bool = True):
        if self._dev.type != "cuda":
            raise RuntimeError("fpkv moves K/V only with its CUDA kernels; this cache lives on "
                               f"{self._dev} and has no CPU path")
        for t in tensors:
            assert t.is_cuda, "tensor must be on the cache's CUDA device"
        if flush:
            self._flush_tables()

    def _status_ptr(self):
        return self._status.data_ptr()

    def check_status(self) -> int:
        """Read and clear the device status word (one synchronising copy).
        Raises if a kernel met an out-of-range index or a bounded wait ran out."""
        bits = int(self._status.item())
        if bits:
            self._status.zero_()
            names = [n for b, n in ((1, "bad slot"), (2, "bad position"), (4, "bad page id"),
                                    (8, "on-chip wait timed out"),
                                    (16, "image span not closed inside its sequence (cut at the sequence's end)"))
                     if bits & b]
            raise RuntimeError("fpkv kernel status: " + ", ".join(names))
        return bits

    # ---------------------------------------------------------------- insert_kv
    def insert_kv(self, layer_id: int, k: Tensor, v: Tensor, input_pos: Tensor | None = None,
                  batch_idx: Tensor | None = None, **kwargs):
        del kwargs
        assert input_pos is not None, "input_pos is required for paged kv cache"
        assert batch_idx is not None, "batch_idx is required for paged kv cache"
        assert batch_idx.ndim in [1, 2], "batch_idx must be 1D (decode) or 2D (prefill 1xL)"
        if batch_idx.ndim == 1:
            return self.assign(layer_id, batch_idx, input_pos, k, v)
        return self.assign_prefill_no_paging(layer_id, k, v, input_pos, batch_idx)

    # ---------------------------------------------------------------- allocator
    def can_reserve(self, size: int, batch_idx_int: int | None = None) -> bool:
        """Host-only check: room for a new request, or for growing an existing one."""
        if batch_idx_int is None:
            return self.num_free_pages * self.page_size >= size and len(self._free_batch_idx) > 0
        return self.reserve(batch_idx_int, None, size, dry_run=True)

    def allocate(self) -> int:
        slot = self._free_batch_idx.pop()
        self.capacity[slot] = 0
        if self._dev.type == "cuda":
            # a free slot's rows are all -1 already (the constructor and erase leave them so)
            self._pending.append((_lib.OP_ALLOCATE, slot, 0, 0))
        else:
            self._physical_to_logical[slot, :] = -1
            self._page_table[slot, :] = -1
        return slot

    @property
    def num_free_pages(self) -> int:
        return len(self._free_pages)

    def reserve(self, batch_idx_int: int, batch_idx: Tensor | None, seq_len: int, dry_run: bool = False) -> bool:
        """Grow slot ``batch_idx_int`` to hold at least ``seq_len`` tokens.
        ``batch_idx`` (the slot as a one-element tensor) is accepted for
        signature compatibility and not needed."""
        if seq_len <= self.capacity[batch_idx_int]:
            return True
        n_new = _cdiv(seq_len - self.capacity[batch_idx_int], self.page_size)
        can = bool(n_new <= self.num_free_pages)
        if dry_run:
            return can
        if not can:
            raise RuntimeError(
                f"Cannot reserve {n_new} pages for a sequence of length {seq_len} "
                f"in batch {batch_idx_int}. Only {self.num_free_pages} pages available. "
                f"Current capacity is {self.capacity[batch_idx_int]} tokens.")
        start = self.capacity[batch_idx_int] // self.page_size
        pages = self._free_pages[-n_new:]
        if self._dev.type == "cuda":
            self._pending.append((_lib.OP_RESERVE, batch_idx_int, start, n_new))
        else:
            for i, pg in enumerate(pages):
                self._page_table[batch_idx_int, start + i] = pg
                self._physical_to_logical[batch_idx_int, pg] = start + i
        self.page_table_cpu[batch_idx_int] += pages
        del self._free_pages[-n_new:]
        self.capacity[batch_idx_int] += n_new * self.page_size
        return True

    def erase(self, batch_idx: int) -> None:
        self._free_batch_idx.append(batch_idx)
        owned = self.page_table_cpu[batch_idx]
        self._free_pages.extend(reversed(owned))
        # cleared on the device too, so padding rows and stale slots read "unmapped"
        if self._dev.type == "cuda":
            self._pending.append((_lib.OP_ERASE, batch_idx, len(owned), 0))
        else:
            self._page_table[batch_idx, :] = -1
            self._physical_to_logical[batch_idx, :] = -1
        self.page_table_cpu[batch_idx] = []
        self.capacity[batch_idx] = 0

    # ------------------------------------------------------------------- append
    def assign(self, layer_id: int, batch_idx: Tensor, input_pos: Tensor, k_val: Tensor, v_val: Tensor):
        """Decode append of (B,H,1,D) rows; returns this layer's K and V pool views."""
        B, H, S, K_D = k_val.shape
        H_cache, MAX_S, D_cache = self.split_q_heads or self.n_heads, self.n_pages * self.page_size, self.head_dim
        assert H_cache == H, "number of heads must match"
        assert MAX_S >= S, "cache must have enough space"
        assert D_cache == K_D, "hidden dim must match"
        assert v_val.shape == k_val.shape, "k and v must have the same shape"
        assert S == 1, "decode append takes one token per row"
        assert input_pos.shape == (B, S), "input_pos must have the same shape as val"
        assert batch_idx.shape == (B,), "batch_idx must have one dimension only"
        assert k_val.dtype == self.dtype and v_val.dtype == self.dtype, "dtype must match the pool"
        self._require_cuda(k_val, v_val, batch_idx, input_pos)
        if batch_idx.dtype != torch.int64:
            batch_idx = batch_idx.to(torch.int64)
        k_val, v_val = self._rows16(k_val), self._rows16(v_val)
        input_pos = input_pos.reshape(-1)
        if not input_pos.is_contiguous():
            input_pos = input_pos.contiguous()
        _lib.check(_lib.lib.fpkv_append_decode(
            ctypes.byref(self._pool), layer_id, batch_idx.data_ptr(), input_pos.data_ptr(), _pos_type(input_pos),
            k_val.data_ptr(), k_val.stride(0), k_val.stride(1), v_val.data_ptr(), v_val.stride(0), v_val.stride(1),
            B, self._status_ptr(), _stream(self._dev)), "fpkv_append_decode")
        if self.split_q_heads:
            return None, None                       # no (1, H, rows, D) views exist of the split regions; attention reads the pool
        return self.kv_cache[layer_id, 0], self.kv_cache[layer_id, 1]

    def assign_prefill_no_paging(self, layer_id: int, k_val: Tensor, v_val: Tensor, input_pos: Tensor,
                                 batch_idx: Tensor):
        """Packed prefill append of (1,H,L,D) rows with per-token (1,L) slot and
        position; returns the fresh k, v (prefill attends over them)."""
        assert batch_idx.ndim == 2, "batch_idx must be a 2D tensor"
        assert batch_idx.shape[0] == 1, "batch_idx must have batch size 1"
        assert input_pos.ndim == 2, "input_pos must be a 2D tensor"
        assert k_val.ndim == 4, "k_val must be a 4D tensor"
        assert v_val.ndim == 4, "v_val must be a 4D tensor"
        assert k_val.shape[0] == 1 and k_val.shape[1] == (self.split_q_heads or self.n_heads) and k_val.shape[3] == self.head_dim
        assert v_val.shape == k_val.shape and k_val.shape[2] == batch_idx.shape[1] == input_pos.shape[1]
        assert k_val.dtype == self.dtype and v_val.dtype == self.dtype, "dtype must match the pool"
        self._require_cuda(k_val, v_val, batch_idx, input_pos)
        if batch_idx.dtype != torch.int64:
            batch_idx = batch_idx.to(torch.int64)
        kk, vv = self._rows16(k_val), self._rows16(v_val)
        bi, ip = batch_idx.reshape(-1), input_pos.reshape(-1)
        bi = bi if bi.is_contiguous() else bi.contiguous()
        ip = ip if ip.is_contiguous() else ip.contiguous()
        _lib.check(_lib.lib.fpkv_append_packed(
            ctypes.byref(self._pool), layer_id, bi.data_ptr(), ip.data_ptr(), _pos_type(ip),
            kk.data_ptr(), kk.stride(1), kk.stride(2), vv.data_ptr(), vv.stride(1), vv.stride(2),
            kk.shape[2], self._status_ptr(), _stream(self._dev)), "fpkv_append_packed")
        return k_val, v_val

    def pre_attention_append(self, layer_id: int, qkv: Tensor, n_q_heads: int, n_kv_heads: int, freqs_cis: Tensor,
                             freqs_cis_2d: Tensor | None, batch_idx: Tensor, input_pos: Tensor,
                             eps: float | None = None) -> Tensor:
        """Norm, rotary embedding and K/V append in one kernel: everything
        ``Attention._pre_attention`` does behind the QKV projection
        (``falcon_perception/model.py:107-120``) plus the ``insert_kv`` that
        follows (``model.py:150-155``).  qkv (B,S,(Hq+2*Hkv)*D) is the projection
        output; freqs_cis (B,S,D/4) complex64 the 1-D rotary table indexed by
        position; freqs_cis_2d (B,S,Hq,D/4) complex64 or None; batch_idx /
        input_pos as ``insert_kv`` takes them ((B,) and (B,1) in a decode step,
        (1,L) each in a packed prefill).  Returns the normalised, rotated
        queries as a (B,Hq,S,D) view; K and V are in the pool.  The pool holds
        n_q_heads heads (the reference's expanded copies) or n_kv_heads heads
        (each key head once; exact when no 2-D table is in use or its
        frequencies agree within a GQA group)."""
        B, S, W = qkv.shape
        D = self.head_dim
        assert W == (n_q_heads + 2 * n_kv_heads) * D, "qkv width must be (Hq + 2*Hkv) * head_dim"
        if self.split_q_heads:
            assert (self.split_q_heads, self.n_heads) == (n_q_heads, n_kv_heads), "head counts must match the split pool"
        else:
            assert self.n_heads in (n_q_heads, n_kv_heads), "the pool must hold the query or the KV head count"
        assert qkv.dtype == self.dtype, "dtype must match the pool"
        assert freqs_cis.shape == (B, S, D // 4) and freqs_cis.dtype == torch.complex64
        if freqs_cis_2d is not None:
            assert freqs_cis_2d.shape == (B, S, n_q_heads, D // 4) and freqs_cis_2d.dtype == torch.complex64
        decode_mode = batch_idx.ndim == 1
        if decode_mode:
            assert S == 1 and batch_idx.shape == (B,), "a decode step appends one token per row"
        else:
            assert B == 1 and batch_idx.shape == (1, S), "a packed prefill is one row of (1, L) indices"
        self._require_cuda(qkv, batch_idx, input_pos, freqs_cis)
        T = B * S
        x = qkv.reshape(T, W)
        if x.stride(1) != 1 or x.data_ptr() % 16 or (x.stride(0) * x.element_size()) % 16:
            x = x.contiguous()
        bi = batch_idx.reshape(-1)
        bi = bi if bi.dtype == torch.int64 else bi.to(torch.int64)
        bi = bi if bi.is_contiguous() else bi.contiguous()
        ip = input_pos.reshape(-1)
        ip = ip if ip.is_contiguous() else ip.contiguous()
        assert bi.numel() == T and ip.numel() == T
        fc = torch.view_as_real(freqs_cis.reshape(T, D // 4)).contiguous()
        fc2 = torch.view_as_real(freqs_cis_2d.reshape(T, n_q_heads, D // 4)).contiguous() if freqs_cis_2d is not None else None
        q_out = torch.empty((B, S, n_q_heads, D), dtype=self.dtype, device=qkv.device)
        if eps is None:
            eps = torch.finfo(torch.float32).eps
        _lib.check(_lib.lib.fpkv_pre_append(
            ctypes.byref(self._pool), layer_id, x.data_ptr(), x.stride(0), n_q_heads, n_kv_heads, fc.data_ptr(),
            fc2.data_ptr() if fc2 is not None else None, bi.data_ptr(), ip.data_ptr(), _pos_type(ip), T,
            1 if decode_mode else 0, q_out.data_ptr(), D, n_q_heads * D, float(eps), self._status_ptr(),
            _stream(self._dev)), "fpkv_pre_append")
        return q_out.permute(0, 2, 1, 3)

    def _rows16(self, t: Tensor) -> Tensor:
        """The kernels read whole head_dim rows with 16-byte accesses through
        arbitrary outer strides (so the model's permuted views need no copy);
        only a row that is not contiguous or not 16-byte aligned is repacked."""
        es = t.element_size()
        ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all((s * es) % 16 == 0 for s in t.stride()[:-1])
        return t if ok else t.contiguous()

    # ------------------------------------------------------------------- gather
    def gather(self, layer_id: int, slot: int, n_tokens: int):
        """K and V of logical positions [0, n_tokens) of a slot as two
        (n_heads, n_tokens, head_dim) tensors read through the page table."""
        self._require_cuda()
        # split layout: K per query head (put together as the reference's expanded cache holds it), V per KV head
        k = torch.empty((self.split_q_heads or self.n_heads, n_tokens, self.head_dim), dtype=self.dtype, device=self._dev)
        v = torch.empty((self.n_heads, n_tokens, self.head_dim), dtype=self.dtype, device=self._dev)
        _lib.check(_lib.lib.fpkv_gather(ctypes.byref(self._pool), layer_id, slot, n_tokens, k.data_ptr(),
                                        v.data_ptr(), self._status_ptr(), _stream(self._dev)), "fpkv_gather")
        return k, v

    # --------------------------------------------------------- decode attention
    def _get_workspace(self, B: int, Hq: int) -> Tensor:
        need = ctypes.c_size_t(0)
        _lib.check(_lib.lib.fpkv_decode_workspace_bytes(ctypes.byref(self._pool), B, Hq, int(self.decode_kernel),
                                                        ctypes.byref(need)), "fpkv_decode_workspace_bytes")
        if self._workspace is None or self._workspace.numel() < need.value:
            # zero-filled once: the head of the workspace holds arrival counters the kernel leaves at zero
            self._workspace = torch.zeros(need.value, dtype=torch.uint8, device=self._dev)
        return self._workspace

    def decode_step(self, layer_id: int, q: Tensor, k: Tensor, v: Tensor, batch_idx: Tensor, input_pos: Tensor,
                    sm_scale: float | None = None, out: Tensor | None = None, lse: Tensor | None = None,
                    sinks: Tensor | None = None):
        """Append k, v (B,H,1,D) and attend with q (B,Hq,1,D) in one go: what
        ``Attention.forward`` does per layer in a decode step (``insert_kv``
        followed by the attention call, ``falcon_perception/model.py:150-162``).
        Same results as the two separate calls; because the attention kernel
        knows that the append is what runs right before it, its set-up overlaps
        the append instead of waiting for it.  With ``sinks`` (n_q_heads,) the
        returned out is already ``out * sigmoid(lse - sinks)``, the gate of
        ``_post_attention`` (``model.py:122-128``); viewed as (B, 1, Hq*D) it is
        what the output projection takes."""
        B = q.shape[0]
        self.assign(layer_id, batch_idx, input_pos.reshape(B, 1), k, v)
        return self.decode_attention(layer_id, q, batch_idx, input_pos, sm_scale, out, lse, sinks=sinks,
                                     _after_append=True)

    def decode_attention(self, layer_id: int, q: Tensor, batch_idx: Tensor, input_pos: Tensor,
                         sm_scale: float | None = None, out: Tensor | None = None, lse: Tensor | None = None,
                         sinks: Tensor | None = None, _after_append: bool = False):
        """One query token per row against keys 0..input_pos[b] of slot
        batch_idx[b].  q (B,Hq,1,D) -> out (B,Hq,1,D) in q's dtype, lse (B,Hq,1)
        fp32.  Call after ``insert_kv`` of the same step, as the model does."""
        B, Hq, S, D = q.shape
        assert S == 1, "decode attention takes one query token per row"
        assert D == self.head_dim and Hq % self.n_heads == 0, "head layout must match the pool"
        assert not self.split_q_heads or Hq == self.split_q_heads, "a split pool serves exactly split_q_heads query heads"
        assert q.dtype == self.dtype, "q dtype must match the pool"
        assert batch_idx.shape == (B,), "batch_idx must have one dimension only"
        input_pos = input_pos.reshape(-1)
        assert input_pos.shape == (B,), "input_pos must have one entry per row"
        self._require_cuda(q, batch_idx, input_pos)
        q_in, bi_in, ip_in = q, batch_idx, input_pos
        if batch_idx.dtype != torch.int64:
            batch_idx = batch_idx.to(torch.int64)
        if not input_pos.is_contiguous():
            input_pos = input_pos.contiguous()
        q = self._rows16(q)
        if q is not q_in or batch_idx is not bi_in or input_pos is not ip_in:
            _after_append = False                      # a conversion kernel now sits between append and attention
        if out is None:
            out = torch.empty((B, Hq, 1, D), dtype=q.dtype, device=q.device)
        if lse is None:
            lse = torch.empty((B, Hq, 1), dtype=torch.float32, device=q.device)
        ws = self._get_workspace(B, Hq)
        scale = (1.0 / math.sqrt(D)) if sm_scale is None else float(sm_scale)
        flags = int(self.decode_kernel) | (_lib.DECODE_AFTER_APPEND if _after_append else 0)
        epi = _epilogue(sinks)
        _lib.check(_lib.lib.fpkv_decode_attn(
            ctypes.byref(self._pool), layer_id, out.data_ptr(), lse.data_ptr(), q.data_ptr(), q.stride(0),
            q.stride(1), batch_idx.data_ptr(), input_pos.data_ptr(), _pos_type(input_pos), B, Hq, scale,
            ws.data_ptr(), ws.numel(), flags, ctypes.byref(epi) if epi is not None else None, self._status_ptr(),
            _stream(self._dev)),
            "fpkv_decode_attn")
        return out, lse

    def prefill_attention(self, layer_id: int, q: Tensor, batch_idx: Tensor, input_pos: Tensor, mask: PrefillMask,
                          sm_scale: float | None = None, sinks: Tensor | None = None, token_major: bool = False):
        """Attention of a packed prefill row (or of a chunk of one) against the
        pages: q (1,Hq,L,D), batch_idx / input_pos (1,L) as given to
        ``insert_kv``, ``mask`` from ``create_prefill_blockmask``.  Call it
        after ``insert_kv`` of the same tokens.  Returns out (1,Hq,L,D) in q's
        dtype and lse (1,Hq,L) fp32; pad rows give 0 / -inf.  ``sinks``
        (n_q_heads,) applies the gate of ``_post_attention`` to out;
        ``token_major`` returns out as (1,L,Hq,D), i.e. (1,L,Hq*D) for the
        output projection, without the reference's permute + copy."""
        _, Hq, L, D = q.shape
        assert q.shape[0] == 1 and D == self.head_dim and Hq % self.n_heads == 0 and q.dtype == self.dtype
        assert not self.split_q_heads or Hq == self.split_q_heads, "a split pool serves exactly split_q_heads query heads"
        assert batch_idx.shape[-1] == L and input_pos.shape[-1] == L and mask.L == L
        self._require_cuda(q, batch_idx, input_pos)
        bi = batch_idx.reshape(-1)
        if bi.dtype != torch.int64:
            bi = bi.to(torch.int64)
        bi = bi if bi.is_contiguous() else bi.contiguous()
        ext = mask.extent(input_pos, self._status)
        q = self._rows16(q)
        out = torch.empty((1, L, Hq, D) if token_major else (1, Hq, L, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((1, Hq, L), dtype=torch.float32, device=q.device)
        scale = (1.0 / math.sqrt(D)) if sm_scale is None else float(sm_scale)
        epi = _epilogue(sinks, token_major)
        _lib.check(_lib.lib.fpkv_prefill_attn(
            ctypes.byref(self._pool), layer_id, out.data_ptr(), lse.data_ptr(), q.data_ptr(), q.stride(1),
            q.stride(2), bi.data_ptr(), ext.data_ptr(), L, Hq, scale, int(self.prefill_kernel),
            ctypes.byref(epi) if epi is not None else None, self._status_ptr(), _stream(self._dev)),
            "fpkv_prefill_attn")
        return out, lse

    def decode_attention_noalloc(self, layer_id: int, q: Tensor, batch_idx: Tensor, input_pos: Tensor,
                                 out: Tensor, lse: Tensor, sm_scale: float | None = None):
        """``decode_attention`` for code that must not allocate on the device:
        an engine whose page pool already holds all free HBM, a decode loop
        that cannot take ``cudaMalloc``'s device-wide stall, a host whose
        memory manager forbids it.  Nothing is allocated here, by torch or by
        CUDA: the caller passes ``out`` (B,Hq,1,D) and ``lse`` (B,Hq,1) and
        already-typed index tensors (int64 ``batch_idx``, contiguous int32 or
        int64 ``input_pos``), and the kernel's scratch is a 4 MiB array built
        into the library and shared by every call on this GPU -- so calls that
        overlap on the GPU race, and head layouts that need more scratch
        (head_dim 128 with more than 4 query heads per stored head) are refused."""
        B, Hq, S, D = q.shape
        assert S == 1 and D == self.head_dim and Hq % self.n_heads == 0 and q.dtype == self.dtype
        assert batch_idx.dtype == torch.int64 and batch_idx.shape == (B,) and batch_idx.is_contiguous()
        input_pos = input_pos.view(-1)
        assert input_pos.shape == (B,) and input_pos.is_contiguous()
        assert tuple(out.shape) == (B, Hq, 1, D) and out.is_contiguous() and out.dtype == q.dtype
        assert tuple(lse.shape) == (B, Hq, 1) and lse.is_contiguous() and lse.dtype == torch.float32
        self._require_cuda(q, batch_idx, input_pos, out, lse, flush=False)
        assert not self._pending, "page-table edits are pending: call flush_tables() before the no-allocation region"
        scale = (1.0 / math.sqrt(D)) if sm_scale is None else float(sm_scale)
        _lib.check(_lib.lib.fpkv_decode_attn_static(
            ctypes.byref(self._pool), layer_id, out.data_ptr(), lse.data_ptr(), q.data_ptr(), q.stride(0),
            q.stride(1), batch_idx.data_ptr(), input_pos.data_ptr(), _pos_type(input_pos), B, Hq, scale,
            self._status_ptr(), _stream(self._dev)), "fpkv_decode_attn_static")
        return out, lse

    # ------------------------------------------------------------ mask builders
    def create_causal_blockmask(self, B: int, L: int) -> CausalDecodeMask:
        """Logical causal mask for decode steps with page_size blocks."""
        return CausalDecodeMask(B, L, self.page_size)

    def convert_logical_block_mask(self, block_mask, batch_idx: Tensor | None = None):
        """Logical -> physical conversion.  The kernels walk the page table
        themselves, so the step mask only has to carry slot and position; a
        mask whose column block differs from page_size is rejected as in the
        reference."""
        if isinstance(block_mask, CausalDecodeMask):
            raise RuntimeError("slice the causal mask for this step first: mask.for_step(batch_idx, input_pos)")
        if block_mask.page_size != self.page_size:
            raise RuntimeError(
                f"Expect block_mask has the same column block size as page_size"
                f"but got size={block_mask.page_size} and size={self.page_size}")
        if batch_idx is not None:
            assert batch_idx.ndim == 1, "batch_idx must be a 1D tensor"
            assert batch_idx.shape[0] == block_mask.batch_idx.shape[0], \
                "batch_idx must have the same shape as block_mask"
            assert batch_idx.shape[0] <= self.max_batch_size, \
                "batch_idx must be less than or equal to max_batch_size"
            return DecodeStepMask(batch_idx, block_mask.input_pos, self.page_size)
        return block_mask

    def get_logical_kv_idx(self, physical_batch_idx: Tensor, physical_kv_idx: Tensor, batch_idx: Tensor):
        """Physical token address -> (is_valid, logical position) for the slot
        of each row; index arithmetic only, on the tables' device."""
        slot = batch_idx[physical_batch_idx]
        page = physical_kv_idx // self.page_size
        logical_page = self.physical_to_logical[slot, page]
        logical = logical_page * self.page_size + physical_kv_idx % self.page_size
        return logical_page >= 0, logical.clamp(min=0)

    def get_mask_mod(self, mask_mod, batch_idx: Tensor):
        """Wrap a logical ``mask_mod(b, h, q_idx, kv_idx)`` so that it takes
        physical key addresses."""
        def new_mask_mod(b, h, q_idx, physical_kv_idx):
            ok, logical = self.get_logical_kv_idx(b, physical_kv_idx, batch_idx)
            inner = True if mask_mod is None else mask_mod(b, h, q_idx, logical)
            return ok & inner
        return new_mask_mod

    def create_prefill_blockmask(self, batch_idx: Tensor, input_ids: Tensor, soi_id: int, eoi_id: int,
                                 BLOCK_SIZE: int = 128) -> PrefillMask:
        """Document-causal OR same-image mask of a packed prefill row."""
        assert batch_idx.ndim == 2 and batch_idx.shape[0] == 1
        doc = batch_idx.reshape(-1).to(torch.int32)
        return PrefillMask(doc, image_span_ids(input_ids, soi_id, eoi_id), BLOCK_SIZE)


def paged_attention(q: Tensor, kv_cache: PagedKVCache, layer_id: int, batch_idx: Tensor, input_pos: Tensor,
                    mask=None, sm_scale: float | None = None):
    """Attention entry that replaces the reference's ``flex_fn(xq, xk, xv,
    block_mask=..., return_aux=AuxRequest(lse=True))`` call
    (``falcon_perception/model.py:156-162``).  Returns ``(out, lse)`` with out
    shaped and typed like q and lse (B,Hq,S) fp32.

    Decode: q (B,Hq,1,D), batch_idx (B,), input_pos (B,) or (B,1); ``mask`` may
    be the step's DecodeStepMask (its tensors are used when given).
    Prefill: q (1,Hq,L,D), batch_idx and input_pos (1,L), ``mask`` the
    PrefillMask of the packed row; keys are read from the pages, so call it
    after ``insert_kv``.
    """
    if batch_idx.ndim == 1:
        if isinstance(mask, DecodeStepMask):
            batch_idx, input_pos = mask.batch_idx, mask.input_pos
        return kv_cache.decode_attention(layer_id, q, batch_idx, input_pos, sm_scale)
    assert isinstance(mask, PrefillMask), "prefill needs the mask from create_prefill_blockmask"
    return kv_cache.prefill_attention(layer_id, q, batch_idx, input_pos, mask, sm_scale)
