"""CPU: the C-ABI library loads, exports what include/fpkv.h declares, and
validates arguments on the host before touching a device."""

import ctypes
import os
import re

import torch

from fpkv import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fpkv.h")).read()
    return sorted(set(re.findall(r"FPKV_API\s+[\w\s\*]+?\b(fpkv_\w+)\s*\(", text)))


def test_header_symbols_are_exported():
    names = declared_symbols()
    assert len(names) >= 7
    assert sorted(_lib.EXPORTS) == names, "the ctypes binding must cover exactly the header's entry points"
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert getattr(raw, n) is not None


def test_library_matches_the_sources():
    """The loaded binary carries the hash of the sources it was compiled from; the loader refuses another."""
    from fpkv._srchash import source_hash
    assert _lib.build_id() == source_hash() and len(_lib.build_id()) == 16


def test_alloc_step_validation():
    L = _lib.lib
    p, buf = _pool()
    ptr = buf.data_ptr()
    st = _lib.FpkvAllocState(ptr, ptr, ptr)
    assert L.fpkv_alloc_step(None, ctypes.byref(st), ptr, 1, None, None) == -1
    assert L.fpkv_alloc_step(ctypes.byref(p), None, ptr, 1, None, None) == -1
    assert L.fpkv_alloc_step(ctypes.byref(p), ctypes.byref(_lib.FpkvAllocState(0, ptr, ptr)), ptr, 1, None, None) == -1
    assert L.fpkv_alloc_step(ctypes.byref(p), ctypes.byref(st), ptr, -1, None, None) == -1
    assert L.fpkv_alloc_step(ctypes.byref(p), ctypes.byref(st), 0, 1, None, None) == -1
    assert L.fpkv_alloc_step(ctypes.byref(p), ctypes.byref(st), ptr + 4, 1, None, None) == -3
    assert L.fpkv_alloc_step(ctypes.byref(p), ctypes.byref(st), ptr, 0, None, None) == 0      # nothing queued
    if not torch.cuda.is_available():
        assert L.fpkv_alloc_step(ctypes.byref(p), ctypes.byref(st), ptr, 1, None, None) == -4


def test_version_and_strerror():
    assert _lib.lib.fpkv_version() >= 100
    assert _lib.strerror(0) == "ok"
    for code in range(-7, 0):
        assert "unknown" not in _lib.strerror(code)
    assert "unknown" in _lib.strerror(-99)


def _pool(**kw):
    buf = torch.zeros(64, dtype=torch.int64)       # any 16-byte aligned host memory: never dereferenced
    d = dict(data=buf.data_ptr(), page_table=buf.data_ptr(), physical_to_logical=buf.data_ptr(), num_layers=1,
             n_heads=2, n_pages=4, page_size=16, head_dim=64, max_batch_size=3, dtype=_lib.FPKV_BF16, split_q_heads=0)
    d.update(kw)
    return _lib.FpkvPool(**d), buf


def test_validation_happens_before_any_launch():
    L = _lib.lib
    p, buf = _pool()
    ptr = buf.data_ptr()
    call = lambda pool, **kw: L.fpkv_append_decode(ctypes.byref(pool), kw.get("layer", 0), kw.get("bi", ptr), ptr,
                                                   kw.get("pt", 0), kw.get("k", ptr), kw.get("sb", 128), 64, ptr,
                                                   128, 64, kw.get("B", 2), None, None)
    assert L.fpkv_append_decode(None, 0, ptr, ptr, 0, ptr, 128, 64, ptr, 128, 64, 2, None, None) == -1
    assert call(_pool(data=0)[0]) == -1                      # null pool data
    assert call(_pool(dtype=9)[0]) == -7                     # bad dtype
    assert call(_pool(head_dim=96)[0]) == -2                 # unsupported head_dim
    assert call(_pool(page_size=24)[0]) == -2                # page_size not a multiple of 16
    assert call(p, layer=1) == -1                            # layer out of range
    assert call(p, B=-1) == -1
    assert call(p, pt=5) == -1                               # bad position type
    assert call(p, bi=0) == -1                               # null batch_idx
    assert call(p, k=ptr + 2) == -3                          # misaligned rows
    assert call(p, sb=100) == -3                             # stride not a multiple of 16 bytes
    assert call(p, B=0) == 0                                 # empty batch is a no-op
    need = ctypes.c_size_t(0)
    assert L.fpkv_decode_workspace_bytes(ctypes.byref(p), 4, 3, 0, ctypes.byref(need)) == -2   # 3 % 2 heads
    assert L.fpkv_decode_workspace_bytes(ctypes.byref(p), 4, 4, 0, ctypes.byref(need)) == 0 and need.value > 0
    # the portable kernel's need follows the batch (its split count shrinks as the batch grows), it is not a fixed maximum
    small, big = ctypes.c_size_t(0), ctypes.c_size_t(0)
    assert L.fpkv_decode_workspace_bytes(ctypes.byref(p), 4, 4, _lib.DECODE_PORTABLE, ctypes.byref(small)) == 0
    assert L.fpkv_decode_workspace_bytes(ctypes.byref(p), 1024, 4, _lib.DECODE_PORTABLE, ctypes.byref(big)) == 0
    assert big.value < 1024 // 4 * small.value
    assert L.fpkv_decode_workspace_bytes(ctypes.byref(p), 4, 4, _lib.DECODE_TMA, ctypes.byref(need)) == -2   # page 16
    # decode: workspace too small is caught on the host
    assert L.fpkv_decode_attn(ctypes.byref(p), 0, ptr, ptr, ptr, 256, 64, ptr, ptr, 0, 2, 4, 0.125, ptr, 16, 0,
                              None, None, None) == -6
    if not torch.cuda.is_available():
        # valid arguments but no device: refused, never a silent CPU path
        assert call(p) == -4


def test_pre_append_validation():
    """fpkv_pre_append checks head counts, layout, strides and alignment on the host."""
    L = _lib.lib
    p, buf = _pool(n_heads=2, head_dim=64)                    # pool of 2 stored heads
    ptr = buf.data_ptr()
    width = (4 + 2 * 2) * 64                                  # 4 query heads, 2 KV heads

    def call(pool=p, hq=4, hkv=2, stride=width, n_tok=3, qkv=ptr, fc=ptr, fc2=None, q_out=ptr, qs=(64, 256),
             eps=1e-6, pt=0, bi=ptr):
        return L.fpkv_pre_append(ctypes.byref(pool), 0, qkv, stride, hq, hkv, fc, fc2, bi, ptr, pt, n_tok, 1,
                                 q_out, qs[0], qs[1], eps, None, None)
    assert call(hq=3, hkv=2) == -2                            # query heads not a multiple of KV heads
    assert call(hq=8, hkv=4, stride=(8 + 8) * 64) == -2       # pool holds neither 8 nor 4 heads
    assert call(stride=width - 64) == -2                      # row shorter than (Hq + 2 Hkv) * D
    assert call(pool=_pool(n_heads=2, head_dim=32)[0]) == -2  # head_dim outside {64, 128}
    assert call(n_tok=-1) == -1 and call(pt=7) == -1 and call(eps=-1.0) == -1
    assert call(qkv=0) == -1 and call(fc=0) == -1 and call(q_out=0) == -1 and call(bi=0) == -1
    assert call(qkv=ptr + 2) == -3 and call(stride=width + 3) == -3 and call(qs=(64, 250)) == -3
    assert call(fc=ptr + 4) == -3 and call(fc2=ptr + 4) == -3   # rotary tables are read as 8-byte pairs
    assert call(n_tok=0) == 0                                 # nothing to do
    if not torch.cuda.is_available():
        assert call() == -4                                   # valid arguments, no device: refused
