"""GPU: the allocation-free decode entry point (scratch built into the library)
against the ordinary one.

Collected last on purpose (pytest orders files by name): if it fails, a run
that stops at the first failure has already run every other test.  It builds
its own cache and does not depend on what ran before it.
"""

import ctypes
import math

import pytest
import torch

from fpkv import _lib
import workloads as wl
from helpers import MAX_ABS, LSE_ABS, product_from_case

pytestmark = pytest.mark.gpu


def _call_static(c, q, bidx, pos, out, lse):
    """Straight through the C ABI: no Python-side helper in between."""
    B, Hq, _, D = q.shape
    rc = _lib.lib.fpkv_decode_attn_static(
        ctypes.byref(c._pool), 0, out.data_ptr(), lse.data_ptr(), q.data_ptr(), q.stride(0), q.stride(1),
        bidx.data_ptr(), pos.data_ptr(), _lib.FPKV_I32, B, Hq, 1.0 / math.sqrt(D), c._status.data_ptr(),
        torch.cuda.current_stream().cuda_stream)
    return rc


def test_static_scratch_entry_matches_workspace_entry_twice():
    # lengths chosen so that many (row, head) segments are cut by work-unit boundaries: the scratch
    # (partials, work counter) is really used, not just passed along
    case = wl.make_decode_case(31337, B=24, Hq=16, Hkv=8, D=128, P=128, n_pages=400, max_batch_size=26,
                               len_lo=100, len_hi=1900, dtype=torch.bfloat16)
    c, slots, bidx, pos, k, v, q = product_from_case(case)
    c.decode_kernel = _lib.DECODE_TMA
    B = case.B
    gen = torch.Generator().manual_seed(9)
    qs = [q, torch.randn(B, 16, 1, 128, generator=gen).bfloat16().cuda()]
    out = torch.empty((B, 16, 1, 128), dtype=torch.bfloat16, device="cuda")
    lse = torch.empty((B, 16, 1), dtype=torch.float32, device="cuda")
    for call, qi in enumerate(qs):                     # two calls in a row share the built-in scratch
        ref_out, ref_lse = c.decode_attention(0, qi, bidx, pos)
        out.fill_(float("nan")); lse.fill_(float("nan"))
        assert _call_static(c, qi, bidx, pos, out, lse) == 0
        torch.cuda.synchronize()
        d = (out.float() - ref_out.float()).abs().max().item()
        dl = (lse - ref_lse).abs().max().item()
        assert d <= MAX_ABS and dl <= LSE_ABS, (call, d, dl)
        # same kernel, same unit schedule, different scratch bytes: the results are in fact identical
        assert torch.equal(out, ref_out) and torch.equal(lse, ref_lse)
    c.check_status()


def test_static_scratch_python_wrapper_and_limits():
    case = wl.make_decode_case(31338, B=5, Hq=16, Hkv=8, D=128, P=128, n_pages=64, max_batch_size=7,
                               len_lo=1, len_hi=700, dtype=torch.bfloat16)
    c, slots, bidx, pos, k, v, q = product_from_case(case)
    out = torch.empty_like(q); lse = torch.empty((5, 16, 1), dtype=torch.float32, device="cuda")
    ref_out, ref_lse = c.decode_attention(0, q, bidx, pos)
    c.decode_attention_noalloc(0, q, bidx, pos, out, lse)
    assert torch.equal(out, ref_out) and torch.equal(lse, ref_lse)
    # 8 query heads per stored head at head_dim 128 needs more than the 4 MiB built in: a clear refusal
    wide = wl.make_decode_case(31339, B=2, Hq=16, Hkv=2, D=128, P=128, n_pages=16, max_batch_size=4,
                               len_lo=10, len_hi=100, dtype=torch.bfloat16)
    cw, _, wb, wp, _, _, wq = product_from_case(wide)
    wo = torch.empty_like(wq); wl_ = torch.empty((2, 16, 1), dtype=torch.float32, device="cuda")
    assert _call_static(cw, wq, wb, wp, wo, wl_) == _lib.ESTATIC
    assert "built-in static array" in _lib.strerror(_lib.ESTATIC)
    # a shape the TMA kernel does not take (fp32 pool) is refused, not served by another path
    f32 = wl.make_decode_case(31340, B=2, Hq=4, Hkv=2, D=64, P=128, n_pages=16, max_batch_size=4,
                              len_lo=10, len_hi=100, dtype=torch.float32)
    cf, _, fb, fp_, _, _, fq = product_from_case(f32)
    fo = torch.empty_like(fq); fl = torch.empty((2, 4, 1), dtype=torch.float32, device="cuda")
    assert _call_static(cf, fq, fb, fp_, fo, fl) == -2
    c.check_status()
