"""GPU: the append and decode-attention entry points can be captured in a CUDA
graph (no allocation, no synchronisation, lengths read on the device) and a
replay with new positions equals the eager result."""

import pytest
import torch

import workloads as wl
from helpers import product_from_case

pytestmark = pytest.mark.gpu


def test_decode_step_in_cuda_graph():
    case = wl.make_decode_case(808, B=10, Hq=16, Hkv=8, D=128, P=128, n_pages=120, max_batch_size=12,
                               len_lo=50, len_hi=1000, dtype=torch.bfloat16)
    c, slots, bidx, pos, k, v, q = product_from_case(case)
    e, *_ = product_from_case(case)                          # eager twin
    for s in slots:
        c.reserve(s, None, 1200); e.reserve(s, None, 1200)
    B = case.B
    out = torch.empty((B, 16, 1, 128), dtype=torch.bfloat16, device="cuda")
    lse = torch.empty((B, 16, 1), dtype=torch.float32, device="cuda")
    spos = pos.clone()                                        # static buffers the graph reads
    sq, sk, sv = q.clone(), k.clone(), v.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        c.decode_step(0, sq, sk, sv, bidx, spos, out=out, lse=lse)     # sizes the workspace outside capture
    side.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        c.decode_step(0, sq, sk, sv, bidx, spos, out=out, lse=lse)
    gen = torch.Generator().manual_seed(4)
    for step in range(1, 5):
        kn, vn, qn = (torch.randn(B, n, 1, 128, generator=gen).bfloat16().cuda() for n in (8, 8, 16))
        p = pos + step
        spos.copy_(p); sq.copy_(qn); sk.copy_(kn); sv.copy_(vn)
        g.replay()
        ref_out, ref_lse = e.decode_step(0, qn, kn, vn, bidx, p)
        torch.cuda.synchronize()
        assert torch.equal(out, ref_out) and torch.equal(lse, ref_lse)
    # the eager twin also replays step 0's write (the warm-up and capture ran it), so the pools match
    e.insert_kv(0, k, v, input_pos=pos.view(-1, 1), batch_idx=bidx)
    assert torch.equal(c.kv_cache, e.kv_cache)
    c.check_status()
