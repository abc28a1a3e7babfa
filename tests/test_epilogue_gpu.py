"""GPU: the sink gate and token-major layout fused into the attention kernels'
output stage, against the oracle's restatement of Attention._post_attention
applied to the un-fused results."""

import pytest
import torch

from fpkv import _lib
import workloads as wl
from fpkv.paged_attention import PagedKVCache, paged_attention
from oracle import paged_kv_oracle as orc
from helpers import product_from_case

pytestmark = pytest.mark.gpu
T = wl.image_text_tokens


def close_to_gated(got, want, what):
    """The kernels evaluate the sigmoid with the fast exponential, so a product can land on the other
    side of a rounding boundary: allow one unit in the last place of the 16-bit result, nothing more."""
    got, want = got.float().cpu(), want.float().cpu()
    ulp = want.abs() * 2.0 ** -7 + 1e-30
    bad = (got - want).abs() > ulp
    assert not bad.any(), f"{what}: {int(bad.sum())} elements differ by more than one ulp"
    assert (got != want).float().mean().item() < 0.02, f"{what}: too many last-place differences"


@pytest.mark.parametrize("kernel", [_lib.DECODE_TMA, _lib.DECODE_PORTABLE])
def test_decode_sink_gate(kernel):
    case = wl.make_decode_case(606, B=20, Hq=16, Hkv=8, D=128, P=128, n_pages=300, max_batch_size=23,
                               len_lo=1, len_hi=1700, dtype=torch.bfloat16)      # long enough for cut segments
    c, slots, bidx, pos, k, v, q = product_from_case(case, pad_rows=2)
    c.decode_kernel = kernel
    sinks = (torch.randn(16) * 2).bfloat16().cuda()
    out, lse = c.decode_attention(0, q, bidx, pos)
    gout, glse = c.decode_attention(0, q, bidx, pos, sinks=sinks)
    assert torch.equal(lse, glse)                                  # lse is returned ungated
    want = orc.post_attention_gate(out.cpu(), lse.cpu(), sinks.cpu())                 # (B, 1, Hq*D)
    close_to_gated(gout.view(case.B + 2, 1, -1), want, "decode gate")
    assert gout[-1].abs().max().item() == 0                        # padding rows: sigmoid(-inf) = 0
    # the fused step takes the same path
    gout2, _ = c.decode_step(0, q, k, v, bidx, pos, sinks=sinks)
    assert torch.equal(gout2, gout)
    # fp32 sinks are accepted too
    gout3, _ = c.decode_attention(0, q, bidx, pos, sinks=sinks.float())
    assert torch.equal(gout3, gout)
    c.check_status()


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("kernel", [_lib.PREFILL_TC, _lib.PREFILL_PORTABLE])
def test_prefill_sink_gate_and_token_major_layout(kernel, D):
    case = wl.make_prefill_case(707, [T(2, 200, 40), T(0, 0, 90)], Hq=16, Hkv=8, D=D, dtype=torch.bfloat16)
    c = PagedKVCache(16, 128, 4, 8, D, 1, torch.bfloat16, "cuda")
    c.prefill_kernel = kernel
    slots = []
    for toks in case.seq_tokens:
        s = c.allocate(); slots.append(s); c.reserve(s, None, len(toks))
    bidx, ipos = case.batch_idx_for(slots).cuda(), case.input_pos.cuda()
    q = case.q.cuda()
    mask = c.create_prefill_blockmask(bidx, case.input_ids.cuda(), wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    c.insert_kv(0, case.k.cuda(), case.v.cuda(), input_pos=ipos, batch_idx=bidx)
    sinks = (torch.randn(16) * 2).bfloat16().cuda()
    out, lse = paged_attention(q, c, 0, bidx, ipos, mask)
    gout, glse = c.prefill_attention(0, q, bidx, ipos, mask, sinks=sinks, token_major=True)
    assert tuple(gout.shape) == (1, case.L, 16, D) and torch.equal(lse, glse)
    want = orc.post_attention_gate(out.cpu(), lse.cpu(), sinks.cpu())                 # (1, L, Hq*D)
    close_to_gated(gout.view(1, case.L, -1), want, "prefill gate, token-major")
    # layout alone, no gate: a pure permutation of the head-major result
    tout, _ = c.prefill_attention(0, q, bidx, ipos, mask, token_major=True)
    assert torch.equal(tout, out.permute(0, 2, 1, 3))
    c.check_status()
