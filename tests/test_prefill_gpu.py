"""GPU: paged prefill attention (tcgen05 kernel) through the C ABI against the
golden vectors recorded from the reference and against the CPU oracle."""

import numpy as np
import pytest
import torch

from fpkv import _lib
import workloads as wl
from fpkv.paged_attention import PagedKVCache, paged_attention
from oracle import paged_kv_oracle as orc
from helpers import assert_attention_close, golden
from test_oracle_golden import PREFILL_CASES

pytestmark = pytest.mark.gpu
T = wl.image_text_tokens


def run_product(case, n_pages, max_batch, dtype=torch.bfloat16, kernel=0, poison=False):
    c = PagedKVCache(n_pages, case.P, max_batch, case.Hkv, case.D, 1, dtype, "cuda")
    if poison:                                     # every row that is never appended holds NaN bit patterns
        c.kv_cache.view(torch.int16).fill_(-1)
    c.prefill_kernel = kernel
    slots = []
    for toks in case.seq_tokens:
        s = c.allocate(); slots.append(s); c.reserve(s, None, len(toks))
    bidx = case.batch_idx_for(slots).cuda()
    ipos = case.input_pos.cuda()
    q, k, v = case.q.to(dtype).cuda(), case.k.to(dtype).cuda(), case.v.to(dtype).cuda()
    mask = c.create_prefill_blockmask(bidx, case.input_ids.cuda(), wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    c.insert_kv(0, k, v, input_pos=ipos, batch_idx=bidx)
    out, lse = paged_attention(q, c, 0, bidx, ipos, mask)
    return c, slots, bidx, ipos, mask, out, lse


def oracle_prefill(case, slots, dtype=torch.bfloat16):
    bidx = case.batch_idx_for(slots)
    img = orc.image_span_ids(case.input_ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    q, k, v = (x.to(dtype).float() for x in (case.q, case.k, case.v))
    return orc.prefill_attention(q, k, v, bidx, img)


def compare_live_rows(case, out, lse, ref_out, ref_lse, what):
    live = case.seq_index.view(-1) > 0
    assert_attention_close(out[0][:, live], lse[0][:, live], torch.as_tensor(ref_out)[0][:, live],
                           torch.as_tensor(ref_lse)[0][:, live], what)
    # pad rows are never consumed; the kernel writes zeros / -inf there
    if (~live).any():
        assert out[0][:, ~live].abs().max().item() == 0 and torch.isneginf(lse[0][:, ~live]).all()


@pytest.mark.parametrize("name,kernel", [("prefill_img_d128", _lib.PREFILL_TC), ("prefill_img_d128", _lib.PREFILL_PORTABLE),
                                         ("prefill_mixed_d64", _lib.PREFILL_TC), ("prefill_mixed_d64", _lib.PREFILL_PORTABLE),
                                         ("prefill_mixed_d64", _lib.PREFILL_AUTO)])
def test_prefill_against_reference_golden(name, kernel):
    """Both kernels against the reference's own output, head_dim 128 and 64."""
    make, n_pages, mb = PREFILL_CASES[name]
    case = make()
    g = golden(name)
    c, slots, bidx, ipos, mask, out, lse = run_product(case, n_pages, mb, kernel=kernel)
    assert slots == g["slots"].tolist()
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == tuple(case.q.shape) and tuple(lse.shape) == (1, 4, case.L)
    compare_live_rows(case, out, lse, g["out"], g["lse"], name)
    c.check_status()


def test_prefill_fp32_pool_portable():
    case = wl.make_prefill_case(5, [T(2, 70, 30), T(0, 0, 140)], Hq=8, Hkv=4, D=64, P=16, align=128, dtype=torch.float32)
    c, slots, bidx, ipos, mask, out, lse = run_product(case, 40, 4, dtype=torch.float32)
    ref_out, ref_lse = oracle_prefill(case, slots, dtype=torch.float32)
    live = case.seq_index.view(-1) > 0
    assert (out[0][:, live].cpu() - ref_out[0][:, live]).abs().max().item() < 1e-4
    assert (lse[0][:, live].cpu() - ref_lse[0][:, live]).abs().max().item() < 1e-4
    c.check_status()


@pytest.mark.parametrize("name,seqs,scale", [
    ("text_only", [T(0, 0, 300), T(0, 0, 77)], 1.0),
    ("image_then_text", [T(0, 1024, 63)] * 2, 1.0),                       # the config-3 sequence layout
    ("config3_scaling", [T(0, 1024, 63)], 128 ** -0.5),
    ("mixed", [T(3, 100, 20), T(0, 0, 50), T(5, 200, 30) + T(2, 37, 9), T(0, 128, 0), T(1, 129, 1)], 1.0),
    ("short", [T(0, 0, 1), T(0, 2, 0), T(0, 0, 127), T(0, 0, 128), T(0, 0, 129)], 1.0),
])
def test_prefill_against_oracle(name, seqs, scale):
    case = wl.make_prefill_case(777, seqs, Hq=16, Hkv=8, D=128, P=128, dtype=torch.bfloat16, value_scale=scale)
    n_pages = sum((len(s) + 127) // 128 for s in seqs) + 2
    c, slots, bidx, ipos, mask, out, lse = run_product(case, n_pages, len(seqs) + 2)
    ref_out, ref_lse = oracle_prefill(case, slots)
    compare_live_rows(case, out, lse, ref_out, ref_lse, name)
    c.check_status()


@pytest.mark.parametrize("kernel", [_lib.PREFILL_TC, _lib.PREFILL_PORTABLE])
def test_prefill_row_of_any_length(kernel):
    """A packed row that ends with its last token instead of padding, its length no multiple of the query tile,
    of a warp's 32 rows or of 8: the last tile's rows past the end are neither read nor written, in either
    output layout.  (Sequences still start on tile boundaries: a query tile holds rows of one sequence.)"""
    seqs = [T(0, 0, 301), T(2, 70, 30), T(0, 0, 77)]
    case = wl.make_prefill_case(2024, seqs, Hq=16, Hkv=8, D=128, P=128, align=128, dtype=torch.bfloat16)
    L = case.offsets[-1] + len(seqs[-1])
    assert L == 384 + 128 + 77 and L % 8
    case.input_ids, case.input_pos, case.seq_index = (x[:, :L].contiguous() for x in (case.input_ids, case.input_pos, case.seq_index))
    case.q, case.k, case.v = (x[:, :, :L].contiguous() for x in (case.q, case.k, case.v))
    c, slots, bidx, ipos, mask, out, lse = run_product(case, 8, 5, kernel=kernel)
    ref_out, ref_lse = oracle_prefill(case, slots)
    compare_live_rows(case, out, lse, ref_out, ref_lse, "unpadded row")
    # the token-major output layout holds the same numbers
    tout, tlse = c.prefill_attention(0, case.q.to(torch.bfloat16).cuda(), bidx, ipos, mask, token_major=True)
    assert tuple(tout.shape) == (1, L, 16, 128)
    assert torch.equal(tout.transpose(1, 2), out) and torch.equal(tlse, lse)
    c.check_status()


@pytest.mark.parametrize("n_tokens", [1, 5, 33])
def test_prefill_row_shorter_than_a_tile(n_tokens):
    """A packed row of a few tokens (shorter than the 128-row query tile and the 32-row output piece) on the
    tensor-core kernel, both output layouts."""
    seqs = [T(0, 0, n_tokens)]
    case = wl.make_prefill_case(77 + n_tokens, seqs, Hq=16, Hkv=8, D=128, P=128, align=1, dtype=torch.bfloat16)
    assert case.L == n_tokens
    c, slots, bidx, ipos, mask, out, lse = run_product(case, 4, 3, kernel=_lib.PREFILL_TC)
    ref_out, ref_lse = oracle_prefill(case, slots)
    compare_live_rows(case, out, lse, ref_out, ref_lse, "short row")
    tout, tlse = c.prefill_attention(0, case.q.to(torch.bfloat16).cuda(), bidx, ipos, mask, token_major=True)
    assert torch.equal(tout.transpose(1, 2), out) and torch.equal(tlse, lse)
    c.check_status()


def test_chunked_prefill_equals_whole_prompt():
    """Queries of a prompt processed 512 rows at a time against the pages (all K/V appended first, as the
    bidirectional image span needs) give the rows of the unchunked result; so does a reordered packing."""
    seqs = [T(0, 1024, 63), T(4, 300, 200)]
    case = wl.make_prefill_case(4321, seqs, Hq=16, Hkv=8, D=128, P=128, dtype=torch.bfloat16)
    c, slots, bidx, ipos, mask, out, lse = run_product(case, 24, 4)
    ext = mask.extent(ipos)
    q = case.q.cuda()
    for off, toks, slot in zip(case.offsets, case.seq_tokens, slots):
        Ls = len(toks)
        for c0 in range(0, Ls, 512):
            c1 = min(Ls, c0 + 512)
            from fpkv.attention import PrefillMask
            chunk_mask = PrefillMask(mask.doc_id[off + c0:off + c1], mask.img_id[off + c0:off + c1])
            chunk_mask._extent = ext[off + c0:off + c1].contiguous()       # extents are properties of the tokens
            o2, l2 = c.prefill_attention(0, q[:, :, off + c0:off + c1], bidx[:, off + c0:off + c1],
                                         ipos[:, off + c0:off + c1], chunk_mask)
            assert torch.equal(o2, out[:, :, off + c0:off + c1]) and torch.equal(l2, lse[:, :, off + c0:off + c1])
    c.check_status()


def test_fp16_and_unmapped_rows():
    case = wl.make_prefill_case(99, [T(0, 40, 100), T(0, 0, 200)], Hq=8, Hkv=8, D=128, dtype=torch.float16)
    c, slots, bidx, ipos, mask, out, lse = run_product(case, 8, 4, dtype=torch.float16)
    ref_out, ref_lse = oracle_prefill(case, slots, dtype=torch.float16)
    compare_live_rows(case, out, lse, ref_out, ref_lse, "fp16")
    c.check_status()
    # a slot whose pages were erased has nothing visible: zeros and -inf, no fault
    c.erase(slots[1])
    out2, lse2 = paged_attention(case.q.half().cuda(), c, 0, bidx, ipos, mask)
    off = case.offsets[1]
    assert out2[0, :, off:off + 200].abs().max().item() == 0 and torch.isneginf(lse2[0, :, off:off + 200]).all()
    assert torch.equal(out2[0, :, :140], out[0, :, :140])
    c.check_status()


def test_long_prompts_many_key_tiles():
    """Thousands of keys per row: 20+ key tiles, query tiles whose rows have very different extents."""
    seqs = [T(0, 0, 2900), T(50, 2000, 300)]
    case = wl.make_prefill_case(31, seqs, Hq=4, Hkv=2, D=128, dtype=torch.bfloat16)
    c, slots, bidx, ipos, mask, out, lse = run_product(case, 48, 4)
    ref_out, ref_lse = oracle_prefill(case, slots)
    compare_live_rows(case, out, lse, ref_out, ref_lse, "long prompts")
    c.check_status()


@pytest.mark.parametrize("seed", range(6))
def test_random_prompt_layouts(seed):
    """Random mixes of text, images (with a few leading register-like tokens folded into the span) and
    several images per prompt, both kernels."""
    rng = np.random.default_rng(500 + seed)
    seqs = []
    for _ in range(int(rng.integers(1, 5))):
        toks = []
        for _ in range(int(rng.integers(1, 4))):
            toks += T(int(rng.integers(0, 40)), int(rng.integers(0, 2)) * int(rng.integers(2, 400)), int(rng.integers(0, 150)))
        seqs.append(toks or T(0, 0, 1))
    # odd seeds at head_dim 64 (fp16 for one of them), three query heads per stored head for another
    D, Hq, Hkv = (64, 8, 4) if seed % 2 else ((128, 6, 2) if seed == 4 else (128, 8, 4))
    dtype = torch.float16 if seed == 3 else torch.bfloat16
    case = wl.make_prefill_case(900 + seed, seqs, Hq=Hq, Hkv=Hkv, D=D, dtype=dtype)
    n_pages = sum((len(s) + 127) // 128 for s in seqs) + 2
    for kernel in (_lib.PREFILL_TC, _lib.PREFILL_PORTABLE):
        c, slots, bidx, ipos, mask, out, lse = run_product(case, n_pages, len(seqs) + 2, dtype=dtype, kernel=kernel)
        ref_out, ref_lse = oracle_prefill(case, slots, dtype=dtype)
        compare_live_rows(case, out, lse, ref_out, ref_lse, f"random layout {seed}, kernel {kernel}")
        c.check_status()


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("kernel", [_lib.PREFILL_TC, _lib.PREFILL_PORTABLE])
def test_rows_never_appended_may_hold_anything(kernel, D):
    """A pool that was not zero-filled: the tails of the sequences' last pages (fetched with the page) and
    reserved page 0 hold NaN bit patterns; no result is touched by them."""
    seqs = [T(0, 100, 30), T(0, 0, 129), T(3, 250, 1), T(0, 0, 5)]
    case = wl.make_prefill_case(4141, seqs, Hq=8, Hkv=4, D=D, dtype=torch.bfloat16)
    c, slots, bidx, ipos, mask, out, lse = run_product(case, 12, 6, kernel=kernel, poison=True)
    ref_out, ref_lse = oracle_prefill(case, slots)
    live = case.seq_index.view(-1) > 0
    assert torch.isfinite(out[0][:, live].float()).all()
    compare_live_rows(case, out, lse, ref_out, ref_lse, f"NaN-filled pool, kernel {kernel}")
    c.check_status()
