"""Shared builders for the parity tests: the same seeded case is loaded into
the CUDA cache (product) and into the CPU oracle (checker)."""

import os

import numpy as np
import torch

from oracle import paged_kv_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# BASELINE tolerance for attention outputs of the 16-bit kernels against the fp32 reference
MAX_ABS, MEAN_ABS, LSE_ABS, REL_MAX = 2e-2, 2e-3, 2e-2, 2e-2


def golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def oracle_from_case(case, dtype=None, pad_rows=0):
    """Oracle cache after reserve + packed history append + decode append.
    Returns (cache, slots, batch_idx, input_pos, k_new, v_new, q) with pad rows
    (slot 0, position 0, zero vectors) appended to the decode batch."""
    dtype = dtype or case.dtype
    o = orc.OraclePagedKVCache(case.n_pages, case.P, case.max_batch_size, case.Hkv, case.D, 1, dtype)
    o.free_pages = list(case.free_pages)
    slots = []
    for L, kh, vh in zip(case.lens, case.k_hist, case.v_hist):
        s = o.allocate(); slots.append(s)
        o.reserve(s, L + 1)
        if L:
            o.append_packed(0, torch.full((1, L), s), torch.arange(L).view(1, L), kh.to(dtype), vh.to(dtype))
    bidx = torch.tensor(slots + [0] * pad_rows, dtype=torch.int64)
    pos = torch.tensor(list(case.lens) + [0] * pad_rows, dtype=torch.int32)

    def pad(x):
        x = x.to(dtype)
        return torch.cat([x, torch.zeros((pad_rows,) + tuple(x.shape[1:]), dtype=dtype)]) if pad_rows else x
    k, v, q = pad(case.k_new), pad(case.v_new), pad(case.q)
    o.append_decode(0, bidx, pos, k, v)
    return o, slots, bidx, pos, k, v, q


def product_from_case(case, device="cuda", pad_rows=0, num_layers=1, layer=0):
    """The CUDA cache driven through the public API with the same case."""
    from fpkv.paged_attention import PagedKVCache
    c = PagedKVCache(case.n_pages, case.P, case.max_batch_size, case.Hkv, case.D, num_layers, case.dtype, device)
    c.free_pages = list(case.free_pages)
    slots = []
    for L, kh, vh in zip(case.lens, case.k_hist, case.v_hist):
        s = c.allocate(); slots.append(s)
        c.reserve(s, torch.tensor([s], device=device), L + 1)
        if L:
            c.insert_kv(layer, kh.to(device), vh.to(device), input_pos=torch.arange(L, device=device).view(1, L),
                        batch_idx=torch.full((1, L), s, device=device))
    B = case.B + pad_rows
    bidx = torch.tensor(slots + [0] * pad_rows, dtype=torch.int64, device=device)
    pos = torch.tensor(list(case.lens) + [0] * pad_rows, dtype=torch.int32, device=device)

    def pad(x):
        x = x.to(device)
        return torch.cat([x, torch.zeros((pad_rows,) + tuple(x.shape[1:]), dtype=x.dtype, device=device)]) \
            if pad_rows else x
    k, v, q = pad(case.k_new), pad(case.v_new), pad(case.q)
    c.insert_kv(layer, k, v, input_pos=pos.view(B, 1), batch_idx=bidx)
    return c, slots, bidx, pos, k, v, q


def assert_attention_close(out, lse, ref_out, ref_lse, what=""):
    """out/lse from the kernel against a reference computed in fp32."""
    out, ref_out = out.float().cpu(), torch.as_tensor(ref_out).float()
    lse, ref_lse = lse.float().cpu(), torch.as_tensor(ref_lse).float()
    assert out.shape == ref_out.shape and lse.shape == ref_lse.shape, what
    d = (out - ref_out).abs()
    assert d.max().item() <= MAX_ABS, f"{what}: max abs {d.max().item()}"
    assert d.mean().item() <= MEAN_ABS, f"{what}: mean abs {d.mean().item()}"
    # relative bound: the absolute tolerances alone would pass an all-zero output on small-valued cases
    denom = ref_out.abs().max().item()
    if denom > 0:
        assert d.max().item() / denom <= REL_MAX, f"{what}: rel max {d.max().item() / denom}"
    fin = torch.isfinite(ref_lse)
    assert torch.equal(fin, torch.isfinite(lse)), f"{what}: lse finiteness differs"
    assert torch.equal(lse[~fin], ref_lse[~fin]), f"{what}: masked rows must give lse=-inf"
    if fin.any():
        dl = (lse[fin] - ref_lse[fin]).abs().max().item()
        assert dl <= LSE_ABS, f"{what}: lse abs {dl}"
    # rows without any visible key: out exactly zero
    dead = ~fin
    if dead.any():
        assert out[dead].abs().max().item() == 0.0, f"{what}: masked rows must give out=0"
