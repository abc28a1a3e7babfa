"""CPU: property tests of the allocator (hypothesis): arbitrary interleavings of
allocate / reserve / erase keep the product's host class equal to the oracle,
and both keep the invariants the kernels rely on."""

import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from fpkv.paged_attention import PagedKVCache
from oracle import paged_kv_oracle as orc

N_PAGES, P, MB = 20, 8, 6

ops = st.lists(st.tuples(st.sampled_from(["allocate", "reserve", "erase", "can"]), st.integers(0, 200),
                         st.integers(0, 10)), min_size=1, max_size=60)


def invariants(c):
    pt = c.page_table.numpy() if torch.is_tensor(c.page_table) else c.page_table
    p2l = c.physical_to_logical.numpy() if torch.is_tensor(c.physical_to_logical) else c.physical_to_logical
    used = [p for row in c.page_table_cpu for p in row]
    assert len(used) == len(set(used)) and 0 not in used                      # a page has one owner; page 0 is nobody's
    assert sorted(used + list(c.free_pages)) == list(range(1, N_PAGES))        # nothing leaks, nothing is duplicated
    assert (pt[0] == 0).all() and (p2l[0] == -1).all()                         # slot 0 stays the no-op slot
    for s in range(1, MB):
        row = c.page_table_cpu[s]
        assert c.capacity[s] == len(row) * P
        assert pt[s, :len(row)].tolist() == row and (pt[s, len(row):] == -1).all() or s in c.free_batch_idx
        for j, pg in enumerate(row):
            assert p2l[s, pg] == j                                             # the inverse table inverts the table
    assert sorted(set(c.free_batch_idx)) == sorted(c.free_batch_idx)           # a slot is freed once


@settings(max_examples=150, deadline=None)
@given(ops)
def test_random_interleavings(seq):
    c = PagedKVCache(N_PAGES, P, MB, 1, 64, 1, torch.float32, "cpu")
    o = orc.OraclePagedKVCache(N_PAGES, P, MB, 1, 64, 1, torch.float32)
    live = []
    for kind, n, pick in seq:
        if kind == "allocate":
            if not c.free_batch_idx:
                continue
            s = c.allocate(); assert o.allocate() == s; live.append(s)
        elif kind == "reserve" and live:
            s = live[pick % len(live)]
            ok = c.can_reserve(n, s)
            assert ok == o.can_reserve(n, s)
            if ok:
                assert c.reserve(s, None, n) and o.reserve(s, n)
            else:
                for cache, call in ((c, lambda: c.reserve(s, None, n)), (o, lambda: o.reserve(s, n))):
                    try:
                        call(); raise AssertionError("over-reserve must raise")
                    except RuntimeError as e:
                        assert "Cannot reserve" in str(e)
        elif kind == "erase" and live:
            s = live.pop(pick % len(live))
            c.erase(s); o.erase(s)
        elif kind == "can":
            assert c.can_reserve(n) == o.can_reserve(n)
        assert list(c.free_pages) == list(o.free_pages) and list(c.free_batch_idx) == list(o.free_batch_idx)
        assert c.page_table_cpu == o.page_table_cpu and list(c.capacity) == list(o.capacity)
        assert np.array_equal(c.page_table.numpy(), o.page_table)
        assert np.array_equal(c.physical_to_logical.numpy(), o.physical_to_logical)
        invariants(c)
