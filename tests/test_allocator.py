"""CPU: the product's host-side allocator against the reference traces.

The cache is built on the CPU device here: its tables and free lists are host
logic shared with the CUDA build; only the K/V data path needs a GPU."""

import json
import os

import pytest
import torch

from fpkv.paged_attention import PagedKVCache
from fpkv.attention import CausalDecodeMask, DecodeStepMask, PrefillMask, image_span_ids
import workloads as wl
from helpers import GOLDEN


def snapshot(c):
    return dict(free_pages=list(c.free_pages), free_batch_idx=list(c.free_batch_idx), capacity=list(c.capacity),
                page_table_cpu=[list(r) for r in c.page_table_cpu],
                page_table=c.page_table.cpu().tolist(), physical_to_logical=c.physical_to_logical.cpu().tolist())


def replay(tr, device):
    n_pages, P, mb = tr["ctor"]
    c = PagedKVCache(n_pages, P, mb, 1, 64, 1, torch.float32, device)
    for step in tr["steps"]:
        op = step["op"]
        if op == "init":
            pass
        elif op[0] == "allocate":
            assert c.allocate() == step["result"]
        elif op[0] == "reserve":
            slot_t = torch.tensor([op[1]], device=device)
            if step["error"] is not None:
                with pytest.raises(RuntimeError) as e:
                    c.reserve(op[1], slot_t, op[2])
                assert str(e.value) == step["error"]
            else:
                assert c.reserve(op[1], slot_t, op[2]) == step["result"]
        elif op[0] == "can_reserve":
            assert bool(c.can_reserve(op[1], op[2])) == step["result"]
        elif op[0] == "erase":
            c.erase(op[1])
        assert snapshot(c) == step["state"], op


def test_allocator_traces_cpu():
    for tr in json.load(open(os.path.join(GOLDEN, "allocator_traces.json"))):
        replay(tr, "cpu")


@pytest.mark.gpu
def test_allocator_traces_cuda():
    for tr in json.load(open(os.path.join(GOLDEN, "allocator_traces.json"))):
        replay(tr, "cuda")


def test_constructor_state_and_shapes():
    c = PagedKVCache(10, 16, 5, 2, 64, 3, torch.bfloat16, "cpu")
    assert c.kv_shape == (3, 2, 1, 2, 160, 64) and tuple(c.kv_cache.shape) == c.kv_shape
    assert c.kv_cache.dtype == torch.bfloat16 and c.page_table.dtype == torch.int64
    assert c.free_pages == [9, 8, 7, 6, 5, 4, 3, 2, 1] and c.free_batch_idx == [4, 3, 2, 1]
    assert c.num_free_pages == 9 and c.capacity == [0] * 5 and c.page_size == 16
    assert (c.page_table[0] == 0).all() and (c.page_table[1:] == -1).all()
    assert (c.physical_to_logical == -1).all()


def test_insert_kv_argument_errors():
    c = PagedKVCache(10, 16, 5, 2, 64, 1, torch.float32, "cpu")
    k = torch.zeros(2, 2, 1, 64)
    with pytest.raises(AssertionError, match="input_pos is required"):
        c.insert_kv(0, k, k, batch_idx=torch.zeros(2, dtype=torch.int64))
    with pytest.raises(AssertionError, match="batch_idx is required"):
        c.insert_kv(0, k, k, input_pos=torch.zeros(2, 1, dtype=torch.int32))
    with pytest.raises(AssertionError, match="1D .decode. or 2D"):
        c.insert_kv(0, k, k, input_pos=torch.zeros(2, 1), batch_idx=torch.zeros(1, 1, 2, dtype=torch.int64))
    with pytest.raises(AssertionError, match="number of heads must match"):
        c.insert_kv(0, torch.zeros(2, 3, 1, 64), torch.zeros(2, 3, 1, 64),
                    input_pos=torch.zeros(2, 1, dtype=torch.int32), batch_idx=torch.zeros(2, dtype=torch.int64))
    with pytest.raises(AssertionError, match="input_pos must have the same shape"):
        c.insert_kv(0, k, k, input_pos=torch.zeros(2, dtype=torch.int32), batch_idx=torch.zeros(2, dtype=torch.int64))


def test_no_cpu_data_path():
    """A CPU cache can do bookkeeping, but K/V only ever moves through the CUDA kernels."""
    c = PagedKVCache(10, 16, 5, 2, 64, 1, torch.float32, "cpu")
    k = torch.zeros(2, 2, 1, 64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        c.insert_kv(0, k, k, input_pos=torch.zeros(2, 1, dtype=torch.int32),
                    batch_idx=torch.zeros(2, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="no CPU path"):
        c.decode_attention(0, torch.zeros(2, 4, 1, 64), torch.zeros(2, dtype=torch.int64),
                           torch.zeros(2, dtype=torch.int32))


def test_mask_builders():
    c = PagedKVCache(10, 16, 5, 2, 64, 1, torch.float32, "cpu")
    m = c.create_causal_blockmask(B=5, L=160)
    assert isinstance(m, CausalDecodeMask) and m.BLOCK_SIZE == (16, 16) and m.seq_lengths == (160, 160)
    bidx, pos = torch.tensor([1, 2]), torch.tensor([3, 40], dtype=torch.int32)
    step = m.for_step(bidx, pos)
    assert isinstance(c.convert_logical_block_mask(step, bidx), DecodeStepMask)
    with pytest.raises(RuntimeError, match="same column block size"):
        c.convert_logical_block_mask(DecodeStepMask(bidx, pos, 128), bidx)
    # prefill mask ids follow the image-span rule
    toks = wl.image_text_tokens(2, 5, 3) + wl.image_text_tokens(0, 3, 1)
    ids = torch.tensor(toks).view(1, -1)
    pm = c.create_prefill_blockmask(torch.ones_like(ids), ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    assert isinstance(pm, PrefillMask)
    assert pm.img_id.tolist() == [0, 0, 1, 1, 1, 1, 1, 0, 0, 0, 0, 2, 2, 2, 0, 0]
    assert pm.doc_id.tolist() == [1] * 16
    assert image_span_ids(ids, wl.IMG_CLS_ID, wl.END_OF_IMG_ID).dtype == torch.int32


def test_logical_index_helpers():
    c = PagedKVCache(10, 4, 5, 1, 64, 1, torch.float32, "cpu")
    c.free_pages = [9, 1, 5, 3, 7]
    s = c.allocate(); c.reserve(s, None, 10)           # pages [5, 3, 7] in list order
    assert c.page_table_cpu[s] == [5, 3, 7]
    bidx = torch.tensor([s])
    phys = torch.tensor([5 * 4 + 1, 3 * 4 + 0, 7 * 4 + 3, 9 * 4])
    ok, logical = c.get_logical_kv_idx(torch.zeros(4, dtype=torch.int64), phys, bidx)
    assert ok.tolist() == [True, True, True, False] and logical.tolist()[:3] == [1, 4, 11]
    mod = c.get_mask_mod(lambda b, h, q, kv: kv <= 4, bidx)
    assert mod(torch.zeros(4, dtype=torch.int64), 0, 0, phys).tolist() == [True, True, False, False]


@pytest.mark.gpu
def test_allocator_calls_are_batched_and_ordered():
    """allocate / reserve / erase on a CUDA cache queue one record each; one launch applies a whole batch in
    order (a slot reserved, erased, allocated and reserved again), the device stacks follow the host lists,
    and bad records are reported, not applied."""
    import ctypes
    from fpkv import _lib
    c = PagedKVCache(16, 8, 4, 1, 64, 1, torch.float32, "cuda")
    a = c.allocate(); c.reserve(a, None, 20)
    c.erase(a)
    b = c.allocate(); assert b == a
    c.reserve(b, None, 9)
    assert len(c._pending) == 5                             # nothing has touched the device yet
    pt = c.page_table                                       # flushes
    assert not c._pending
    assert pt[b, :2].tolist() == c.page_table_cpu[b] and (pt[b, 2:] == -1).all()
    p2l = c.physical_to_logical[b]
    assert sorted((p2l >= 0).nonzero().view(-1).tolist()) == sorted(c.page_table_cpu[b])
    assert (pt[0] == 0).all()                               # slot 0 is never edited
    n_pg, n_sl = c._alloc_counts.tolist()
    assert c._free_pages_dev[:n_pg].tolist() == c.free_pages and c._free_slots_dev[:n_sl].tolist() == c.free_batch_idx
    # records naming slot 0, page 0, ids out of range, a pop of the wrong slot or more pages than are free are
    # skipped and flagged
    bad = torch.tensor([[3, 0, 0, 3], [3, 2, 1, 0], [3, 2, 99, 3], [4, 7, 0, 0], [0, 3, 0, 0], [1, 2, 0, 99]],
                       dtype=torch.int32, device="cuda")
    before, counts = c._page_table.clone(), c._alloc_counts.clone()
    assert _lib.lib.fpkv_alloc_step(ctypes.byref(c._pool), ctypes.byref(c._alloc), bad.data_ptr(), 6,
                                    c._status.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert torch.equal(before, c._page_table) and torch.equal(counts, c._alloc_counts)
    with pytest.raises(RuntimeError, match="bad slot, bad page id"):
        c.check_status()
    # direct edits (for callers with their own free lists) and a full clear
    ok = torch.tensor([[3, 2, 5, 9], [3, 2, 6, 4], [4, 2, 0, 0], [3, 2, 1, 7]], dtype=torch.int32, device="cuda")
    assert _lib.lib.fpkv_alloc_step(ctypes.byref(c._pool), ctypes.byref(c._alloc), ok.data_ptr(), 4,
                                    c._status.data_ptr(), None) == 0
    assert c._page_table[2].tolist() == [-1, 7] + [-1] * 14 and c._physical_to_logical[2, 7].item() == 1
    c.check_status()


@pytest.mark.gpu
def test_device_stacks_follow_the_host_lists():
    """Random allocate / reserve / erase traffic, flushed at random moments: the device free stacks and tables
    always equal the host lists and the oracle's tables."""
    import random
    from oracle import paged_kv_oracle as orc
    rnd = random.Random(7)
    c = PagedKVCache(200, 16, 12, 1, 64, 1, torch.float32, "cuda")
    o = orc.OraclePagedKVCache(200, 16, 12, 1, 64, 1, torch.float32)
    perm = list(range(1, 200)); rnd.shuffle(perm)
    c.free_pages = list(perm); o.free_pages = list(perm)
    live = {}
    for step in range(400):
        r = rnd.random()
        if r < 0.25 and c.free_batch_idx:
            s = c.allocate(); assert o.allocate() == s; live[s] = 0
        elif r < 0.7 and live:
            s = rnd.choice(list(live)); want = live[s] + rnd.randint(1, 300)
            if c.can_reserve(want, s):
                c.reserve(s, None, want); o.reserve(s, want); live[s] = want
        elif live:
            s = rnd.choice(list(live)); del live[s]; c.erase(s); o.erase(s)
        if rnd.random() < 0.2 or step == 399:
            assert torch.equal(c.page_table.cpu(), torch.as_tensor(o.page_table))
            assert torch.equal(c.physical_to_logical.cpu(), torch.as_tensor(o.physical_to_logical))
            n_pg, n_sl = c._alloc_counts.tolist()
            assert c._free_pages_dev[:n_pg].tolist() == list(o.free_pages) == c.free_pages
            assert c._free_slots_dev[:n_sl].tolist() == list(o.free_batch_idx) == c.free_batch_idx
    c.check_status()
