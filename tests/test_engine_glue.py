"""CPU: the engine-side glue (step state, mixed-step planning, packed prefill rows) on a bookkeeping-only cache."""

from collections import deque

import torch

from fpkv.engine_glue import MixedStepPlanner, SlotState, decoding_block_mask, pack_prefill_rows
from fpkv.paged_attention import PagedKVCache


class Seq:
    def __init__(self, n, spans=()):
        self.tokens = list(range(100, 100 + n))
        self.batch_idx = None
        self.image_spans = list(spans)
        self.generated = 0

    @property
    def total_length(self):
        return len(self.tokens) + self.generated


def test_slot_state_one_upload_per_step():
    st = SlotState(8, "cpu")
    st.begin(3, 41, 57, 900)          # a sequence of 42 tokens whose first sampled token is 900
    st.begin(5, 9, 9, 901)
    n = st.stage([5, 3], bucket=4)    # padded to a graph bucket of 4 with slot 0
    assert n == 4 and st.batch_idx[:4].tolist() == [5, 3, 0, 0]
    bi, pos, rope, ids = st.step_inputs(4)
    assert pos.tolist() == [9, 41, 0, 0] and pos.dtype == torch.int32
    assert rope.tolist() == [9, 57, 0, 0] and ids.tolist() == [901, 900, 0, 0]
    st.advance(4, torch.tensor([11, 12, 13, 14]))
    _, pos, rope, ids = st.step_inputs(4)
    assert pos.tolist() == [10, 42, 0, 0] and rope.tolist() == [10, 58, 0, 0] and ids.tolist() == [11, 12, 0, 0]
    assert st.input_pos[0].item() == 0 and st.last_token[0].item() == 0          # the padding slot never moves
    st.stage([3])                     # the other sequence finished; nothing restarted
    assert st.step_inputs(1)[1].tolist() == [42]
    m = decoding_block_mask(PagedKVCache(8, 16, 8, 1, 64, 1, torch.float32, "cpu").create_causal_blockmask(8, 128),
                            *st.step_inputs(1)[:2])
    assert m.batch_idx.tolist() == [3] and m.input_pos.tolist() == [42]


def test_planner_mixes_prefill_chunks_with_decode_rows():
    c = PagedKVCache(40, 16, 6, 1, 64, 1, torch.float32, "cpu")             # 39 usable pages of 16 tokens
    pl = MixedStepPlanner(c, chunk_tokens=64, prefill_token_budget=96)
    a, b = Seq(150, spans=[(40, 100)]), Seq(30)
    pl.add(a); pl.add(b)
    p1 = pl.plan()
    assert p1.kind == "prefill" and p1.admitted == [a, b] and (a.batch_idx, b.batch_idx) == (1, 2)
    assert c.capacity[1] == 160 and c.capacity[2] == 32
    # a's first chunk would end at 64, inside the image span [40, 100): extended to 100; the budget of 96 is then spent
    assert [(ch.seq, ch.start, ch.end) for ch in p1.prefill] == [(a, 0, 100)]
    pl.commit(p1)
    p2 = pl.plan()
    assert [(ch.seq, ch.start, ch.end) for ch in p2.prefill] == [(a, 100, 150), (b, 0, 30)]
    pl.commit(p2)
    assert list(pl.running) == [a, b] and not pl.prefilling
    d = Seq(60)
    pl.add(d)
    p3 = pl.plan()                                                            # a newcomer is prefilled while a and b decode
    assert p3.kind == "mixed" and p3.decode == [a, b] and [(ch.seq, ch.start, ch.end) for ch in p3.prefill] == [(d, 0, 60)]
    pl.commit(p3)
    a.generated += 11; b.generated += 3                                       # a crosses a page boundary: 161 > 160
    p4 = pl.plan()
    assert p4.kind == "decode" and p4.decode == [a, b, d] and c.capacity[1] == 176
    pl.finish(b)
    assert list(pl.running) == [a, d] and 2 in c.free_batch_idx and c.capacity[2] == 0


def test_planner_preempts_the_newest_when_the_pool_is_exhausted():
    c = PagedKVCache(9, 16, 6, 1, 64, 1, torch.float32, "cpu")               # 8 usable pages
    pl = MixedStepPlanner(c, chunk_tokens=512)
    a, b = Seq(64), Seq(64)
    pl.add(a); pl.add(b)
    p = pl.plan(); pl.commit(p)
    assert list(pl.running) == [a, b] and c.num_free_pages == 0
    waiting = Seq(10)
    pl.add(waiting)
    a.generated = 1                                                          # a needs a fifth page; none is free
    p = pl.plan()
    assert p.preempted == [b] and p.decode == [a] and list(pl.waiting)[0] is b and c.capacity[a.batch_idx] == 80
    # b's pages came back; the queue's head (b itself) does not fit beside a again, so nothing is admitted
    assert not p.admitted and c.num_free_pages == 3


def test_packed_rows_follow_the_reference_layout():
    c = PagedKVCache(40, 16, 6, 1, 64, 1, torch.float32, "cpu")
    pl = MixedStepPlanner(c, chunk_tokens=100, prefill_token_budget=1000)
    a, b = Seq(150), Seq(30)
    pl.add(a); pl.add(b)
    p = pl.plan(); pl.commit(p)
    p = pl.plan()                                                             # a's rows 100..149 only
    ids, pos, bidx, offsets, last = pack_prefill_rows(p.prefill, lambda s: s.tokens, pad_id=7, align=128)
    assert ids.shape == (1, 128) and offsets == [0] and last == {id(a): 49}
    assert ids[0, :50].tolist() == a.tokens[100:150] and (ids[0, 50:] == 7).all()
    assert pos[0, :50].tolist() == list(range(100, 150)) and (pos[0, 50:] == 0).all()
    assert (bidx[0, :50] == a.batch_idx).all() and (bidx[0, 50:] == 0).all()
