"""CPU, world_size 2 over gloo: the multi-GPU plan has no data-path collective;
each rank owns a shard of the job (the same seeded amount of work in its own
pool with its own page permutation and free lists) and the report is MAX-of-times / SUM-of-work over ranks."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    from fpkv.paged_attention import PagedKVCache
    # the rank's shard: its own draw, its own (CPU, bookkeeping-only) cache and allocator state
    case = bench.rank_case(rank, batch=8, n_pages=512, len_lo=100, len_hi=900)
    cache = PagedKVCache(512, 128, 9, 8, 128, 1, torch.bfloat16, "cpu")
    cache.free_pages = list(case.free_pages)
    slots = []
    for L in case.lens:
        s = cache.allocate(); cache.reserve(s, None, L + 1); slots.append(s)
    my_bytes = float(bench.step_bytes(case.lens))
    my_ms = 1.0 + rank                                 # the slower rank defines the job's time
    (ms,), (total_bytes, tokens) = bench.reduce_over_ranks([my_ms], [my_bytes, 8.0], torch.device("cpu"), world)
    gathered = [None] * world
    dist.all_gather_object(gathered, dict(lens=case.lens, pages=[cache.page_table_cpu[s] for s in slots],
                                          bytes=my_bytes))
    if rank == 0:
        out.put(dict(ms=ms, total_bytes=total_bytes, tokens=tokens, ranks=gathered))
    dist.destroy_process_group()


def test_two_rank_shards_and_report():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = out.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    r0, r1 = res["ranks"]
    assert res["ms"] == 2.0                             # MAX over ranks
    assert res["tokens"] == 16.0                        # SUM over ranks
    assert abs(res["total_bytes"] - (r0["bytes"] + r1["bytes"])) < 1e-6
    assert r0["lens"] == r1["lens"]                     # weak scaling: the same work on every rank ...
    assert r0["pages"] != r1["pages"]                   # ... in its own pool with its own page permutation
    import bench
    assert r0["lens"] == bench.rank_case(0, batch=8, n_pages=512, len_lo=100, len_hi=900).lens
    # every rank allocates from its own pool: page ids overlap freely between ranks, never within one
    for r in (r0, r1):
        flat = [p for seq in r["pages"] for p in seq]
        assert len(flat) == len(set(flat)) and 0 not in flat
