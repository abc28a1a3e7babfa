"""Benchmark of the paged KV-cache decode path (append + paged decode attention).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl fpkv|reference]

Workload (one "step" = one decode step of one layer over the whole batch):
bf16, batch 64 per GPU, 16 query heads over 8 stored heads, head_dim 128,
page 128, context lengths uniform in [1024, 8192], page ids permuted over a
65 536-page pool (32 GiB), values N(0,1)/sqrt(128); every step appends one
token per sequence and runs one paged decode attention, then positions advance
by one.  Inputs are synthetic and seeded; nothing is read from disk or network.

  value      algorithmic KV GB/s of the whole job: bytes the step must move
             (K/V of every visible key once, the appended rows, q, out, lse)
             divided by the device time of K steps, summed over GPUs, with the
             step inputs already resident in HBM.
  e2e        the same through the public Python API with the step's inputs
             (q, k, v, slots, positions) copied from pinned host memory and
             out / lse written to pinned host memory every step, the host
             waiting for each step's result.
  roofline   the decode-attention kernel alone (its two launches) against the
             measured HBM copy bandwidth.
  cpu_baseline / --impl reference
             the CPU restatement of the reference path (oracle/), timed on the
             host cores with torch's threads on a bounded sample.

Multi-GPU: one process per GPU (torchrun), each with its own pool and its own
batch of 64 sequences (weak scaling); no collective on the data path, NCCL is
used only for the timing barrier and to combine the per-rank numbers.
"""

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "falcon-perception_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

HQ, HKV, D, P = 16, 8, 128, 128
BATCH = 64
LEN_LO, LEN_HI = 1024, 8192
N_PAGES = 65536
FALLBACK_HBM_GBS = 6650.0
WINDOW = 64          # positions cycle through L .. L+63
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_tma_kernel launch on this workload, from the
# ncu capture summarised in profiles/decode_tma_kernel_config2.md
NCU_TRAFFIC_BYTES = 1.1731e9


def step_bytes(lens_before_append):
    """Algorithmic bytes of one step: K and V of every visible key (context +
    the appended token) once, the appended K/V rows read and written, q read,
    out written, lse written.  bf16."""
    s = 2
    B = len(lens_before_append)
    kv = sum((L + 1) * 2 * HKV * D * s for L in lens_before_append)
    return kv + 2 * B * 2 * HKV * D * s + 2 * B * HQ * D * s + 4 * B * HQ


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """SM clock and throttle reasons sampled through NVML (read-only queries)
    every few milliseconds while the timed regions run."""
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, device_index, period_s=0.004):
        self.period, self.samples, self.bits, self.stop_flag, self.thread = period_s, [], 0, False, None
        self.handle = self.max_mhz = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception as e:                      # no NVML: report that instead of guessing
            self.error = repr(e)
            self.handle = None

    def _loop(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.handle is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()

    def stop(self):
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable: " + getattr(self, "error", "?")],
                    "samples": 0}
        self.stop_flag = True
        self.thread.join(timeout=2)
        v = sorted(self.samples)
        return {"sm_mhz": v[len(v) // 2] if v else None, "sm_max_mhz": self.max_mhz,
                "reasons": [n for n, b in self.REASONS if self.bits & b], "samples": len(v)}


def rank_case(rank, batch=BATCH, n_pages=N_PAGES, len_lo=LEN_LO, len_hi=LEN_HI, seed=2002):
    """The shard of the job that rank ``rank`` owns.  Weak scaling: every rank gets the same amount of work
    -- the seeded context lengths of the single-GPU workload -- in its own pool, with its own page
    permutation (so the page tables differ from rank to rank); rank 0 alone is the single-GPU workload."""
    import numpy as np
    from fpkv import workloads as wl
    case = wl.config2_case(B=batch, n_pages=n_pages, len_lo=len_lo, len_hi=len_hi, seed=seed)
    if rank:
        case.free_pages = (np.random.default_rng(seed + 7919 * rank).permutation(n_pages - 1) + 1).tolist()
    return case


def reduce_over_ranks(times_ms, work, device, world):
    """Whole-job numbers from per-rank ones: a time is the MAX over ranks (the job ends when the slowest
    rank does), work (bytes, tokens) is the SUM.  The only communication of the benchmark."""
    import torch.distributed as dist
    t = torch.tensor(times_ms, dtype=torch.float64, device=device)
    w = torch.tensor(work, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(w, op=dist.ReduceOp.SUM)
    return t.tolist(), w.tolist()


def build_gpu_workload(rank, device, n_steps, n_pages=N_PAGES, batch=BATCH, len_lo=LEN_LO, len_hi=LEN_HI):
    """Cache with 64 seeded sequences whose context pages hold random values."""
    from fpkv import workloads as wl
    from fpkv.paged_attention import PagedKVCache
    case = rank_case(rank, batch, n_pages, len_lo, len_hi)
    cache = PagedKVCache(n_pages, P, batch + 1, HKV, D, 1, torch.bfloat16, device)
    cache.free_pages = list(case.free_pages)
    slots = []
    for L in case.lens:
        s = cache.allocate(); slots.append(s)
        cache.reserve(s, None, L + 1 + n_steps)
    gen = torch.Generator(device=device).manual_seed(7 + rank)
    view = cache.kv_cache.view(2, HKV, n_pages, P, D)
    for s in slots:                                    # context values ~ N(0,1)/sqrt(D), written page-wise
        pages = torch.tensor(cache.page_table_cpu[s], device=device)
        view[:, :, pages] = (torch.randn((2, HKV, pages.numel(), P, D), device=device, generator=gen)
                             * D ** -0.5).to(torch.bfloat16)
    return case, cache, slots


def run_fpkv(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path for the product"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    K, W = args.steps, args.warmup
    case, cache, slots = build_gpu_workload(rank, device, WINDOW, args.pool_pages, args.batch, args.len_lo, args.len_hi)
    B = args.batch
    lens = torch.tensor(case.lens, dtype=torch.int32)
    bidx_h = torch.tensor(slots, dtype=torch.int64).pin_memory()
    bidx = bidx_h.to(device)
    gen = torch.Generator(device="cpu").manual_seed(99 + rank)
    NV = 4                                             # distinct step inputs, cycled
    q_h = (torch.randn((NV, B, HQ, 1, D), generator=gen) * D ** -0.5).to(torch.bfloat16).pin_memory()
    k_h = (torch.randn((NV, B, HKV, 1, D), generator=gen) * D ** -0.5).to(torch.bfloat16).pin_memory()
    v_h = (torch.randn((NV, B, HKV, 1, D), generator=gen) * D ** -0.5).to(torch.bfloat16).pin_memory()
    # positions advance by one per step and wrap after WINDOW steps, so that the context stays in range
    pos_h = (lens.view(1, B) + torch.arange(WINDOW, dtype=torch.int32).view(-1, 1)).contiguous().pin_memory()
    q_d, k_d, v_d, pos_d = q_h.to(device), k_h.to(device), v_h.to(device), pos_h.to(device)
    out = torch.empty((B, HQ, 1, D), dtype=torch.bfloat16, device=device)
    lse = torch.empty((B, HQ, 1), dtype=torch.float32, device=device)
    stream = torch.cuda.current_stream(device)

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---------------- device-resident timing -------------------------------
    # One step = the fused public call (append, then attention whose set-up overlaps the append).
    def step_resident(i):
        j = i % NV
        cache.decode_step(0, q_d[j], k_d[j], v_d[j], bidx, pos_d[i % WINDOW], out=out, lse=lse)

    step = 0
    for _ in range(W):
        step_resident(step); step += 1
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first_timed = step
    t0.record(stream)
    for i in range(K):
        step_resident(step); step += 1
    t1.record(stream)
    barrier()
    ms_total = t0.elapsed_time(t1)
    cache.check_status()
    bytes_timed = sum(step_bytes([L + (first_timed + i) % WINDOW for L in case.lens]) for i in range(K))

    # The decode-attention call alone (main kernel + its finish kernel), same positions as the timed
    # steps, K launches back to back between one pair of events on the launching stream: the average
    # launch duration is the roofline's denominator.  (Events between the launches would serialise what
    # the kernels overlap on their own, so they bracket the loop, not each launch.)
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a0.record(stream)
    for i in range(K):
        j = (first_timed + i) % NV
        cache.decode_attention(0, q_d[j], bidx, pos_d[(first_timed + i) % WINDOW], out=out, lse=lse)
    a1.record(stream)
    barrier()
    attn_ms = a0.elapsed_time(a1) / K
    attn_bytes = bytes_timed / K - 2 * B * 2 * HKV * D * 2          # attention alone: no append traffic

    # ---------------- end to end through the public API, host buffers ------
    # One pinned staging buffer per direction: the step's q, k, v, positions and slots travel in one
    # host-to-device copy, out and lse come back in one device-to-host copy; the API gets views.
    nq, nk = B * HQ * D * 2, B * HKV * D * 2
    in_bytes = (nq + 2 * nk + B * 4 + B * 8 + 15) // 16 * 16           # rows of the staging array stay 16-byte aligned
    in_h = torch.empty((NV, in_bytes), dtype=torch.uint8).pin_memory()
    in_d = torch.empty(in_bytes, dtype=torch.uint8, device=device)
    # The result needs no staging copy: out and lse are pinned host memory that the kernels write directly
    # (the device can address pinned memory), so the step's result is on the host when the stream is idle.
    res_h = torch.empty(nq + B * HQ * 4, dtype=torch.uint8).pin_memory()

    def views(buf):
        o = 0
        q = buf[o:o + nq].view(torch.bfloat16).view(B, HQ, 1, D); o += nq
        k = buf[o:o + nk].view(torch.bfloat16).view(B, HKV, 1, D); o += nk
        v = buf[o:o + nk].view(torch.bfloat16).view(B, HKV, 1, D); o += nk
        bi = buf[o:o + B * 8].view(torch.int64); o += B * 8
        ps = buf[o:o + B * 4].view(torch.int32)
        return q, k, v, bi, ps
    host_pos = []
    for j in range(NV):                                # the NV distinct step inputs, staged in pinned memory
        hq, hk, hv, hbi, hps = views(in_h[j])
        hq.copy_(q_h[j]); hk.copy_(k_h[j]); hv.copy_(v_h[j]); hbi.copy_(bidx_h); hps.copy_(pos_h[0])
        host_pos.append(hps)
    q_s, k_s, v_s, bidx_s, pos_s = views(in_d)
    out_s = res_h[:nq].view(torch.bfloat16).view(B, HQ, 1, D)
    lse_s = res_h[nq:].view(torch.float32).view(B, HQ, 1)

    # As the reference engine does for decode, the step (copy in, append + attention writing its result to
    # host memory) is captured once per staging buffer in a CUDA graph and replayed; the host writes the
    # step's positions into pinned memory, replays, and waits for the result.
    graphs = []
    if not args.kernels_only:
        side = torch.cuda.Stream(device)
        for j in range(NV):
            side.wait_stream(stream)
            with torch.cuda.stream(side):              # warm the path on the capture stream first
                in_d.copy_(in_h[j], non_blocking=True)
                cache.decode_step(0, q_s, k_s, v_s, bidx_s, pos_s, out=out_s, lse=lse_s)
            side.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=side):
                in_d.copy_(in_h[j], non_blocking=True)
                cache.decode_step(0, q_s, k_s, v_s, bidx_s, pos_s, out=out_s, lse=lse_s)
            graphs.append(gr)
        torch.cuda.synchronize(device)

    def step_e2e(i):
        j = i % NV
        host_pos[j].copy_(pos_h[i % WINDOW])          # this step's positions, written by the host
        graphs[j].replay()
        torch.cuda.current_stream(device).synchronize()   # the step's result is on the host before the next step

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first_e2e = step
    if args.kernels_only:                              # profiling runs: device-resident loop only
        ms_e2e = float("nan")
    else:
        for _ in range(W):
            step_e2e(step); step += 1
        barrier()
        first_e2e = step
        e0.record(stream)
        for _ in range(K):
            step_e2e(step); step += 1
        e1.record(stream)
        barrier()
        ms_e2e = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    cache.check_status()
    bytes_e2e = sum(step_bytes([L + (first_e2e + i) % WINDOW for L in case.lens]) for i in range(K))
    h2d, d2h = in_d.numel(), res_h.numel()

    # ---------------- combine ranks: max time, summed work -----------------
    (ms_total, ms_e2e, attn_ms_max), (bytes_all, bytes_e2e_all, tokens_all) = reduce_over_ranks(
        [ms_total, ms_e2e, attn_ms], [bytes_timed, bytes_e2e, float(B * K)], device, world)

    if rank == 0:
        peak, peak_src = measured_peak()
        headline = (args.batch, args.len_lo, args.len_hi) == (BATCH, LEN_LO, LEN_HI)
        achieved = attn_bytes / (attn_ms * 1e-3) / 1e9
        line = {
            "metric": "paged_decode_attn_kv_gbps", "value": bytes_all / (ms_total * 1e-3) / 1e9, "unit": "GB/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_total / K, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "config 2: bf16 paged decode, batch 64 per GPU, 16 q heads / 8 kv heads, "
                                   "head_dim 128, page 128, context uniform [1024,8192], 65536-page pool, "
                                   "1 append + 1 decode attention per sequence per step",
                       "batch_per_gpu": B, "layers": 1, "l2": "inputs larger than L2 (about 1.2 GB of KV read per step)",
                       "seed": 2002},
            "decode_tokens_per_s": tokens_all / (ms_total * 1e-3),
            "pct_of_nominal_hbm_8000": 100.0 * bytes_all / world / (ms_total * 1e-3) / 1e9 / 8000.0,
            "e2e": {"value": bytes_e2e_all / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / K,
                    "decode_tokens_per_s": tokens_all / (ms_e2e * 1e-3)},
            "gpu_launches": 3 * K,                       # per rank and step: append, decode attention, its finish kernel
            "roofline": {"bound": "hbm", "kernel": "decode_tma_kernel + decode_tma_finish_kernel (one decode-attention call), timed alone",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_src, "traffic": NCU_TRAFFIC_BYTES if headline else None,
                         "bytes_per_launch": attn_bytes,
                         "ms_per_launch": attn_ms},
            "clocks": clocks,
        }
        if world == 1 and not args.kernels_only:
            line["cpu_baseline"] = cpu_baseline_sample()
        if args.pool_pages != N_PAGES:
            line["config"]["pool_pages"] = args.pool_pages
        if (args.batch, args.len_lo, args.len_hi) != (BATCH, LEN_LO, LEN_HI):      # not the headline workload
            line["config"]["workload"] = (f"variant: bf16 paged decode, batch {args.batch} per GPU, 16 q heads / 8 kv "
                                          f"heads, head_dim 128, page 128, context uniform [{args.len_lo},{args.len_hi}]")
            line["config"]["batch_per_gpu"] = args.batch
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------- CPU arm
def build_cpu_workload(n_seq):
    """The same workload shape on the CPU oracle, on a pool compacted to the
    pages in use (the full 32 GiB pool is not needed to time the path)."""
    from fpkv import workloads as wl
    from oracle import paged_kv_oracle as orc
    case = wl.config2_case(B=BATCH, n_pages=N_PAGES, len_lo=LEN_LO, len_hi=LEN_HI, seed=2002)
    lens = case.lens[:n_seq]
    n_pages = sum((L + 1 + 64 + P - 1) // P for L in lens) + 1
    o = orc.OraclePagedKVCache(n_pages, P, n_seq + 1, HKV, D, 1, torch.bfloat16)
    perm = torch.randperm(n_pages - 1, generator=torch.Generator().manual_seed(1)) + 1
    o.free_pages = perm.tolist()
    slots = []
    for L in lens:
        s = o.allocate(); o.reserve(s, L + 1 + 64); slots.append(s)
    g = torch.Generator().manual_seed(2)
    o.kv_cache.copy_((torch.randn((1, 1, 1, 1, n_pages * P, D), generator=g) * D ** -0.5).to(torch.bfloat16)
                     .expand(o.kv_shape))
    q = (torch.randn((n_seq, HQ, 1, D), generator=g) * D ** -0.5).to(torch.bfloat16)
    k = (torch.randn((n_seq, HKV, 1, D), generator=g) * D ** -0.5).to(torch.bfloat16)
    v = (torch.randn((n_seq, HKV, 1, D), generator=g) * D ** -0.5).to(torch.bfloat16)
    return o, slots, lens, q, k, v


def time_cpu_path(steps, warmup, n_seq=BATCH, budget_s=25.0):
    from oracle import paged_kv_oracle as orc
    o, slots, lens, q, k, v = build_cpu_workload(n_seq)
    bidx = torch.tensor(slots)
    times, nbytes = [], []
    t_start = time.perf_counter()
    for i in range(warmup + steps):
        pos = torch.tensor([L + i for L in lens], dtype=torch.int32)
        t0 = time.perf_counter()
        o.append_decode(0, bidx, pos, k, v)
        orc.decode_attention(o, 0, q, bidx, pos)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt); nbytes.append(step_bytes([L + i for L in lens]))
        if i >= warmup and time.perf_counter() - t_start > budget_s:
            break
    total = sum(times)
    return {"gbps": sum(nbytes) / total / 1e9, "ms_per_step": 1e3 * total / len(times), "steps": len(times),
            "tokens_per_s": n_seq * len(times) / total, "cores": torch.get_num_threads(), "n_seq": n_seq}


def cpu_baseline_sample():
    r = time_cpu_path(steps=5, warmup=1)
    return {"value": r["gbps"], "unit": "GB/s", "cores": r["cores"], "kind": "port",
            "sample": f"{r['steps']} steps of all {r['n_seq']} sequences on a compacted pool, "
                      f"{r['ms_per_step']:.0f} ms per step, host has {os.cpu_count()} logical cores"}


def run_reference(args):
    """The reference project is Python on torch FlexAttention; its checkout is
    not present on the benchmark machine, so this arm times the CPU port of its
    path (oracle/) with all host threads torch uses."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1; this arm is meant to use the host cores it can get
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    r = time_cpu_path(steps=args.steps, warmup=min(args.warmup, 2), budget_s=120.0)
    line = {
        "impl": "reference", "metric": "paged_decode_attn_kv_gbps", "value": r["gbps"], "unit": "GB/s",
        "n_gpus": world, "steps": r["steps"], "warmup": min(args.warmup, 2), "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, fp32 math",
        "data": "synthetic",
        "config": {"workload": "config 2: bf16 paged decode, batch 64, 16 q heads / 8 kv heads, head_dim 128, "
                               "page 128, context uniform [1024,8192], pool compacted to the pages in use, "
                               "1 append + 1 decode attention per sequence per step", "seed": 2002},
        "decode_tokens_per_s": r["tokens_per_s"],
        "cpu_baseline": {"value": r["gbps"], "unit": "GB/s", "cores": r["cores"], "kind": "port",
                         "sample": f"{r['steps']} steps of all {r['n_seq']} sequences, "
                                   f"host has {os.cpu_count()} logical cores"},
        "e2e": {"value": r["gbps"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_prefill(args):
    """Secondary workload (config 3's prefill part): 8 sequences of 1024 image-patch tokens + 64 text
    tokens, packed with 128-alignment (9216 rows), bf16, 16 q heads / 8 kv heads, head_dim 128.  One step =
    packed append of the row's K/V into pages + paged prefill attention under the image-prefix mask.
    Tensor-core bound: the metric is TFLOP/s over 4 * Hq * D * (allowed query-key pairs)."""
    from fpkv import workloads as wl
    from fpkv.paged_attention import PagedKVCache, paged_attention
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path for the product"
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    K, W = args.steps, args.warmup
    case = wl.config3_prefill_case()
    cache = PagedKVCache(256, P, 16, HKV, D, 1, torch.bfloat16, device)
    slots = []
    for toks in case.seq_tokens:
        s = cache.allocate(); slots.append(s); cache.reserve(s, None, len(toks))
    bidx, ipos = case.batch_idx_for(slots).to(device), case.input_pos.to(device)
    q, k, v = case.q.to(device), case.k.to(device), case.v.to(device)
    mask = cache.create_prefill_blockmask(bidx, case.input_ids.to(device), wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    ext = mask.extent(ipos)
    pairs = int(ext.to(torch.int64).sum().item())          # every row sees a prefix of extent[t] keys
    flops = 4.0 * HQ * D * pairs
    stream = torch.cuda.current_stream(device)

    def step():
        cache.insert_kv(0, k, v, input_pos=ipos, batch_idx=bidx)
        return paged_attention(q, cache, 0, bidx, ipos, mask)
    for _ in range(W):
        step()
    torch.cuda.synchronize(device)
    sampler = ClockSampler(device.index); sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(K):
        step()
    e1.record(stream)
    torch.cuda.synchronize(device)
    ms_step = e0.elapsed_time(e1) / K
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record(stream)
    for _ in range(K):
        paged_attention(q, cache, 0, bidx, ipos, mask)
    a1.record(stream)
    torch.cuda.synchronize(device)
    ms_attn = a0.elapsed_time(a1) / K
    # the fused norm + rotary embedding + append step on the same packed row (reported beside the headline)
    gen = torch.Generator(device="cpu").manual_seed(3004)
    L = q.shape[2]
    qkv = (torch.randn(1, L, (HQ + 2 * HKV) * D, generator=gen) * 1.7).to(torch.bfloat16).to(device)
    ang = torch.randn(1, L, D // 4, generator=gen).to(device)
    fc = torch.polar(torch.ones_like(ang), ang)
    for _ in range(3):
        cache.pre_attention_append(0, qkv, HQ, HKV, fc, None, bidx, ipos)
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record(stream)
    for _ in range(min(K, 200)):
        cache.pre_attention_append(0, qkv, HQ, HKV, fc, None, bidx, ipos)
    p1.record(stream)
    torch.cuda.synchronize(device)
    ms_pre = p0.elapsed_time(p1) / min(K, 200)
    pre_bytes = L * ((HQ + 2 * HKV) * D * 2 + HQ * D * 2 + 2 * HKV * D * 2 + (D // 4) * 8)
    clocks = sampler.stop()
    cache.check_status()
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, src = float(json.load(f)["bf16_tflops"]), "measured (burst)"
    except Exception:
        peak, src = 1590.0, "fallback"
    tf = flops / (ms_attn * 1e-3) / 1e12
    print(json.dumps({
        "metric": "paged_prefill_attn_tflops", "value": flops / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "config 3 (prefill part): 8 x (1024 image + 64 text tokens) packed to 9216 rows, "
                               "16 q heads / 8 kv heads, head_dim 128, page 128, image-prefix mask; "
                               "packed append + paged prefill attention", "allowed_pairs": pairs, "seed": 3003},
        "gpu_launches": 2 * K,
        "roofline": {"bound": "tensor", "kernel": "prefill_tc_kernel, timed alone", "achieved": tf, "peak": peak,
                     "unit": "TFLOP/s", "frac": tf / peak, "peak_source": src, "traffic": None,
                     "flops_per_launch": flops, "ms_per_launch": ms_attn},
        "pre_append": {"what": "fused per-head norm + 1-D rotary embedding + K/V append of the same packed row "
                               "(includes the wrapper's table repacking)", "ms": ms_pre,
                       "algorithmic_bytes": pre_bytes, "gbps": pre_bytes / (ms_pre * 1e-3) / 1e9},
        "clocks": clocks}), flush=True)


def run_stack(args):
    """Secondary workload (config 5): decode steps of a 28-layer random-init dense GQA decoder stack (hidden 2048,
    16 q heads / 8 kv heads, head_dim 128, gated squared-ReLU FFN of 6144, bf16) over 64 sequences per GPU with
    context uniform in [2048, 8192]; every layer does append + paged attention through fpkv, the projections and
    the FFN are torch GEMMs (library code, not part of the path under test).  The whole step is replayed from a
    CUDA graph.  Metric: decode tokens/s of the whole job (512 sequences at 8 GPUs, 64 per GPU: weak scaling)."""
    import torch.distributed as dist
    import torch.nn.functional as F
    from fpkv import workloads as wl
    from fpkv.paged_attention import PagedKVCache
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path for the product"
    torch.cuda.set_device(local); device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    NL, HID, FFN, B = 28, 2048, 6144, BATCH
    K, W = min(args.steps, 256), args.warmup
    case = rank_case(rank, B, 4352, 2048, 8192, seed=5005)
    cache = PagedKVCache(4352, P, B + 1, HKV, D, NL, torch.bfloat16, device)      # 61 GB of pool per GPU
    cache.free_pages = list(case.free_pages)
    slots = []
    for L in case.lens:
        s = cache.allocate(); slots.append(s); cache.reserve(s, None, L + 1 + WINDOW)
    cache.kv_cache.normal_(0, D ** -0.5)
    g = torch.Generator(device=device).manual_seed(5005 + rank)
    w = lambda *shape: (torch.randn(shape, device=device, generator=g) * 0.02).to(torch.bfloat16)
    layers = [dict(qkv=w(HID, (HQ + 2 * HKV) * D), wo=w(HQ * D, HID), up=w(HID, 2 * FFN), down=w(FFN, HID))
              for _ in range(NL)]
    bidx = torch.tensor(slots, dtype=torch.int64, device=device)
    pos = torch.tensor(case.lens, dtype=torch.int32, device=device)
    x0 = torch.randn((B, HID), device=device, generator=g).to(torch.bfloat16)
    attn_out = torch.empty((B, HQ, 1, D), dtype=torch.bfloat16, device=device)
    lse = torch.empty((B, HQ, 1), dtype=torch.float32, device=device)

    def step(x, attention_only=False):
        for li, lw in enumerate(layers):
            if attention_only:
                qkv = x_qkv
            else:
                qkv = F.rms_norm(x, (HID,)) @ lw["qkv"]
            q = qkv[:, :HQ * D].view(B, 1, HQ, D).permute(0, 2, 1, 3)
            k = qkv[:, HQ * D:(HQ + HKV) * D].view(B, 1, HKV, D).permute(0, 2, 1, 3)
            v = qkv[:, (HQ + HKV) * D:].view(B, 1, HKV, D).permute(0, 2, 1, 3)
            cache.decode_step(li, q, k, v, bidx, pos, out=attn_out, lse=lse)
            if attention_only:
                continue
            x = x + attn_out.view(B, HQ * D) @ lw["wo"]
            gu = F.rms_norm(x, (HID,)) @ lw["up"]
            x = x + (F.relu(gu[:, :FFN]).square() * gu[:, FFN:]) @ lw["down"]
        return x
    x_qkv = (torch.randn((B, (HQ + 2 * HKV) * D), device=device, generator=g) * D ** -0.5).to(torch.bfloat16)

    def timed(attention_only):
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            step(x0, attention_only)
        side.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=side):
            y = step(x0, attention_only)
        for _ in range(W):
            gr.replay()
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(K):
            pos.add_(1 if (i % WINDOW) != WINDOW - 1 else -(WINDOW - 1))     # positions advance and wrap (device op)
            gr.replay()
        e1.record()
        torch.cuda.synchronize(device)
        pos.copy_(torch.tensor(case.lens, dtype=torch.int32))
        return e0.elapsed_time(e1) / K
    ms_full = timed(False)
    ms_attn = timed(True)
    cache.check_status()
    kv_bytes = float(NL * sum((L + WINDOW // 2) * 2 * HKV * D * 2 for L in case.lens))
    (ms_full, ms_attn), (tokens, kvb) = reduce_over_ranks([ms_full, ms_attn], [float(B), kv_bytes], device, world)
    if rank == 0:
        print(json.dumps({
            "metric": "stack_decode_tokens_per_s", "value": tokens / (ms_full * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_full, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "config 5: 28-layer random-init dense GQA decoder stack, hidden 2048, 16 q / 8 kv "
                                   "heads, head_dim 128, FFN 6144, 64 sequences per GPU, context uniform [2048,8192]; "
                                   "append + paged attention per layer through fpkv, projections/FFN torch GEMMs, "
                                   "CUDA-graph replay", "seed": 5005},
            "attention_only": {"tokens_per_s": tokens / (ms_attn * 1e-3), "ms_per_step": ms_attn,
                               "kv_gbps": kvb / (ms_attn * 1e-3) / 1e9,
                               "pct_of_nominal_hbm_8000": 100.0 * kvb / world / (ms_attn * 1e-3) / 1e9 / 8000.0},
            "gpu_launches": 3 * NL * K}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="fpkv", choices=["fpkv", "reference"])
    ap.add_argument("--pool-pages", type=int, default=N_PAGES,
                    help="pages in the pool (default 65536 = 32 GiB; profiling captures use a small pool)")
    ap.add_argument("--batch", type=int, default=BATCH, help="sequences per GPU (default 64: the headline workload)")
    ap.add_argument("--len-lo", type=int, default=LEN_LO)
    ap.add_argument("--len-hi", type=int, default=LEN_HI)
    ap.add_argument("--kernels-only", action="store_true",
                    help="run only the device-resident loop (no host-buffer loop, no CPU baseline): for profilers")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "stack"],
                    help="decode = config 2 (the headline metric); prefill = config 3's prefill part (tensor-bound); "
                         "stack = config 5's 28-layer decoder stack (decode tokens/s)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "stack":
        run_stack(args)
    else:
        run_fpkv(args)


if __name__ == "__main__":
    main()
