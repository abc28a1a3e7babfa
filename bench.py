"""Benchmark of the paged KV-cache hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl fpkv|reference] [--only PART]
    python bench.py --impl engine --engine-cache reference|expanded|split|compact     (opt-in, for context)

Headline workload (one "step" = one decode step of one layer over the whole
batch): bf16, batch 64 per GPU, 16 query heads over 8 stored heads, head_dim
128, page 128, context lengths uniform in [1024, 8192], page ids permuted over
a 65 536-page pool (32 GiB), values N(0,1)/sqrt(128); every step appends one
token per sequence and runs one paged decode attention, then positions advance
by one.  Inputs are synthetic and seeded; nothing is read from disk or network.

  value      algorithmic KV GB/s of the whole job: bytes the step must move
             (K/V of every visible key once, the appended rows, q, out, lse)
             divided by the device time of K steps, summed over GPUs, with the
             step inputs already resident in HBM.  The K-step region is timed
             several times (`blocks`) and the median block is reported.
  e2e        the same through the public Python API with the step's inputs
             (q, k, v, slots, positions) copied from pinned host memory and
             out / lse written to pinned host memory every step, the host
             waiting for each step's result.
  roofline   the decode-attention call alone (its two launches) against the
             measured HBM copy bandwidth.
  cpu_baseline / --impl reference
             the reference project's own CPU path (its PagedKVCache on "cpu",
             its decode mask pipeline and its flex-attention call in eager
             mode), timed on the host cores on a bounded sample; the CPU
             restatement under oracle/ only when the reference is not there.

Beside the headline the line carries one object per further workload, each
with its own roofline: `prefill` (the multimodal prefill of 8 x 1088 tokens:
packed append + tensor-core attention), `mixed_step` (the same prompts
prefilled in 512-row chunks while 56 other sequences decode in the same step),
`long_context` (batch 32 at 16K-32K context with sequences finishing and new
ones admitted into the freed pages every 64 steps) and `stack` (decode
tokens/s of a 28-layer decoder stack, 64 sequences per GPU).

Multi-GPU: one process per GPU (torchrun), each with its own pool and its own
shard of the sequences (weak scaling); no collective on the data path, NCCL is
used only for the timing barrier and to combine the per-rank numbers.
"""

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

_impl = next((sys.argv[i + 1] for i, a in enumerate(sys.argv[:-1]) if a == "--impl"),
             next((a.split("=", 1)[1] for a in sys.argv if a.startswith("--impl=")), "fpkv"))
if _impl == "reference":                            # the reference's compiled handles must run eagerly on the CPU;
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")   # the switch is read when torch is imported

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "falcon-perception_b200"), os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

HQ, HKV, D, P = 16, 8, 128, 128
BATCH = 64
LEN_LO, LEN_HI = 1024, 8192
N_PAGES = 65536
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TFLOPS = 1590.0
WINDOW = 64          # positions cycle through L .. L+63
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_tma_kernel launch on the headline workload, from an
# ncu capture of this program (one launch, small pool)
NCU_TRAFFIC_BYTES = 1.1731e9
WORKLOAD = ("config 2: bf16 paged decode, batch 64 per GPU, 16 q heads / 8 kv heads, head_dim 128, page 128, "
            "context uniform [1024,8192], 1 append + 1 decode attention per sequence per step")


def step_bytes(lens_before_append):
    """Algorithmic bytes of one step: K and V of every visible key (context +
    the appended token) once, the appended K/V rows read and written, q read,
    out written, lse written.  bf16."""
    s = 2
    B = len(lens_before_append)
    kv = sum((L + 1) * 2 * HKV * D * s for L in lens_before_append)
    return kv + 2 * B * 2 * HKV * D * s + 2 * B * HQ * D * s + 4 * B * HQ


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, FALLBACK_TFLOPS, "fallback"


def median(xs):
    v = sorted(xs)
    return v[len(v) // 2] if len(v) % 2 else 0.5 * (v[len(v) // 2 - 1] + v[len(v) // 2])


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


def reduce_over_ranks(times_ms, work, device, world):
    """Whole-job numbers from per-rank ones: a time is the MAX over ranks (the job ends when the slowest
    rank does), work (bytes, tokens, flops) is the SUM.  The only communication of the benchmark."""
    import torch.distributed as dist
    t = torch.tensor(times_ms, dtype=torch.float64, device=device)
    w = torch.tensor(work, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(w, op=dist.ReduceOp.SUM)
    return t.tolist(), w.tolist()


class Ranks:
    """One process per GPU, launched by torchrun; rank, device, the timing barrier and the report reduction."""

    def __init__(self):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path for the product"
        torch.cuda.set_device(self.local)
        self.device = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.device)

    def barrier(self):
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize(self.device)

    def reduce(self, times_ms, work):
        return reduce_over_ranks(times_ms, work, self.device, self.world)

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def timed_blocks(rk, stream, n_blocks, n_steps, step_fn, first_step):
    """n_blocks regions of exactly n_steps steps each, every region bracketed by barrier + synchronize on both
    sides and timed with CUDA events on the launching stream.  Returns the per-block times in ms."""
    out, step = [], first_step
    for _ in range(n_blocks):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        rk.barrier()
        e0.record(stream)
        for _ in range(n_steps):
            step_fn(step); step += 1
        e1.record(stream)
        rk.barrier()
        out.append(e0.elapsed_time(e1))
    return out, step


def time_loop(rk, stream, n, fn, warm=3):
    """Average device time of fn over n back-to-back calls after `warm` untimed ones (ms)."""
    for _ in range(warm):
        fn()
    rk.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(n):
        fn()
    e1.record(stream)
    rk.barrier()
    return e0.elapsed_time(e1) / n


def rank_case(rank, batch=BATCH, n_pages=N_PAGES, len_lo=LEN_LO, len_hi=LEN_HI, seed=2002):
    """The shard of the job that rank ``rank`` owns.  Weak scaling: every rank gets the same amount of work
    -- the seeded context lengths of the single-GPU workload -- in its own pool, with its own page
    permutation (so the page tables differ from rank to rank); rank 0 alone is the single-GPU workload."""
    import numpy as np
    import workloads as wl
    case = wl.config2_case(B=batch, n_pages=n_pages, len_lo=len_lo, len_hi=len_hi, seed=seed)
    if rank:
        case.free_pages = (np.random.default_rng(seed + 7919 * rank).permutation(n_pages - 1) + 1).tolist()
    return case


def build_gpu_workload(rank, device, n_steps, n_pages=N_PAGES, batch=BATCH, len_lo=LEN_LO, len_hi=LEN_HI, seed=2002):
    """Cache with the seeded sequences whose context pages hold random values."""
    from fpkv.paged_attention import PagedKVCache
    case = rank_case(rank, batch, n_pages, len_lo, len_hi, seed)
    cache = PagedKVCache(n_pages, P, batch + 9, HKV, D, 1, torch.bfloat16, device)
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


# ------------------------------------------------------------------ headline
def bench_decode(rk, args):
    """Config 2: the headline numbers (value, e2e, roofline of the attention call)."""
    device, rank = rk.device, rk.rank
    K, W = args.steps, args.warmup
    R = max(1, min(10, math.ceil(200 / K)))            # short regions are repeated and the median block is reported
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

    def block_bytes(first):
        return [float(sum(step_bytes([L + (first + r * K + i) % WINDOW for L in case.lens]) for i in range(K)))
                for r in range(R)]

    # ---------------- device-resident timing -------------------------------
    # One step = the fused public call (append, then attention whose set-up overlaps the append).
    def step_resident(i):
        cache.decode_step(0, q_d[i % NV], k_d[i % NV], v_d[i % NV], bidx, pos_d[i % WINDOW], out=out, lse=lse)

    step = 0
    for _ in range(W):
        step_resident(step); step += 1
    first_timed = step
    ms_blocks, step = timed_blocks(rk, stream, R, K, step_resident, step)
    cache.check_status()
    bytes_blocks = block_bytes(first_timed)

    # The decode-attention call alone (main kernel + its finish kernel), same positions as the timed
    # steps, K launches back to back between one pair of events on the launching stream: the average
    # launch duration is the roofline's denominator.  (Events between the launches would serialise what
    # the kernels overlap on their own, so they bracket the loop, not each launch.)
    def step_attn(i):
        cache.decode_attention(0, q_d[i % NV], bidx, pos_d[i % WINDOW], out=out, lse=lse)
    attn_blocks, _ = timed_blocks(rk, stream, R, K, step_attn, first_timed)
    append_bytes = 2 * B * 2 * HKV * D * 2
    attn_rates = [(b - K * append_bytes) / (t * 1e-3) / 1e9 for b, t in zip(bytes_blocks, attn_blocks)]
    mid = sorted(range(R), key=lambda r: attn_rates[r])[R // 2]
    attn_ms, attn_bytes = attn_blocks[mid] / K, bytes_blocks[mid] / K - append_bytes

    # ---------------- end to end through the public API, host buffers ------
    # One pinned staging buffer per direction: the step's q, k, v, positions and slots travel in one
    # host-to-device copy; out and lse are pinned host memory that the kernels write directly (the device
    # can address pinned memory), so the step's result is on the host when the stream is idle.
    nq, nk = B * HQ * D * 2, B * HKV * D * 2
    in_bytes = (nq + 2 * nk + B * 4 + B * 8 + 15) // 16 * 16           # rows of the staging array stay 16-byte aligned
    e2e_blocks, bytes_e2e = [float("nan")] * R, [0.0] * R
    h2d = d2h = 0
    if not args.kernels_only:
        in_h = torch.empty((NV, in_bytes), dtype=torch.uint8).pin_memory()
        in_d = torch.empty(in_bytes, dtype=torch.uint8, device=device)
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
        for _ in range(W):
            step_e2e(step); step += 1
        first_e2e = step
        e2e_blocks, step = timed_blocks(rk, stream, R, K, step_e2e, step)
        bytes_e2e = block_bytes(first_e2e)
        h2d, d2h = in_d.numel(), res_h.numel()
        del graphs
    cache.check_status()
    del cache
    torch.cuda.empty_cache()

    # ---------------- combine ranks: max time, summed work, block by block --
    t_all, w_all = rk.reduce(ms_blocks + e2e_blocks + [attn_ms], bytes_blocks + bytes_e2e + [float(B)])
    ms_b, e2e_b, attn_ms_max = t_all[:R], t_all[R:2 * R], t_all[2 * R]
    by_b, bye_b, rows_all = w_all[:R], w_all[R:2 * R], w_all[2 * R]
    rate = [b / (t * 1e-3) / 1e9 for b, t in zip(by_b, ms_b)]
    m = sorted(range(R), key=lambda r: rate[r])[R // 2]
    if args.kernels_only:
        e2e = None
    else:
        rate_e = [b / (t * 1e-3) / 1e9 for b, t in zip(bye_b, e2e_b)]
        me = sorted(range(R), key=lambda r: rate_e[r])[R // 2]
        e2e = {"value": rate_e[me], "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_b[me] / K, "decode_tokens_per_s": rows_all * K / (e2e_b[me] * 1e-3),
               "blocks_gbps": [round(x, 1) for x in rate_e]}
    peak, _, peak_src = measured_peaks()
    achieved = attn_bytes / (attn_ms * 1e-3) / 1e9
    headline = (args.batch, args.len_lo, args.len_hi) == (BATCH, LEN_LO, LEN_HI)
    line = {
        "metric": "paged_decode_attn_kv_gbps", "value": rate[m], "unit": "GB/s",
        "n_gpus": rk.world, "steps": K, "warmup": W, "ms_per_step": ms_b[m] / K, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "pool": f"{args.pool_pages}-page pool ({args.pool_pages * P * HKV * D * 4 >> 30} GiB), page ids permuted over it",
                   "batch_per_gpu": B, "layers": 1, "l2": "inputs larger than L2 (about 1.2 GB of KV read per step)",
                   "seed": 2002},
        "blocks": {"n": R, "steps_each": K, "reported": "median block",
                   "gbps": [round(x, 1) for x in rate], "ms_per_step": [round(t / K, 5) for t in ms_b]},
        "decode_tokens_per_s": rows_all * K / (ms_b[m] * 1e-3),
        "pct_of_nominal_hbm_8000": 100.0 * rate[m] / rk.world / 8000.0,
        "e2e": e2e,
        "gpu_launches": 3 * K,                       # per rank and K-step region: append, decode attention, its finish kernel
        "roofline": {"bound": "hbm", "kernel": "decode_tma_kernel + decode_tma_finish_kernel (one decode-attention call), timed alone",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_src, "traffic": NCU_TRAFFIC_BYTES if headline else None,
                     "traffic_source": "ncu capture of one launch of this program on a small pool; not observed by this run",
                     "bytes_per_launch": attn_bytes, "ms_per_launch": attn_ms, "ms_per_launch_max_over_ranks": attn_ms_max},
    }
    if not headline:
        line["config"]["workload"] = (f"variant: bf16 paged decode, batch {args.batch} per GPU, 16 q heads / 8 kv "
                                      f"heads, head_dim 128, page 128, context uniform [{args.len_lo},{args.len_hi}]")
    return line


# ------------------------------------------------------------------ prefill
def prefill_inputs(device, n_seq=8):
    import workloads as wl
    case = wl.config3_prefill_case(n_seq=n_seq)
    return case, case.input_pos.to(device), case.q.to(device), case.k.to(device), case.v.to(device)


def bench_prefill(rk, args, n=100):
    """Config 3's prefill part: 8 sequences of 1024 image-patch tokens + 64 text tokens, packed with 128-alignment
    (9216 rows).  One step = packed append of the row's K/V into pages + paged prefill attention under the
    image-prefix mask.  Tensor-core bound: TFLOP/s over 4 * Hq * D * (allowed query-key pairs)."""
    import workloads as wl
    from fpkv.paged_attention import PagedKVCache, paged_attention
    device = rk.device
    stream = torch.cuda.current_stream(device)
    case, ipos, q, k, v = prefill_inputs(device)
    cache = PagedKVCache(256, P, 16, HKV, D, 1, torch.bfloat16, device)
    slots = []
    for toks in case.seq_tokens:
        s = cache.allocate(); slots.append(s); cache.reserve(s, None, len(toks))
    bidx = case.batch_idx_for(slots).to(device)
    mask = cache.create_prefill_blockmask(bidx, case.input_ids.to(device), wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    ext = mask.extent(ipos)
    pairs = int(ext.to(torch.int64).sum().item())          # every row sees a prefix of extent[t] keys
    flops = 4.0 * HQ * D * pairs

    def both():
        cache.insert_kv(0, k, v, input_pos=ipos, batch_idx=bidx)
        paged_attention(q, cache, 0, bidx, ipos, mask)
    ms_step = time_loop(rk, stream, n, both)
    ms_attn = time_loop(rk, stream, n, lambda: paged_attention(q, cache, 0, bidx, ipos, mask))
    ms_append = time_loop(rk, stream, n, lambda: cache.insert_kv(0, k, v, input_pos=ipos, batch_idx=bidx))
    # the fused norm + rotary embedding + append step on the same packed row
    gen = torch.Generator(device="cpu").manual_seed(3004)
    L = q.shape[2]
    qkv = (torch.randn(1, L, (HQ + 2 * HKV) * D, generator=gen) * 1.7).to(torch.bfloat16).to(device)
    ang = torch.randn(1, L, D // 4, generator=gen).to(device)
    fc = torch.polar(torch.ones_like(ang), ang)
    ms_pre = time_loop(rk, stream, n, lambda: cache.pre_attention_append(0, qkv, HQ, HKV, fc, None, bidx, ipos))
    pre_bytes = L * ((HQ + 2 * HKV) * D * 2 + HQ * D * 2 + 2 * HKV * D * 2 + (D // 4) * 8)
    append_bytes = int((bidx > 0).sum().item()) * 2 * HKV * D * 2 * 2        # live rows read and written
    cache.check_status()
    # one long causal prompt: the per-tile set-up is amortised over many key tiles
    T16 = 16384
    lcache = PagedKVCache(T16 // P + 2, P, 3, HKV, D, 1, torch.bfloat16, device)
    ls = lcache.allocate(); lcache.reserve(ls, None, T16)
    lb = torch.full((1, T16), ls, dtype=torch.int64, device=device); lp = torch.arange(T16, device=device).view(1, -1)
    g = torch.Generator(device=device).manual_seed(16)
    lq, lk, lv = ((torch.randn((1, h, T16, D), device=device, generator=g) * D ** -0.5).bfloat16() for h in (HQ, HKV, HKV))
    lmask = lcache.create_prefill_blockmask(lb, torch.full((1, T16), wl.TEXT_ID, device=device), wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    lcache.insert_kv(0, lk, lv, input_pos=lp, batch_idx=lb)
    ms_long = time_loop(rk, stream, 20, lambda: paged_attention(lq, lcache, 0, lb, lp, lmask))
    flops_long = 4.0 * HQ * D * (T16 * (T16 + 1) / 2)
    lcache.check_status()
    del cache, lcache
    torch.cuda.empty_cache()
    (ms_step, ms_attn, ms_append, ms_pre, ms_long), (fl, fl_long) = rk.reduce(
        [ms_step, ms_attn, ms_append, ms_pre, ms_long], [flops, flops_long])
    _, peak, src = measured_peaks()
    tf = flops / (ms_attn * 1e-3) / 1e12               # per GPU: the slowest rank's launch time
    tf_long = flops_long / (ms_long * 1e-3) / 1e12
    return {
        "metric": "paged_prefill_attn_tflops", "value": fl / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": n,
        "ms_per_step": ms_step,
        "workload": "config 3, prefill part: 8 x (1024 image + 64 text tokens) per GPU packed to 9216 rows, 16 q heads / "
                    "8 kv heads, head_dim 128, page 128, image-prefix mask; packed append + paged prefill attention",
        "allowed_pairs": pairs,
        "roofline": {"bound": "tensor", "kernel": "prefill_tc_kernel, timed alone (slowest GPU)", "achieved": tf, "peak": peak,
                     "unit": "TFLOP/s", "frac": tf / peak, "peak_source": src + " (burst)", "traffic": None,
                     "flops_per_launch": flops, "ms_per_launch": ms_attn},
        "packed_append": {"ms": ms_append, "algorithmic_bytes": append_bytes, "gbps": append_bytes / (ms_append * 1e-3) / 1e9},
        "pre_append": {"what": "fused per-head norm + 1-D rotary embedding + K/V append of the same packed row "
                               "(includes the wrapper's table repacking)", "ms": ms_pre,
                       "algorithmic_bytes": pre_bytes, "gbps": pre_bytes / (ms_pre * 1e-3) / 1e9},
        "causal_16k": {"what": "one 16384-token causal prompt per GPU, attention alone", "ms": ms_long,
                       "tflops": tf_long, "frac": tf_long / peak},
    }


# --------------------------------------------------------------- mixed step
def bench_mixed(rk, args, rounds=30):
    """Config 3 as written: 8 prompts of 1088 tokens are prefilled in 512-row chunks (K/V into pages first, as
    the bidirectional image span needs) while 56 other sequences with 1K-8K context decode in the same step.
    A prompt takes three steps (query rows 0-511, 512-1023, 1024-1087 of every prompt); each step also appends
    one token to, and attends for, the 56 decoders.  Prefill work goes to a second stream, the step ends when
    both streams are done.  The three steps of a round are timed together."""
    import workloads as wl
    from fpkv.attention import PrefillMask
    device = rk.device
    main = torch.cuda.current_stream(device)
    side = torch.cuda.Stream(device)
    case, ipos, q, k, v = prefill_inputs(device)
    # the decoders share the pool with the prompts, as they would in the engine
    Bd = 56
    dcase, cache, dslots = build_gpu_workload(rk.rank, device, WINDOW, 4096, Bd, LEN_LO, LEN_HI, seed=3003)
    pslots = []
    for toks in case.seq_tokens:
        s = cache.allocate(); pslots.append(s); cache.reserve(s, None, len(toks))
    bidx = case.batch_idx_for(pslots).to(device)
    mask = cache.create_prefill_blockmask(bidx, case.input_ids.to(device), wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    ext = mask.extent(ipos)
    chunks = []
    for c0 in (0, 512, 1024):                              # rows [c0, c0 + 512) of every prompt, gathered into one packed row
        # (the last chunk takes the prompt's 64 pad rows along: a 128-row tile holds rows of one prompt only)
        idx = torch.cat([torch.arange(off + c0, off + min(c0 + 512, (len(t) + 127) // 128 * 128), device=device)
                         for off, t in zip(case.offsets, case.seq_tokens)])
        assert idx.numel() % 128 == 0
        m = PrefillMask(mask.doc_id[idx], mask.img_id[idx]); m._extent = ext[idx].contiguous()
        chunks.append((q[:, :, idx].contiguous(), bidx[:, idx].contiguous(), ipos[:, idx].contiguous(), m))
    dbi = torch.tensor(dslots, dtype=torch.int64, device=device)
    dlens = torch.tensor(dcase.lens, dtype=torch.int32)
    pos_d = (dlens.view(1, Bd) + torch.arange(WINDOW, dtype=torch.int32).view(-1, 1)).to(device)
    g = torch.Generator(device=device).manual_seed(33 + rk.rank)
    dq, dk, dv = ((torch.randn((Bd, h, 1, D), device=device, generator=g) * D ** -0.5).bfloat16() for h in (HQ, HKV, HKV))
    dout = torch.empty((Bd, HQ, 1, D), dtype=torch.bfloat16, device=device)
    dlse = torch.empty((Bd, HQ, 1), dtype=torch.float32, device=device)
    done = torch.cuda.Event()
    cache.flush_tables()

    def prefill_part(ci):
        if ci == 0:
            cache.insert_kv(0, k, v, input_pos=ipos, batch_idx=bidx)
        cq, cb, cp, cm = chunks[ci]
        cache.prefill_attention(0, cq, cb, cp, cm)

    def decode_part(i):
        cache.decode_step(0, dq, dk, dv, dbi, pos_d[i % WINDOW], out=dout, lse=dlse)
    counter = [0]

    def mixed_round(two_streams):
        r = counter[0]; counter[0] += 1
        for ci in range(3):
            if two_streams:
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    prefill_part(ci)
                    done.record(side)
                decode_part(3 * r + ci)
                main.wait_event(done)
            else:
                prefill_part(ci)
                decode_part(3 * r + ci)

    def decode_round():
        r = counter[0]; counter[0] += 1
        for ci in range(3):
            decode_part(3 * r + ci)
    ms_mixed = time_loop(rk, main, rounds, lambda: mixed_round(True))
    ms_serial = time_loop(rk, main, rounds, lambda: mixed_round(False))
    ms_prefill = time_loop(rk, main, rounds, lambda: [prefill_part(ci) for ci in range(3)])
    ms_decode = time_loop(rk, main, rounds, decode_round)
    cache.check_status()
    pairs = int(ext.to(torch.int64).sum().item())
    flops = 4.0 * HQ * D * pairs
    dbytes = float(sum(step_bytes([L + WINDOW // 2 for L in dcase.lens]) for _ in range(3)))
    del cache
    torch.cuda.empty_cache()
    (ms_mixed, ms_serial, ms_prefill, ms_decode), (fl, by) = rk.reduce([ms_mixed, ms_serial, ms_prefill, ms_decode], [flops, dbytes])
    hbm, tfl, src = measured_peaks()
    # time the round would need if each part ran alone at its own roofline, one after the other
    floor_ms = (flops / (tfl * 1e12) + dbytes / (hbm * 1e9)) * 1e3
    return {
        "metric": "mixed_step_ms", "value": ms_mixed / 3, "unit": "ms per step (a third of a three-step round)",
        "rounds": rounds, "higher_is_better": False, "ms_per_step": ms_mixed / 3,
        "workload": "config 3: 8 prompts of 1024 image + 64 text tokens per GPU prefilled in 512-row chunks "
                    "(three steps per prompt, K/V appended to pages in the first) while 56 sequences with context "
                    "uniform [1024,8192] decode in the same step",
        "round_ms": {"two_streams": ms_mixed, "one_stream": ms_serial, "prefill_parts_alone": ms_prefill,
                     "decode_parts_alone": ms_decode},
        "prefill_tflops_in_step": fl / (ms_mixed * 1e-3) / 1e12, "decode_gbps_in_step": by / (ms_mixed * 1e-3) / 1e9,
        "decode_tokens_per_s": 3 * Bd * rk.world / (ms_mixed * 1e-3),
        "roofline": {"bound": "tensor + hbm", "kernel": "prefill_tc_kernel and decode_tma_kernel in one step",
                     "achieved": floor_ms / ms_mixed, "peak": 1.0, "unit": "(flops / tensor peak + bytes / hbm peak) / measured time",
                     "frac": floor_ms / ms_mixed, "peak_source": src, "traffic": None,
                     "flops_per_round": flops, "bytes_per_round": dbytes, "floor_ms": floor_ms},
    }


# ------------------------------------------------------------- long context
def time_alloc_launch(device, n_pages=10240, B=32):
    """Device time (us) of the allocator launch of one admission at config 4's size -- 8 sequences of about
    190 pages erased, 8 slots allocated and given 17 pages each -- as the 24 records the cache queues for it,
    and as the same table edits spelled out entry by entry (16 full-row clears, 136 single-entry maps), which is
    what had to be uploaded and applied before the free stacks lived on the device."""
    import ctypes
    from fpkv import _lib
    from fpkv.paged_attention import PagedKVCache
    stream = torch.cuda.current_stream(device)
    c = PagedKVCache(n_pages, P, B + 1, 1, 64, 1, torch.bfloat16, device)      # only its tables and stacks are used
    slots = []
    for _ in range(B):
        s = c.allocate(); slots.append(s); c.reserve(s, None, 190 * P)
    c.flush_tables()
    state = (c._page_table, c._physical_to_logical, c._free_pages_dev, c._free_slots_dev, c._alloc_counts)
    snap = [t.clone() for t in state]
    gone = slots[::4]
    for s in gone:
        c.erase(s)
    new = []
    for _ in gone:
        s = c.allocate(); c.reserve(s, None, 17 * P); new.append(s)
    records = list(c._pending)
    c._pending = []                                        # applied by hand below, several times
    entries = [(_lib.OP_CLEAR, s, 0, 0) for s in gone + new]
    entries += [(_lib.OP_MAP, s, j, pg) for s in new for j, pg in enumerate(c.page_table_cpu[s])]

    def launch(recs):
        ops = torch.tensor(recs, dtype=torch.int32, device=device)
        ts = []
        for _ in range(7):
            for dst, src in zip(state, snap):
                dst.copy_(src)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            _lib.check(_lib.lib.fpkv_alloc_step(ctypes.byref(c._pool), ctypes.byref(c._alloc), ops.data_ptr(), len(recs),
                                                c._status.data_ptr(), stream.cuda_stream), "fpkv_alloc_step")
            b.record(stream)
            torch.cuda.synchronize(device)
            ts.append(a.elapsed_time(b) * 1e3)
        return median(ts)
    us_records, us_entries = launch(records), launch(entries)
    c.check_status()
    return {"records": len(records), "records_us": us_records, "entry_edits": len(entries), "entry_edits_us": us_entries,
            "what": "one allocator launch for an admission of 8 sequences (8 erases of 190 pages, 8 allocates, 8 reserves of 17 "
                    "pages) as queued records, and as the same table edits entry by entry (16 row clears + 136 maps)"}


def bench_long_context(rk, args, steps=256, period=64):
    """Config 4's shape: batch 32, context uniform [16384, 32768], a 10 240-page pool; every `period` steps a seeded
    quarter of the sequences finishes, is erased, and new 2048-token sequences are admitted (packed append) into
    the freed pages, so the page tables become non-contiguous.  The whole loop is timed, host bookkeeping,
    allocator launches and admissions included."""
    import numpy as np
    from fpkv.paged_attention import PagedKVCache
    device = rk.device
    stream = torch.cuda.current_stream(device)
    B, n_pages, NEW = 32, 10240, 2048
    rng = np.random.default_rng(4004 + rk.rank)
    cache = PagedKVCache(n_pages, P, B + 1, HKV, D, 1, torch.bfloat16, device)
    cache.free_pages = (rng.permutation(n_pages - 1) + 1).tolist()
    lens = rng.integers(16384, 32769, size=B).tolist()
    slots = []
    for L in lens:
        s = cache.allocate(); slots.append(s); cache.reserve(s, None, L + 1)
    cache.kv_cache.normal_(0, D ** -0.5)
    g = torch.Generator(device=device).manual_seed(44 + rk.rank)
    NV = 4
    q, k, v = ((torch.randn((NV, B, h, 1, D), device=device, generator=g) * D ** -0.5).bfloat16() for h in (HQ, HKV, HKV))
    ak, av = ((torch.randn((1, HKV, NEW, D), device=device, generator=g) * D ** -0.5).bfloat16() for _ in range(2))
    apos = torch.arange(NEW, device=device).view(1, -1)
    aslot = torch.empty((1, NEW), dtype=torch.int64, device=device)
    out = torch.empty((B, HQ, 1, D), dtype=torch.bfloat16, device=device)
    lse = torch.empty((B, HQ, 1), dtype=torch.float32, device=device)
    # slots and positions of a step travel through two pinned buffers used in turn
    idx_h = [torch.empty(3 * B, dtype=torch.int32).pin_memory() for _ in range(2)]
    idx_d = [torch.empty(3 * B, dtype=torch.int32, device=device) for _ in range(2)]
    idx_ev = [torch.cuda.Event(), torch.cuda.Event()]

    def churn():
        gone = rng.permutation(B)[:B // 4].tolist()
        for i in gone:
            cache.erase(slots[i])
        for i in gone:
            s = cache.allocate(); cache.reserve(s, None, NEW + 1)
            slots[i], lens[i] = s, NEW
        for i in gone:
            aslot.fill_(slots[i])
            cache.insert_kv(0, ak, av, input_pos=apos, batch_idx=aslot)
        return len(gone)

    def one_step(i):
        for j, s in enumerate(slots):                     # grow by a page when the next token needs one
            cache.reserve(s, None, lens[j] + 1)
        t = i & 1
        idx_ev[t].synchronize()                           # the copy that last read this pinned buffer
        h = idx_h[t].numpy()
        h[:2 * B].view(np.int64)[:] = slots; h[2 * B:] = lens
        idx_d[t].copy_(idx_h[t], non_blocking=True)
        idx_ev[t].record(stream)
        cache.decode_step(0, q[i % NV], k[i % NV], v[i % NV], idx_d[t][:2 * B].view(torch.int64), idx_d[t][2 * B:], out=out, lse=lse)
        for j in range(B):
            lens[j] += 1
    for i in range(3):
        one_step(i)
    rk.barrier()
    nbytes, admitted, t_churn = 0.0, 0, []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        if i and i % period == 0:
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0.record(stream)
            admitted += churn()
            c1.record(stream)
            t_churn.append((c0, c1))
        nbytes += step_bytes(lens)
        one_step(i)
    e1.record(stream)
    rk.barrier()
    ms_total = e0.elapsed_time(e1)
    churn_ms = [a.elapsed_time(b) for a, b in t_churn]
    cache.check_status()
    nbytes += admitted * NEW * 2 * HKV * D * 2 * 2         # admitted K/V rows read and written
    del cache
    torch.cuda.empty_cache()
    alloc = time_alloc_launch(device) if rk.rank == 0 else None
    (ms_total, churn_max), (by, toks) = rk.reduce([ms_total, max(churn_ms) if churn_ms else 0.0], [nbytes, float(B * steps)])
    peak, _, src = measured_peaks()
    gbps = by / (ms_total * 1e-3) / 1e9
    return {
        "metric": "long_context_decode_kv_gbps", "value": gbps, "unit": "GB/s", "steps": steps, "ms_per_step": ms_total / steps,
        "workload": f"config 4: batch 32 per GPU, context uniform [16384,32768], 10240-page pool, {steps} decode steps; every "
                    f"{period} steps 8 sequences are erased and 8 new 2048-token sequences admitted into the freed pages; "
                    "host bookkeeping, allocator launches and admissions inside the timed region",
        "decode_tokens_per_s": toks / (ms_total * 1e-3), "pct_of_nominal_hbm_8000": 100.0 * gbps / rk.world / 8000.0,
        "admission_ms": {"each": [round(x, 3) for x in churn_ms], "max_over_ranks": churn_max,
                         "what": "device time of one admission: allocator launch + 8 packed appends of 2048 tokens"},
        "alloc_launch": alloc,
        "roofline": {"bound": "hbm", "kernel": "decode_tma_kernel inside the whole loop (host work included)",
                     "achieved": gbps / rk.world, "peak": peak, "unit": "GB/s", "frac": gbps / rk.world / peak,
                     "peak_source": src, "traffic": None},
    }


# -------------------------------------------------------------------- stack
def bench_stack(rk, args, steps=64):
    """Config 5: decode steps of a 28-layer random-init dense GQA decoder stack (hidden 2048, 16 q heads / 8 kv
    heads, head_dim 128, gated squared-ReLU FFN of 6144, bf16) over 64 sequences per GPU with context uniform in
    [2048, 8192]; every layer does append + paged attention through fpkv, the projections and the FFN are torch
    GEMMs (library code, not part of the path under test).  The whole step is replayed from a CUDA graph.
    Decode tokens/s of the whole job (512 sequences at 8 GPUs, 64 per GPU: weak scaling)."""
    import torch.nn.functional as F
    from fpkv.paged_attention import PagedKVCache
    device, rank = rk.device, rk.rank
    NL, HID, FFN, B = 28, 2048, 6144, BATCH
    K, W = steps, 3
    case = rank_case(rank, B, 4352, 2048, 8192, seed=5005)
    cache = PagedKVCache(4352, P, B + 1, HKV, D, NL, torch.bfloat16, device)      # 61 GB of pool per GPU
    cache.free_pages = list(case.free_pages)
    slots = []
    for L in case.lens:
        s = cache.allocate(); slots.append(s); cache.reserve(s, None, L + 1 + WINDOW)
    cache.kv_cache.normal_(0, D ** -0.5)
    cache.flush_tables()
    g = torch.Generator(device=device).manual_seed(5005 + rank)
    w = lambda *shape: (torch.randn(shape, device=device, generator=g) * 0.02).to(torch.bfloat16)
    layers = [dict(qkv=w(HID, (HQ + 2 * HKV) * D), wo=w(HQ * D, HID), up=w(HID, 2 * FFN), down=w(FFN, HID))
              for _ in range(NL)]
    bidx = torch.tensor(slots, dtype=torch.int64, device=device)
    pos = torch.tensor(case.lens, dtype=torch.int32, device=device)
    x0 = torch.randn((B, HID), device=device, generator=g).to(torch.bfloat16)
    attn_out = torch.empty((B, HQ, 1, D), dtype=torch.bfloat16, device=device)
    lse = torch.empty((B, HQ, 1), dtype=torch.float32, device=device)
    x_qkv = (torch.randn((B, (HQ + 2 * HKV) * D), device=device, generator=g) * D ** -0.5).to(torch.bfloat16)

    def step(x, attention_only=False):
        for li, lw in enumerate(layers):
            qkv = x_qkv if attention_only else F.rms_norm(x, (HID,)) @ lw["qkv"]
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

    def timed(attention_only):
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            step(x0, attention_only)
        side.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=side):
            step(x0, attention_only)
        for _ in range(W):
            gr.replay()
        rk.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(K):
            pos.add_(1 if (i % WINDOW) != WINDOW - 1 else -(WINDOW - 1))     # positions advance and wrap (device op)
            gr.replay()
        e1.record()
        rk.barrier()
        pos.copy_(torch.tensor(case.lens, dtype=torch.int32))
        ms = e0.elapsed_time(e1) / K
        del gr
        return ms
    ms_full = timed(False)
    ms_attn = timed(True)
    cache.check_status()
    kv_bytes = float(NL * sum((L + WINDOW // 2) * 2 * HKV * D * 2 for L in case.lens))
    del cache, layers
    torch.cuda.empty_cache()
    (ms_full, ms_attn), (tokens, kvb) = rk.reduce([ms_full, ms_attn], [float(B), kv_bytes])
    peak, _, src = measured_peaks()
    rate = kvb / rk.world / (ms_attn * 1e-3) / 1e9
    return {
        "metric": "stack_decode_tokens_per_s", "value": tokens / (ms_full * 1e-3), "unit": "tokens/s", "steps": K,
        "ms_per_step": ms_full,
        "workload": "config 5: 28-layer random-init dense GQA decoder stack, hidden 2048, 16 q / 8 kv heads, head_dim 128, "
                    "FFN 6144, 64 sequences per GPU, context uniform [2048,8192]; append + paged attention per layer "
                    "through fpkv, projections/FFN torch GEMMs, CUDA-graph replay",
        "attention_only": {"tokens_per_s": tokens / (ms_attn * 1e-3), "ms_per_step": ms_attn,
                           "kv_gbps": kvb / (ms_attn * 1e-3) / 1e9, "pct_of_nominal_hbm_8000": 100.0 * rate / 8000.0},
        "gpu_launches": 3 * NL * K,
        "roofline": {"bound": "hbm", "kernel": "append + decode attention of all 28 layers (attention-only step)",
                     "achieved": rate, "peak": peak, "unit": "GB/s", "frac": rate / peak, "peak_source": src, "traffic": None},
    }


def bench_split_layout(rk, args, n_pages=4096):
    """Config 2's decode step over a split pool (first half of K and V once per KV head, second half of K once per
    query head): the layout that is exact under per-query-head 2-D rotary, at 5/8 of the bytes of the expanded
    cache the reference keeps for that case.  Reports the step, the attention call alone, and its rate on the bytes
    the split layout holds (640 B per key and KV group at these head counts)."""
    from fpkv.paged_attention import PagedKVCache
    device, rank = rk.device, rk.rank
    stream = torch.cuda.current_stream(device)
    B, K = BATCH, 20
    case = rank_case(rank, B, n_pages, LEN_LO, LEN_HI, 2002)
    cache = PagedKVCache(n_pages, P, B + 9, HKV, D, 1, torch.bfloat16, device, split_q_heads=HQ)
    cache.free_pages = list(case.free_pages)
    slots = []
    for L in case.lens:
        s = cache.allocate(); slots.append(s); cache.reserve(s, None, L + 1 + WINDOW)
    cache.kv_cache.normal_(0, D ** -0.5)
    g = torch.Generator(device=device).manual_seed(55 + rank)
    NV = 4
    q, k, v = ((torch.randn((NV, B, HQ, 1, D), device=device, generator=g) * D ** -0.5).bfloat16() for _ in range(3))
    bidx = torch.tensor(slots, dtype=torch.int64, device=device)
    pos = (torch.tensor(case.lens, dtype=torch.int32).view(1, B) + torch.arange(WINDOW, dtype=torch.int32).view(-1, 1)).to(device)
    out = torch.empty((B, HQ, 1, D), dtype=torch.bfloat16, device=device)
    lse = torch.empty((B, HQ, 1), dtype=torch.float32, device=device)

    def step(i):
        cache.decode_step(0, q[i % NV], k[i % NV], v[i % NV], bidx, pos[i % WINDOW], out=out, lse=lse)

    def attn(i):
        cache.decode_attention(0, q[i % NV], bidx, pos[i % WINDOW], out=out, lse=lse)
    for i in range(5):
        step(i)
    R = 10
    step_blocks, _ = timed_blocks(rk, stream, R, K, step, 5)
    attn_blocks, _ = timed_blocks(rk, stream, R, K, attn, 5)
    cache.check_status()
    del cache
    torch.cuda.empty_cache()
    # config 3's packed prefill row on a split pool: single-head items in the tensor-core kernel
    import workloads as wl
    from fpkv.paged_attention import paged_attention
    pcase, pipos, pq, pk, pv = prefill_inputs(device)
    pcache = PagedKVCache(256, P, 16, HKV, D, 1, torch.bfloat16, device, split_q_heads=HQ)
    pslots = []
    for toks in pcase.seq_tokens:
        s = pcache.allocate(); pslots.append(s); pcache.reserve(s, None, len(toks))
    pbidx = pcase.batch_idx_for(pslots).to(device)
    pmask = pcache.create_prefill_blockmask(pbidx, pcase.input_ids.to(device), wl.IMG_CLS_ID, wl.END_OF_IMG_ID)
    pairs = int(pmask.extent(pipos).to(torch.int64).sum().item())
    n_rep = HQ // HKV
    pcache.insert_kv(0, pk.repeat_interleave(n_rep, 1).contiguous(), pv.repeat_interleave(n_rep, 1).contiguous(),
                     input_pos=pipos, batch_idx=pbidx)
    ms_prefill = time_loop(rk, stream, 50, lambda: paged_attention(pq, pcache, 0, pbidx, pipos, pmask))
    pcache.check_status()
    del pcache
    torch.cuda.empty_cache()
    per_key = (HKV * (D // 2) + HQ * (D // 2) + HKV * D) * 2          # bytes of one key position in the split layout
    keys = [sum(L + 1 + (5 + r * K + i) % WINDOW for L in case.lens for i in range(K)) for r in range(R)]
    rates = [kk * per_key / (t * 1e-3) / 1e9 for kk, t in zip(keys, attn_blocks)]
    mid = sorted(range(R), key=lambda r: rates[r])[R // 2]
    hbm_peak, _, which = measured_peaks()
    (t_attn, t_step, ms_prefill), (work,) = rk.reduce([attn_blocks[mid], step_blocks[mid], ms_prefill], [float(keys[mid] * per_key)])
    gbs = work / (t_attn * 1e-3) / 1e9
    return {"workload": "config 2's decode step on a split pool (16 q heads / 8 kv heads, head_dim 128, page 128, "
                        f"batch {B}, context uniform [{LEN_LO},{LEN_HI}], pool {n_pages} pages)",
            "metric": "split_layout_decode_attention_bandwidth", "value": round(gbs, 1), "unit": "GB/s",
            "bytes_per_key_and_kv_group": per_key // HKV, "expanded_cache_bytes_per_key_and_kv_group": 2 * (HQ // HKV) * D * 2,
            "attn_ms": round(t_attn / K, 4), "step_ms": round(t_step / K, 4), "steps": K, "blocks": R,
            "roofline": {"bound": "hbm", "kernel": "decode_tma_kernel (split instantiation) + decode_tma_finish_kernel, timed alone",
                         "achieved": round(gbs, 1), "peak": hbm_peak * rk.world, "unit": "GB/s",
                         "frac": round(gbs / (hbm_peak * rk.world), 3), "peak_source": which,
                         "traffic": 1.4807e9, "traffic_source": "ncu capture of one launch of this workload; not observed by this run",
                         "bytes_per_launch": work / K / rk.world, "ms_per_launch": round(t_attn / K, 4)},
            "expanded_equivalent_gbs": round(gbs * (2 * HQ * D * 2) / per_key, 1),
            "prefill_config3_row": {"ms": round(ms_prefill, 4), "tflops_per_gpu": round(4.0 * HQ * D * pairs / (ms_prefill * 1e-3) / 1e12, 1),
                                    "what": "paged prefill attention of config 3's packed row over the split pool (single-head items)"},
            "gpu_launches_per_step": 3}


PARTS = {"prefill": bench_prefill, "mixed_step": bench_mixed, "long_context": bench_long_context, "stack": bench_stack,
         "split_layout": bench_split_layout}


def run_fpkv(args):
    from fpkv import _lib
    rk = Ranks()
    sampler = ClockSampler(rk.local)
    if rk.rank == 0:
        sampler.start()
    line = None
    if args.only in ("all", "decode"):
        line = bench_decode(rk, args)
    extras = {}
    if not args.kernels_only:
        for name, fn in PARTS.items():
            if args.only in ("all", name):
                t0 = time.perf_counter()
                try:
                    extras[name] = fn(rk, args)
                except torch.cuda.OutOfMemoryError as e:      # a smaller GPU: say so instead of losing the headline
                    extras[name] = {"unavailable": "out of device memory: " + str(e).split("\n")[0]}
                    torch.cuda.empty_cache()
                extras[name]["wall_s"] = round(time.perf_counter() - t0, 1)
    clocks = sampler.stop() if rk.rank == 0 else None
    if rk.rank == 0:
        if line is None:                                    # one of the further workloads on its own
            name, line = next(iter(extras.items()))
            line = dict(line)
            line.update({"n_gpus": rk.world, "warmup": 3, "higher_is_better": line.get("higher_is_better", True),
                         "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic"})
            line["config"] = {"workload": line.pop("workload", name)}
        else:
            line.update(extras)
        line["clocks"] = clocks
        line["build_id"] = _lib.build_id()
        if rk.world == 1 and not args.kernels_only and args.only == "all":
            line["cpu_baseline"] = cpu_baseline_sample()
            line["gpu_competitor"] = gpu_competitor_sample()
        print(json.dumps(line), flush=True)
    rk.close()


# ---------------------------------------------------------------- CPU arm
def reference_root():
    """Where the reference project can be imported from: the offline install under baseline/_ref, or a checkout
    named by FALCON_PERCEPTION_SRC.  None when neither is there."""
    for cand in (os.path.join(ROOT, "baseline", "_ref"), os.environ.get("FALCON_PERCEPTION_SRC", "")):
        if cand and os.path.isdir(os.path.join(cand, "falcon_perception")):
            return cand
    return None


SAMPLE_SEQS = 4


def time_reference_cpu(steps, warmup, budget_s):
    """The reference's own decode path on the host cores: its PagedKVCache on "cpu" (16 expanded heads, as it
    stores them), its per-step mask slicing and logical-to-physical conversion, and its flex-attention call,
    eager.  Its attention scores every row against every token of the pool, so time and memory grow with
    batch x pool: the sample is the first SAMPLE_SEQS of the 64 seeded sequences in a pool holding just their
    pages (the full batch asks for a 180 GB temporary).  Bytes are counted as for the GPU arm (8 real KV heads)."""
    import types
    import workloads as wl
    sys.path.insert(0, reference_root())
    stub = types.ModuleType("pycocotools"); stub.mask = types.ModuleType("pycocotools.mask")   # post-processing only
    sys.modules.setdefault("pycocotools", stub); sys.modules.setdefault("pycocotools.mask", stub.mask)
    from torch.nn.attention.flex_attention import AuxRequest
    from falcon_perception.attention import compiled_flex_attn_decode
    from falcon_perception.paged_attention import PagedKVCache as RefCache
    from falcon_perception.paged_inference import PagedInferenceEngine
    case = wl.config2_case(B=BATCH, n_pages=N_PAGES, len_lo=LEN_LO, len_hi=LEN_HI, seed=2002)
    lens = case.lens[:SAMPLE_SEQS]
    n = len(lens)
    n_pages = sum((L + 1 + WINDOW + P - 1) // P for L in lens) + 1
    c = RefCache(n_pages, P, n + 1, HQ, D, 1, torch.bfloat16, "cpu")
    c.free_pages = (torch.randperm(n_pages - 1, generator=torch.Generator().manual_seed(1)) + 1).tolist()
    slots = []
    for L in lens:
        s = c.allocate(); c.reserve(s, torch.tensor([s]), L + 1 + WINDOW); slots.append(s)
    g = torch.Generator().manual_seed(2)
    c.kv_cache.copy_((torch.randn((1, 1, 1, 1, n_pages * P, D), generator=g) * D ** -0.5).to(torch.bfloat16).expand(c.kv_shape))
    q = (torch.randn((n, HQ, 1, D), generator=g) * D ** -0.5).to(torch.bfloat16)
    k = (torch.randn((n, HKV, 1, D), generator=g) * D ** -0.5).to(torch.bfloat16).repeat_interleave(HQ // HKV, dim=1)
    v = (torch.randn((n, HKV, 1, D), generator=g) * D ** -0.5).to(torch.bfloat16).repeat_interleave(HQ // HKV, dim=1)
    engine = types.SimpleNamespace(block_mask=c.create_causal_blockmask(B=n + 1, L=(LEN_HI // P + 2) * P))
    bidx = torch.tensor(slots)
    times, nbytes = [], []
    t_start = time.perf_counter()
    for i in range(warmup + steps):
        pos = torch.tensor([L + i % WINDOW for L in lens], dtype=torch.int32)
        t0 = time.perf_counter()
        mask = PagedInferenceEngine.get_decoding_block_mask(engine, bidx, pos)          # paged_inference.py:783-826
        mask = c.convert_logical_block_mask(mask, bidx)                                  # paged_attention.py:234-301
        xk, xv = c.insert_kv(0, k, v, input_pos=pos.view(-1, 1), batch_idx=bidx)         # paged_attention.py:184-232
        compiled_flex_attn_decode(q, xk, xv, block_mask=mask, return_aux=AuxRequest(lse=True))   # model.py:156-162
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt); nbytes.append(step_bytes([L + i % WINDOW for L in lens]))
            if time.perf_counter() - t_start > budget_s:
                break
    total = sum(times)
    return {"gbps": sum(nbytes) / total / 1e9, "ms_per_step": 1e3 * total / len(times), "steps": len(times),
            "tokens_per_s": n * len(times) / total, "cores": torch.get_num_threads(), "n_seq": n, "kind": "reference",
            "sample": f"{len(times)} steps of the first {n} of the 64 seeded sequences through the reference's own CPU path "
                      f"(PagedKVCache on cpu with 16 expanded heads, mask slicing + conversion, eager flex attention) in a "
                      f"pool of their {n_pages} pages; its cost grows with batch x pool, so the full batch would be slower "
                      f"per byte; host has {os.cpu_count()} logical cores"}


def time_port_cpu(steps, warmup, budget_s, n_seq=BATCH):
    """The CPU restatement (oracle/) of the same step on all 64 sequences, pool compacted to the pages in use."""
    import workloads as wl
    from oracle import paged_kv_oracle as orc
    case = wl.config2_case(B=BATCH, n_pages=N_PAGES, len_lo=LEN_LO, len_hi=LEN_HI, seed=2002)
    lens = case.lens[:n_seq]
    n_pages = sum((L + 1 + WINDOW + P - 1) // P for L in lens) + 1
    o = orc.OraclePagedKVCache(n_pages, P, n_seq + 1, HKV, D, 1, torch.bfloat16)
    o.free_pages = (torch.randperm(n_pages - 1, generator=torch.Generator().manual_seed(1)) + 1).tolist()
    slots = []
    for L in lens:
        s = o.allocate(); o.reserve(s, L + 1 + WINDOW); slots.append(s)
    g = torch.Generator().manual_seed(2)
    o.kv_cache.copy_((torch.randn((1, 1, 1, 1, n_pages * P, D), generator=g) * D ** -0.5).to(torch.bfloat16).expand(o.kv_shape))
    q = (torch.randn((n_seq, HQ, 1, D), generator=g) * D ** -0.5).to(torch.bfloat16)
    k = (torch.randn((n_seq, HKV, 1, D), generator=g) * D ** -0.5).to(torch.bfloat16)
    v = (torch.randn((n_seq, HKV, 1, D), generator=g) * D ** -0.5).to(torch.bfloat16)
    bidx = torch.tensor(slots)
    times, nbytes = [], []
    t_start = time.perf_counter()
    for i in range(warmup + steps):
        pos = torch.tensor([L + i % WINDOW for L in lens], dtype=torch.int32)
        t0 = time.perf_counter()
        o.append_decode(0, bidx, pos, k, v)
        orc.decode_attention(o, 0, q, bidx, pos)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt); nbytes.append(step_bytes([L + i % WINDOW for L in lens]))
            if time.perf_counter() - t_start > budget_s:
                break
    total = sum(times)
    return {"gbps": sum(nbytes) / total / 1e9, "ms_per_step": 1e3 * total / len(times), "steps": len(times),
            "tokens_per_s": n_seq * len(times) / total, "cores": torch.get_num_threads(), "n_seq": n_seq, "kind": "port",
            "sample": f"{len(times)} steps of all {n_seq} sequences through the CPU restatement of the path (oracle/), pool "
                      f"compacted to the pages in use; host has {os.cpu_count()} logical cores"}


def cpu_baseline_sample():
    """The CPU arm on a bounded sample, in its own process (it needs torch imported with dynamo off and all host
    threads, neither of which this process should change)."""
    try:
        env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "OMP_NUM_THREADS")}
        res = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", "5", "--warmup", "3"],
                             capture_output=True, text=True, timeout=300, env=env)
        ref = json.loads(res.stdout.strip().splitlines()[-1])
        out = dict(ref["cpu_baseline"])
        if "cpu_port" in ref:
            out["port"] = ref["cpu_port"]
        return out
    except Exception as e:
        return {"value": None, "unit": "GB/s", "cores": None, "kind": "reference", "sample": "failed: " + repr(e)[:200]}


def gpu_competitor_sample():
    """The reference's own GPU path on this box, in its own process (it compiles FlexAttention with
    torch.compile; a failure or a slow first compile must not take the benchmark down)."""
    try:
        env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "TORCHDYNAMO_DISABLE")}
        res = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-gpu", "--steps", "50", "--warmup", "3"],
                             capture_output=True, text=True, timeout=300, env=env)
        return json.loads(res.stdout.strip().splitlines()[-1])
    except Exception as e:
        return {"impl": "reference-gpu", "unavailable": repr(e)[:200]}


def run_reference_gpu(args):
    """--impl reference-gpu: the reference's own GPU path for the same step, for context (not the target and not
    the reference arm): its PagedKVCache on the device with 16 expanded heads, its per-step mask slicing and
    conversion, its append and its compiled FlexAttention decode call, on the 64 seeded sequences in a pool
    compacted to the pages in use (the reference's mask conversion allocates batch x n_pages index tensors, and
    its kernel walks them, so the pool size is part of its cost)."""
    import types
    import workloads as wl
    root = reference_root()
    if root is None:
        print(json.dumps({"impl": "reference-gpu", "unavailable": "the reference project is not installed under baseline/_ref"}))
        return
    assert torch.cuda.is_available()
    sys.path.insert(0, root)
    stub = types.ModuleType("pycocotools"); stub.mask = types.ModuleType("pycocotools.mask")
    sys.modules.setdefault("pycocotools", stub); sys.modules.setdefault("pycocotools.mask", stub.mask)
    from torch.nn.attention.flex_attention import AuxRequest
    from falcon_perception.attention import compiled_flex_attn_decode
    from falcon_perception.paged_attention import PagedKVCache as RefCache
    from falcon_perception.paged_inference import PagedInferenceEngine
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    case = wl.config2_case(B=BATCH, n_pages=N_PAGES, len_lo=LEN_LO, len_hi=LEN_HI, seed=2002)
    lens, n = case.lens, BATCH
    n_pages = sum((L + 1 + WINDOW + P - 1) // P for L in lens) + 1
    c = RefCache(n_pages, P, n + 1, HQ, D, 1, torch.bfloat16, device)
    c.free_pages = (torch.randperm(n_pages - 1, generator=torch.Generator().manual_seed(1)) + 1).tolist()
    slots = []
    for L in lens:
        s = c.allocate(); c.reserve(s, torch.tensor([s], device=device), L + 1 + WINDOW); slots.append(s)
    c.kv_cache.normal_(0, D ** -0.5)
    g = torch.Generator(device=device).manual_seed(2)
    q = (torch.randn((n, HQ, 1, D), device=device, generator=g) * D ** -0.5).bfloat16()
    k = (torch.randn((n, HQ, 1, D), device=device, generator=g) * D ** -0.5).bfloat16()
    v = (torch.randn((n, HQ, 1, D), device=device, generator=g) * D ** -0.5).bfloat16()
    engine = types.SimpleNamespace(block_mask=c.create_causal_blockmask(B=n + 1, L=(LEN_HI // P + 2) * P))
    bidx = torch.tensor(slots, device=device)
    pos_all = (torch.tensor(lens, dtype=torch.int32).view(1, n) + torch.arange(WINDOW, dtype=torch.int32).view(-1, 1)).to(device)

    def step(i):
        pos = pos_all[i % WINDOW]
        mask = PagedInferenceEngine.get_decoding_block_mask(engine, bidx, pos)
        mask = c.convert_logical_block_mask(mask, bidx)
        xk, xv = c.insert_kv(0, k, v, input_pos=pos.view(-1, 1), batch_idx=bidx)
        return compiled_flex_attn_decode(q, xk, xv, block_mask=mask, return_aux=AuxRequest(lse=True))
    t0 = time.perf_counter()
    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    compile_s = time.perf_counter() - t0
    K = args.steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / K
    # the same step replayed from a CUDA graph, as the reference engine runs decode (paged_inference.py:865-952)
    ms_graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=side):
            step(0)
        torch.cuda.synchronize()
        e0.record()
        for i in range(K):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        ms_graph = e0.elapsed_time(e1) / K
    except Exception as e:
        ms_graph = "capture failed: " + repr(e)[:120]
    nbytes = sum(step_bytes([L + i % WINDOW for L in lens]) for i in range(K)) / K
    best = ms_graph if isinstance(ms_graph, float) else ms
    print(json.dumps({
        "impl": "reference-gpu", "metric": "paged_decode_attn_kv_gbps", "value": nbytes / (best * 1e-3) / 1e9, "unit": "GB/s",
        "ms_per_step": ms, "ms_per_step_graph_replay": ms_graph, "steps": K, "first_calls_s": round(compile_s, 1),
        "config": {"workload": WORKLOAD, "pool": f"{n_pages}-page pool (compacted to the pages in use), 16 expanded heads"},
        "what": "the reference's own GPU path: mask slicing + conversion, append (PagedKVCache.assign), compiled FlexAttention "
                "decode; bytes counted as for fpkv (8 real KV heads), so the figure is comparable with `value`; it reads "
                "twice those bytes"}), flush=True)


def run_engine(args):
    """--impl engine (opt-in, N = 1, for context): the reference's own PagedInferenceEngine.generate on its
    flagship-sized model (28 layers, 16 / 8 heads, head_dim 128, random weights, bf16) with its own cache and compiled
    FlexAttention, or -- `--engine-cache split` / `compact` -- with fpkv.PagedKVCache substituted (the substitutions
    of tests/test_engine_dropin_gpu.py).  64 requests of 8000 tokens; prefill is timed as a generate() that stops
    after the first token, decode as the difference to one that goes on for 64 more.  One JSON line."""
    import types
    root = reference_root()
    if root is None:
        print(json.dumps({"impl": "engine", "unavailable": "the reference project is not installed under baseline/_ref"}))
        return
    assert torch.cuda.is_available()
    sys.path.insert(0, root)
    stub = types.ModuleType("pycocotools"); stub.mask = types.ModuleType("pycocotools.mask")
    sys.modules.setdefault("pycocotools", stub); sys.modules.setdefault("pycocotools.mask", stub.mask)
    import falcon_perception.model as ref_model
    import falcon_perception.paged_inference as eng_mod
    from falcon_perception import ModelArgs
    which = args.engine_cache
    n_seq, prompt, new = 64, 8000, 64

    class Tok:                                               # what the engine and ModelArgs.update read; requests arrive tokenised
        padding_side = "right"
        pad_token_id, eos_token_id, bos_id = 0, 1, None
        start_of_image_token_id, image_cls_token_id, end_of_image_token_id, image_token_id = 2, 3, 4, 5
        image_row_sep_token_id = 7
        image_reg_1_token_id, image_reg_2_token_id, image_reg_3_token_id, image_reg_4_token_id = 8, 9, 10, 11
        seg_token_id, coord_token_id, size_token_id = 12, 13, 14
    margs = ModelArgs(perception_heads=False, do_segmentation=False, max_seq_len=8192)
    margs.update(Tok())
    torch.manual_seed(1)
    model = ref_model.FalconPerception(margs)
    with torch.no_grad():
        for name, prm in model.named_parameters():
            if prm.dim() >= 2: prm.normal_(0, 0.02)
            elif "norm" in name: prm.fill_(1.0)
            else: prm.zero_()
        for name, buf in model.named_buffers():
            if buf.is_floating_point() and not torch.isfinite(buf).all(): buf.zero_()
    model = model.to(device="cuda", dtype=torch.bfloat16).eval()
    if which != "reference":
        from fpkv.engine_glue import decoding_block_mask, install_attention
        from fpkv.paged_attention import PagedKVCache

        def fpkv_cache(**kw):
            if which == "split": kw = dict(kw, n_heads=margs.n_kv_heads, split_q_heads=margs.n_heads)
            if which == "compact": kw = dict(kw, n_heads=margs.n_kv_heads)
            return PagedKVCache(**kw)
        eng_mod.PagedKVCache = fpkv_cache
        eng_mod.PagedInferenceEngine.get_decoding_block_mask = \
            lambda self, batch_idx, input_pos: decoding_block_mask(self.block_mask, batch_idx, input_pos)
        install_attention(ref_model.Attention, fused=True)
    if args.engine_batched_setup:
        from fpkv.engine_glue import install_decode_setup
        install_decode_setup(eng_mod.PagedInferenceEngine)
    pages = n_seq * ((prompt + new + P - 1) // P + 1) + 8
    t0 = time.perf_counter()
    eng = eng_mod.PagedInferenceEngine(model, Tok(), None, max_batch_size=n_seq + 1, max_seq_length=8192, n_pages=pages,
                                       seed=0, enable_hr_cache=False, capture_cudagraph=True, prefill_length_limit=32768)
    ready_s = time.perf_counter() - t0

    def requests():
        gen = torch.Generator().manual_seed(3)
        out = []
        for i in range(n_seq):
            r = eng_mod.Sequence(text="", image=None, request_idx=i, task="detection")
            r.input_ids = torch.randint(20, 60000, (prompt,), generator=gen)
            r.rope_pos_t = torch.arange(prompt, dtype=torch.long)
            r.rope_pos_hw = torch.zeros(prompt, 2)
            out.append(r)
        return out

    def timed(n_new):
        sp = eng_mod.SamplingParams(max_new_tokens=n_new, stop_token_ids=[1])
        torch.cuda.synchronize(); t = time.perf_counter()
        done = eng.generate(requests(), sampling_params=sp)
        torch.cuda.synchronize()
        return time.perf_counter() - t, done
    timed(2)                                                 # compilation and autotuning of whatever is compiled
    t_pre = min(timed(1)[0] for _ in range(2))
    t_all, done = timed(1 + new)
    finite = all(bool(torch.isfinite(r.output_probs).all()) for r in done)
    print(json.dumps({
        "impl": "engine", "cache": which, "batched_decode_setup": bool(args.engine_batched_setup), "n_gpus": 1, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"the reference's PagedInferenceEngine.generate, 28-layer model (16 q / 8 kv heads, head_dim 128, "
                               f"random weights), {n_seq} requests of {prompt} tokens, {new} decode steps, CUDA graphs"},
        "engine_ready_s": round(ready_s, 1),
        "prefill_ms": round(t_pre * 1e3, 1), "prefill_tokens_per_s": round(n_seq * prompt / t_pre),
        "decode_ms_per_step": round((t_all - t_pre) / new * 1e3, 2), "decode_tokens_per_s": round(n_seq * new / (t_all - t_pre)),
        "outputs_finite": finite, "first_tokens": [int(r.output_ids[0]) for r in done[:4]]}), flush=True)


def run_reference(args):
    """--impl reference: the reference's own CPU implementation of the path on the host cores, same metric and
    workload string as the GPU arm.  Rank 0 alone runs it; its throughput does not depend on how many GPU
    processes were launched beside it (the host cores are the same), so the line says n_gpus 1."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1; this arm is meant to use the host cores it can get
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    extra = {}
    if reference_root() is not None:
        r = time_reference_cpu(args.steps, args.warmup, budget_s=150.0)
        port = time_port_cpu(3, 1, budget_s=20.0)
        extra["cpu_port"] = {"value": port["gbps"], "unit": "GB/s", "kind": "port", "cores": port["cores"], "sample": port["sample"]}
        pool = f"pool holding the {SAMPLE_SEQS} sampled sequences' pages only"
    else:
        r = time_port_cpu(args.steps, args.warmup, budget_s=120.0)
        extra["note"] = "the reference project is not installed under baseline/_ref: timed the CPU restatement (oracle/) instead"
        pool = "pool compacted to the pages in use"
    line = {
        "impl": "reference", "metric": "paged_decode_attn_kv_gbps", "value": r["gbps"], "unit": "GB/s",
        "n_gpus": 1, "launched_world_size": world, "steps": r["steps"], "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, fp32/fp64 math",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "pool": pool, "seed": 2002, "sampled_sequences": r["n_seq"]},
        "decode_tokens_per_s": r["tokens_per_s"],
        "cpu_baseline": {"value": r["gbps"], "unit": "GB/s", "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]},
        "e2e": {"value": r["gbps"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    line.update(extra)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="fpkv", choices=["fpkv", "reference", "reference-gpu", "engine"])
    ap.add_argument("--engine-batched-setup", action="store_true",
                    help="--impl engine: also batch the engine's per-request decode set-up copies (fpkv.engine_glue.install_decode_setup)")
    ap.add_argument("--engine-cache", default="split", choices=["reference", "expanded", "split", "compact"],
                    help="--impl engine: the cache the reference's engine runs on (its own, or fpkv's in one of its layouts)")
    ap.add_argument("--pool-pages", type=int, default=N_PAGES,
                    help="pages in the pool (default 65536 = 32 GiB; profiling captures use a small pool)")
    ap.add_argument("--batch", type=int, default=BATCH, help="sequences per GPU (default 64: the headline workload)")
    ap.add_argument("--len-lo", type=int, default=LEN_LO)
    ap.add_argument("--len-hi", type=int, default=LEN_HI)
    ap.add_argument("--kernels-only", action="store_true",
                    help="device-resident loops only (no host-buffer loop, no further workloads, no CPU baseline): for profilers")
    ap.add_argument("--only", default="all", choices=["all", "decode"] + sorted(PARTS),
                    help="run one part: decode = config 2 (the headline metric), or one of the further workloads")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    elif args.impl == "engine":
        run_engine(args)
    else:
        run_fpkv(args)


if __name__ == "__main__":
    main()
