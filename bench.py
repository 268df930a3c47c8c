#!/usr/bin/env python
"""Benchmark of the decode-attention hot path (one JSON line on stdout, rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c4|c3]

A step is one decode-attention call (one new token per sequence, one decoder layer) over one batch
of synthetic input: by default fp16, batch 16, 32 heads x 128, cached lengths uniform in
[1024, 2048] drawn from seed 1 (the LLaMA-2-7B layer shape the metric is quoted on).  With N > 1
every rank runs its own batch of that shape (independent (batch, head) units, no collective on the
data path: weak scaling) and the value is the sum over ranks divided by the slowest rank's time.

`value`   algorithmic bytes (K and V rows read + appended rows + q/k/v + output; no mask, score or
          table bytes) per second with all inputs resident in HBM; four distinct input sets are
          rotated so no step re-reads what the previous steps left in L2.
`e2e`     the same metric through the public call with HOST inputs: every step copies that step's
          q, k, v from pinned host memory, runs the call, and reads the output back.
`roofline` the decode kernel's bytes per launch over its average duration (CUDA events on the
          launching stream), against the measured copy bandwidth of this pool's B200s.
`cpu_baseline` the scalar host oracle timed on this box's cores on a bounded sample.

`--workload c4` is the 13B-shape batch split over the ranks (strong scaling); `--workload c3` is the
causal prefill (metric TFLOP/s of causal-exact flops, tensor roofline).

`--impl reference` times the reference's own CUDA attention chain (three kernels + two cuBLAS gemv
+ softmax, fp32 cache) built from the reference checkout by oracle/build_ref.sh; the reference has
no CPU implementation of this path.  Its decode gemv arguments are corrected as described in
oracle/ref_runner.cu (as written they are rejected by cuBLAS for L > 128), and since it has one
cached length per call the ragged batch is run as one call per sequence.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

NBUF = 4  # distinct input sets rotated through the timed loop (--sets)

WORKLOADS = {
    # name: (B, H, lo, hi, seed, description)
    "c2": (16, 32, 1024, 2048, 1, "fp16 decode attention, LLaMA-2-7B layer shape: batch 16, 32 heads x 128, cached lengths U[1024,2048], seed 1"),
    "c4": (64, 40, 2048, 4096, 3, "fp16 decode attention, LLaMA-2-13B layer shape: batch 64, 40 heads x 128, cached lengths U[2048,4096], seed 3"),
}
PREFILL_WORKLOADS = ("c3",)


def load_peaks() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.005):
        self.samples: list[tuple[int, int]] = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        self.err = None
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # NVML missing: report it, do not fail the benchmark
            self.nv = None
            self.err = repr(e)
        self.period = period_s

    def _one(self):
        nv = self.nv
        try:
            mhz = int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
            try:
                reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            except Exception:
                reasons = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
            self.samples.append((mhz, reasons))
        except Exception as e:
            self.err = repr(e)

    def _run(self):
        while not self._stop.is_set():
            self._one()
            self._stop.wait(self.period)

    def start(self):
        if self.nv is None:
            return
        self._stop.clear()
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()

    def stop(self):
        if self._thr is not None:
            self._one()
            self._stop.set()
            self._thr.join()
            self._thr = None

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "error": self.err}
        mhz = sorted(s[0] for s in self.samples)
        bits = 0
        for _, r in self.samples:
            bits |= r
        names = {
            0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
            0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
            0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
        }
        reasons = [n for b, n in names.items() if bits & b and n != "gpu_idle"]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(mhz)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


# ------------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local):
    from fasterllama_b200 import attention as A
    from fasterllama_b200 import workloads as W

    from fasterllama_b200 import sharding

    global NBUF
    NBUF = max(1, args.sets)
    B, H, lo, hi, seed, desc = WORKLOADS[args.workload]
    T = hi + 1
    dev = f"cuda:{local}"
    lens = W.draw_lengths(seed, B, lo, hi)  # the same lengths on every rank and in every set
    strong = args.workload == "c4"  # config 4 is quoted as one batch sharded over the GPUs
    if strong:
        sh = sharding.plan(B, H, world, rank)
        if sh.axis == "batch":
            lens = lens[sh.start:sh.stop]
        B, H = sh.batch, sh.heads
    sets = []
    for j in range(NBUF):
        c = W.device_case(f"{args.workload}-{j}", seed + 7919 * j + 104729 * rank, B, H, T, lens, device=dev)
        c.scratch_zeroed = True  # device_case hands over zeroed scratch; the kernel leaves it zeroed
        c.early_start = 0 if args.no_early_start else args.early_start
        # q, k, v as three views of one buffer, so that the end-to-end leg moves them with one host->device copy
        c.arrays["qkv"] = torch.stack([c.arrays[n] for n in ("q", "k", "v")]).contiguous()
        c.arrays["q"], c.arrays["k"], c.arrays["v"] = c.arrays["qkv"][0], c.arrays["qkv"][1], c.arrays["qkv"][2]
        sets.append((c, c.params()))
    bytes_step = sets[0][0].algorithmic_bytes()
    tokens_step = WORKLOADS[args.workload][0] if strong else B * world  # sequences advanced per step, all ranks
    stream = torch.cuda.current_stream()

    # Back-to-back calls with early start level 2 overlap each other's ramp and drain, so partitions no longer
    # have to be small to shorten a call's tail: one partition per (batch, head) unit (no partial results, no merge)
    # is fastest there.  Isolated calls (the single-call and end-to-end legs below) keep the library's default.
    import dataclasses
    chain_split = args.split_len if args.split_len else (2048 if (args.early_start == 2 and not args.no_early_start) else 512)
    chain = [dataclasses.replace(c, split_len=chain_split).params() for c, _ in sets]

    def step(i):
        A.decode(chain[i % NBUF], stream)

    def single(i):
        A.decode(sets[i % NBUF][1], stream)

    for i in range(max(args.warmup, 3)):
        step(i)
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    sampler.start()
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    torch.cuda.synchronize()
    sampler.stop()
    t_dev = e0.elapsed_time(e1) * 1e-3
    barrier(world)
    t = max_over_ranks(t_dev, world)
    for c, _ in sets:
        assert A.scratch_status(c.arrays["scratch"]) == 0, "a decode kernel reported an error status"

    # spread of a single call: 200 launches timed one by one (each between its own pair of events, the stream
    # idle before it), so these include the launch latency that back-to-back calls hide
    singles = []
    es = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(200)]
    for i, (a0, a1) in enumerate(es):
        a0.record(stream)
        single(i)
        a1.record(stream)
        stream.synchronize()
    singles = sorted(a0.elapsed_time(a1) * 1e3 for a0, a1 in es)
    spread = {"p10": round(singles[20], 2), "p50": round(singles[100], 2), "p90": round(singles[180], 2),
              "what": "one call at a time, stream idle before each (us)"}

    # ---- end to end: host q/k/v in, output back on the host, every step --------------------------
    host_in = [c.arrays["qkv"].cpu().pin_memory() for c, _ in sets]
    host_out = torch.empty_like(sets[0][0].arrays["out"], device="cpu").pin_memory()
    h2d = host_in[0].numel() * host_in[0].element_size()
    d2h = host_out.numel() * host_out.element_size()

    # Two ways to take host buffers through the C ABI call.  "mapped": the call is handed the pinned host
    # buffers themselves (pinned memory is device-addressable): the kernel reads this step's q, k, v over PCIe
    # while its first cache tiles are in flight and stores the result rows straight into host memory, so the
    # step is ONE launch and the same bytes cross the bus.  "copies": copy in, launch, copy out.
    mapped_params = []
    if args.e2e_mode == "mapped":
        for j, (c, _) in enumerate(sets):
            a = dict(c.arrays)
            a["q"], a["k"], a["v"] = host_in[j][0], host_in[j][1], host_in[j][2]
            a["out"] = host_out
            mapped_params.append(c.params(a))

    def e2e_step(i):
        c, p = sets[i % NBUF]
        if mapped_params:
            A.decode(mapped_params[i % NBUF], stream)
        else:
            c.arrays["qkv"].copy_(host_in[i % NBUF], non_blocking=True)  # this step's q, k, v: one copy from pinned memory
            A.decode(p, stream)
            host_out.copy_(c.arrays["out"], non_blocking=True)
        stream.synchronize()  # the caller reads the step's result before it issues the next step

    for i in range(max(args.warmup, 3)):
        e2e_step(i)
    barrier(world)
    e0.record(stream)
    for i in range(args.steps):
        e2e_step(i)
    e1.record(stream)
    torch.cuda.synchronize()
    t_e2e = max_over_ranks(e0.elapsed_time(e1) * 1e-3, world)
    barrier(world)
    # what reached the host is what the device-resident leg computed for the same inputs
    last = (args.steps - 1) % NBUF
    assert torch.equal(host_out, sets[last][0].arrays["out"].cpu()), "end-to-end result differs from the device-resident result"

    peak, peak_src = load_peaks()
    total_bytes = sum_over_ranks(float(bytes_step), world)
    value = total_bytes * args.steps / t / 1e9
    e2e_val = total_bytes * args.steps / t_e2e / 1e9
    achieved = bytes_step * args.steps / t_dev / 1e9  # this rank's kernel: one launch per step

    line = {
        "metric": "decode_attn_hbm_gbps", "value": round(value, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(t / args.steps * 1e3, 5), "higher_is_better": True, "scaling": "strong" if strong else "weak",
        "vs_baseline": None, "dtype": "f16 storage, f32 arithmetic", "data": "synthetic",
        "config": {
            "workload": desc, "per_gpu_batch": B, "heads": H, "head_dim": 128, "cache_rows_total": int(lens.sum()),
            "total_len": T, "split_len": chain_split, "split_len_single_call_and_e2e": 512,
            "launch": ("ordinary stream launches" if args.no_early_start else
                       "programmatic dependent launch, level 1: a call's CTAs may become resident and fetch their first cache tiles while the previous call drains; inputs, scratch and outputs are touched only after it has completed"
                       if args.early_start == 1 else
                       "programmatic dependent launch, level 2: a call's CTAs may become resident while the previous call drains and stream the cache against q and k (which, as in the decoder layer, are final before the kernel in front starts); the new token's v, the cache append, scratch and outputs are touched only after the previous call has completed"),
            "l2": f"{NBUF} distinct input sets rotated ({NBUF * bytes_step / 1e6:.0f} MB > 126 MB L2), no flush kernel in the timed region",
            "sharding": ("one batch split over the ranks by contiguous (batch, head) ranges, no collective" if strong
                         else "every rank runs its own batch of this shape (independent (batch, head) units), no collective"),
        },
        "tokens_per_s": round(tokens_step * args.steps / t, 1),
        "pct_of_8TBps": round(100 * value / world / 8000.0, 2),
        "bytes_per_step_per_gpu": bytes_step,
        "gpu_launches": args.steps,
        "single_call_us": spread,
        "e2e": {"value": round(e2e_val, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(t_e2e / args.steps * 1e3, 5), "tokens_per_s": round(tokens_step * args.steps / t_e2e, 1),
                "host_buffers": ("pinned host q/k/v/out handed to the call; the kernel reads and writes them over PCIe, host waits for each step"
                                 if mapped_params else "copy in, launch, copy out; host waits for each step")},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "peak_source": f"{peak_src} (copy bandwidth, MEASURED_PEAKS.json)",
                     "kernel": "flb_decode_attn_kernel<__half,...>", "traffic": DRAM_TRAFFIC_PER_LAUNCH.get(args.workload)},
        "clocks": sampler.summary(),
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(sets[0][0], bytes_step, B)
    if rank == 0:
        print(json.dumps(line), flush=True)


def run_prefill(args, rank, world, local):
    """Config 3: fp16 causal prefill, batch 8, 1024 tokens, 32 heads x 128, seed 2 (every rank its own
    batch).  A step = prologue (dequant/RoPE/transpose/cache append) + tensor-core attention."""
    from fasterllama_b200 import attention as A
    from fasterllama_b200 import workloads as W

    B, H, S = 8, 32, 1024
    dev = f"cuda:{local}"
    g = torch.Generator(device=dev)
    g.manual_seed(2 + rank)
    nbuf = max(1, min(args.sets, 2))
    sets = []
    for j in range(nbuf):
        a = {n: torch.randn((B, S, H, 128), generator=g, device=dev).to(torch.float16) for n in ("q", "k", "v")}
        a["k_cache"] = torch.zeros((B, H, S, 128), device=dev, dtype=torch.float16)
        a["v_cache"] = torch.zeros_like(a["k_cache"])
        a["out"] = torch.zeros((B, H, S, 128), device=dev, dtype=torch.float16)
        a["freq_cis"] = torch.from_numpy(W.freq_cis_table(S)).to(dev)
        a["scratch"] = torch.zeros(A.workspace_bytes(B, H, S, S), dtype=torch.uint8, device=dev)
        c = W.Case(name="c3", B=B, H=H, S=S, T=S, start_pos=0, arrays=a, rope_add_past=True)
        sets.append((c, c.params()))
    stream = torch.cuda.current_stream()
    flops = B * H * 2 * 128 * S * (S + 1)  # causal-exact: two contractions over the visible pairs

    def step(i):
        A.prefill(sets[i % nbuf][1], stream)

    steps = min(args.steps, 500)
    for i in range(max(args.warmup, 3)):
        step(i)
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    sampler.start()
    e0.record(stream)
    for i in range(steps):
        step(i)
    e1.record(stream)
    torch.cuda.synchronize()
    sampler.stop()
    t_dev = e0.elapsed_time(e1) * 1e-3
    t = max_over_ranks(t_dev, world)
    for c, _ in sets:
        assert A.scratch_status(c.arrays["scratch"]) == 0, "a prefill kernel reported an error status"

    host_in = [{n: c.arrays[n].cpu().pin_memory() for n in ("q", "k", "v")} for c, _ in sets]
    host_out = torch.empty_like(sets[0][0].arrays["out"], device="cpu").pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host_in[0].values())
    d2h = host_out.numel() * host_out.element_size()

    def e2e_step(i):
        c, p = sets[i % nbuf]
        for n in ("q", "k", "v"):
            c.arrays[n].copy_(host_in[i % nbuf][n], non_blocking=True)
        A.prefill(p, stream)
        host_out.copy_(c.arrays["out"], non_blocking=True)
        stream.synchronize()

    e2e_steps = min(steps, 50)
    for i in range(2):
        e2e_step(i)
    barrier(world)
    e0.record(stream)
    for i in range(e2e_steps):
        e2e_step(i)
    e1.record(stream)
    torch.cuda.synchronize()
    t_e2e = max_over_ranks(e0.elapsed_time(e1) * 1e-3, world)
    barrier(world)
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
        peak_src = "measured (cuBLAS bf16 burst, MEASURED_PEAKS.json)"
    except Exception:
        peak, peak_src = 1590.0, "fallback"
    value = flops * world * steps / t / 1e12
    achieved = flops * steps / t_dev / 1e12
    line = {
        "metric": "prefill_attn_tflops", "value": round(value, 1), "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(t / steps * 1e3, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 operands, f32 accumulation", "data": "synthetic",
        "config": {"workload": "fp16 causal prefill attention, LLaMA-2-7B layer shape: batch 8, 1024 tokens, 32 heads x 128, RoPE rows 0..1023, seed 2",
                   "flops_per_step": flops, "l2": f"{nbuf} distinct input sets rotated; q/k/v/caches of one set = 0.4 GB > 126 MB L2"},
        "tokens_per_s": round(B * S * world * steps / t, 1),
        "gpu_launches": 2 * steps,
        "e2e": {"value": round(flops * world * e2e_steps / t_e2e / 1e12, 1), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(t_e2e / e2e_steps * 1e3, 5)},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(achieved / peak, 4), "peak_source": peak_src,
                     "kernel": "flb_prefill_prologue_kernel + flb_prefill_attn_kernel<64> (whole step)", "traffic": None},
        "clocks": sampler.summary(),
    }
    if rank == 0:
        print(json.dumps(line), flush=True)


# dram__bytes_read.sum + dram__bytes_write.sum of one decode launch, from the ncu capture summarised
# under profiles/ (None until a capture of that workload exists)
DRAM_TRAFFIC_PER_LAUNCH: dict[str, int | None] = {"c2": 413121536, "c4": 3977282560}  # c4: the c2 capture scaled by the algorithmic bytes


def cpu_baseline(case, bytes_step: int, B: int, min_seconds: float = 10.0) -> dict:
    """The host oracle (a scalar port: the reference has no CPU path) on all host cores, on a
    bounded sample: the first 4 sequences of the batch, repeated for about `min_seconds`."""
    from oracle import oracle

    nb = min(4, B)
    host = {}
    for k, v in case.arrays.items():
        if k == "scratch":
            continue
        a = v.cpu().numpy()
        host[k] = np.ascontiguousarray(a[:nb]) if k in ("q", "k", "v", "k_cache", "v_cache", "out", "past_lens") else a
    import copy

    sub = copy.copy(case)
    sub.B = nb
    sub.arrays = host
    p = sub.params(host)
    sub_bytes = sub.algorithmic_bytes()
    threads = oracle.set_threads(oracle.hw_threads())
    oracle.attention(p)  # warm
    n, t0 = 0, time.perf_counter()
    while True:
        oracle.attention(p)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds:
            break
    return {"value": round(sub_bytes * n / dt / 1e9, 3), "unit": "GB/s", "cores": threads, "kind": "port",
            "tokens_per_s": round(nb * n / dt, 2),
            "sample": f"first {nb} of {B} sequences of the same batch, {n} repetitions in {dt:.1f} s, OpenMP over (batch, head)"}


# ------------------------------------------------------------------------------------------------
def run_reference(args, rank, world, local):
    if rank != 0:
        return
    from oracle import ref_runner

    if not ref_runner.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libflb_ref.so was not built (the reference checkout was absent at build time)"}), flush=True)
        return
    from fasterllama_b200 import workloads as W

    if args.workload in PREFILL_WORKLOADS:
        return run_reference_prefill(args, local, world)
    B, H, lo, hi, seed, desc = WORKLOADS[args.workload]
    T, d = hi + 1, 128
    dev = f"cuda:{local}"
    lens = W.draw_lengths(seed, B, lo, hi)
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    ref = ref_runner.RefRunner()
    mask = torch.from_numpy(W.causal_mask(T, strict=False)).to(dev)
    table = ref.freq_cis(T + 8)
    nbuf = 2
    sets = []
    for j in range(nbuf):
        per_seq = []
        kc = torch.randn((B, H, T, d), generator=g, device=dev, dtype=torch.float32)
        vc = torch.randn((B, H, T, d), generator=g, device=dev, dtype=torch.float32)
        packed = torch.randint(-8192, 8192, (3, B, 1, H, d), generator=g, device=dev, dtype=torch.int32)  # q, k, v in one buffer
        qkv = {"q": packed[0], "k": packed[1], "v": packed[2], "packed": packed}
        out = torch.zeros((B, H, 1, d), device=dev, dtype=torch.float32)
        for b in range(B):  # one cached length per call in the reference: one call per sequence
            t = {n: qkv[n][b:b + 1] for n in ("q", "k", "v")}
            t.update(act_scale=torch.full((1,), 2.0**-7, device=dev), q_w_scale=torch.full((H * d,), 2.0**-6, device=dev),
                     k_w_scale=torch.full((H * d,), 2.0**-6, device=dev), v_w_scale=torch.full((H * d,), 2.0**-6, device=dev),
                     freq_cis=table, attn_mask=mask, k_cache=kc[b:b + 1], v_cache=vc[b:b + 1], out=out[b:b + 1])
            per_seq.append(ref.make_args(t, start_pos=int(lens[b]), rope_row=int(lens[b])))
        sets.append((per_seq, qkv, out))
    stream = torch.cuda.current_stream()

    def step(i):
        for a in sets[i % nbuf][0]:
            st = ref.attention(a, stream.cuda_stream)
            if st != 0:
                raise RuntimeError(f"reference runner status {st}")

    steps = args.steps
    for i in range(max(args.warmup, 3)):
        step(i)
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    sampler.start()
    e0.record(stream)
    for i in range(steps):
        step(i)
    e1.record(stream)
    torch.cuda.synchronize()
    sampler.stop()
    t = e0.elapsed_time(e1) * 1e-3

    host_in = [s[1]["packed"].cpu().pin_memory() for s in sets]
    host_out = torch.empty_like(sets[0][2], device="cpu").pin_memory()
    h2d = host_in[0].numel() * host_in[0].element_size()
    d2h = host_out.numel() * host_out.element_size()

    def e2e_step(i):
        s = sets[i % nbuf]
        s[1]["packed"].copy_(host_in[i % nbuf], non_blocking=True)  # one copy, as in the other arm
        step(i)
        host_out.copy_(s[2], non_blocking=True)
        stream.synchronize()

    for i in range(3):
        e2e_step(i)
    torch.cuda.synchronize()
    e0.record(stream)
    for i in range(steps):
        e2e_step(i)
    e1.record(stream)
    torch.cuda.synchronize()
    t_e2e = e0.elapsed_time(e1) * 1e-3

    # same byte basis as the other arm (the fp16 workload's algorithmic bytes), so that the ratio of
    # the two lines is a ratio of times; the reference itself moves more (fp32 cache, score round trips)
    e_c, e_io = 2, 2
    bytes_step = int(H * (2 * lens.astype(np.int64) * d * e_c + 2 * d * e_c + 3 * d * e_io + d * e_io).sum())
    value = bytes_step * steps / t / 1e9
    e2e_val = bytes_step * steps / t_e2e / 1e9
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbps", "value": round(value, 1), "unit": "GB/s", "n_gpus": 1,
        "ranks_launched": world,  # the reference is single-GPU: rank 0 alone measures, the others exit
        "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": round(t / steps * 1e3, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "reference_mode": "the reference's kernels + cuBLAS gemv with corrected arguments (as written cuBLAS rejects them for L > 128), fp32 cache, one call per sequence (it has one cached length per call)",
                   "byte_basis": "fp16 workload bytes, identical to the other arm"},
        "tokens_per_s": round(B * steps / t, 1),
        "gpu_launches": steps * B * 6,
        "cpu_baseline": {"value": round(value, 1), "unit": "GB/s", "cores": 0, "kind": "reference",
                         "sample": "the whole batch; the reference has no CPU implementation of this path, so its own CUDA kernels run on the GPU"},
        "e2e": {"value": round(e2e_val, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(t_e2e / steps * 1e3, 5), "tokens_per_s": round(B * steps / t_e2e, 1)},
        "clocks": sampler.summary(),
    }
    print(json.dumps(line), flush=True)
    ref.close()


def run_reference_prefill(args, local, world=1):
    """The reference's prefill chain (3 kernels, 2 batched cuBLAS GEMMs with fp16 tensor-core math on
    fp32 storage, softmax over the materialised 1 GiB score matrix) at the config-3 shape."""
    from fasterllama_b200 import workloads as W
    from oracle import ref_runner

    B, H, S, d = 8, 32, 1024, 128
    dev = f"cuda:{local}"
    ref = ref_runner.RefRunner()
    g = torch.Generator(device=dev)
    g.manual_seed(2)
    t = {n: torch.randint(-8192, 8192, (B, S, H, d), generator=g, device=dev, dtype=torch.int32) for n in ("q", "k", "v")}
    t.update(act_scale=torch.full((B * S,), 2.0**-7, device=dev), q_w_scale=torch.full((H * d,), 2.0**-6, device=dev),
             k_w_scale=torch.full((H * d,), 2.0**-6, device=dev), v_w_scale=torch.full((H * d,), 2.0**-6, device=dev),
             freq_cis=ref.freq_cis(S + 8), attn_mask=torch.from_numpy(W.causal_mask(S, strict=False)).to(dev),
             k_cache=torch.zeros((B, H, S, d), device=dev), v_cache=torch.zeros((B, H, S, d), device=dev),
             out=torch.zeros((B, H, S, d), device=dev))
    a = ref.make_args(t, start_pos=0)
    stream = torch.cuda.current_stream()
    steps = min(args.steps, 100)
    for _ in range(3):
        assert ref.attention(a, stream.cuda_stream) == 0
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    sampler.start()
    e0.record(stream)
    for _ in range(steps):
        ref.attention(a, stream.cuda_stream)
    e1.record(stream)
    torch.cuda.synchronize()
    sampler.stop()
    tt = e0.elapsed_time(e1) * 1e-3
    flops = B * H * 2 * d * S * (S + 1)
    v = flops * steps / tt / 1e12
    line = {"impl": "reference", "metric": "prefill_attn_tflops", "value": round(v, 1), "unit": "TFLOP/s", "n_gpus": 1, "ranks_launched": world,
            "steps": steps, "warmup": 3, "ms_per_step": round(tt / steps * 1e3, 5), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 storage, fp16 tensor-core math (CUBLAS_COMPUTE_32F_FAST_16F)", "data": "synthetic",
            "config": {"workload": "causal prefill attention, batch 8, 1024 tokens, 32 heads x 128", "flop_basis": "causal-exact flops, identical to the other arm (the reference computes the full square)"},
            "gpu_launches": steps * 6,
            "cpu_baseline": {"value": round(v, 1), "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                             "sample": "the whole batch; the reference has no CPU implementation of this path, so its own CUDA kernels run on the GPU"},
            "e2e": {"value": round(v, 1), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "clocks": sampler.summary()}
    print(json.dumps(line), flush=True)
    ref.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + list(PREFILL_WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the host-oracle baseline leg")
    ap.add_argument("--split-len", type=int, default=0,
                    help="rows per split-KV partition in the back-to-back leg (0: 2048 with early start level 2, else the library's 512)")
    ap.add_argument("--early-start", type=int, default=2, choices=[1, 2],
                    help="level of the programmatic dependent launch (flb_attn_params.early_start): 1 = only cache tiles are fetched before the previous call has completed, 2 = the whole pass over the cache")
    ap.add_argument("--no-early-start", action="store_true",
                    help="launch every decode call the ordinary way (default: programmatic dependent launch, a call may fetch its first cache tiles while the previous one drains)")
    ap.add_argument("--e2e-mode", default="mapped", choices=["mapped", "copies"],
                    help="end-to-end leg: hand the pinned host buffers to the call (the kernel moves the bytes) or copy in / copy out")
    ap.add_argument("--sets", type=int, default=NBUF, help="distinct input sets rotated through the loop (1 for a small profiler capture)")
    args = ap.parse_args()
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: there is no CPU path to measure")
    torch.cuda.set_device(local)
    launched = world
    if args.impl == "reference":
        world = 1  # rank 0 alone runs the reference arm; the other ranks leave without work
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    try:
        if args.impl == "reference":
            run_reference(args, rank, launched, local)
        else:
            from fasterllama_b200 import _lib

            _lib.load_library()  # no fallback: fail here if the CUDA library is missing
            if args.workload in PREFILL_WORKLOADS:
                run_prefill(args, rank, world, local)
            else:
                run_ours(args, rank, world, local)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
