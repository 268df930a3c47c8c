#!/usr/bin/env python
"""Benchmark of the attention hot path (one JSON line on stdout, rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4]

Headline (`--workload c2`, the default): a step is one decode-attention call (one new token per sequence,
one decoder layer) over one batch of synthetic input: fp16, batch 16, 32 heads x 128, cached lengths uniform in
[1024, 2048] drawn from seed 1 (the LLaMA-2-7B layer shape the metric is quoted on).  With N > 1 every rank runs
its own batch of that shape (independent (batch, head) units, no collective on the data path: weak scaling) and
the value is the sum over ranks divided by the slowest rank's time.

`value`    algorithmic bytes (K and V rows read + appended rows + q/k/v + output; no mask, score or table
           bytes) per second with all inputs resident in HBM, calls launched the ORDINARY way with the library's
           default partition length — what any caller of flb_attn_decode() gets back to back.  Four distinct
           input sets are rotated so no step re-reads what the previous steps left in L2.
`chain`    the same loop with programmatic dependent launch level 2 and one partition per (batch, head) unit:
           consecutive attention calls overlap each other's ramp and drain.  Only attention calls that follow
           attention calls get this; it is reported beside the headline, not as it.
`single_call_us`  one call at a time with an idle stream in front of it.
`e2e`      the headline metric through the public call with HOST inputs: every step hands the call that step's
           q, k, v and output buffer in pinned host memory and waits for the result.
`roofline` the decode kernel's bytes per launch over its average duration (CUDA events on the launching
           stream), against the measured copy bandwidth of this pool's B200s.
`cpu_baseline` the scalar host oracle timed on this box's cores on a bounded sample.
`legs`     the other configurations of the metric, each measured the same way in the same run:
             in_layer  the decode call where it sits in the decoder layer: an INT8 GEMM of the V-projection
                       shape in front of it and the attention-output quantisation behind it, at the end-to-end
                       configuration's layer shape (batch 32, 32 heads, 640 cached rows, fp16 cache);
             c3        causal prefill (batch 8, 1024 tokens), TFLOP/s of causal-exact flops, tensor roofline;
             c4        the LLaMA-2-13B decode batch (64 x 40 heads, lengths U[2048,4096]): whole on one GPU,
                       split over the ranks by contiguous (batch, head) ranges at N > 1 (strong scaling);
             exchange  (N > 1) the head-split layer's decode step: decode kernel alone, with peer stores +
                       exchange kernel, and with an NCCL all-gather behind it.
A timed region shorter than 50 ms is repeated (at least 20 times, each repeat bracketed like the first) and the
median is reported; `steps` stays what was asked for.

`--impl reference` times the reference's own CUDA attention chain (three kernels + two cuBLAS gemv + softmax,
fp32 cache) built from the reference checkout by oracle/build_ref.sh; the reference has no CPU implementation of
this path.  Its decode gemv arguments are corrected as described in oracle/ref_runner.cu (as written they are
rejected by cuBLAS for L > 128).  It has one cached length per call, so `value` runs the ragged batch as one call
per sequence; `uniform_Lmax` is its best case, one call with every sequence at the maximum length (more rows than
the workload holds, credited with the workload's bytes only).
"""
from __future__ import annotations

import argparse
import dataclasses
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

WORKLOADS = {
    # name: (B, H, lo, hi, seed, description)
    "c2": (16, 32, 1024, 2048, 1, "fp16 decode attention, LLaMA-2-7B layer shape: batch 16, 32 heads x 128, cached lengths U[1024,2048], seed 1"),
    "c4": (64, 40, 2048, 4096, 3, "fp16 decode attention, LLaMA-2-13B layer shape: batch 64, 40 heads x 128, cached lengths U[2048,4096], seed 3"),
}
PREFILL_WORKLOADS = ("c3",)
C3_DESC = "fp16 causal prefill attention, LLaMA-2-7B layer shape: batch 8, 1024 tokens, 32 heads x 128, RoPE rows 0..1023, seed 2"
MIN_REGION_MS = 50.0   # a timed region shorter than this is repeated
MIN_REPEATS = 20


def load_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured (MEASURED_PEAKS.json)"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_traffic(workload: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per decode launch from the ncu capture summarised under
    profiles/ (None when no capture of that workload is recorded there)."""
    try:
        d = json.load(open(os.path.join(ROOT, "profiles", "decode_attn_traffic.json")))
        e = d.get(workload)
        return (int(e["dram_bytes_per_launch"]), e.get("capture")) if e else (None, None)
    except Exception:
        return None, None


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


def timed(step, steps: int, warmup: int, world: int, stream, sampler: ClockSampler | None = None, sync_each: bool = False):
    """Times exactly `steps` calls of step(i) on `stream`: barrier + synchronize, event, the steps, event,
    synchronize + barrier; the region's time is the max over ranks.  A region shorter than MIN_REGION_MS is
    repeated (every repeat bracketed the same way) until at least MIN_REPEATS regions and ~MIN_REGION_MS * 4 of
    device time have been seen; the median region is reported.  Returns (seconds per region on this rank's
    device clock, seconds per region max over ranks, number of regions)."""
    for i in range(warmup):
        step(i)
        if sync_each:
            stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    own, worst = [], []
    if sampler is not None:
        sampler.start()
    while True:
        barrier(world)
        e0.record(stream)
        for i in range(steps):
            step(i)
            if sync_each:
                stream.synchronize()
        e1.record(stream)
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) * 1e-3
        own.append(t)
        worst.append(max_over_ranks(t, world))
        barrier(world)
        # every rank takes the same decision: it is taken on the max-over-ranks times
        if worst[0] * 1e3 >= MIN_REGION_MS:
            break
        if len(worst) >= MIN_REPEATS and sum(worst) * 1e3 >= 4 * MIN_REGION_MS:
            break
        if len(worst) >= 2000:
            break
    if sampler is not None:
        sampler.stop()
    k = len(worst) // 2
    order = sorted(range(len(worst)), key=lambda j: worst[j])
    return own[order[k]], worst[order[k]], len(worst)


def single_call_spread(call, stream, n: int = 200) -> dict:
    """n launches timed one by one (each between its own pair of events, the stream idle before it): these
    include the launch latency that back-to-back calls hide."""
    es = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    for i, (a0, a1) in enumerate(es):
        a0.record(stream)
        call(i)
        a1.record(stream)
        stream.synchronize()
    s = sorted(a0.elapsed_time(a1) * 1e3 for a0, a1 in es)
    return {"p10": round(s[n // 10], 2), "p50": round(s[n // 2], 2), "p90": round(s[n * 9 // 10], 2),
            "what": "one call at a time, stream idle before each (us); ordinary launch, default partition length"}


# ------------------------------------------------------------------------------------------------
# decode legs
# ------------------------------------------------------------------------------------------------
def make_decode_sets(workload: str, rank: int, world: int, local: int, nbuf: int, strong: bool):
    from fasterllama_b200 import sharding
    from fasterllama_b200 import workloads as W

    B, H, lo, hi, seed, desc = WORKLOADS[workload]
    T = hi + 1
    dev = f"cuda:{local}"
    lens = W.draw_lengths(seed, B, lo, hi)  # the same lengths on every rank and in every set
    if strong:
        sh = sharding.plan(B, H, world, rank)
        if sh.axis == "batch":
            lens = lens[sh.start:sh.stop]
        B, H = sh.batch, sh.heads
    sets = []
    for j in range(nbuf):
        c = W.device_case(f"{workload}-{j}", seed + 7919 * j + 104729 * rank, B, H, T, lens, device=dev)
        c.scratch_zeroed = True  # device_case hands over zeroed scratch; the kernel leaves it zeroed
        # q, k, v as three views of one buffer, so that a copying end-to-end leg moves them with one host->device copy
        c.arrays["qkv"] = torch.stack([c.arrays[n] for n in ("q", "k", "v")]).contiguous()
        c.arrays["q"], c.arrays["k"], c.arrays["v"] = c.arrays["qkv"][0], c.arrays["qkv"][1], c.arrays["qkv"][2]
        sets.append(c)
    return sets, B, H, T, lens, desc


def decode_numbers(sets, steps, warmup, world, stream, sampler, split_len=0, early_start=0):
    """Back-to-back decode calls over the rotating sets.  Returns (own s/region, max-over-ranks s/region, regions)."""
    from fasterllama_b200 import attention as A

    ps = [dataclasses.replace(c, split_len=split_len, early_start=early_start).params() for c in sets]
    n = len(ps)
    res = timed(lambda i: A.decode(ps[i % n], stream), steps, warmup, world, stream, sampler)
    for c in sets:
        assert A.scratch_status(c.arrays["scratch"]) == 0, "a decode kernel reported an error status"
    return res


def run_ours(args, rank, world, local):
    from fasterllama_b200 import attention as A

    nbuf = max(1, args.sets)
    strong = args.workload == "c4"  # config 4 is quoted as one batch sharded over the GPUs
    sets, B, H, T, lens, desc = make_decode_sets(args.workload, rank, world, local, nbuf, strong)
    bytes_step = sets[0].algorithmic_bytes()
    tokens_step = WORKLOADS[args.workload][0] if strong else B * world  # sequences advanced per step, all ranks
    stream = torch.cuda.current_stream()
    warmup = max(args.warmup, 3)
    peaks = load_peaks()

    # ---- headline: ordinary launches, library defaults -------------------------------------------
    sampler = ClockSampler(local)
    t_own, t, regions = decode_numbers(sets, args.steps, warmup, world, stream, sampler, split_len=args.split_len, early_start=0)
    total_bytes = sum_over_ranks(float(bytes_step), world)
    value = total_bytes * args.steps / t / 1e9
    achieved = bytes_step * args.steps / t_own / 1e9  # this rank's kernel: one launch per step

    # ---- the attention-after-attention chain (programmatic dependent launch level 2, one partition per unit) ---
    chain = None
    if not args.no_chain:
        c_own, c_t, c_reg = decode_numbers(sets, args.steps, warmup, world, stream, None, split_len=T - 1 if args.chain_split == 0 else args.chain_split, early_start=2)
        chain = {"value": round(total_bytes * args.steps / c_t / 1e9, 1), "unit": "GB/s", "ms_per_step": round(c_t / args.steps * 1e3, 5),
                 "pct_of_8TBps": round(100 * total_bytes * args.steps / c_t / 1e9 / world / 8000.0, 2), "regions": c_reg,
                 "frac_of_measured_peak": round(bytes_step * args.steps / c_own / 1e9 / peaks["hbm_gbs"], 4),
                 "what": "calls launched with programmatic dependent launch level 2 (flb_attn_params.early_start = 2) and one partition per (batch, head) unit: a call streams the cache against q and k while the call in front drains; holds only where the kernel in front is another attention call"}

    # ---- single calls ----------------------------------------------------------------------------
    single_ps = [c.params() for c in sets]
    spread = single_call_spread(lambda i: A.decode(single_ps[i % nbuf], stream), stream)

    # ---- end to end: host q/k/v in, output back on the host, every step --------------------------
    host_in = [c.arrays["qkv"].cpu().pin_memory() for c in sets]
    host_out = torch.empty_like(sets[0].arrays["out"], device="cpu").pin_memory()
    h2d = host_in[0].numel() * host_in[0].element_size()
    d2h = host_out.numel() * host_out.element_size()
    # Two ways to take host buffers through the C ABI call.  "mapped": the call is handed the pinned host
    # buffers themselves (pinned memory is device-addressable): the kernel reads this step's q, k, v over PCIe
    # while its first cache tiles are in flight and stores the result rows straight into host memory, so the
    # step is ONE launch and the same bytes cross the bus.  "copies": copy in, launch, copy out.
    mapped_params = []
    if args.e2e_mode == "mapped":
        for j, c in enumerate(sets):
            a = dict(c.arrays)
            a["q"], a["k"], a["v"] = host_in[j][0], host_in[j][1], host_in[j][2]
            a["out"] = host_out
            mapped_params.append(c.params(a))

    def e2e_step(i):
        c = sets[i % nbuf]
        if mapped_params:
            A.decode(mapped_params[i % nbuf], stream)
        else:
            c.arrays["qkv"].copy_(host_in[i % nbuf], non_blocking=True)  # this step's q, k, v: one copy from pinned memory
            A.decode(single_ps[i % nbuf], stream)
            host_out.copy_(c.arrays["out"], non_blocking=True)

    # the caller reads the step's result before it issues the next step: a stream sync per step
    _, t_e2e, e_reg = timed(e2e_step, args.steps, warmup, world, stream, None, sync_each=True)
    # what reached the host is what the device-resident leg computed for the same inputs
    last = (args.steps - 1) % nbuf
    assert torch.equal(host_out, sets[last].arrays["out"].cpu()), "end-to-end result differs from the device-resident result"
    e2e_val = total_bytes * args.steps / t_e2e / 1e9

    traffic, capture = load_traffic(args.workload)
    line = {
        "metric": "decode_attn_hbm_gbps", "value": round(value, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(t / args.steps * 1e3, 5), "higher_is_better": True, "scaling": "strong" if strong else "weak",
        "vs_baseline": None, "dtype": "f16 storage, f32 arithmetic", "data": "synthetic",
        "config": {
            "workload": desc, "per_gpu_batch": B, "heads": H, "head_dim": 128, "cache_rows_total": int(lens.sum()),
            "total_len": T, "split_len": args.split_len or "library default",
            "value_is": "back-to-back calls, ORDINARY stream launches, library-default partition length (what every caller of flb_attn_decode gets); the overlapped attention-after-attention figure is `chain`",
            "l2": f"{nbuf} distinct input sets rotated ({nbuf * bytes_step / 1e6:.0f} MB > 126 MB L2), no flush kernel in the timed region",
            "timed_regions": regions,
            "region_rule": f"a region of `steps` calls shorter than {MIN_REGION_MS:.0f} ms is repeated (>= {MIN_REPEATS} regions); ms_per_step is the median region / steps",
            "sharding": ("one batch split over the ranks by contiguous (batch, head) ranges, no collective" if strong
                         else "every rank runs its own batch of this shape (independent (batch, head) units), no collective"),
        },
        "tokens_per_s": round(tokens_step * args.steps / t, 1),
        "pct_of_8TBps": round(100 * value / world / 8000.0, 2),
        "bytes_per_step_per_gpu": bytes_step,
        "gpu_launches": args.steps,
        "single_call_us": spread,
        "e2e": {"value": round(e2e_val, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(t_e2e / args.steps * 1e3, 5), "tokens_per_s": round(tokens_step * args.steps / t_e2e, 1), "regions": e_reg,
                "host_buffers": ("pinned host q/k/v/out handed to the call; the kernel reads and writes them over PCIe, host waits for each step"
                                 if mapped_params else "copy in, launch, copy out; host waits for each step")},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": f"{peaks['source']}: copy bandwidth",
                     "kernel": "flb_decode_attn_kernel<__half,...>", "traffic": traffic, "traffic_capture": capture},
        "clocks": sampler.summary(),
    }
    if chain is not None:
        line["chain"] = chain
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(sets[0], bytes_step, B)

    # ---- the other configurations ----------------------------------------------------------------
    legs = {}
    if not args.no_legs and args.workload == "c2":
        del sets, single_ps, mapped_params
        torch.cuda.empty_cache()
        legs["in_layer"] = leg_in_layer(local, world, stream, peaks)
        legs["c3"] = prefill_numbers(args, rank, world, local, peaks, brief=True)
        torch.cuda.empty_cache()
        legs["c4"] = leg_c4(args, rank, world, local, stream, peaks)
        torch.cuda.empty_cache()
        if world > 1:
            legs["exchange"] = leg_exchange(rank, world, local, stream)
        line["legs"] = legs
    if rank == 0:
        print(json.dumps(line), flush=True)


def leg_c4(args, rank, world, local, stream, peaks) -> dict:
    """Config 4: the one 64 x 40-head batch, whole on one GPU, split over the ranks at N > 1 (strong scaling)."""
    sets, B, H, T, lens, desc = make_decode_sets("c4", rank, world, local, 2, strong=True)
    bytes_rank = sets[0].algorithmic_bytes()
    total = sum_over_ranks(float(bytes_rank), world)
    own, t, reg = decode_numbers(sets, args.steps, max(args.warmup, 3), world, stream, None)
    c_own, c_t, c_reg = decode_numbers(sets, args.steps, max(args.warmup, 3), world, stream, None, split_len=T - 1, early_start=2)
    return {"workload": desc, "scaling": "strong", "n_gpus": world, "per_gpu_batch": B, "heads": H,
            "value": round(total * args.steps / t / 1e9, 1), "unit": "GB/s", "ms_per_step": round(t / args.steps * 1e3, 5),
            "tokens_per_s": round(WORKLOADS["c4"][0] * args.steps / t, 1), "pct_of_8TBps_per_gpu": round(100 * total * args.steps / t / 1e9 / world / 8000.0, 2),
            "roofline_frac_of_measured_peak": round(bytes_rank * args.steps / own / 1e9 / peaks["hbm_gbs"], 4), "regions": reg,
            "chain_ms_per_step": round(c_t / args.steps * 1e3, 5), "chain_value": round(total * args.steps / c_t / 1e9, 1),
            "what": "value: ordinary launches, default partition length; chain_*: programmatic dependent launch level 2, one partition per unit"}


def leg_in_layer(local, world, stream, peaks) -> dict:
    """The decode call where the decoder layer has it: behind an INT8 GEMM of the V-projection shape
    (fasterLlama/cuda/open_decoder.cu:126-136: [B, 4096] x [4096, 4096] int8 -> int32, which produces this call's
    v), in front of the attention-output quantisation (open_decoder.cu:245), at the end-to-end configuration's
    layer shape: batch 32, 32 heads, 640 cached rows, fp16 cache, int32 q/k/v with scales.  Events sit between
    the three launches of a layer-step; the queue is kept full (no host sync inside the loop)."""
    from fasterllama_b200 import attention as A
    from fasterllama_b200 import workloads as W

    B, H, L, T, d = 32, 32, 640, 768, 128
    dev = f"cuda:{local}"
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    lens = np.full(B, L, dtype=np.int32)
    nset = 3
    sets = []
    x8 = torch.randint(-127, 128, (B, H * d), generator=g, device=dev, dtype=torch.int8)
    w8 = torch.randint(-127, 128, (H * d, H * d), generator=g, device=dev, dtype=torch.int8)
    gemm = "torch._int_mm (cuBLASLt INT8 GEMM, int32 result written into this call's v)"
    mode = "int8_out"
    try:
        torch._int_mm(x8, w8, out=torch.empty((B, H * d), dtype=torch.int32, device=dev))
    except Exception:
        try:
            torch._int_mm(x8, w8)
            mode, gemm = "int8", "torch._int_mm (cuBLASLt INT8 GEMM, int32 result in a buffer of its own)"
        except Exception as e:  # pragma: no cover - depends on the installed cuBLASLt
            mode, gemm = "f16", f"fp16 matmul of the same shape (torch._int_mm unavailable: {type(e).__name__})"
            x8, w8 = x8.half(), w8.half()
    for j in range(nset):
        c = W.device_case(f"layer-{j}", 50 + j, B, H, T, lens, device=dev, out_dtype="float32")
        a = c.arrays
        for n in ("q", "k", "v"):
            a[n] = torch.randint(-8192, 8192, (B, 1, H, d), generator=g, device=dev, dtype=torch.int32)
        a["act_scale"] = torch.full((B,), 2.0**-7, device=dev)
        for n in ("q_w_scale", "k_w_scale", "v_w_scale"):
            a[n] = torch.full((H * d,), 2.0**-6, device=dev)
        a["q8"] = torch.empty((B, H * d), dtype=torch.int8, device=dev)
        a["q8_scale"] = torch.empty((B,), dtype=torch.float32, device=dev)
        c.scratch_zeroed = True
        sets.append(c)
    nbytes = sets[0].algorithmic_bytes()
    out = {"shape": "batch 32 x 32 heads x 128, 640 cached rows, fp16 cache, int32 q/k/v + scales", "gemm_in_front": gemm,
           "bytes_per_call": nbytes, "what": "us from the completion of the GEMM in front to the completion of the decode kernel, median over 300 layer-steps with the queue kept full"}

    def gemm_into_v(c):
        if mode == "int8_out":
            torch._int_mm(x8, w8, out=c.arrays["v"].view(B, H * d))
        elif mode == "int8":
            torch._int_mm(x8, w8)
        else:
            torch.matmul(x8, w8)

    for label, es in (("ordinary", 0), ("early_start_1", 1)):
        ps = [dataclasses.replace(c, early_start=es).params() for c in sets]
        n_it = 300
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_it)]
        for i in range(n_it + 10):
            c = sets[i % nset]
            gemm_into_v(c)
            if i >= 10:
                ev[i - 10][0].record(stream)
            A.decode(ps[i % nset], stream)
            if i >= 10:
                ev[i - 10][1].record(stream)
            A.quantize(c.arrays["out"], c.arrays["q8"], c.arrays["q8_scale"], stream)
        torch.cuda.synchronize()
        us = sorted(a.elapsed_time(b) * 1e3 for a, b in ev)
        med = us[n_it // 2]
        out[label] = {"us": round(med, 2), "p10": round(us[n_it // 10], 2), "p90": round(us[n_it * 9 // 10], 2),
                      "gbps": round(nbytes / med / 1e3, 1), "pct_of_8TBps": round(100 * nbytes / med / 1e3 / 8000.0, 2),
                      "frac_of_measured_peak": round(nbytes / med / 1e3 / peaks["hbm_gbs"], 4)}
    for c in sets:
        assert A.scratch_status(c.arrays["scratch"]) == 0
    return out


def leg_exchange(rank, world, local, stream) -> dict:
    """The head-split layer's decode step at the end-to-end configuration's shard shape (batch 32, 32/N local
    heads, 640 cached rows, fp32 cache and output as in the reference): the decode kernel alone, the decode kernel
    storing its rows into every rank's receive slot + the exchange kernel (flag hand-shake over NVLink, no
    collective call), and the decode kernel + an NCCL all-gather.  us per layer-step, max over ranks."""
    import torch.distributed as dist

    from fasterllama_b200 import attention as A
    from fasterllama_b200 import workloads as W
    from fasterllama_b200.tensor_parallel import HeadShardedAttention, PeerWindow

    B, H, T, L = 32, 32, 768, 640
    if H % world:
        return {"skipped": f"{H} heads do not divide over {world} ranks"}
    dev = f"cuda:{local}"
    hl = H // world
    lens = np.full(B, L, dtype=np.int32)
    c = W.device_case("exchange", 7 + rank, B, hl, T, lens, device=dev, in_dtype="float32", cache_dtype="float32", out_dtype="float32")
    c.scratch_zeroed = True
    loc = c.arrays
    layer = HeadShardedAttention(B, H, world, rank, attend=None)
    win = PeerWindow(B * H * 128 * 4, world, rank)
    full = torch.zeros((B, H, 1, 128), device=dev)
    mk = lambda l, peers, total, off: c.params(l, out_peers=peers, out_head_total=total, out_head_offset=off)  # noqa: E731
    p_local = c.params()
    parts = [torch.empty_like(loc["out"]) for _ in range(world)]

    def step_push(i):
        layer.forward_push(loc, win, mk, full, status=loc["scratch"], stream=stream)

    def step_nccl(i):
        A.decode(p_local, stream)
        dist.all_gather(parts, loc["out"])

    def step_none(i):
        A.decode(p_local, stream)

    res = {"shape": f"batch {B} x {hl} local heads of {H}, {L} cached rows, fp32 cache, {world} GPUs"}
    for name, fn in (("decode_only_us", step_none), ("decode_nccl_all_gather_us", step_nccl), ("decode_peer_stores_exchange_us", step_push)):
        _, t, _ = timed(fn, 200, 20, world, stream)
        res[name] = round(t / 200 * 1e6, 2)
    # The prefill gather of the same layer (batch 32 x 512 tokens): what the binding does today — an all-gather of the fp32
    # head outputs, 256 MiB per layer — against the exchange that moves a quarter of the bytes and is bit-exact too:
    # all-reduce(max) of the per-token absmax, quantise locally, all-gather the int8 rows.  Collectives only: this sizes
    # what a change of the prefill exchange could save, it is not a second code path.
    S = 512
    shard = torch.empty((B * S * hl * 128,), dtype=torch.float32, device=dev)
    full32 = torch.empty((world, shard.numel()), dtype=torch.float32, device=dev)
    amax = torch.rand((B * S,), device=dev)
    shard8 = torch.empty((shard.numel(),), dtype=torch.int8, device=dev)
    full8 = torch.empty((world, shard.numel()), dtype=torch.int8, device=dev)

    def gather32(i):
        dist.all_gather_into_tensor(full32, shard)

    def gather8(i):
        dist.all_reduce(amax, op=dist.ReduceOp.MAX)
        dist.all_gather_into_tensor(full8, shard8)

    _, t32, _ = timed(gather32, 20, 3, world, stream)
    _, t8, _ = timed(gather8, 20, 3, world, stream)
    res["prefill_gather"] = {"tokens": B * S, "fp32_all_gather_us": round(t32 / 20 * 1e6, 1), "fp32_bytes_per_rank": shard.numel() * 4 * world,
                             "absmax_all_reduce_plus_int8_all_gather_us": round(t8 / 20 * 1e6, 1), "int8_bytes_per_rank": shard.numel() * world,
                             "what": "NCCL collectives alone, per layer, at the end-to-end configuration's prefill (32 x 512 tokens)"}
    del shard, full32, shard8, full8
    res["exchange_status"] = int(A.scratch_status(loc["scratch"]))
    # what the push delivered is what the all-gather delivered
    step_nccl(0)
    step_push(0)
    torch.cuda.synchronize()
    res["push_equals_all_gather"] = bool(torch.equal(full, torch.cat(parts, dim=1)))
    win.close()
    return res


# ------------------------------------------------------------------------------------------------
# prefill
# ------------------------------------------------------------------------------------------------
def prefill_numbers(args, rank, world, local, peaks, brief=False) -> dict:
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
    steps = min(args.steps, 500)
    sampler = ClockSampler(local)
    t_own, t, regions = timed(lambda i: A.prefill(sets[i % nbuf][1], stream), steps, max(args.warmup, 3), world, stream, sampler)
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

    e2e_steps = min(steps, 20)
    _, t_e2e, _ = timed(e2e_step, e2e_steps, 2, world, stream, None, sync_each=True)
    value = flops * world * steps / t / 1e12
    achieved = flops * steps / t_own / 1e12
    res = {
        "metric": "prefill_attn_tflops", "value": round(value, 1), "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(t / steps * 1e3, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 operands, f32 accumulation", "data": "synthetic",
        "config": {"workload": C3_DESC, "flops_per_step": flops, "timed_regions": regions,
                   "l2": f"{nbuf} distinct input sets rotated; q/k/v/caches of one set = 0.4 GB > 126 MB L2"},
        "tokens_per_s": round(B * S * world * steps / t, 1),
        "gpu_launches": 2 * steps,
        "e2e": {"value": round(flops * world * e2e_steps / t_e2e / 1e12, 1), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(t_e2e / e2e_steps * 1e3, 5)},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": round(achieved / peaks["bf16_tflops"], 4), "frac_of_sustained": round(achieved / peaks["bf16_tflops_sustained"], 4),
                     "peak_source": f"{peaks['source']}: cuBLAS bf16 burst",
                     "kernel": "flb_prefill_prologue_kernel + flb_prefill_attn_kernel (whole step)", "traffic": None},
        "clocks": sampler.summary(),
    }
    if brief:
        for k in ("higher_is_better", "vs_baseline", "data", "scaling", "n_gpus", "warmup"):
            res.pop(k, None)
    return res


def run_prefill(args, rank, world, local):
    res = prefill_numbers(args, rank, world, local, load_peaks())
    if rank == 0:
        print(json.dumps(res), flush=True)


def cpu_baseline(case, bytes_step: int, B: int, min_seconds: float = 10.0) -> dict:
    """The host oracle (a scalar port: the reference has no CPU path) on all host cores, on a
    bounded sample: the first 4 sequences of the batch, repeated for about `min_seconds`."""
    from oracle import oracle

    nb = min(4, B)
    host = {}
    for k, v in case.arrays.items():
        if k in ("scratch", "qkv"):
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
# reference arm
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
        line = reference_prefill(args, local, world)
        print(json.dumps(line), flush=True)
        return
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
    scales = dict(q_w_scale=torch.full((H * d,), 2.0**-6, device=dev), k_w_scale=torch.full((H * d,), 2.0**-6, device=dev),
                  v_w_scale=torch.full((H * d,), 2.0**-6, device=dev))
    for j in range(nbuf):
        per_seq = []
        kc = torch.randn((B, H, T, d), generator=g, device=dev, dtype=torch.float32)
        vc = torch.randn((B, H, T, d), generator=g, device=dev, dtype=torch.float32)
        packed = torch.randint(-8192, 8192, (3, B, 1, H, d), generator=g, device=dev, dtype=torch.int32)  # q, k, v in one buffer
        qkv = {"q": packed[0], "k": packed[1], "v": packed[2], "packed": packed}
        out = torch.zeros((B, H, 1, d), device=dev, dtype=torch.float32)
        for b in range(B):  # one cached length per call in the reference: one call per sequence
            t = {n: qkv[n][b:b + 1] for n in ("q", "k", "v")}
            t.update(act_scale=torch.full((1,), 2.0**-7, device=dev), freq_cis=table, attn_mask=mask,
                     k_cache=kc[b:b + 1], v_cache=vc[b:b + 1], out=out[b:b + 1], **scales)
            per_seq.append(ref.make_args(t, start_pos=int(lens[b]), rope_row=int(lens[b])))
        # best case for the reference: ONE call, every sequence at the longest length it can hold (T - 1 rows)
        tu = {n: qkv[n] for n in ("q", "k", "v")}
        tu.update(act_scale=torch.full((B,), 2.0**-7, device=dev), freq_cis=table, attn_mask=mask, k_cache=kc, v_cache=vc, out=out, **scales)
        uniform = ref.make_args(tu, start_pos=T - 1, rope_row=T - 1)
        sets.append((per_seq, qkv, out, uniform))
    stream = torch.cuda.current_stream()

    def step(i):
        for a in sets[i % nbuf][0]:
            st = ref.attention(a, stream.cuda_stream)
            if st != 0:
                raise RuntimeError(f"reference runner status {st}")

    def step_uniform(i):
        st = ref.attention(sets[i % nbuf][3], stream.cuda_stream)
        if st != 0:
            raise RuntimeError(f"reference runner status {st}")

    steps = args.steps
    warmup = max(args.warmup, 3)
    sampler = ClockSampler(local)
    _, t, regions = timed(step, steps, warmup, 1, stream, sampler)
    _, t_uni, _ = timed(step_uniform, steps, warmup, 1, stream, None)

    host_in = [s[1]["packed"].cpu().pin_memory() for s in sets]
    host_out = torch.empty_like(sets[0][2], device="cpu").pin_memory()
    h2d = host_in[0].numel() * host_in[0].element_size()
    d2h = host_out.numel() * host_out.element_size()

    def e2e_step(i):
        s = sets[i % nbuf]
        s[1]["packed"].copy_(host_in[i % nbuf], non_blocking=True)  # one copy, as in the other arm
        step(i)
        host_out.copy_(s[2], non_blocking=True)

    _, t_e2e, _ = timed(e2e_step, steps, 3, 1, stream, None, sync_each=True)

    # same byte basis as the other arm (the fp16 workload's algorithmic bytes), so that the ratio of
    # the two lines is a ratio of times; the reference itself moves more (fp32 cache, score round trips)
    e_c, e_io = 2, 2
    bytes_step = int(H * (2 * lens.astype(np.int64) * d * e_c + 2 * d * e_c + 3 * d * e_io + d * e_io).sum())
    value = bytes_step * steps / t / 1e9
    e2e_val = bytes_step * steps / t_e2e / 1e9
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbps", "value": round(value, 1), "unit": "GB/s", "n_gpus": 1,
        "ranks_launched": world,  # the reference is single-GPU: rank 0 alone measures, the others exit
        "steps": steps, "warmup": warmup, "ms_per_step": round(t / steps * 1e3, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": desc, "reference_mode": "the reference's kernels + cuBLAS gemv with corrected arguments (as written cuBLAS rejects them for L > 128), fp32 cache",
                   "value_is": "one call per sequence (the reference has one cached length per call): 16 calls x 6 launches per step; `uniform_Lmax` is its single-call best case",
                   "byte_basis": "fp16 workload bytes, identical to the other arm", "timed_regions": regions},
        "tokens_per_s": round(B * steps / t, 1),
        "gpu_launches": steps * B * 6,
        "uniform_Lmax": {"value": round(bytes_step * steps / t_uni / 1e9, 1), "unit": "GB/s", "ms_per_step": round(t_uni / steps * 1e3, 5),
                         "gpu_launches": steps * 6,
                         "what": f"ONE call per step with every sequence at {T - 1} cached rows (the reference's best case: no per-sequence launches, but {B * (T - 1)} rows instead of the workload's {int(lens.sum())}); credited with the workload's bytes only"},
        "cpu_baseline": {"value": round(value, 1), "unit": "GB/s", "cores": 0, "kind": "reference",
                         "sample": "the whole batch; the reference has no CPU implementation of this path, so its own CUDA kernels run on the GPU"},
        "e2e": {"value": round(e2e_val, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(t_e2e / steps * 1e3, 5), "tokens_per_s": round(B * steps / t_e2e, 1)},
        "clocks": sampler.summary(),
    }
    del sets
    torch.cuda.empty_cache()
    if not args.no_legs and args.workload == "c2":
        c3 = reference_prefill(args, local, world)
        line["legs"] = {"c3": {k: c3[k] for k in ("metric", "value", "unit", "steps", "ms_per_step", "dtype", "config", "gpu_launches")}}
    print(json.dumps(line), flush=True)
    ref.close()


def reference_prefill(args, local, world=1) -> dict:
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

    def step(i):
        st = ref.attention(a, stream.cuda_stream)
        if st != 0:
            raise RuntimeError(f"reference runner status {st}")

    sampler = ClockSampler(local)
    _, tt, regions = timed(step, steps, 3, 1, stream, sampler)
    flops = B * H * 2 * d * S * (S + 1)
    v = flops * steps / tt / 1e12
    line = {"impl": "reference", "metric": "prefill_attn_tflops", "value": round(v, 1), "unit": "TFLOP/s", "n_gpus": 1, "ranks_launched": world,
            "steps": steps, "warmup": 3, "ms_per_step": round(tt / steps * 1e3, 5), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 storage, fp16 tensor-core math (CUBLAS_COMPUTE_32F_FAST_16F)", "data": "synthetic",
            "config": {"workload": "causal prefill attention, batch 8, 1024 tokens, 32 heads x 128", "timed_regions": regions,
                       "flop_basis": "causal-exact flops, identical to the other arm (the reference computes the full square)"},
            "gpu_launches": steps * 6,
            "cpu_baseline": {"value": round(v, 1), "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                             "sample": "the whole batch; the reference has no CPU implementation of this path, so its own CUDA kernels run on the GPU"},
            "e2e": {"value": round(v, 1), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "clocks": sampler.summary()}
    ref.close()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + list(PREFILL_WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the host-oracle baseline leg")
    ap.add_argument("--no-legs", action="store_true", help="skip the in-layer, prefill, 13B-shape and exchange legs")
    ap.add_argument("--no-chain", action="store_true", help="skip the attention-after-attention (early start level 2) figure")
    ap.add_argument("--split-len", type=int, default=0, help="rows per split-KV partition of the headline loop (0: the library's default)")
    ap.add_argument("--chain-split", type=int, default=0, help="rows per partition in the chain figure (0: one partition per unit)")
    ap.add_argument("--e2e-mode", default="mapped", choices=["mapped", "copies"],
                    help="end-to-end leg: hand the pinned host buffers to the call (the kernel moves the bytes) or copy in / copy out")
    ap.add_argument("--sets", type=int, default=4, help="distinct input sets rotated through the loop (1 for a small profiler capture)")
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
