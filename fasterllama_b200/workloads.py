"""Seeded synthetic inputs for the attention path, shaped like one decoder layer of LLaMA-2.

The reference measures on no dataset and ships no inputs (its samples draw random weights), so
every workload here is synthetic: N(0,1) values from a seeded generator with the shapes the
benchmark configurations name.  `host_case` draws with numpy (tests, oracle); `device_case` draws
the large tensors on the GPU (benchmark sizes)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import numpy as np

from . import attention as A

HEAD_DIM = 128


def freq_cis_table(rows: int, d: int = HEAD_DIM, base: float = 10000.0) -> np.ndarray:
    """RoPE table in the reference's layout (fasterLlama/cuda/decoding_kernels.cu:85-114):
    row = position, [2i] = cos, [2i+1] = sin of pos * base^(-2i/d); evaluated in double here.
    Both the CUDA path and the oracle take the table as input, so its rounding never enters a
    comparison."""
    pos = np.arange(rows, dtype=np.float64)[:, None]
    i2 = np.arange(0, d, 2, dtype=np.float64)[None, :]
    theta = pos * np.power(base, -i2 / d)
    t = np.empty((rows, d), dtype=np.float32)
    t[:, 0::2] = np.cos(theta)
    t[:, 1::2] = np.sin(theta)
    return t


def causal_mask(T: int, strict: bool, masked: float = -np.finfo(np.float32).max) -> np.ndarray:
    """Additive [T, T] mask as the reference's programs build it: strict keeps key < query
    (samples/llama_fp16.cu:73-81), inclusive keeps key <= query."""
    r = np.arange(T)[:, None]
    c = np.arange(T)[None, :]
    keep = (c < r) if strict else (c <= r)
    return np.where(keep, np.float32(0), np.float32(masked)).astype(np.float32)


@dataclass
class Case:
    """One call's worth of inputs.  `arrays` holds numpy arrays or torch tensors."""

    name: str
    B: int
    H: int
    S: int
    T: int
    start_pos: int
    arrays: dict[str, Any]
    rope_pos0: int = 0
    rope_add_past: bool = False
    mask_mode: int = A.FLB_MASK_CAUSAL_INCLUSIVE
    softmax_scale: float = 1.0 / math.sqrt(HEAD_DIM)
    split_len: int = 0
    max_past_len: int = 0
    scratch_zeroed: bool = False
    early_start: int = 0  # decode: programmatic dependent launch, level 0 / 1 / 2 (see flb_attn_params.early_start)
    meta: dict[str, Any] = field(default_factory=dict)

    def params(self, arrays: dict[str, Any] | None = None, out_peers=None, out_head_total: int = 0, out_head_offset: int = 0):
        """The parameter block of this case on `arrays`.  With `out_peers` (device addresses of every rank's
        [B, out_head_total, 1, d] buffer) the decode call pushes its rows there instead of writing `out`."""
        a = arrays if arrays is not None else self.arrays
        return A.make_params(
            q=a["q"], k=a["k"], v=a["v"], k_cache=a["k_cache"], v_cache=a["v_cache"],
            out=(None if out_peers is not None else a["out"]), out_peers=out_peers, out_head_total=out_head_total,
            out_head_offset=out_head_offset, out_dtype=str(a["out"].dtype).replace("torch.", ""),
            scratch=a.get("scratch"), start_pos=self.start_pos, past_lens=a.get("past_lens"),
            max_past_len=self.max_past_len, act_scale=a.get("act_scale"), q_w_scale=a.get("q_w_scale"),
            k_w_scale=a.get("k_w_scale"), v_w_scale=a.get("v_w_scale"), freq_cis=a.get("freq_cis"),
            rope_pos0=self.rope_pos0, rope_add_past=self.rope_add_past, mask_mode=self.mask_mode,
            attn_mask=a.get("attn_mask"), softmax_scale=self.softmax_scale,
            scratch_zeroed=self.scratch_zeroed, split_len=self.split_len, early_start=self.early_start,
            out_q8=a.get("out_q8"), out_q8_scale=a.get("out_q8_scale"),
        )

    def algorithmic_bytes(self) -> int:
        """Bytes a decode call must move: K and V cache rows read, the appended rows written, q/k/v
        read and the output written — no mask, score or table bytes."""
        a = self.arrays
        e_c = 2 if "16" in str(a["k_cache"].dtype) else 4
        e_in = {"int32": 4, "float32": 4, "float16": 2}[str(a["q"].dtype).replace("torch.", "")]
        e_out = 2 if "16" in str(a["out"].dtype) else 4
        d = int(a["q"].shape[-1])
        if "past_lens" in a and a["past_lens"] is not None:
            pl = a["past_lens"]
            lens = pl.cpu().numpy() if hasattr(pl, "cpu") else np.asarray(pl)
        else:
            lens = np.full(self.B, self.start_pos)
        per_seq = 2 * lens.astype(np.int64) * d * e_c + 2 * d * e_c + 3 * d * e_in + d * e_out
        return int(self.H * per_seq.sum())


def host_case(
    name: str,
    seed: int,
    B: int,
    H: int,
    T: int,
    *,
    S: int = 1,
    past=0,
    in_dtype: str = "float32",
    cache_dtype: str = "float32",
    out_dtype: str = "float32",
    rope: str = "past",
    mask_mode: int = A.FLB_MASK_CAUSAL_INCLUSIVE,
    split_len: int = 0,
    uniform_start_pos: bool | None = None,
    d: int = HEAD_DIM,
) -> Case:
    """Draws a case with numpy.  `past` is an int (same cached length for every sequence, the
    reference's start_pos) or an int array [B] (per-sequence lengths).  `rope`: "past" rotates at
    the absolute position, "reference" at the chunk-relative row like the reference, "none"."""
    rng = np.random.default_rng(seed)
    per_seq = not np.isscalar(past)
    lens = np.asarray(past, dtype=np.int32) if per_seq else np.full(B, int(past), dtype=np.int32)
    if uniform_start_pos is None:
        uniform_start_pos = not per_seq
    arrays: dict[str, Any] = {}
    if in_dtype == "int32":
        for n in ("q", "k", "v"):
            arrays[n] = np.rint(rng.standard_normal((B, S, H, d)) * 4096.0).astype(np.int32)
        arrays["act_scale"] = (rng.uniform(0.5, 1.5, B * S) / 64.0).astype(np.float32)
        for n in ("q_w_scale", "k_w_scale", "v_w_scale"):
            arrays[n] = (rng.uniform(0.5, 1.5, H * d) / 64.0).astype(np.float32)
    else:
        for n in ("q", "k", "v"):
            arrays[n] = rng.standard_normal((B, S, H, d)).astype(np.float32).astype(in_dtype)
    kc = np.zeros((B, H, T, d), dtype=cache_dtype)
    vc = np.zeros((B, H, T, d), dtype=cache_dtype)
    for b in range(B):
        n = int(lens[b])
        kc[b, :, :n] = rng.standard_normal((H, n, d)).astype(np.float32).astype(cache_dtype)
        vc[b, :, :n] = rng.standard_normal((H, n, d)).astype(np.float32).astype(cache_dtype)
    arrays["k_cache"], arrays["v_cache"] = kc, vc
    arrays["out"] = np.zeros((B, H, S, d), dtype=out_dtype)
    if rope != "none":
        arrays["freq_cis"] = freq_cis_table(T, d)
    if mask_mode == A.FLB_MASK_GENERIC:
        # a generic additive mask: inclusive causal plus a random finite bias and some dropped keys
        m = causal_mask(T, strict=False)
        bias = rng.uniform(-2.0, 0.0, (T, T)).astype(np.float32)
        drop = rng.uniform(size=(T, T)) < 0.1
        m = np.where(m == 0, np.where(drop, np.float32(-np.finfo(np.float32).max), bias), m).astype(np.float32)
        arrays["attn_mask"] = m
    if not uniform_start_pos:
        arrays["past_lens"] = lens
    c = Case(
        name=name, B=B, H=H, S=S, T=T, start_pos=int(lens[0]) if uniform_start_pos else 0, arrays=arrays,
        rope_pos0=0, rope_add_past=(rope == "past"), mask_mode=mask_mode, split_len=split_len,
        max_past_len=int(lens.max()) if not uniform_start_pos else 0, softmax_scale=1.0 / math.sqrt(d),
    )
    c.meta["seed"] = seed
    return c


def to_device(case: Case, device: str = "cuda:0") -> dict[str, Any]:
    """Copies a host case to the GPU and adds the scratch buffer the call needs."""
    import torch

    dev = {k: torch.from_numpy(np.ascontiguousarray(v)).to(device) for k, v in case.arrays.items()}
    if "_merged" in case.arrays:
        # q, k, v are column blocks of one [B, S, row] buffer (a merged QKV projection's output): keep that layout
        B, S, H, d = case.arrays["q"].shape
        buf = dev["_merged"]
        for i, name in enumerate(("q", "k", "v")):
            dev[name] = buf[:, :, i * H * d:(i + 1) * H * d].unflatten(2, (H, d))
    n = A.workspace_bytes(case.B, case.H, case.T, case.S, case.split_len, size_per_head=int(case.arrays["q"].shape[-1]))
    dev["scratch"] = torch.empty(n, dtype=torch.uint8, device=device)
    return dev


def device_case(
    name: str,
    seed: int,
    B: int,
    H: int,
    T: int,
    lens,
    *,
    device: str = "cuda:0",
    in_dtype: str = "float16",
    cache_dtype: str = "float16",
    out_dtype: str = "float16",
    split_len: int = 0,
    mask_mode: int = A.FLB_MASK_CAUSAL_INCLUSIVE,
) -> Case:
    """Decode case drawn on the GPU (benchmark sizes): every cache row is N(0,1) — rows at or
    beyond a sequence's length are never read — q/k/v N(0,1), RoPE at the absolute position."""
    import torch

    g = torch.Generator(device=device)
    g.manual_seed(seed)
    tdt = {"float16": torch.float16, "float32": torch.float32}
    d = HEAD_DIM
    arrays: dict[str, Any] = {}
    for n in ("q", "k", "v"):
        arrays[n] = torch.randn((B, 1, H, d), generator=g, device=device, dtype=torch.float32).to(tdt[in_dtype])
    for n in ("k_cache", "v_cache"):
        c = torch.empty((B, H, T, d), device=device, dtype=tdt[cache_dtype])
        for b in range(B):  # per-sequence draws keep the peak fp32 temporary small
            c[b] = torch.randn((H, T, d), generator=g, device=device, dtype=torch.float32).to(tdt[cache_dtype])
        arrays[n] = c
    arrays["out"] = torch.zeros((B, H, 1, d), device=device, dtype=tdt[out_dtype])
    arrays["freq_cis"] = torch.from_numpy(freq_cis_table(T, d)).to(device)
    lens = np.asarray(lens, dtype=np.int32)
    arrays["past_lens"] = torch.from_numpy(lens).to(device)
    n = A.workspace_bytes(B, H, T, 1, split_len)
    arrays["scratch"] = torch.zeros(n, dtype=torch.uint8, device=device)
    c = Case(
        name=name, B=B, H=H, S=1, T=T, start_pos=0, arrays=arrays, rope_pos0=0, rope_add_past=True,
        mask_mode=mask_mode, split_len=split_len, max_past_len=int(lens.max()),
    )
    c.meta["seed"] = seed
    return c


def draw_lengths(seed: int, B: int, lo: int, hi: int) -> np.ndarray:
    """Per-sequence cached lengths, uniform in [lo, hi]."""
    return np.random.default_rng(seed).integers(lo, hi + 1, size=B).astype(np.int32)
