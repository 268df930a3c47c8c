"""Loads the committed golden vectors (outputs of the reference's own kernels) and turns a golden
case into a Case for the oracle or the CUDA path."""
from __future__ import annotations

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import golden_cases as G  # noqa: E402

from fasterllama_b200 import attention as A  # noqa: E402
from fasterllama_b200 import workloads as W  # noqa: E402

_GOLD = None

# The reference's prefill contractions use fp16 tensor-core math on fp32 storage
# (CUBLAS_COMPUTE_32F_FAST_16F, fasterLlama/cuda/common.h:71): measured on the golden inputs its
# result is up to 2.5e-3 away from exact arithmetic, so comparisons AGAINST THE REFERENCE's prefill
# output use this bound (reference noise + the 2e-3 allowed to the implementation under test).
REF_PREFILL_ABS = 5e-3


class _Fixtures:
    """The committed fixtures as one mapping: ref_golden.npz (head size 128) and ref_golden_head_sizes.npz."""

    def __init__(self):
        self.files = [np.load(os.path.join(HERE, "golden", n)) for n in ("ref_golden.npz", "ref_golden_head_sizes.npz")
                      if os.path.exists(os.path.join(HERE, "golden", n))]

    def __getitem__(self, key):
        for f in self.files:
            if key in f.files:
                return f[key]
        raise KeyError(key)


def gold():
    global _GOLD
    if _GOLD is None:
        _GOLD = _Fixtures()
    return _GOLD


def head_size_fixture_present() -> bool:
    return os.path.exists(os.path.join(HERE, "golden", "ref_golden_head_sizes.npz"))


def notes() -> dict:
    return json.loads(bytes(gold()["notes_json"]).decode())


def case_from_golden(name: str, mask_mode: str = "generic", cache_dtype: str = "float32", out_dtype: str = "float32") -> W.Case:
    """The golden case `name` as call parameters.  `mask_mode`: "generic" hands over the additive
    [T,T] mask exactly like the reference; "index" uses the index-computed mode that the mask
    classifies as."""
    c = G.case(name)
    a = G.build(name)
    S, T, sp = c["S"], c["T"], c["start_pos"]
    d = c.get("d", G.D)
    # table with the stored rows placed where the call will look for them
    table = np.zeros((T + 8, d), dtype=np.float32)
    table[c["rope_row"]:c["rope_row"] + S] = gold()[f"{name}/freq_rows"]
    a["freq_cis"] = table
    if cache_dtype != "float32":
        a["k_cache"] = a["k_cache"].astype(cache_dtype)
        a["v_cache"] = a["v_cache"].astype(cache_dtype)
    a["out"] = a["out"].astype(out_dtype)
    if c["mask"] == "none":
        mm = A.FLB_MASK_NONE
    elif mask_mode == "generic":
        mm = A.FLB_MASK_GENERIC
    else:
        mm = A.FLB_MASK_CAUSAL_STRICT if c["mask"] == "strict" else A.FLB_MASK_CAUSAL_INCLUSIVE
        a.pop("attn_mask", None)
    return W.Case(name=name, B=c["B"], H=c["H"], S=S, T=T, start_pos=sp, arrays=a,
                  rope_pos0=c["rope_row"], rope_add_past=False, mask_mode=mm, softmax_scale=1.0 / float(np.sqrt(d)))


def compare_with_golden(name: str, out: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, *, tol_out_abs: float | None,
                        rel: float = 1e-5, cache_tol: float = 1e-6) -> None:
    """Checks an implementation's result against the reference's stored result.  Rows where the
    reference produced NaN (fully masked rows: 0/0 in its softmax) must be exactly zero here."""
    from util import assert_abs_close, assert_fp32_close

    c = G.case(name)
    S, sp = c["S"], c["start_pos"]
    hs = list(G.PREFILL_HEADS_KEPT) if S > 1 else list(range(c["H"]))
    want = gold()[f"{name}/out"]
    got = np.asarray(out, dtype=np.float32)[:, hs]
    nan_rows = np.isnan(want).any(axis=-1)
    if nan_rows.any():
        assert c["mask"] == "strict", "only the strict mask has fully masked rows"
        assert not got[nan_rows].any(), "a fully masked row must come out as zeros"
    ok = ~nan_rows
    if tol_out_abs is None:
        assert_fp32_close(got[ok], want[ok], rel=rel, what=name + " out vs reference")
    else:
        assert_abs_close(got[ok], want[ok], tol_out_abs, what=name + " out vs reference")
    kr = np.asarray(k_cache, dtype=np.float32)[:, hs, sp:sp + S]
    vr = np.asarray(v_cache, dtype=np.float32)[:, hs, sp:sp + S]
    wk, wv = gold()[f"{name}/k_rows"], gold()[f"{name}/v_rows"]
    assert np.abs(kr - wk).max() <= cache_tol * max(1.0, np.abs(wk).max()), name + " appended K rows"
    assert np.abs(vr - wv).max() <= cache_tol * max(1.0, np.abs(wv).max()), name + " appended V rows"
