"""Helpers shared by the parity tests."""
from __future__ import annotations

import numpy as np

from fasterllama_b200 import attention as A
from fasterllama_b200 import workloads as W

# tolerances of the parity contract: fp32 within 1e-5 relative, fp16 within 2e-3 absolute
FP32_REL = 1e-5
FP16_ABS = 2e-3


def assert_fp32_close(got: np.ndarray, want: np.ndarray, rel: float = FP32_REL, what: str = "") -> None:
    """|got - want| <= rel * max(|want|, rms(want)): relative to each element, with the tensor's own
    scale as the floor so that outputs that cancel to ~0 are judged against their magnitude class."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    floor = float(np.sqrt(np.mean(want * want))) or 1.0
    bound = rel * np.maximum(np.abs(want), floor)
    err = np.abs(got - want)
    bad = err > bound
    if bad.any():
        i = np.unravel_index(np.argmax(err / bound), err.shape)
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} beyond {rel:g} rel; worst at {i}: got {got[i]!r} want {want[i]!r}")


def assert_abs_close(got: np.ndarray, want: np.ndarray, tol: float = FP16_ABS, what: str = "") -> None:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got - want)
    if err.max() > tol:
        i = np.unravel_index(np.argmax(err), err.shape)
        raise AssertionError(f"{what}: max abs err {err.max():.3e} > {tol:g} at {i}: got {got[i]!r} want {want[i]!r}")


def run_oracle(case: W.Case, f16_operands: bool = False) -> dict[str, np.ndarray]:
    """Runs the host oracle on copies of the case's arrays; returns out and the updated caches."""
    from oracle import oracle

    arrays = {k: np.array(v, copy=True) for k, v in case.arrays.items()}
    p = case.params(arrays)
    oracle.attention(p, acc_double=True, f16_operands=f16_operands)
    return {"out": arrays["out"], "k_cache": arrays["k_cache"], "v_cache": arrays["v_cache"]}


def run_cuda(case: W.Case, device: str = "cuda:0", calls: int = 1, canary: bool = True) -> dict[str, np.ndarray]:
    """Runs the CUDA path through the C ABI on device copies; returns out, caches and the kernels'
    status word.  With `canary`, the output is pre-filled with a sentinel to catch unwritten
    elements."""
    import torch

    dev = W.to_device(case, device)
    if canary:
        dev["out"].fill_(float("nan"))
        dev["scratch"].fill_(0xA5)
    p = case.params(dev)
    for _ in range(calls):
        A.forward(p)
    torch.cuda.synchronize()
    st = A.scratch_status(dev["scratch"])
    return {
        "out": dev["out"].float().cpu().numpy(),
        "k_cache": dev["k_cache"].float().cpu().numpy(),
        "v_cache": dev["v_cache"].float().cpu().numpy(),
        "status": st,
        "dev": dev,
    }
