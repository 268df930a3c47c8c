"""Parity of the CUDA prefill attention (tensor-core kernel, through the C ABI) against the host
oracle (2e-3 absolute: fp16 operands, fp32 accumulation) and the reference's golden vectors."""
import numpy as np
import pytest

from fasterllama_b200 import attention as A
from fasterllama_b200 import workloads as W

import golden_util as GU
from util import assert_abs_close, run_cuda, run_oracle

pytestmark = pytest.mark.gpu

PREFILL_ABS = 2e-3


def _check(case, cuda, orc, cache16):
    assert cuda["status"] == 0, f"kernel status word {cuda['status']:#x}"
    assert_abs_close(cuda["out"], orc["out"].astype(np.float32), PREFILL_ABS, case.name + " out")
    S = case.S
    ko = orc["k_cache"].astype(np.float32)[:, :, :S]
    vo = orc["v_cache"].astype(np.float32)[:, :, :S]
    tol = 2e-3 if cache16 else 1e-5
    assert np.abs(cuda["k_cache"][:, :, :S] - ko).max() <= tol * max(1.0, np.abs(ko).max())
    assert np.array_equal(cuda["v_cache"][:, :, :S], vo)
    # rows beyond the prompt stay untouched
    assert not cuda["k_cache"][:, :, S:].any() and not cuda["v_cache"][:, :, S:].any()


@pytest.mark.parametrize("S", [2, 17, 64, 127, 128, 129, 200, 255, 256, 257, 300, 383, 384, 385, 513, 640, 1000])
def test_prefill_lengths_fp16_cache(cuda_device, S):
    case = W.host_case(f"pf16-S{S}", 400 + S, 1, 2, S + 40, S=S, past=0, in_dtype="float16", cache_dtype="float16",
                       out_dtype="float32", rope="past")
    _check(case, run_cuda(case), run_oracle(case), cache16=True)


@pytest.mark.parametrize("S", [5, 128, 260, 520])
def test_prefill_fp32_cache_int32_inputs(cuda_device, S):
    """The reference's data path: int32 accumulators + scales in, fp32 cache, fp32 output.  The
    tensor cores take fp16 operands (as the reference's own FAST_16F GEMMs do), so the oracle is
    asked for the same operand rounding; the cache rows must still be the unrounded fp32 values."""
    case = W.host_case(f"pf32-S{S}", 500 + S, 2, 4, S + 9, S=S, past=0, in_dtype="int32", rope="reference")
    _check(case, run_cuda(case), run_oracle(case, f16_operands=True), cache16=False)


@pytest.mark.parametrize("mask_mode", [A.FLB_MASK_NONE, A.FLB_MASK_GENERIC, A.FLB_MASK_CAUSAL_INCLUSIVE, A.FLB_MASK_CAUSAL_STRICT])
@pytest.mark.parametrize("S", [100, 256, 400])
def test_prefill_mask_modes(cuda_device, mask_mode, S):
    case = W.host_case(f"pmask{mask_mode}-S{S}", 600 + S, 1, 4, S + 3, S=S, past=0, in_dtype="float32", cache_dtype="float16",
                       mask_mode=mask_mode)
    cuda, orc = run_cuda(case), run_oracle(case)
    _check(case, cuda, orc, cache16=True)
    if mask_mode == A.FLB_MASK_CAUSAL_STRICT:
        assert not cuda["out"][:, :, 0].any()  # row 0 sees no key: zeros (the reference gives NaN)


@pytest.mark.parametrize("mask_mode", [A.FLB_MASK_NONE, A.FLB_MASK_GENERIC, A.FLB_MASK_CAUSAL_INCLUSIVE, A.FLB_MASK_CAUSAL_STRICT])
@pytest.mark.parametrize("S", [60, 256, 300, 700])
def test_prefill_half_inputs_half_cache_every_mask(cuda_device, mask_mode, S):
    """fp16 q/k/v into an fp16 cache: the V tiles are read from the caller's rows and appended to the cache by the attention
    kernel itself (each key tile once, whatever the mask lets the query blocks see); the appended rows must be the input
    bit for bit and the rows behind the prompt untouched."""
    case = W.host_case(f"pv-direct{mask_mode}-S{S}", 650 + S, 2, 3, S + 70, S=S, past=0, in_dtype="float16", cache_dtype="float16",
                       out_dtype="float16", mask_mode=mask_mode)
    cuda, orc = run_cuda(case), run_oracle(case)
    _check(case, cuda, orc, cache16=True)
    v_in = np.transpose(case.arrays["v"].astype(np.float32), (0, 2, 1, 3))  # [B,S,H,d] -> [B,H,S,d]
    assert np.array_equal(cuda["v_cache"][:, :, :S], v_in)


@pytest.mark.parametrize("name", [c for c in GU.G.CASES if c.startswith("prefill")])
@pytest.mark.parametrize("mask_mode", ["generic", "index"])
def test_prefill_matches_reference_golden(cuda_device, name, mask_mode):
    case = GU.case_from_golden(name, mask_mode=mask_mode)
    r = run_cuda(case)
    assert r["status"] == 0
    GU.compare_with_golden(name, r["out"], r["k_cache"], r["v_cache"], tol_out_abs=GU.REF_PREFILL_ABS)


def test_prefill_fp16_output_and_repeat(cuda_device):
    import torch
    case = W.host_case("pf-out16", 77, 2, 4, 400, S=384, past=0, in_dtype="float16", cache_dtype="float16", out_dtype="float16")
    r = run_cuda(case)
    _check(case, r, run_oracle(case), cache16=True)
    dev = r["dev"]
    first = dev["out"].clone()
    A.forward(case.params(dev))
    torch.cuda.synchronize()
    assert torch.equal(first, dev["out"]), "prefill must be deterministic"


def test_prefill_then_decode_continues_the_cache(cuda_device):
    """Prefill S tokens, then decode one token on the same cache: equals the oracle doing the same."""
    import torch
    S, T, B, H = 150, 200, 2, 4
    pre = W.host_case("pd-pre", 81, B, H, T, S=S, past=0, in_dtype="float16", cache_dtype="float16", out_dtype="float32")
    host = {k: np.array(v, copy=True) for k, v in pre.arrays.items()}
    from oracle import oracle
    oracle.attention(pre.params(host))
    dev = W.to_device(pre)
    A.forward(pre.params(dev))
    dec = W.host_case("pd-dec", 82, B, H, T, past=S, in_dtype="float16", cache_dtype="float16", out_dtype="float32")
    hd = {k: np.array(v, copy=True) for k, v in dec.arrays.items()}
    hd["k_cache"], hd["v_cache"] = host["k_cache"], host["v_cache"]
    oracle.attention(dec.params(hd))
    dd = W.to_device(dec)
    dd["k_cache"], dd["v_cache"] = dev["k_cache"], dev["v_cache"]
    A.forward(dec.params(dd))
    torch.cuda.synchronize()
    assert A.scratch_status(dd["scratch"]) == 0
    assert_abs_close(dd["out"].cpu().numpy(), hd["out"], 2e-3, "decode after prefill")


def test_config3_shape_sampled_heads(cuda_device):
    """fp16 causal prefill at the LLaMA-2-7B layer shape (batch 8, 1024 tokens, 32 heads x 128, seed 2),
    full size on the GPU; the oracle checks a sample of the (batch, head) units."""
    import torch
    B, H, S = 8, 32, 1024
    case = W.host_case("config3", 2, B, H, S, S=S, past=0, in_dtype="float16", cache_dtype="float16", out_dtype="float16")
    r = run_cuda(case)
    assert r["status"] == 0
    for (b, h) in [(0, 0), (3, 17), (7, 31)]:
        sub = W.Case(name="c3-sub", B=1, H=1, S=S, T=S, start_pos=0, rope_add_past=True, mask_mode=case.mask_mode,
                     arrays={k: (np.ascontiguousarray(v[b:b + 1, :, h:h + 1]) if k in ("q", "k", "v") else
                                 np.ascontiguousarray(v[b:b + 1, h:h + 1]) if k in ("k_cache", "v_cache", "out") else v)
                             for k, v in case.arrays.items()})
        o = run_oracle(sub)
        assert_abs_close(r["out"][b, h], o["out"][0, 0].astype(np.float32), PREFILL_ABS, f"config3 unit ({b},{h})")


@pytest.mark.parametrize("S,mask_mode", [(1500, A.FLB_MASK_CAUSAL_INCLUSIVE), (2049, A.FLB_MASK_CAUSAL_STRICT), (1300, A.FLB_MASK_NONE)])
def test_long_prompts(cuda_device, S, mask_mode):
    """Prompts well beyond the benchmark's 1024 tokens (up to 33 key tiles per query tile, ragged last tiles):
    the barrier phases, the ring indices and the lazy rescaling have run many times over by the end."""
    case = W.host_case(f"long-S{S}", 900 + S, 1, 1, S + 7, S=S, past=0, in_dtype="float16", cache_dtype="float16",
                       out_dtype="float32", rope="past", mask_mode=mask_mode)
    _check(case, run_cuda(case), run_oracle(case, f16_operands=True), cache16=True)
