"""The optional fused epilogue: the reference's attention-output quantisation + transpose
(launchAttnQuantizedTransposeKernel, decoder_kernels.cu:1179-1300).  Integer work: bit-exact."""
import numpy as np
import pytest

from fasterllama_b200 import attention as A
from fasterllama_b200 import workloads as W
from oracle import oracle, ref_runner


def test_oracle_quantize_closed_form():
    a = np.zeros((1, 2, 1, 4), dtype=np.float32)
    a[0, 0, 0] = [1.0, -2.0, 0.5, 0.0]
    a[0, 1, 0] = [4.0, -4.0, 0.0157, 2.5 * 4 / 127]   # absmax 4 -> scale 4/127; 2.5 codes -> ties to even = 2
    q8, sc = oracle.attn_quantize(a)
    assert np.isclose(sc[0], 4.0 / 127.0)
    assert q8.shape == (1, 1, 8)
    assert q8[0, 0].tolist() == [32, -64, 16, 0, 127, -127, 0, 2]
    # an all-zero row (e.g. a fully masked query): absmax 0, scale 0, 0 * 127 / 0 = NaN converts to code 0
    q8, sc = oracle.attn_quantize(np.zeros((1, 1, 1, 4), dtype=np.float32))
    assert sc[0] == 0 and not q8.any()


def _with_q8(case, dev):
    import torch
    dev["out_q8"] = torch.full((case.B, case.S, case.H * 128), 99, dtype=torch.int8, device="cuda")
    dev["out_q8_scale"] = torch.full((case.B * case.S,), float("nan"), dtype=torch.float32, device="cuda")
    return dev


@pytest.mark.gpu
@pytest.mark.parametrize("lens", [[0, 5, 300], [600, 1500, 513, 31]])
def test_decode_fused_quantisation(cuda_device, lens):
    import torch
    lens = np.array(lens, dtype=np.int32)
    case = W.host_case("q8-dec", 61, len(lens), 8, 1600, past=lens, in_dtype="int32")
    dev = _with_q8(case, W.to_device(case))
    p = case.params(dev)
    for _ in range(2):  # twice: the per-sequence counters must have been left at zero
        A.forward(p)
    torch.cuda.synchronize()
    assert A.scratch_status(dev["scratch"]) == 0
    out = dev["out"].cpu().numpy()
    want_q8, want_sc = oracle.attn_quantize(out)
    assert np.array_equal(dev["out_q8_scale"].cpu().numpy(), want_sc)
    assert np.array_equal(dev["out_q8"].cpu().numpy(), want_q8)
    if ref_runner.available():
        ref = ref_runner.RefRunner()
        if hasattr(ref.lib, "ref_attn_quant"):
            rq, rs = ref.attn_quant(dev["out"])
            torch.cuda.synchronize()
            assert torch.equal(rq, dev["out_q8"]) and torch.equal(rs, dev["out_q8_scale"])
        ref.close()


@pytest.mark.gpu
@pytest.mark.parametrize("mask_mode", [A.FLB_MASK_CAUSAL_INCLUSIVE, A.FLB_MASK_CAUSAL_STRICT])
def test_prefill_quantisation_kernel(cuda_device, mask_mode):
    import torch
    case = W.host_case("q8-pre", 62, 2, 8, 200, S=150, past=0, in_dtype="int32", mask_mode=mask_mode)
    dev = _with_q8(case, W.to_device(case))
    A.forward(case.params(dev))
    torch.cuda.synchronize()
    out = dev["out"].cpu().numpy()
    want_q8, want_sc = oracle.attn_quantize(out)
    assert np.array_equal(dev["out_q8_scale"].cpu().numpy(), want_sc)
    assert np.array_equal(dev["out_q8"].cpu().numpy(), want_q8)
    if ref_runner.available():
        ref = ref_runner.RefRunner()
        if hasattr(ref.lib, "ref_attn_quant"):
            rq, rs = ref.attn_quant(dev["out"])
            torch.cuda.synchronize()
            assert torch.equal(rq, dev["out_q8"]) and torch.equal(rs, dev["out_q8_scale"])
        ref.close()


def test_quantisation_needs_fp32_output_and_both_pointers():
    from fasterllama_b200 import _lib
    c = W.host_case("v", 1, 2, 4, 64, past=10, out_dtype="float16", in_dtype="float16", cache_dtype="float16")
    c.arrays["scratch"] = np.zeros(A.workspace_bytes(2, 4, 64), dtype=np.uint8)
    c.arrays["out_q8"] = np.zeros((2, 1, 512), dtype=np.int8)
    c.arrays["out_q8_scale"] = np.zeros(2, dtype=np.float32)
    assert A.validate(c.params()) == _lib.FLB_ERR_UNSUPPORTED
    c2 = W.host_case("v", 1, 2, 4, 64, past=10)
    c2.arrays["scratch"] = np.zeros(A.workspace_bytes(2, 4, 64), dtype=np.uint8)
    c2.arrays["out_q8"] = np.zeros((2, 1, 512), dtype=np.int8)
    assert A.validate(c2.params()) == _lib.FLB_ERR_NULL_POINTER
