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


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(3, 8, 1), (2, 5, 37), (1, 32, 1)])
def test_standalone_quantize_call(cuda_device, shape):
    """flb_attn_quantize on a tensor the caller assembled itself (e.g. after an all-gather): bit-exact against the
    oracle, including an all-zero row (a fully masked query)."""
    import torch
    B, H, S = shape
    g = torch.Generator(device="cuda")
    g.manual_seed(9)
    attn = torch.randn((B, H, S, 128), generator=g, device="cuda") * 3.0
    attn[0, :, 0] = 0.0
    q8 = torch.full((B, S, H * 128), 99, dtype=torch.int8, device="cuda")
    sc = torch.full((B * S,), float("nan"), device="cuda")
    A.quantize(attn, q8, sc)
    torch.cuda.synchronize()
    want_q8, want_sc = oracle.attn_quantize(attn.cpu().numpy())
    assert np.array_equal(sc.cpu().numpy(), want_sc)
    assert np.array_equal(q8.cpu().numpy(), want_q8)


@pytest.mark.gpu
def test_exchange_kernel_quantises_what_it_received(cuda_device):
    """The exchange step of the head-split decode layer with the quantisation folded in (one rank: no waiting):
    rows [B, H*d] in the receive slot -> int8 codes + scales, no fp32 copy."""
    import torch
    B, H = 5, 12
    g = torch.Generator(device="cuda")
    g.manual_seed(10)
    recv = torch.randn((B, H, 1, 128), generator=g, device="cuda") * 2.0
    recv[3] = 0.0
    q8 = torch.full((B, 1, H * 128), 99, dtype=torch.int8, device="cuda")
    sc = torch.full((B,), float("nan"), device="cuda")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    A.peer_exchange(rank=0, size=1, epoch=1, flags_local=flags.data_ptr(), flags_peer=[0], recv=recv.data_ptr(), nbytes=recv.numel() * 4,
                    out_q8=q8.data_ptr(), out_q8_scale=sc.data_ptr(), q8_rows=B, q8_row_elems=H * 128)
    torch.cuda.synchronize()
    want_q8, want_sc = oracle.attn_quantize(recv.cpu().numpy())
    assert np.array_equal(sc.cpu().numpy(), want_sc)
    assert np.array_equal(q8.cpu().numpy(), want_q8)
