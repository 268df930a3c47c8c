"""Attention at the head sizes other than 128 that the call accepts: decode at 64 and 256 (the reference's kernels take
size_per_head <= 128 on their warp forms and 256 on their block forms, fasterLlama/cuda/decoder_kernels.cu:563-589),
prefill at 64.
CPU: the oracle against the vectors the reference's own kernels produced at these sizes
(tests/golden/ref_golden_head_sizes.npz), and the argument checks.  GPU: the CUDA path against the oracle and against
those vectors."""
import numpy as np
import pytest

from fasterllama_b200 import _lib
from fasterllama_b200 import attention as A
from fasterllama_b200 import workloads as W

import golden_util as GU
from util import FP16_ABS, assert_abs_close, assert_fp32_close, run_cuda, run_oracle

HEAD_SIZES = [64, 256]
GOLDEN = [c for c in GU.G.HEAD_SIZE_CASES if c.startswith("decode")]
GOLDEN_PREFILL = [c for c in GU.G.HEAD_SIZE_CASES if c.startswith("prefill")]
needs_fixture = pytest.mark.skipif(not GU.head_size_fixture_present(), reason="tests/golden/ref_golden_head_sizes.npz not generated")


# ---------------------------------------------------------------------------------------------------- CPU
@needs_fixture
@pytest.mark.parametrize("name", GOLDEN)
def test_oracle_matches_reference_golden_at_other_head_sizes(name):
    """The oracle's decode path against the reference's own kernels (corrected gemv arguments), 1e-5 relative."""
    case = GU.case_from_golden(name)
    r = run_oracle(case)
    GU.compare_with_golden(name, r["out"], r["k_cache"], r["v_cache"], tol_out_abs=None, rel=1e-5)


@needs_fixture
@pytest.mark.parametrize("name", GOLDEN_PREFILL)
def test_oracle_matches_reference_golden_prefill_at_head_size_64(name):
    """The oracle's prefill path against the reference's chain, within what the reference's fp16 tensor-core
    contractions leave (measured up to 2.5e-3 from exact arithmetic)."""
    case = GU.case_from_golden(name)
    r = run_oracle(case)
    GU.compare_with_golden(name, r["out"], r["k_cache"], r["v_cache"], tol_out_abs=GU.REF_PREFILL_ABS)


@needs_fixture
def test_head_size_fixture_notes():
    """Every case of the fixture ran through the reference's kernels with status 0."""
    import json
    import os
    f = np.load(os.path.join(GU.HERE, "golden", "ref_golden_head_sizes.npz"))
    notes = json.loads(bytes(f["notes_json"]).decode())
    assert all(notes[c]["status"] == 0 and notes[c]["nan_rows"] == 0 for c in GOLDEN), notes
    # a strict mask leaves token 0 of every (batch, head) without a key: the reference's softmax gives NaN there
    for c in GOLDEN_PREFILL:
        kept = GU.G.case(c)
        want_nan = kept["B"] * kept["H"] if kept["mask"] == "strict" else 0
        assert notes[c]["status"] == 0 and notes[c]["nan_rows"] == want_nan, notes


def _validate(case, arrays):
    import ctypes
    return _lib.load_library().flb_attn_validate(ctypes.byref(case.params(arrays)))


@pytest.mark.parametrize("d,S,want", [(64, 1, "ok"), (256, 1, "ok"), (128, 1, "ok"), (64, 4, "ok"), (128, 4, "ok"), (256, 4, "unsupported"),
                                      (96, 1, "unsupported"), (96, 4, "unsupported"), (512, 1, "unsupported")])
def test_which_head_sizes_the_call_accepts(d, S, want):
    """Host-side argument check only (no launch): decode takes 64, 128 and 256; prefill is built for 64 and 128."""
    case = W.host_case("hs", 1, 1, 4, 64, S=S, past=0 if S > 1 else 9, d=d)
    arrays = dict(case.arrays)
    arrays["scratch"] = np.zeros(1 << 20, dtype=np.uint8)
    st = _validate(case, arrays)
    assert st == (_lib.FLB_OK if want == "ok" else _lib.FLB_ERR_UNSUPPORTED), (d, S, st)


# ---------------------------------------------------------------------------------------------------- GPU
def _check(case, cuda, orc, fp16):
    assert cuda["status"] == 0, f"kernel status word {cuda['status']:#x}"
    if fp16:
        assert_abs_close(cuda["out"], orc["out"].astype(np.float32), FP16_ABS, case.name + " out")
    else:
        assert_fp32_close(cuda["out"], orc["out"], what=case.name + " out")
    kc, ko = cuda["k_cache"], orc["k_cache"].astype(np.float32)
    tol = 2e-3 if fp16 else 1e-5
    assert np.abs(kc - ko).max() <= tol * max(1.0, np.abs(ko).max())
    assert np.array_equal(cuda["v_cache"], orc["v_cache"].astype(np.float32)), "V cache differs (append is a pure copy/round)"


@pytest.mark.gpu
@pytest.mark.parametrize("d", HEAD_SIZES)
@pytest.mark.parametrize("past", [0, 1, 7, 8, 15, 16, 17, 31, 32, 33, 63, 64, 65, 255, 256, 257, 511, 512, 513, 1025])
def test_fp32_decode_lengths(cuda_device, d, past):
    """Every tile boundary of the two sizes' kernels (8 / 32 rows with an fp32 cache) and the partition boundaries."""
    case = W.host_case(f"d{d}-fp32-L{past}", 900 + past + d, 1, 4, 1100, past=past, d=d)
    _check(case, run_cuda(case), run_oracle(case), fp16=False)


@pytest.mark.gpu
@pytest.mark.parametrize("d", HEAD_SIZES)
@pytest.mark.parametrize("past", [0, 3, 15, 16, 17, 63, 64, 65, 127, 128, 129, 511, 512, 513, 900])
def test_fp16_decode_lengths(cuda_device, d, past):
    case = W.host_case(f"d{d}-fp16-L{past}", 1900 + past + d, 2, 4, 1100, past=past, in_dtype="float16", cache_dtype="float16",
                       out_dtype="float16", d=d)
    _check(case, run_cuda(case), run_oracle(case), fp16=True)


@pytest.mark.gpu
@pytest.mark.parametrize("d", HEAD_SIZES)
@pytest.mark.parametrize("mask_mode", [A.FLB_MASK_NONE, A.FLB_MASK_GENERIC, A.FLB_MASK_CAUSAL_INCLUSIVE, A.FLB_MASK_CAUSAL_STRICT])
def test_mask_modes_int32_inputs_ragged_lengths(cuda_device, d, mask_mode):
    """The reference's input form (int32 accumulators + scales), a length per sequence, several partitions, every mask."""
    lens = np.array([0, 5, 300, 1500, 513], dtype=np.int32)
    case = W.host_case(f"d{d}-mask{mask_mode}", 77 + d + mask_mode, len(lens), 8, 1600, past=lens, in_dtype="int32", mask_mode=mask_mode,
                       split_len=512, d=d)
    _check(case, run_cuda(case), run_oracle(case), fp16=False)


@pytest.mark.gpu
@pytest.mark.parametrize("d", HEAD_SIZES)
def test_calls_repeat_bit_for_bit_on_one_scratch(cuda_device, d):
    """Calls on the same scratch (counters left at zero by each) give the same bits, early-start launches included (each
    call appends the same row again)."""
    import dataclasses
    import torch
    lens = np.array([700, 64, 1300], dtype=np.int32)
    case = W.host_case(f"d{d}-repeat", 5 + d, len(lens), 4, 1400, past=lens, d=d, split_len=256)
    dev = W.to_device(case)
    dev["scratch"].zero_()
    outs = []
    for es in (0, 0, 1, 2):
        c = dataclasses.replace(case, early_start=es)
        dev["out"].fill_(float("nan"))
        A.forward(c.params(dev))
        torch.cuda.synchronize()
        assert A.scratch_status(dev["scratch"]) == 0
        outs.append(dev["out"].clone())
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    assert_fp32_close(outs[0].cpu().numpy(), run_oracle(case)["out"], what=f"d{d} out")


@pytest.mark.gpu
@pytest.mark.parametrize("d", HEAD_SIZES)
def test_fused_output_quantisation(cuda_device, d):
    """The reference's next kernel folded into the decode call (absmax over all heads of a row, rni codes): bit-exact
    against the oracle at the other head sizes as well."""
    import torch
    from oracle import oracle
    lens = np.array([0, 5, 300, 1500], dtype=np.int32)
    case = W.host_case(f"d{d}-q8", 61 + d, len(lens), 8, 1600, past=lens, in_dtype="int32", d=d)
    dev = W.to_device(case)
    dev["scratch"].zero_()
    dev["out_q8"] = torch.zeros((case.B, 1, case.H * d), dtype=torch.int8, device="cuda:0")
    dev["out_q8_scale"] = torch.zeros((case.B,), dtype=torch.float32, device="cuda:0")
    p = case.params(dev)
    for _ in range(2):
        A.forward(p)
    torch.cuda.synchronize()
    assert A.scratch_status(dev["scratch"]) == 0
    want_q8, want_sc = oracle.attn_quantize(dev["out"].cpu().numpy())
    assert np.array_equal(dev["out_q8_scale"].cpu().numpy(), want_sc)
    assert np.array_equal(dev["out_q8"].cpu().numpy().reshape(want_q8.shape), want_q8)


@needs_fixture
@pytest.mark.gpu
@pytest.mark.parametrize("name", GOLDEN)
@pytest.mark.parametrize("mask_mode", ["generic", "index"])
def test_decode_matches_reference_golden(cuda_device, name, mask_mode):
    case = GU.case_from_golden(name, mask_mode=mask_mode)
    r = run_cuda(case)
    assert r["status"] == 0
    GU.compare_with_golden(name, r["out"], r["k_cache"], r["v_cache"], tol_out_abs=None, rel=1e-5)


@needs_fixture
@pytest.mark.gpu
@pytest.mark.parametrize("name", GOLDEN)
def test_fp16_cache_decode_matches_reference_golden(cuda_device, name):
    case = GU.case_from_golden(name, mask_mode="index", cache_dtype="float16", out_dtype="float16")
    r = run_cuda(case)
    assert r["status"] == 0
    GU.compare_with_golden(name, r["out"], r["k_cache"], r["v_cache"], tol_out_abs=2e-3, cache_tol=2e-3)


# ---------------------------------------------------------------------------------------------------- GPU, prefill at 64
def _check_prefill(case, cuda, orc, cache16):
    assert cuda["status"] == 0, f"kernel status word {cuda['status']:#x}"
    assert_abs_close(cuda["out"], orc["out"].astype(np.float32), FP16_ABS, case.name + " out")
    S = case.S
    ko = orc["k_cache"].astype(np.float32)[:, :, :S]
    tol = 2e-3 if cache16 else 1e-5
    assert np.abs(cuda["k_cache"][:, :, :S] - ko).max() <= tol * max(1.0, np.abs(ko).max())
    assert np.array_equal(cuda["v_cache"][:, :, :S], orc["v_cache"].astype(np.float32)[:, :, :S])
    assert not cuda["k_cache"][:, :, S:].any() and not cuda["v_cache"][:, :, S:].any()  # rows behind the prompt untouched


@pytest.mark.gpu
@pytest.mark.parametrize("S", [2, 17, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300, 384, 513, 640, 1000])
def test_prefill_d64_lengths_fp16_cache(cuda_device, S):
    """Every boundary of the 64-key tiles, the 128-row query tiles and the 256-row work items."""
    case = W.host_case(f"pf64-S{S}", 2400 + S, 1, 3, S + 40, S=S, past=0, in_dtype="float32", cache_dtype="float16", rope="past", d=64)
    _check_prefill(case, run_cuda(case), run_oracle(case), cache16=True)


@pytest.mark.gpu
@pytest.mark.parametrize("S", [5, 128, 260, 520])
def test_prefill_d64_reference_data_path(cuda_device, S):
    """int32 accumulators + scales in, fp32 cache, fp32 output; the oracle rounds the operands to fp16 as the tensor
    cores (and the reference's own FAST_16F GEMMs) do; the cache rows stay unrounded."""
    case = W.host_case(f"pf64-i32-S{S}", 2500 + S, 2, 4, S + 9, S=S, past=0, in_dtype="int32", rope="reference", d=64)
    _check_prefill(case, run_cuda(case), run_oracle(case, f16_operands=True), cache16=False)


@pytest.mark.gpu
@pytest.mark.parametrize("mask_mode", [A.FLB_MASK_NONE, A.FLB_MASK_GENERIC, A.FLB_MASK_CAUSAL_INCLUSIVE, A.FLB_MASK_CAUSAL_STRICT])
@pytest.mark.parametrize("S", [60, 256, 300, 700])
def test_prefill_d64_half_inputs_half_cache_every_mask(cuda_device, mask_mode, S):
    """fp16 q/k/v into an fp16 cache (the V tiles come from the caller's rows and the kernel appends them to the cache):
    the appended V rows are the input bit for bit."""
    case = W.host_case(f"pf64-direct{mask_mode}-S{S}", 2650 + S, 2, 3, S + 70, S=S, past=0, in_dtype="float16", cache_dtype="float16",
                       out_dtype="float16", mask_mode=mask_mode, d=64)
    cuda = run_cuda(case)
    _check_prefill(case, cuda, run_oracle(case), cache16=True)
    v_in = np.transpose(case.arrays["v"].astype(np.float32), (0, 2, 1, 3))  # [B,S,H,d] -> [B,H,S,d]
    assert np.array_equal(cuda["v_cache"][:, :, :S], v_in)


@pytest.mark.gpu
def test_prefill_d64_then_decode_continues_the_cache(cuda_device):
    """Prefill, then one decode step on the same cache: equals the oracle doing the same."""
    import torch
    from oracle import oracle
    S, T, B, H, d = 150, 200, 2, 4, 64
    pre = W.host_case("pd64-pre", 91, B, H, T, S=S, past=0, in_dtype="float16", cache_dtype="float16", out_dtype="float32", d=d)
    host = {k: np.array(v, copy=True) for k, v in pre.arrays.items()}
    oracle.attention(pre.params(host))
    dev = W.to_device(pre)
    A.forward(pre.params(dev))
    dec = W.host_case("pd64-dec", 92, B, H, T, past=S, in_dtype="float16", cache_dtype="float16", out_dtype="float32", d=d)
    hd = {k: np.array(v, copy=True) for k, v in dec.arrays.items()}
    hd["k_cache"], hd["v_cache"] = host["k_cache"], host["v_cache"]
    oracle.attention(dec.params(hd))
    dd = W.to_device(dec)
    dd["k_cache"], dd["v_cache"] = dev["k_cache"], dev["v_cache"]
    A.forward(dec.params(dd))
    torch.cuda.synchronize()
    assert A.scratch_status(dd["scratch"]) == 0
    assert_abs_close(dd["out"].cpu().numpy(), hd["out"], FP16_ABS, "decode after prefill at head size 64")


@pytest.mark.gpu
def test_prefill_d64_fused_output_quantisation(cuda_device):
    """The reference's quantise + transpose kernel behind the prefill call, and as a call of its own: bit-exact against
    the oracle on the call's own fp32 output."""
    import torch
    from oracle import oracle
    case = W.host_case("pf64-q8", 93, 2, 4, 300, S=260, past=0, in_dtype="int32", d=64)
    dev = W.to_device(case)
    dev["out_q8"] = torch.zeros((case.B, case.S, case.H * 64), dtype=torch.int8, device="cuda:0")
    dev["out_q8_scale"] = torch.zeros((case.B, case.S), dtype=torch.float32, device="cuda:0")
    A.forward(case.params(dev))
    torch.cuda.synchronize()
    assert A.scratch_status(dev["scratch"]) == 0
    want_q8, want_sc = oracle.attn_quantize(dev["out"].cpu().numpy())
    assert np.array_equal(dev["out_q8_scale"].cpu().numpy().reshape(want_sc.shape), want_sc)
    assert np.array_equal(dev["out_q8"].cpu().numpy().reshape(want_q8.shape), want_q8)


@needs_fixture
@pytest.mark.gpu
@pytest.mark.parametrize("name", GOLDEN_PREFILL)
@pytest.mark.parametrize("mask_mode", ["generic", "index"])
def test_prefill_d64_matches_reference_golden(cuda_device, name, mask_mode):
    case = GU.case_from_golden(name, mask_mode=mask_mode)
    r = run_cuda(case)
    assert r["status"] == 0
    GU.compare_with_golden(name, r["out"], r["k_cache"], r["v_cache"], tol_out_abs=GU.REF_PREFILL_ABS)
