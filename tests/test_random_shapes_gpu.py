"""Seeded random shapes, lengths, dtypes, masks and split sizes through the C ABI against the oracle."""
import numpy as np
import pytest

from fasterllama_b200 import attention as A
from fasterllama_b200 import workloads as W

from util import FP16_ABS, assert_abs_close, assert_fp32_close, run_cuda, run_oracle

pytestmark = pytest.mark.gpu
MASKS = [A.FLB_MASK_NONE, A.FLB_MASK_GENERIC, A.FLB_MASK_CAUSAL_INCLUSIVE, A.FLB_MASK_CAUSAL_STRICT]


@pytest.mark.parametrize("seed", range(16))
def test_random_decode(cuda_device, seed):
    rng = np.random.default_rng(1000 + seed)
    B, H = int(rng.integers(1, 6)), int(rng.integers(1, 10))
    T = int(rng.integers(2, 1400))
    per_seq = bool(rng.integers(0, 2))
    past = rng.integers(0, T, size=B).astype(np.int32) if per_seq else int(rng.integers(0, T))
    in_dtype = ["int32", "float32", "float16"][int(rng.integers(0, 3))]
    cache = ["float32", "float16"][int(rng.integers(0, 2))]
    out = "float32" if cache == "float32" else ["float32", "float16"][int(rng.integers(0, 2))]
    case = W.host_case(f"rnd-dec-{seed}", 2000 + seed, B, H, T, past=past, in_dtype=in_dtype, cache_dtype=cache, out_dtype=out,
                       rope=["past", "reference", "none"][int(rng.integers(0, 3))], mask_mode=MASKS[int(rng.integers(0, 4))],
                       split_len=int(rng.choice([0, 32, 64, 128, 256, 1024])))
    cuda, orc = run_cuda(case, calls=2), run_oracle(case)
    assert cuda["status"] == 0
    if cache == "float16" or out == "float16":
        assert_abs_close(cuda["out"], orc["out"].astype(np.float32), FP16_ABS, case.name)
    else:
        assert_fp32_close(cuda["out"], orc["out"], what=case.name)
    assert np.array_equal(cuda["v_cache"], orc["v_cache"].astype(np.float32))


@pytest.mark.parametrize("seed", range(8))
def test_random_decode_early_start(cuda_device, seed):
    """The same kind of draw with zeroed scratch, programmatic dependent launch and three calls in a row."""
    import torch

    rng = np.random.default_rng(5000 + seed)
    B, H = int(rng.integers(1, 6)), int(rng.integers(1, 10))
    T = int(rng.integers(2, 1400))
    per_seq = bool(rng.integers(0, 2))
    past = rng.integers(0, T, size=B).astype(np.int32) if per_seq else int(rng.integers(0, T))
    in_dtype = ["int32", "float32", "float16"][int(rng.integers(0, 3))]
    cache = ["float32", "float16"][int(rng.integers(0, 2))]
    case = W.host_case(f"rnd-early-{seed}", 6000 + seed, B, H, T, past=past, in_dtype=in_dtype, cache_dtype=cache, out_dtype="float32",
                       rope=["past", "reference", "none"][int(rng.integers(0, 3))], mask_mode=MASKS[int(rng.integers(0, 4))],
                       split_len=int(rng.choice([0, 64, 256])))
    orc = run_oracle(case)
    dev = W.to_device(case, cuda_device)
    dev["scratch"].zero_()
    case.scratch_zeroed = True
    case.early_start = 1 + seed % 2
    p = case.params(dev)
    assert p.early_start == 1 + seed % 2 and p.scratch_zeroed == 1
    for _ in range(3):
        A.decode(p)
    torch.cuda.synchronize()
    assert A.scratch_status(dev["scratch"]) == 0
    got = dev["out"].float().cpu().numpy()
    if cache == "float16":
        assert_abs_close(got, orc["out"].astype(np.float32), FP16_ABS, case.name)
    else:
        assert_fp32_close(got, orc["out"], what=case.name)
    assert np.array_equal(dev["v_cache"].float().cpu().numpy(), orc["v_cache"].astype(np.float32))


@pytest.mark.parametrize("seed", range(10))
def test_random_prefill(cuda_device, seed):
    rng = np.random.default_rng(3000 + seed)
    B, H = int(rng.integers(1, 4)), int(rng.integers(1, 7))
    S = int(rng.integers(2, 700))
    T = S + int(rng.integers(0, 50))
    in_dtype = ["int32", "float32", "float16"][int(rng.integers(0, 3))]
    cache = ["float32", "float16"][int(rng.integers(0, 2))]
    case = W.host_case(f"rnd-pre-{seed}", 4000 + seed, B, H, T, S=S, past=0, in_dtype=in_dtype, cache_dtype=cache,
                       out_dtype=["float32", "float16"][int(rng.integers(0, 2))],
                       rope=["past", "reference", "none"][int(rng.integers(0, 3))], mask_mode=MASKS[int(rng.integers(0, 4))])
    cuda, orc = run_cuda(case), run_oracle(case, f16_operands=True)
    assert cuda["status"] == 0
    # value magnitudes of the int32 path reach ~5: the bound scales with them (fp16 rounding of P and V)
    scale = max(1.0, float(np.abs(orc["v_cache"].astype(np.float32)).max()) / 4.0)
    assert_abs_close(cuda["out"], orc["out"].astype(np.float32), FP16_ABS * scale, case.name)
    assert np.array_equal(cuda["v_cache"][:, :, :S], orc["v_cache"].astype(np.float32)[:, :, :S])
