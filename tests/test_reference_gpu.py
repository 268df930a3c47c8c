"""The CUDA path against the REFERENCE's own kernels: the committed golden vectors, and — when the
reference runner library was built and travelled with the tree — a live side-by-side run."""
import numpy as np
import pytest

from fasterllama_b200 import attention as A
from fasterllama_b200 import workloads as W
from oracle import ref_runner

import golden_util as GU
from util import run_cuda

pytestmark = pytest.mark.gpu

DECODE = [c for c in GU.G.CASES if c.startswith("decode")]


@pytest.mark.parametrize("mask_mode", ["generic", "index"])
@pytest.mark.parametrize("name", DECODE)
def test_decode_matches_reference_golden(cuda_device, name, mask_mode):
    """fp32 cache, int32 inputs — the reference's exact data path; 1e-5 relative."""
    case = GU.case_from_golden(name, mask_mode=mask_mode)
    r = run_cuda(case)
    assert r["status"] == 0
    GU.compare_with_golden(name, r["out"], r["k_cache"], r["v_cache"], tol_out_abs=None, rel=1e-5)


@pytest.mark.parametrize("name", DECODE)
def test_fp16_cache_decode_matches_reference_golden(cuda_device, name):
    """fp16 cache (the cached rows of the golden inputs are exact in fp16): 2e-3 absolute."""
    case = GU.case_from_golden(name, mask_mode="index", cache_dtype="float16", out_dtype="float16")
    r = run_cuda(case)
    assert r["status"] == 0
    GU.compare_with_golden(name, r["out"], r["k_cache"], r["v_cache"], tol_out_abs=2e-3, cache_tol=2e-3)


@pytest.mark.skipif(not ref_runner.available(), reason="reference runner library not built")
@pytest.mark.parametrize("past", [0, 127, 256, 1000])
def test_live_reference_decode(cuda_device, past):
    """Seeded random int32 inputs through the reference's kernels (corrected gemv arguments) and
    through the CUDA path, same device buffers' contents; 1e-5 relative."""
    import torch

    B, H, T = 2, 8, 1100
    case = W.host_case(f"live-{past}", 900 + past, B, H, T, past=past, in_dtype="int32", rope="reference",
                       mask_mode=A.FLB_MASK_CAUSAL_INCLUSIVE)
    mine = run_cuda(case)
    assert mine["status"] == 0
    ref = ref_runner.RefRunner()
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).cuda() for k, v in case.arrays.items()}
    t["attn_mask"] = torch.from_numpy(W.causal_mask(T, strict=False)).cuda()
    st = ref.attention(ref.make_args(t, start_pos=past, rope_row=0))
    torch.cuda.synchronize()
    assert st == 0
    from util import assert_fp32_close
    assert_fp32_close(mine["out"], t["out"].cpu().numpy(), what="vs live reference")
    assert np.abs(mine["k_cache"] - t["k_cache"].cpu().numpy()).max() <= 1e-5
    assert np.array_equal(mine["v_cache"], t["v_cache"].cpu().numpy())
    ref.close()
