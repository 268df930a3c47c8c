"""q, k and v as column blocks of one wider buffer (flb_attn_params.qkv_row_stride): the form a merged QKV
projection leaves them in — one [B*S, 3*H*d] buffer instead of the reference's three GEMM outputs
(fasterLlama/cuda/open_decoder.cu:105-136).  Strided inputs must give exactly what dense inputs give."""
import numpy as np
import pytest

from fasterllama_b200 import _lib
from fasterllama_b200 import attention as A
from fasterllama_b200 import workloads as W

from util import run_cuda, run_oracle


def _merged(case, pad: int = 0):
    """The case's q, k, v re-housed as three column blocks of one [B, S, 3*H*d + pad] buffer."""
    a = dict(case.arrays)
    B, S, H, d = a["q"].shape
    row = 3 * H * d + pad
    buf = np.zeros((B, S, row), dtype=a["q"].dtype)
    for i, n in enumerate(("q", "k", "v")):
        buf[:, :, i * H * d:(i + 1) * H * d] = a[n].reshape(B, S, H * d)
        a[n] = buf[:, :, i * H * d:(i + 1) * H * d].reshape(B, S, H, d)  # a view: strides (S*row, row, d, 1)
        assert not a[n].flags["C_CONTIGUOUS"] or (B * S == 1)
    a["_merged"] = buf
    import copy

    c = copy.copy(case)
    c.arrays = a
    return c


@pytest.mark.parametrize("in_dtype,S", [("int32", 1), ("float16", 1), ("float32", 5), ("int32", 70)])
def test_oracle_reads_strided_rows(in_dtype, S):
    past = 0 if S > 1 else np.array([33, 7, 100], dtype=np.int32)
    case = W.host_case("stride", 900 + S, 3, 4, 128 + S, S=S, past=past, in_dtype=in_dtype)
    dense = run_oracle(case)
    merged = run_oracle(_merged(case, pad=8))
    for k in ("out", "k_cache", "v_cache"):
        assert np.array_equal(dense[k], merged[k]), k


def test_params_carry_the_stride_and_validate_checks_it():
    case = W.host_case("stride-v", 7, 2, 4, 64, past=10, in_dtype="float16")
    case.arrays["scratch"] = np.zeros(A.workspace_bytes(2, 4, 64), dtype=np.uint8)
    m = _merged(case)
    p = m.params()
    assert p.qkv_row_stride == 3 * 4 * 128
    assert A.validate(p) == _lib.FLB_OK
    p.qkv_row_stride = 4 * 128 - 8  # rows would overlap
    assert A.validate(p) == _lib.FLB_ERR_BAD_SHAPE
    p.qkv_row_stride = 3 * 4 * 128 + 4  # 8-byte multiple only: breaks the 16-byte rule for fp16 rows
    assert A.validate(p) == _lib.FLB_ERR_MISALIGNED
    assert case.params().qkv_row_stride == 0  # dense inputs leave the field at its default


@pytest.mark.gpu
@pytest.mark.parametrize("in_dtype,cache_dtype", [("int32", "float32"), ("float16", "float16")])
def test_decode_strided_equals_dense(cuda_device, in_dtype, cache_dtype):
    past = np.array([700, 3, 513, 64], dtype=np.int32)
    case = W.host_case("stride-d", 31, 4, 8, 800, past=past, in_dtype=in_dtype, cache_dtype=cache_dtype)
    want, got = run_cuda(case), run_cuda(_merged(case))
    assert want["status"] == 0 and got["status"] == 0
    for k in ("out", "k_cache", "v_cache"):
        assert np.array_equal(want[k], got[k]), k


@pytest.mark.gpu
@pytest.mark.parametrize("in_dtype,cache_dtype", [("int32", "float32"), ("float16", "float16")])
def test_prefill_strided_equals_dense(cuda_device, in_dtype, cache_dtype):
    case = W.host_case("stride-p", 32, 2, 4, 300, S=260, past=0, in_dtype=in_dtype, cache_dtype=cache_dtype, rope="reference")
    want, got = run_cuda(case), run_cuda(_merged(case, pad=16))
    assert want["status"] == 0 and got["status"] == 0
    for k in ("out", "k_cache", "v_cache"):
        assert np.array_equal(want[k], got[k]), k
