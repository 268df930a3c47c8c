"""The allocation-free decode entry point (flb_attn_decode_static_scratch) against the regular one.

Some callers have no device memory of their own to offer as scratch — a plugin that only ever sees
its input and output tensors, or a server that may not call the allocator while it is serving.  For
them the library carries one fixed scratch block per GPU.  This file checks that decoding through
that block gives what the regular entry point gives, twice in a row on different inputs (the
second call finds the first call's leftovers in the block), and that a call too large for the
block is refused before anything is launched.  It is named to be collected last."""
import ctypes as C

import numpy as np
import pytest

from fasterllama_b200 import _lib
from fasterllama_b200 import attention as A
from fasterllama_b200 import workloads as W

from util import FP16_ABS, assert_abs_close


def _run_both(case, device="cuda:0"):
    import torch

    dev = W.to_device(case, device)
    A.decode(case.params(dev))                      # regular entry point, caller's scratch
    torch.cuda.synchronize()
    want = dev["out"].float().cpu().numpy()
    want_k = dev["k_cache"].float().cpu().numpy()

    dev2 = W.to_device(case, device)
    dev2.pop("scratch")                             # nothing to give
    dev2["out"].fill_(float("nan"))
    p = case.params(dev2)
    assert not p.scratch and p.scratch_bytes == 0
    A.decode_static_scratch(p)
    torch.cuda.synchronize()
    got = dev2["out"].float().cpu().numpy()
    got_k = dev2["k_cache"].float().cpu().numpy()
    return got, want, got_k, want_k


@pytest.mark.gpu
def test_static_scratch_matches_regular_entry_point_twice(cuda_device):
    # first call: ragged lengths with several partitions per sequence
    lens = np.array([1500, 3, 600, 1024, 0, 513], dtype=np.int32)
    first = W.host_case("noalloc-1", 41, 6, 8, 1600, past=lens, in_dtype="float16", cache_dtype="float16", out_dtype="float32")
    got, want, gk, wk = _run_both(first)
    assert_abs_close(got, want, FP16_ABS, "static scratch, first call")
    assert np.array_equal(gk, wk)
    # second call straight after, other shapes and lengths: the block still holds the first call's partials
    lens2 = np.array([700, 1100], dtype=np.int32)
    second = W.host_case("noalloc-2", 42, 2, 16, 1200, past=lens2, split_len=256)
    got, want, gk, wk = _run_both(second)
    from util import assert_fp32_close
    assert_fp32_close(got, want, what="static scratch, second call")
    assert np.array_equal(gk, wk)


@pytest.mark.gpu
def test_static_scratch_status_reports_a_bad_length(cuda_device):
    """The kernels' error word lives inside the library's block, out of the caller's reach: the accessor reads it.
    A cached length beyond the slab (a caller bug) is clamped by the kernel and reported as bit 4; the next
    well-formed call through the same entry point starts from a clean word again."""
    import torch

    assert A.static_scratch_status() in (0, 4)  # whatever an earlier test left; never a wait that ran out
    lens = np.array([100, 50], dtype=np.int32)
    case = W.host_case("noalloc-bad", 43, 2, 4, 256, past=lens)
    case.max_past_len = 255
    dev = W.to_device(case, cuda_device)
    dev.pop("scratch")
    good = case.params(dev)
    A.decode_static_scratch(good)
    torch.cuda.synchronize()
    assert A.static_scratch_status() == 0
    want = dev["out"].float().cpu().numpy().copy()
    dev["past_lens"] = torch.tensor([100, 100000], dtype=torch.int32, device=cuda_device)  # second entry is nonsense
    A.decode_static_scratch(case.params(dev))
    torch.cuda.synchronize()
    assert A.static_scratch_status() & 4, "the clamped length was not reported"
    dev["past_lens"] = torch.from_numpy(lens).to(cuda_device)
    A.decode_static_scratch(case.params(dev))
    torch.cuda.synchronize()
    assert A.static_scratch_status() == 0
    assert np.array_equal(dev["out"].float().cpu().numpy()[0], want[0])  # the sequence with a valid length


def test_static_scratch_refuses_what_does_not_fit():
    """Host-side check only: a batch whose partitions overflow the fixed block is refused with
    FLB_ERR_TOO_LARGE before any CUDA call."""
    lib = _lib.load_library()
    c = W.host_case("big", 1, 1, 4, 64, past=10)
    p = c.params()
    # pretend a huge batch: 4096 sequences x 64 heads x 8 partitions of 520 bytes > 16 MiB
    p.batch_size, p.head_num, p.total_len, p.start_pos = 4096, 64, 4097, 4096
    assert lib.flb_attn_decode_static_scratch(C.byref(p), None) == _lib.FLB_ERR_TOO_LARGE
    p = c.params()
    p.seq_len = 2
    assert lib.flb_attn_decode_static_scratch(C.byref(p), None) == _lib.FLB_ERR_BAD_SHAPE
    assert lib.flb_attn_decode_static_scratch(None, None) == _lib.FLB_ERR_NULL_POINTER
