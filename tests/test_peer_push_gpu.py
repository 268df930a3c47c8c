"""The push form of the head-split decode layer on ONE GPU: the kernel stores its rows into several
destination buffers at a head offset, and the exchange kernel's wait is bounded (a flag that nothing sets makes
it run out and report through the status word, with the context still usable).  The two-GPU run of the same
path is in test_tp_gpu.py."""
import numpy as np
import pytest
import torch

from fasterllama_b200 import _lib
from fasterllama_b200 import attention as A
from fasterllama_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("out_dtype", ["float32", "float16"])
@pytest.mark.parametrize("past", [np.array([700, 5, 1299], dtype=np.int32), np.array([0, 64, 31], dtype=np.int32)])
def test_rows_land_in_every_destination_at_the_head_offset(cuda_device, past, out_dtype):
    B, H, T = 3, 8, 1300
    case = W.host_case("push", 21, B, H, T, past=past, in_dtype="float16", cache_dtype="float16", out_dtype=out_dtype)
    dev = W.to_device(case, cuda_device)
    A.forward(case.params(dev))
    torch.cuda.synchronize()
    want = dev["out"].clone()

    # the same heads computed as two "ranks" of 4 heads, each pushing into both full-size buffers
    dt = dev["out"].dtype
    full = [torch.full((B, H, 1, 128), float("nan"), dtype=dt, device=cuda_device) for _ in range(2)]
    half = H // 2
    for r in range(2):
        fresh = W.to_device(case, cuda_device)
        loc = {k: v for k, v in fresh.items()}
        for name in ("q", "k", "v"):
            loc[name] = fresh[name][:, :, r * half:(r + 1) * half].contiguous()
        for name in ("k_cache", "v_cache"):
            loc[name] = fresh[name][:, r * half:(r + 1) * half].contiguous()
        loc["scratch"] = torch.zeros(A.workspace_bytes(B, half, T), dtype=torch.uint8, device=cuda_device)
        part = W.Case(name="p", B=B, H=half, S=1, T=T, start_pos=0, arrays=loc, rope_add_past=True, mask_mode=case.mask_mode,
                      max_past_len=case.max_past_len)
        A.decode(part.params(loc, out_peers=[t.data_ptr() for t in full], out_head_total=H, out_head_offset=r * half))
        torch.cuda.synchronize()
        assert A.scratch_status(loc["scratch"]) == 0
    for t in full:
        assert torch.equal(t, want)


def test_exchange_of_one_rank_is_a_copy(cuda_device):
    src = torch.arange(4096, dtype=torch.float32, device=cuda_device)
    dst = torch.zeros_like(src)
    flags = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    A.peer_exchange(rank=0, size=1, epoch=1, flags_local=flags.data_ptr(), flags_peer=[0], recv=src.data_ptr(), dst=dst.data_ptr(),
                    nbytes=src.numel() * 4)
    torch.cuda.synchronize()
    assert torch.equal(src, dst)


def test_exchange_signals_waits_and_copies(cuda_device):
    """Both directions on one GPU: "rank 1" is a second flag array in local memory.  Rank 0's kernel finds its
    peer's word already at the epoch (set by hand), writes its own word into the peer's array, and copies."""
    mine = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    theirs = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    mine[1] = 5  # rank 1 has published epochs up to 5 here
    src = torch.randn(1000 * 4, device=cuda_device)
    dst = torch.zeros_like(src)
    A.peer_exchange(rank=0, size=2, epoch=5, flags_local=mine.data_ptr(), flags_peer=[0, theirs.data_ptr()], recv=src.data_ptr(),
                    dst=dst.data_ptr(), nbytes=src.numel() * 4, status=status.data_ptr(), timeout_ms=200)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert int(theirs[0]) == 5 and int(theirs[1]) == 0
    assert torch.equal(src, dst)


def test_a_wait_that_runs_out_reports_and_returns(cuda_device):
    mine = torch.zeros(64, dtype=torch.int32, device=cuda_device)  # nobody will ever write word 1
    theirs = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    src = torch.ones(4096, device=cuda_device)
    dst = torch.zeros_like(src)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    A.peer_exchange(rank=0, size=2, epoch=1, flags_local=mine.data_ptr(), flags_peer=[0, theirs.data_ptr()], recv=src.data_ptr(),
                    dst=dst.data_ptr(), nbytes=src.numel() * 4, status=status.data_ptr(), timeout_ms=50)
    t1.record()
    torch.cuda.synchronize()  # returns: the kernel gave up by itself
    assert 40.0 <= t0.elapsed_time(t1) < 1000.0
    assert int(status[0]) & _lib.FLB_STATUS_PEER_WAIT
    assert int(theirs[0]) == 1  # it had signalled before it waited
    assert float(dst.abs().sum()) == 0.0  # no copy of rows that may be incomplete
    # the context is intact: the next call works
    mine[1] = 2
    status.zero_()
    A.peer_exchange(rank=0, size=2, epoch=2, flags_local=mine.data_ptr(), flags_peer=[0, theirs.data_ptr()], recv=src.data_ptr(),
                    dst=dst.data_ptr(), nbytes=src.numel() * 4, status=status.data_ptr(), timeout_ms=50)
    torch.cuda.synchronize()
    assert int(status[0]) == 0 and torch.equal(src, dst)


def test_exchange_argument_checks(cuda_device):
    flags = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    with pytest.raises(_lib.FlbError):
        A.peer_exchange(rank=0, size=2, epoch=0, flags_local=flags.data_ptr(), flags_peer=[0, flags.data_ptr()])  # epoch 0
    with pytest.raises(_lib.FlbError):
        A.peer_exchange(rank=2, size=2, epoch=1, flags_local=flags.data_ptr(), flags_peer=[0, flags.data_ptr()])  # rank
    with pytest.raises(_lib.FlbError):
        A.peer_exchange(rank=0, size=2, epoch=1, flags_local=flags.data_ptr(), flags_peer=[0, 0])  # peer flags missing
    with pytest.raises(_lib.FlbError):
        A.peer_exchange(rank=0, size=1, epoch=1, flags_local=flags.data_ptr(), flags_peer=[0], recv=flags.data_ptr() + 4,
                        dst=flags.data_ptr() + 128, nbytes=64)  # misaligned
