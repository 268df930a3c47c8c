"""Head-sharded attention layer on two GPUs (NCCL): each rank runs the CUDA path on half of the heads,
the head outputs are all-gathered, and the result must be bit-identical to the unsharded call.
Skipped on a box with fewer than two GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    try:
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from fasterllama_b200 import attention as A
        from fasterllama_b200 import workloads as W
        from fasterllama_b200.tensor_parallel import HeadShardedAttention

        dev = f"cuda:{rank}"
        B, H, T = 4, 16, 1300
        lens = np.array([1200, 37, 512, 700], dtype=np.int32)
        case = W.host_case("tp-gpu", 13, B, H, T, past=lens, in_dtype="float16", cache_dtype="float16", out_dtype="float32")
        full_dev = W.to_device(case, dev)
        A.forward(case.params(full_dev))
        torch.cuda.synchronize()
        want = full_dev["out"].clone()

        def attend(loc):
            part = W.Case(name="p", B=B, H=H // world, S=1, T=T, start_pos=0, arrays=loc, rope_add_past=True,
                          mask_mode=case.mask_mode, max_past_len=case.max_past_len)
            loc["scratch"] = torch.empty(A.workspace_bytes(B, H // world, T), dtype=torch.uint8, device=dev)
            A.forward(part.params(loc))

        layer = HeadShardedAttention(B, H, world, rank, attend)
        fresh = W.to_device(case, dev)
        fresh.pop("scratch")
        got = layer.forward(layer.local_arrays(fresh))
        torch.cuda.synchronize()
        ok = torch.equal(got, want)
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            ret.put(bool(flag.item()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_head_sharded_layer_on_two_gpus(cuda_device):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert ret.get(timeout=10)


def _push_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist

    import datetime

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"),
                            timeout=datetime.timedelta(seconds=60))
    window = None
    try:
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from fasterllama_b200 import attention as A
        from fasterllama_b200 import workloads as W
        from fasterllama_b200.tensor_parallel import HeadShardedAttention, PeerWindow

        dev = f"cuda:{rank}"
        B, H, T = 4, 16, 1300
        layer = HeadShardedAttention(B, H, world, rank, attend=None)
        window = PeerWindow(B * H * 128 * 4, world, rank)
        ok = True
        # five steps: the two receive slots are reused, the ranks drift apart and meet again
        for step in range(5):
            lens = np.array([1200 + step, 37 + step, 512, 700 - step], dtype=np.int32)
            case = W.host_case("tp-push", 13 + step, B, H, T, past=lens, in_dtype="float16", cache_dtype="float16", out_dtype="float32")
            full_dev = W.to_device(case, dev)
            A.forward(case.params(full_dev))
            want = full_dev["out"].clone()

            fresh = W.to_device(case, dev)
            fresh.pop("scratch")
            loc = layer.local_arrays(fresh)
            loc["scratch"] = torch.zeros(A.workspace_bytes(B, H // world, T), dtype=torch.uint8, device=dev)
            part = W.Case(name="p", B=B, H=H // world, S=1, T=T, start_pos=0, arrays=loc, rope_add_past=True,
                          mask_mode=case.mask_mode, max_past_len=case.max_past_len)
            got = torch.full((B, H, 1, 128), float("nan"), device=dev)
            if rank == step % world:
                torch.cuda._sleep(2_000_000)  # about a millisecond of head start for the other rank
            layer.forward_push(loc, window, lambda l, peers, total, off: part.params(l, out_peers=peers, out_head_total=total, out_head_offset=off),
                               got, status=loc["scratch"])
            torch.cuda.synchronize()
            ok = ok and torch.equal(got, want) and A.scratch_status(loc["scratch"]) == 0
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            ret.put(bool(flag.item()))
    finally:
        if window is not None:
            window.close()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_head_sharded_decode_with_peer_stores_on_two_gpus(cuda_device):
    """The same layer without a collective library: rows go to the other GPU as peer stores from the decode
    kernel, a flag hand-shake (bounded wait) replaces the all-gather; bit-identical to the unsharded call."""
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_push_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    codes = [p.exitcode for p in procs]
    for p in procs:
        if p.is_alive():
            p.kill()  # exactly the children started above
    assert codes == [0, 0]
    assert ret.get(timeout=10)


E2E_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.skipif(not all(os.path.exists(os.path.join(E2E_DIR, f"libe2e_{v}.so")) for v in ("flb", "tp")),
                    reason="end-to-end libraries not built")
@pytest.mark.parametrize("fuse_quant", [False, True])
@pytest.mark.parametrize("exchange", ["peer stores", "nccl"])
@pytest.mark.parametrize("config", ["small", "medium"])
def test_tensor_parallel_generation_matches_one_gpu(cuda_device, tmp_path, config, exchange, fuse_quant):
    """The reference's DecodingSampling with the tensor-parallel layer (Q/K/V projections on a column slice,
    head-sharded attention, one exchange of head outputs per layer: NCCL all-gather in prefill; in decode either
    peer stores from the decode kernel + flag hand-shake, or NCCL again) on two GPUs samples exactly the
    ids of the one-GPU adaptor run: int32 projections are exact under the column split, each head's
    attention is bit-identical wherever it runs, and the exchange is a copy.  With fuse_quant the layer's next
    step (attention-output quantisation) is done by the exchange kernel on the rows it received (decode) or by
    flb_attn_quantize on the gathered tensor (prefill, NCCL decode) instead of by the reference's kernel."""
    import json
    import subprocess

    root = os.path.dirname(E2E_DIR.rstrip("/"))
    e2e = os.path.join(root, "e2e.py")
    one, two = str(tmp_path / "one.npz"), str(tmp_path / "two.npz")
    r = subprocess.run([sys.executable, e2e, "--variant", "flb", "--config", config, "--out", one], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-1500:]
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), e2e, "--variant", "tp", "--config", config, "--out", two]
                       + (["--no-push"] if exchange == "nccl" else []) + (["--fuse-quant"] if fuse_quant else []),
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1]
    assert json.loads(line)["tp_decode_exchange"] == exchange
    a, b = np.load(one), np.load(two)
    assert np.array_equal(a["seq_len"], b["seq_len"])
    assert np.array_equal(a["ids"], b["ids"])
