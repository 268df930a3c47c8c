"""Head-sharded (tensor-parallel) attention layer: every rank runs the attention path on its slice of the
heads against its own cache shard, then the head outputs are all-gathered so that each rank holds the full
[B, H, S, d] result — which is what the next step of the reference's layer needs: its attention-output
quantisation takes the absmax over ALL heads of a token row
(fasterLlama/cuda/decoder_kernels.cu:1197-1203), so every rank must see every head.

There is no collective inside attention itself; the one all-gather (NCCL over NVLink on GPUs, gloo in
the CPU tests) is the only exchange of the layer.  Outputs are gathered in fp32, so the result is
bit-identical to the unsharded call (the split-KV partition depends on sequence lengths only)."""
from __future__ import annotations

from typing import Any, Callable

from . import sharding


class HeadShardedAttention:
    """Owns the shard plan of one layer.  `attend(arrays)` is the per-rank attention call (the CUDA path in
    production; any callable with the same contract in tests): it takes the rank's slice of the arrays and
    fills `arrays["out"]` ([B, H_local, S, d])."""

    def __init__(self, batch_size: int, head_num: int, world: int, rank: int, attend: Callable[[dict], None], group=None):
        if head_num % world != 0:
            raise ValueError(f"{head_num} heads do not divide over {world} ranks")
        self.world, self.rank, self.group = world, rank, group
        n = head_num // world
        self.shard = sharding.Shard("head", rank * n, (rank + 1) * n, batch_size, n)
        self.attend = attend

    def local_arrays(self, arrays: dict[str, Any]) -> dict[str, Any]:
        """This rank's view of full-size arrays (q/k/v [B,S,H,d], caches/out [B,H,*,d], per-channel scales)."""
        loc = sharding.slice_arrays(arrays, self.shard)
        return {k: (v.contiguous() if hasattr(v, "contiguous") else v) for k, v in loc.items()}

    def forward(self, local: dict[str, Any]):
        """Runs attention on the local heads and returns the gathered [B, H, S, d] output (fp32)."""
        import torch
        import torch.distributed as dist

        self.attend(local)
        mine = local["out"].float().contiguous()
        if self.world == 1:
            return mine
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        return torch.cat(parts, dim=1)

    def forward_push(self, local: dict[str, Any], window: "PeerWindow", make_call: Callable[..., Any], full_out, status=None,
                     stream=None):
        """Decode step without a collective library: the rank's decode kernel stores each finished head row
        into every rank's receive slot (peer stores over NVLink), then one small kernel signals the peers,
        waits (bounded) for theirs and copies the slot into `full_out` [B, H, 1, d].  `make_call(local,
        out_peers, out_head_total, out_head_offset)` builds the parameter block of the CUDA decode call for
        this rank's arrays.  Everything is stream-ordered; nothing synchronises with the host."""
        from . import attention as A

        e = window.next_epoch()
        heads = self.shard.heads * self.world
        p = make_call(local, [window.slot(r, e) for r in range(self.world)], heads, self.rank * self.shard.heads)
        A.decode(p, stream=stream)
        A.peer_exchange(rank=self.rank, size=self.world, epoch=e, flags_local=window.flags(self.rank),
                        flags_peer=[window.flags(r) if r != self.rank else 0 for r in range(self.world)],
                        recv=window.slot(self.rank, e), dst=full_out.data_ptr(),
                        nbytes=full_out.numel() * full_out.element_size(), status=(status.data_ptr() if status is not None else 0),
                        stream=stream)
        return full_out


def _cudart():
    """The CUDA runtime already loaded into this process (torch's), through ctypes."""
    import ctypes as C

    rt = C.CDLL("libcudart.so.12")
    rt.cudaMalloc.argtypes = [C.POINTER(C.c_void_p), C.c_size_t]
    rt.cudaFree.argtypes = [C.c_void_p]
    rt.cudaMemset.argtypes = [C.c_void_p, C.c_int, C.c_size_t]
    rt.cudaIpcGetMemHandle.argtypes = [C.c_void_p, C.c_void_p]
    rt.cudaIpcOpenMemHandle.argtypes = [C.POINTER(C.c_void_p), _IpcHandle, C.c_uint]
    rt.cudaIpcCloseMemHandle.argtypes = [C.c_void_p]
    rt.cudaDeviceSynchronize.argtypes = []
    return rt


def _make_handle_type():
    import ctypes as C

    class IpcHandle(C.Structure):  # cudaIpcMemHandle_t: 64 opaque bytes, passed by value
        _fields_ = [("reserved", C.c_ubyte * 64)]

    return IpcHandle


_IpcHandle = _make_handle_type()


class PeerWindow:
    """One rank's landing area for a head-split decode layer, mapped into every rank of the node.

    Layout of the block (its own cudaMalloc, so that the CUDA IPC handle names exactly this memory): 256 bytes
    of flag words (word r: the last epoch rank r has published here), then two receive slots of `slot_bytes`
    used alternately (slot = epoch & 1).  Peers are opened with cudaIpcOpenMemHandle, which also enables peer
    access from this rank's GPU to theirs.  `group` must span the ranks of ONE node."""

    FLAG_BYTES = 256

    def __init__(self, slot_bytes: int, world: int, rank: int, group=None):
        import ctypes as C

        import torch.distributed as dist

        self.world, self.rank, self.group = world, rank, group
        self.slot_bytes = (int(slot_bytes) + 255) // 256 * 256
        self.epoch = 0
        self._rt = rt = _cudart()
        total = self.FLAG_BYTES + 2 * self.slot_bytes
        own = C.c_void_p()
        self._check(rt.cudaMalloc(C.byref(own), total), "cudaMalloc")
        self._check(rt.cudaMemset(own, 0, total), "cudaMemset")
        self._check(rt.cudaDeviceSynchronize(), "cudaDeviceSynchronize")
        h = _IpcHandle()
        self._check(rt.cudaIpcGetMemHandle(C.byref(h), own), "cudaIpcGetMemHandle")
        handles: list = [None] * world
        dist.all_gather_object(handles, bytes(h), group=group)  # also orders every rank's memset before any use
        self.base = [0] * world
        self._opened = []
        for r in range(world):
            if r == rank:
                self.base[r] = own.value
                continue
            hr = _IpcHandle()
            C.memmove(C.byref(hr), handles[r], 64)
            ptr = C.c_void_p()
            self._check(rt.cudaIpcOpenMemHandle(C.byref(ptr), hr, 1), "cudaIpcOpenMemHandle")  # 1 = lazy peer access
            self.base[r] = ptr.value
            self._opened.append(ptr)
        self._own = own

    @staticmethod
    def _check(err: int, what: str) -> None:
        if err != 0:
            raise RuntimeError(f"{what} failed with CUDA error {err}")

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def flags(self, r: int) -> int:
        return self.base[r]

    def slot(self, r: int, epoch: int) -> int:
        return self.base[r] + self.FLAG_BYTES + (epoch & 1) * self.slot_bytes

    def close(self) -> None:
        """Unmaps the peers' blocks, then (after every rank has done so) frees this rank's."""
        import torch.distributed as dist

        self._check(self._rt.cudaDeviceSynchronize(), "cudaDeviceSynchronize")
        for ptr in self._opened:
            self._rt.cudaIpcCloseMemHandle(ptr)
        self._opened = []
        dist.barrier(group=self.group)
        if self._own is not None:
            self._rt.cudaFree(self._own)
            self._own = None
