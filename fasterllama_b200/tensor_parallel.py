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
