"""Sharding of the attention work over the GPUs of one box.

Every (batch, head) pair is an independent attention problem with its own contiguous cache slab
([B, H, T, d], fasterLlama/open_decoder.h:72-77), so the path shards without any exchange: each rank
owns a contiguous range of sequences (or, when the batch does not divide, of heads) and runs the
same call on its slice.  The split-KV partition of a sequence depends on its length only, so the
per-head results are bit-identical at every GPU count."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    axis: str          # "batch" or "head"
    start: int
    stop: int
    batch: int         # sequences this rank holds
    heads: int         # heads this rank holds

    @property
    def units(self) -> int:
        return self.batch * self.heads


def plan(batch_size: int, head_num: int, world: int, rank: int) -> Shard:
    """Contiguous slice of the batch (preferred: per-sequence lengths travel with it) or of the
    heads for `rank` of `world`.  Raises when neither axis divides."""
    if not (0 <= rank < world):
        raise ValueError("rank outside the world")
    if batch_size % world == 0:
        n = batch_size // world
        return Shard("batch", rank * n, (rank + 1) * n, n, head_num)
    if head_num % world == 0:
        n = head_num // world
        return Shard("head", rank * n, (rank + 1) * n, batch_size, n)
    raise ValueError(f"neither batch {batch_size} nor heads {head_num} divide over {world} ranks")


def slice_arrays(arrays: dict, shard: Shard) -> dict:
    """The rank's slice of a case's arrays (numpy or torch): q/k/v [B,S,H,d], caches and out
    [B,H,*,d], past_lens [B]; tables, masks and scales that are not per-sequence pass through
    (per-channel weight scales are sliced with the heads)."""
    out = {}
    s = slice(shard.start, shard.stop)
    for k, v in arrays.items():
        if v is None:
            out[k] = v
        elif shard.axis == "batch":
            if k in ("q", "k", "v", "k_cache", "v_cache", "out", "past_lens"):
                out[k] = v[s]
            elif k == "act_scale":
                per = v.shape[0] // arrays["q"].shape[0]
                out[k] = v[shard.start * per:shard.stop * per]
            else:
                out[k] = v
        else:
            if k in ("q", "k", "v"):
                out[k] = v[:, :, s]
            elif k in ("k_cache", "v_cache", "out"):
                out[k] = v[:, s]
            elif k in ("q_w_scale", "k_w_scale", "v_w_scale"):
                d = arrays["q"].shape[-1]
                out[k] = v[shard.start * d:shard.stop * d]
            else:
                out[k] = v
    return out
