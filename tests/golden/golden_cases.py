"""Deterministic inputs for the golden vectors.

Inputs come from an integer hash of the element index (no library random generator, so they are
identical on every machine and numpy version) and sit on exact binary grids:
  * q/k/v are int32 accumulators below 2^14 with 4-bit scale mantissas, so the reference's
    dequantisation float(acc)*act_scale*w_scale is exact in fp32 and every implementation sees the
    same values whatever its multiplication order;
  * cache entries are multiples of 1/32 in [-4, 4].
The reference accepts q/k/v only as int32 accumulators + scales, hence this form."""
from __future__ import annotations

import numpy as np

D = 128

# name -> parameters.  mask: "strict" (the reference's samples), "inclusive", "none".
# rope_row: table row used for token 0 of the chunk (the reference's kernels use row s of the
# pointer they are handed; the runner offsets the pointer by rope_row).
CASES = {
    "decode_L128_as_written": dict(B=1, H=8, S=1, T=160, start_pos=127, mask="inclusive", rope_row=127, as_written=True),
    "decode_L128_fixed": dict(B=1, H=8, S=1, T=160, start_pos=127, mask="inclusive", rope_row=127,
                              inputs_of="decode_L128_as_written"),
    "decode_L1": dict(B=2, H=8, S=1, T=64, start_pos=0, mask="inclusive", rope_row=0),
    "decode_L38_none": dict(B=2, H=8, S=1, T=64, start_pos=37, mask="none", rope_row=0),
    "decode_L301_strict": dict(B=2, H=8, S=1, T=400, start_pos=300, mask="strict", rope_row=0),
    "decode_L600_inclusive": dict(B=1, H=8, S=1, T=640, start_pos=599, mask="inclusive", rope_row=599),
    "decode_config1_shape": dict(B=1, H=32, S=1, T=512, start_pos=256, mask="inclusive", rope_row=256),
    "prefill_S64_strict": dict(B=1, H=8, S=64, T=96, start_pos=0, mask="strict", rope_row=0),
    "prefill_S128_inclusive": dict(B=1, H=8, S=128, T=160, start_pos=0, mask="inclusive", rope_row=0),
    "prefill_S200_inclusive": dict(B=1, H=8, S=200, T=256, start_pos=0, mask="inclusive", rope_row=0),
}


# Decode at the other head sizes the call accepts (the reference's kernels take them too: size_per_head <= 128 on
# its warp kernels, 256 on its block kernels, decoder_kernels.cu:563-589), and prefill at head size 64.  Their vectors
# live in a fixture of their own, ref_golden_head_sizes.npz, made by `make_ref_golden.py <out> head_sizes`.
HEAD_SIZE_CASES = {
    "decode_d64_L200_inclusive": dict(B=2, H=8, S=1, T=256, start_pos=199, mask="inclusive", rope_row=199, d=64),
    "decode_d64_L700_strict": dict(B=1, H=8, S=1, T=768, start_pos=699, mask="strict", rope_row=0, d=64),
    "decode_d256_L150_none": dict(B=2, H=8, S=1, T=192, start_pos=149, mask="none", rope_row=149, d=256),
    "decode_d256_L600_inclusive": dict(B=1, H=8, S=1, T=640, start_pos=599, mask="inclusive", rope_row=599, d=256),
    "prefill_d64_S200_inclusive": dict(B=1, H=8, S=200, T=256, start_pos=0, mask="inclusive", rope_row=0, d=64),
    "prefill_d64_S330_strict": dict(B=1, H=8, S=330, T=384, start_pos=0, mask="strict", rope_row=0, d=64),
}


def case(name: str) -> dict:
    return CASES[name] if name in CASES else HEAD_SIZE_CASES[name]


# heads whose results the fixture keeps for the prefill cases
PREFILL_HEADS_KEPT = (0, 5)


def _hash(n: int, salt: int) -> np.ndarray:
    """32-bit mix of the indices 0..n-1 (xorshift-multiply), as uint64 values below 2^32."""
    x = (np.arange(n, dtype=np.uint64) + np.uint64(salt) * np.uint64(0x9E3779B1)) & np.uint64(0xFFFFFFFF)
    for _ in range(2):
        x ^= x >> np.uint64(16)
        x = (x * np.uint64(0x7FEB352D)) & np.uint64(0xFFFFFFFF)
        x ^= x >> np.uint64(15)
        x = (x * np.uint64(0x846CA68B)) & np.uint64(0xFFFFFFFF)
        x ^= x >> np.uint64(16)
    return x


def _centered_sum(n: int, salt: int, terms: int, span: int) -> np.ndarray:
    """Sum of `terms` uniform integers in [0, span) minus the mean: a bell-shaped integer."""
    acc = np.zeros(n, dtype=np.int64)
    for t in range(terms):
        acc += (_hash(n, salt * 16 + t) % np.uint64(span)).astype(np.int64)
    return acc - terms * (span - 1) // 2


def build(name: str) -> dict:
    """Host arrays of one golden case (everything but the RoPE table rows, which the fixture
    stores because they come from the reference's own table kernel)."""
    c = case(name)
    B, H, S, T, sp = c["B"], c["H"], c["S"], c["T"], c["start_pos"]
    D = c.get("d", globals()["D"])  # head size of this case
    salt = sum(ord(ch) for ch in c.get("inputs_of", name))  # "inputs_of": share another case's inputs
    n = B * S * H * D
    a = {}
    for i, nm in enumerate(("q", "k", "v")):
        # about N(0, 1) after scaling: 4 uniform terms on [0, 4096) -> sigma ~ 2365, times ~2^-11
        a[nm] = _centered_sum(n, salt + i, 4, 4096).astype(np.int32).reshape(B, S, H, D)
    a["act_scale"] = ((8 + _hash(B * S, salt + 7) % np.uint64(8)).astype(np.float32) / 8.0 * 2.0**-6).astype(np.float32)
    for i, nm in enumerate(("q_w_scale", "k_w_scale", "v_w_scale")):
        a[nm] = ((8 + _hash(H * D, salt + 8 + i) % np.uint64(8)).astype(np.float32) / 8.0 * 2.0**-6).astype(np.float32)
    m = B * H * T * D
    for i, nm in enumerate(("k_cache", "v_cache")):
        full = (_centered_sum(m, salt + 11 + i, 2, 129).astype(np.float32) / 32.0).reshape(B, H, T, D)
        full[:, :, sp:] = 0.0
        a[nm] = np.ascontiguousarray(full)
    a["out"] = np.zeros((B, H, S, D), dtype=np.float32)
    if c["mask"] != "none":
        r = np.arange(T)[:, None]
        col = np.arange(T)[None, :]
        keep = (col < r) if c["mask"] == "strict" else (col <= r)
        a["attn_mask"] = np.where(keep, np.float32(0), -np.finfo(np.float32).max).astype(np.float32)
    return a
