"""Generates tests/golden/ref_golden.npz by running the REFERENCE's own attention kernels and
cuBLAS calls (oracle/_ref/libflb_ref.so, built by oracle/build_ref.sh from the reference checkout)
on the deterministic inputs of golden_cases.py.  Needs a GPU:

    python tests/golden/make_ref_golden.py <output.npz>                  (ref_golden.npz: the head-size-128 cases)
    python tests/golden/make_ref_golden.py <output.npz> head_sizes       (ref_golden_head_sizes.npz: decode at 64 and 256, prefill at 64)

Stored per case (prefill cases: for the heads in golden_cases.PREFILL_HEADS_KEPT only, to keep
the fixture small): the attention output, the cache rows the call appended, the RoPE table rows it
used (from the reference's own table kernel) and the runner's status.  The decode cases use the
corrected gemv arguments ("fixed"), except the one named as_written, which passes the arguments
exactly as the reference does at the one length (L == size_per_head) where they are consistent.
Also records what the as-written call returns at L = 257."""
from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

import golden_cases as G  # noqa: E402
from oracle.ref_runner import RefRunner  # noqa: E402


def main(out_path: str, which: str = "base") -> None:
    ref = RefRunner()
    store: dict[str, np.ndarray] = {}
    notes: dict[str, object] = {"torch": torch.__version__, "gpu": torch.cuda.get_device_name(0)}
    cases = G.HEAD_SIZE_CASES if which == "head_sizes" else G.CASES
    for name, c in cases.items():
        a = G.build(name)
        t = {k: torch.from_numpy(v).cuda() for k, v in a.items()}
        table = ref.freq_cis(c["T"] + 8, c.get("d", G.D))
        t["freq_cis"] = table
        args = ref.make_args(t, start_pos=c["start_pos"], rope_row=c["rope_row"], as_written=c.get("as_written", False))
        st = ref.attention(args)
        torch.cuda.synchronize()
        sp, S = c["start_pos"], c["S"]
        hs = list(G.PREFILL_HEADS_KEPT) if S > 1 else list(range(c["H"]))  # keep the fixture small
        store[f"{name}/out"] = t["out"][:, hs].cpu().numpy()
        store[f"{name}/k_rows"] = t["k_cache"][:, hs, sp:sp + S].cpu().numpy()
        store[f"{name}/v_rows"] = t["v_cache"][:, hs, sp:sp + S].cpu().numpy()
        store[f"{name}/freq_rows"] = table[c["rope_row"]:c["rope_row"] + S].cpu().numpy()
        notes[name] = {"status": st, "nan_rows": int(torch.isnan(t["out"]).any(dim=-1).sum())}
        print(name, "status", st, "nan rows", notes[name]["nan_rows"], flush=True)
    if which == "head_sizes":
        store["notes_json"] = np.frombuffer(json.dumps(notes).encode(), dtype=np.uint8)
        np.savez_compressed(out_path, **store)
        print("wrote", out_path, os.path.getsize(out_path), "bytes")
        ref.close()
        return
    # what the reference's decode call does, exactly as written, at L = 257 (> size_per_head)
    name = "decode_config1_shape"
    a = G.build(name)
    t = {k: torch.from_numpy(v).cuda() for k, v in a.items()}
    t["freq_cis"] = ref.freq_cis(G.CASES[name]["T"] + 8)
    args = ref.make_args(t, start_pos=256, rope_row=256, as_written=True)
    st = ref.attention(args)
    torch.cuda.synchronize()
    notes["as_written_L257_status"] = st
    print("as written at L=257: status", st, flush=True)
    store["notes_json"] = np.frombuffer(json.dumps(notes).encode(), dtype=np.uint8)
    np.savez_compressed(out_path, **store)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")
    ref.close()


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_golden.npz"), sys.argv[2] if len(sys.argv) > 2 else "base")
