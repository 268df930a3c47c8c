"""End to end through the reference's own classes: DecodingSampling<FP16> + OpenDecoder with the attention
section replaced by the adaptor call (include/flb_open_decoder.h), against the same classes running the
reference's attention (decode gemv arguments corrected).  The libraries are built from a patched copy of
the reference checkout by oracle/make_e2e_variants.py and travel with the tree; without them the tests skip.

What is asserted:
  * teacher-forced parity: inside the reference's generation loop, at every decode call of every layer,
    the adaptor is run on the reference's own state and its output is compared with the reference's
    (the "mix" library, FLB_E2E_USE=4) — 1e-5 of the tensor's magnitude;
  * free-running: both produce the same number of tokens, are deterministic, and agree on a
    large part of the sampled ids.  Bit-identical ids are NOT asserted: the reference's contractions are
    cuBLAS calls whose summation order is not public, its attention outputs are re-quantised to INT8 right
    after, and with random weights the sampled trajectory amplifies a 1e-6 difference within a few steps
    (measured: the reference itself, with its prefill GEMMs switched from fp16 to fp32 tensor-core math,
    agrees with itself on 60-86 % of the ids on these configurations)."""
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not all(os.path.exists(os.path.join(REF_DIR, f"libe2e_{v}.so")) for v in ("ref", "flb", "mix")),
                                 reason="end-to-end libraries not built (oracle/make_e2e_variants.py needs the reference checkout)")]


def _run(variant, config, out, env=None, extra=()):
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "e2e.py"), "--variant", variant, "--config", config, "--out", out, *extra],
                       capture_output=True, text=True, env=e, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


def test_teacher_forced_decode_parity_inside_the_reference_loop(cuda_device, tmp_path):
    out = _run("mix", "medium", str(tmp_path / "mix.npz"), env={"FLB_E2E_USE": "4"})
    rows = re.findall(r"\[cmp (\d+)\] start_pos (\d+) max\|ref-flb\| ([0-9.e+-]+) .* max\|ref\| ([0-9.e+-]+)", out)
    assert len(rows) >= 50, out[-1500:]
    for _, _, diff, amax in rows:
        assert float(diff) <= 1e-5 * max(1.0, float(amax)), (diff, amax)


@pytest.mark.parametrize("mask", ["inclusive", "strict"])
def test_free_running_generation_small(cuda_device, tmp_path, mask):
    a, b, b2 = (str(tmp_path / n) for n in ("ref.npz", "flb.npz", "flb2.npz"))
    _run("ref", "small", a, extra=("--mask", mask))
    _run("flb", "small", b, extra=("--mask", mask))
    _run("flb", "small", b2, extra=("--mask", mask))
    ra, rb, rb2 = np.load(a), np.load(b), np.load(b2)
    assert np.array_equal(rb["ids"], rb2["ids"]), "the adaptor path must be deterministic"
    assert np.array_equal(ra["seq_len"], rb["seq_len"])
    n = int(ra["seq_len"].max())
    match = (ra["ids"][:, :n] == rb["ids"][:, :n]).mean()
    print(json.dumps({"mask": mask, "id_match_fraction": float(match)}))
    assert match >= 0.5, f"only {match:.2f} of the sampled ids agree with the reference"
    # the prompt is teacher-forced by both, so the very first sampled token depends on prefill only
    assert (ra["ids"][:, 0] == rb["ids"][:, 0]).mean() >= 0.5


def test_adaptor_switches_do_not_change_the_ids(cuda_device, tmp_path):
    """Fused attention-output quantisation (FLB_FUSE_QUANT=1) and ordinary launches with a counter memset per call
    (FLB_EARLY_START=0) are different ways to issue the same arithmetic: the sampled ids must not move."""
    base, fused, plain = (str(tmp_path / n) for n in ("base.npz", "fused.npz", "plain.npz"))
    _run("flb", "medium", base)
    _run("flb", "medium", fused, extra=("--fuse-quant",))
    _run("flb", "medium", plain, env={"FLB_EARLY_START": "0"})
    a, b, c = np.load(base), np.load(fused), np.load(plain)
    assert np.array_equal(a["ids"], b["ids"]) and np.array_equal(a["seq_len"], b["seq_len"])
    assert np.array_equal(a["ids"], c["ids"]) and np.array_equal(a["seq_len"], c["seq_len"])


def test_fp16_cache_generation_runs_and_is_deterministic(cuda_device, tmp_path):
    """FLB_CACHE_F16=1 keeps the caches as halves inside the caller's float slabs: a different (coarser) cache
    format, so ids may differ from the fp32-cache run, but the run is deterministic and complete."""
    a, b = (str(tmp_path / n) for n in ("h1.npz", "h2.npz"))
    _run("flb", "small", a, extra=("--cache-f16",))
    _run("flb", "small", b, extra=("--cache-f16",))
    ra, rb = np.load(a), np.load(b)
    assert np.array_equal(ra["ids"], rb["ids"]) and np.array_equal(ra["seq_len"], rb["seq_len"])
    assert int(ra["seq_len"].max()) > 0
