"""End to end through the reference's own classes: DecodingSampling<FP16> + OpenDecoder with the attention
section replaced by the adaptor call (include/flb_open_decoder.h), against the same classes running the
reference's attention (decode gemv arguments corrected).  The libraries are built from a patched copy of
the reference checkout by oracle/make_e2e_variants.py and travel with the tree; without them the tests skip.

What is asserted:
  * teacher-forced parity: inside the reference's generation loop, at the prefill call and at every decode call of
    every layer, the adaptor is run on the reference's own state and its output is compared with the reference's
    (the "mix" library, FLB_E2E_USE=4) — decode 1e-5 of the tensor's magnitude, prefill 5e-3;
  * teacher-forced logits: with the reference's ids fed to every variant, each step's logits row and the top-4 set the
    sampler draws from, against the distance the reference has from itself when its prefill GEMMs compute in fp32;
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


def _json_lines(out):
    res = []
    for line in out.splitlines():
        if line.startswith("{"):
            try:
                res.append(json.loads(line))
            except ValueError:
                pass
    return res


def test_teacher_forced_parity_inside_the_reference_loop(cuda_device, tmp_path):
    """Every attention call of the run — the prefill call and all decode calls of every layer — with the adaptor run
    on the reference's own state beside the reference's code.  Decode: 1e-5 of the tensor's magnitude (the
    reference's gemv is true fp32).  Prefill: 5e-3 absolute, the bound of the golden prefill cases (the reference's own
    GEMMs there use fp16 tensor-core math on fp32 storage, fasterLlama/cuda/common.h:71)."""
    out = _run("mix", "medium", str(tmp_path / "mix.npz"), env={"FLB_E2E_USE": "4"})
    stats = [j["mix"] for j in _json_lines(out) if "mix" in j]
    assert stats, out[-1500:]
    m = stats[-1]
    cfg_layers, cfg_steps = 4, 48
    assert m["decode_calls"] == cfg_layers * (cfg_steps - 1), m   # every decode call of every layer
    assert m["prefill_calls"] == cfg_layers, m
    assert m["nan_rows_not_zero"] == 0
    assert m["decode_max_abs_diff"] <= 1e-5 * max(1.0, m["decode_max_abs_ref"]), m
    assert m["prefill_max_abs_diff"] <= 5e-3 * max(1.0, m["prefill_max_abs_ref"] / 4.0), m


def test_teacher_forced_logits_and_top4_sets(cuda_device, tmp_path):
    """What can be said about sampled ids without the reference's summation order: with the SAME token history (the
    reference's own ids fed to every variant), the logits the sampler reads and the top-4 set it draws from.  The
    reference with its prefill GEMMs in true fp32 (ref32) is the noise floor: the adaptor must not sit further from
    the reference than the reference sits from itself."""
    e = dict(os.environ)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "e2e.py"), "--variant", "ref", "--config", "medium", "--out", str(tmp_path / "x.npz"),
                        "--compare-logits", "ref32,flb"], capture_output=True, text=True, env=e, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    res = _json_lines(r.stdout)[-1]
    print(json.dumps(res))
    flb, floor = res["flb"], res["ref32"]
    assert flb["max_abs_diff"] <= max(2.0 * floor["max_abs_diff"], 1e-3 * res["max_abs_logit"]), res
    assert flb["top4_set_same"] >= min(0.98, floor["top4_set_same"] - 0.02), res
    assert flb["argmax_same"] >= min(0.98, floor["argmax_same"] - 0.02), res


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


@pytest.mark.skipif(not os.path.exists(os.path.join(REF_DIR, "libe2e_opt.so")), reason="libe2e_opt.so not built")
def test_merged_qkv_projection_gives_the_same_ids(cuda_device, tmp_path):
    """One INT8 GEMM for the Q, K and V projections, its int32 output read in place by the attention call (row stride
    3 x hidden), is the same integer arithmetic as the reference's three GEMMs: ids must be identical.  The other changes
    of that variant (LM head over the last rows only, lagged finished check, fp16-sized slab) are exercised on the way."""
    three, one, one16 = (str(tmp_path / n) for n in ("three.npz", "one.npz", "one16.npz"))
    for cfg in ("small", "medium"):
        _run("opt", cfg, three)
        _run("opt", cfg, one, extra=("--merged-qkv",))
        a, b = np.load(three), np.load(one)
        assert np.array_equal(a["ids"], b["ids"]) and np.array_equal(a["seq_len"], b["seq_len"]), cfg
    _run("opt", "medium", one16, extra=("--merged-qkv", "--cache-f16"))
    assert int(np.load(one16)["seq_len"].max()) > 0
    # against the plain adaptor build: the LM head now runs as a 8-row GEMM instead of a 1280-row one (another cuBLAS
    # kernel, another summation order), so only agreement is reported, not identity
    flb = str(tmp_path / "flb.npz")
    _run("flb", "medium", flb)
    f, o = np.load(flb), np.load(three)
    n = int(f["seq_len"].max())
    print(json.dumps({"opt_vs_flb_id_match": float((f["ids"][:, :n] == o["ids"][:, :n]).mean())}))
    assert np.array_equal(f["seq_len"], o["seq_len"])


def test_fp16_cache_generation_runs_and_is_deterministic(cuda_device, tmp_path):
    """FLB_CACHE_F16=1 keeps the caches as halves inside the caller's float slabs: a different (coarser) cache
    format, so ids may differ from the fp32-cache run, but the run is deterministic and complete."""
    a, b = (str(tmp_path / n) for n in ("h1.npz", "h2.npz"))
    _run("flb", "small", a, extra=("--cache-f16",))
    _run("flb", "small", b, extra=("--cache-f16",))
    ra, rb = np.load(a), np.load(b)
    assert np.array_equal(ra["ids"], rb["ids"]) and np.array_equal(ra["seq_len"], rb["seq_len"])
    assert int(ra["seq_len"].max()) > 0
