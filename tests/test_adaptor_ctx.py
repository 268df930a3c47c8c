"""The reference-side binding (include/flb_open_decoder.h) keeps its state per object: two decoders with different
masks, scratch buffers and streams in one process each get their own answers.  The header is plain C/C++ with
static inline functions, so it is exercised by a small compiled probe."""
import os
import subprocess

import pytest

from fasterllama_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HERE = os.path.dirname(os.path.abspath(__file__))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build(tmp_path) -> str:
    exe = str(tmp_path / "adaptor_probe")
    pkg = os.path.join(ROOT, "fasterllama_b200")
    subprocess.run(["g++", "-std=c++17", "-O1", os.path.join(HERE, "adaptor_probe.cpp"), "-I", os.path.join(ROOT, "include"),
                    "-I", os.path.join(CUDA, "include"), "-L", pkg, "-lflb_attn", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
                    "-Wl,-rpath," + pkg, "-Wl,-rpath," + os.path.join(CUDA, "lib64"), "-o", exe], check=True)
    return exe


def test_probe_compiles_as_plain_cxx(tmp_path):
    """No GPU needed: the header must compile and link against the library from ordinary host C++."""
    _lib.load_library()
    assert os.path.exists(_build(tmp_path))


@pytest.mark.gpu
def test_two_contexts_keep_their_own_state(cuda_device, tmp_path):
    exe = _build(tmp_path)
    env = dict(os.environ)
    for k in ("FLB_MASK_MODE", "FLB_EARLY_START", "FLB_CACHE_F16", "FLB_FUSE_QUANT"):
        env.pop(k, None)
    out = subprocess.run([exe], check=True, capture_output=True, text=True, env=env).stdout
    got = dict(line.split(" ", 1) for line in out.strip().splitlines())
    assert got["mask_a"] == str(_lib.FLB_MASK_CAUSAL_STRICT)
    assert got["mask_b"] == str(_lib.FLB_MASK_CAUSAL_INCLUSIVE)
    assert got["first_call_zeroed_a"] == "0 early_a 0"        # first decode call on a scratch: counters get cleared
    assert got["second_call_zeroed_a"] == "1 early_a 1"       # then they are known to be zero; level 1 is the default
    assert got["other_stream_zeroed_a"] == "0 early_a 0"      # another stream: start over
    assert got["mask_a_changed"] == str(_lib.FLB_MASK_CAUSAL_INCLUSIVE)
    assert got["b_unaffected"] == f"{_lib.FLB_MASK_CAUSAL_INCLUSIVE} zeroed_b 1"
    assert got["row_stride"] == f"{4 * 128} validate 0"
    assert got["cuda"] == "0"
