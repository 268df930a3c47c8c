"""In-tree build of the native pieces: the CUDA attention library (sm_100a only) and, for the
tests, the host oracle.  Run as `python -m fasterllama_b200.build` or through
`__graft_entry__.build()`.  Nothing here needs a GPU: nvcc cross-compiles."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libflb_attn.so")
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_LIB = os.path.join(ORACLE_DIR, "libflb_oracle.so")

CUDA_SOURCES = ["decode_attn.cu", "prefill_attn.cu", "launch.cu", "static_scratch.cu", "peer_exchange.cu"]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the attention library cannot be built")
    return cand


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    deps = srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    deps.append(os.path.join(ROOT, "include", "flb_attn.h"))
    if not force and _newer(LIB_PATH, deps):
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", LIB_PATH, *srcs]
    subprocess.run(cmd, check=True)
    return LIB_PATH


def build_oracle(force: bool = False) -> str:
    src = os.path.join(ORACLE_DIR, "attn_oracle.cpp")
    if not force and _newer(ORACLE_LIB, [src, os.path.join(ROOT, "include", "flb_attn.h")]):
        return ORACLE_LIB
    cmd = ["g++", "-O2", "-std=c++17", "-fopenmp", "-shared", "-fPIC", src, "-o", ORACLE_LIB]
    subprocess.run(cmd, check=True)
    return ORACLE_LIB


def reference_root() -> str | None:
    """Where the reference checkout lies on this machine: FLB_REFERENCE_ROOT, else a directory named `reference`
    beside this repository.  None when neither exists (the prebuilt files under oracle/_ref are then used as they are)."""
    cand = os.environ.get("FLB_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
    return cand if os.path.isdir(os.path.join(cand, "fasterLlama", "cuda")) else None


def build_reference(force: bool = False) -> str | None:
    """Compiles the reference's own CUDA kernels (from the read-only reference checkout, where
    present) plus the runner in oracle/ref_runner.cu into oracle/_ref/.  Returns None when the
    reference sources are not on this machine."""
    script = os.path.join(ORACLE_DIR, "build_ref.sh")
    if not os.path.exists(script):
        return None
    out = os.path.join(ORACLE_DIR, "_ref", "libflb_ref.so")
    ref_root = reference_root()
    if ref_root is None:
        return out if os.path.exists(out) else None
    if not force and os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(os.path.join(ORACLE_DIR, "ref_runner.cu")):
        return out
    subprocess.run(["bash", script, ref_root], check=True)
    return out


E2E_VARIANTS = ("ref", "flb", "ref32", "mix", "tp", "opt")


def build_e2e_variants(force: bool = False) -> list[str]:
    """End-to-end libraries around the reference's own DecodingSampling/OpenDecoder classes (test and baseline
    infrastructure, oracle/make_e2e_variants.py).  Built only where the reference checkout exists; stale ones are
    rebuilt when the runner, the patch script or the binding headers changed."""
    ref_root = reference_root()
    out_dir = os.path.join(ORACLE_DIR, "_ref")
    libs = [os.path.join(out_dir, f"libe2e_{v}.so") for v in E2E_VARIANTS]
    if ref_root is None:
        return [l for l in libs if os.path.exists(l)]
    deps = [os.path.join(ORACLE_DIR, "e2e_runner.cu"), os.path.join(ORACLE_DIR, "make_e2e_variants.py"),
            os.path.join(ROOT, "include", "flb_open_decoder.h"), os.path.join(ROOT, "include", "flb_attn.h")]
    stale = [v for v, l in zip(E2E_VARIANTS, libs) if force or not _newer(l, deps)]
    if stale:
        subprocess.run([sys.executable, os.path.join(ORACLE_DIR, "make_e2e_variants.py"), ref_root, *stale], check=True)
    return libs


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    build_oracle(force)
    build_reference(force)
    build_e2e_variants(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", LIB_PATH)
