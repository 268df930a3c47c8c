"""ctypes binding of oracle/attn_oracle.cpp (the scalar host restatement of the reference's
attention math).  TEST INFRASTRUCTURE: only tests, the smoke check and the benchmark's
CPU-baseline leg import this module; the product path never does."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libflb_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "attn_oracle.cpp")
    hdr = os.path.join(os.path.dirname(HERE), "include", "flb_attn.h")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        subprocess.run(["g++", "-O2", "-std=c++17", "-fopenmp", "-shared", "-fPIC", src, "-o", LIB], check=True)
    return LIB


def load():
    global _lib
    if _lib is None:
        build()
        lib = C.CDLL(LIB)
        lib.orc_attention.restype = C.c_int
        lib.orc_attention.argtypes = [C.c_void_p, C.c_int]
        lib.orc_set_threads.restype = C.c_int
        lib.orc_set_threads.argtypes = [C.c_int]
        lib.orc_hw_threads.restype = C.c_int
        lib.orc_rope_row.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        lib.orc_softmax_row.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.POINTER(C.c_int)]
        lib.orc_freq_cis.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_double]
        lib.orc_attn_quantize.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
        _lib = lib
    return _lib


def attention(params, acc_double: bool = True, f16_operands: bool = False) -> None:
    """Runs the whole path on the host.  `params` is a flb_attn_params block whose pointers are
    HOST memory (numpy arrays); the caches and `out` arrays are written in place.
    `f16_operands` rounds the prefill operands to fp16 first (the precision of the reference's
    own fp16 tensor-core prefill GEMMs); decode ignores it."""
    st = load().orc_attention(C.addressof(params), int(acc_double) | (2 if f16_operands else 0))
    if st != 0:
        raise RuntimeError(f"oracle rejected the parameters: status {st}")


def set_threads(n: int) -> int:
    return int(load().orc_set_threads(int(n)))


def hw_threads() -> int:
    return int(load().orc_hw_threads())


def rope_row(x: np.ndarray, freq_row: np.ndarray) -> np.ndarray:
    y = np.ascontiguousarray(x, dtype=np.float32).copy()
    f = np.ascontiguousarray(freq_row, dtype=np.float32)
    load().orc_rope_row(y.ctypes.data, f.ctypes.data, int(y.size))
    return y


def softmax_row(scores: np.ndarray, mask_row: np.ndarray | None, scaler: float):
    y = np.ascontiguousarray(scores, dtype=np.float32).copy()
    m = None if mask_row is None else np.ascontiguousarray(mask_row, dtype=np.float32)
    fm = C.c_int(0)
    load().orc_softmax_row(y.ctypes.data, None if m is None else m.ctypes.data, int(y.size), float(scaler), C.byref(fm))
    return y, bool(fm.value)


def freq_cis(rows: int, d: int = 128, base: float = 10000.0) -> np.ndarray:
    t = np.empty((rows, d), dtype=np.float32)
    load().orc_freq_cis(t.ctypes.data, rows, d, float(base))
    return t


def attn_quantize(attn: np.ndarray):
    """The reference's attention-output quantisation on the host: attn [B,H,S,d] fp32 ->
    (codes int8 [B,S,H*d], scale fp32 [B*S])."""
    a = np.ascontiguousarray(attn, dtype=np.float32)
    B, H, S, d = a.shape
    q8 = np.empty((B, S, H * d), dtype=np.int8)
    sc = np.empty((B * S,), dtype=np.float32)
    load().orc_attn_quantize(a.ctypes.data, q8.ctypes.data, sc.ctypes.data, B, H, S, d)
    return q8, sc
