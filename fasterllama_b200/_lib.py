"""ctypes binding of the C ABI in include/flb_attn.h.

The shared library is built in-tree by `fasterllama_b200.build` (nvcc, sm_100a).  There is no
fallback of any kind: if the library is missing, loading raises, and every compute call goes to
the CUDA kernels."""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libflb_attn.so")

# enums of include/flb_attn.h
FLB_OK = 0
FLB_ERR_NULL_POINTER = -1
FLB_ERR_BAD_SHAPE = -2
FLB_ERR_UNSUPPORTED = -3
FLB_ERR_MISALIGNED = -4
FLB_ERR_SCRATCH_TOO_SMALL = -5
FLB_ERR_LAUNCH = -6
FLB_ERR_BAD_ENUM = -7
FLB_ERR_DEVICE = -8
FLB_ERR_TOO_LARGE = -9

FLB_IN_INT32, FLB_IN_F32, FLB_IN_F16 = 0, 1, 2
FLB_F32, FLB_F16 = 0, 1
FLB_MAX_PEERS = 8
FLB_STATUS_PEER_WAIT = 0x100
FLB_MASK_NONE, FLB_MASK_GENERIC, FLB_MASK_CAUSAL_INCLUSIVE, FLB_MASK_CAUSAL_STRICT = 0, 1, 2, 3


class FlbAttnParams(C.Structure):
    """struct flb_attn_params, field for field."""

    _fields_ = [
        ("batch_size", C.c_int),
        ("head_num", C.c_int),
        ("size_per_head", C.c_int),
        ("seq_len", C.c_int),
        ("start_pos", C.c_int),
        ("total_len", C.c_int),
        ("past_lens", C.c_void_p),
        ("max_past_len", C.c_int),
        ("input_mode", C.c_int),
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("act_scale", C.c_void_p),
        ("q_w_scale", C.c_void_p),
        ("k_w_scale", C.c_void_p),
        ("v_w_scale", C.c_void_p),
        ("freq_cis", C.c_void_p),
        ("rope_pos0", C.c_int),
        ("rope_add_past", C.c_int),
        ("mask_mode", C.c_int),
        ("attn_mask", C.c_void_p),
        ("mask_row_stride", C.c_int),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("cache_dtype", C.c_int),
        ("out", C.c_void_p),
        ("out_dtype", C.c_int),
        ("softmax_scale", C.c_float),
        ("scratch", C.c_void_p),
        ("scratch_bytes", C.c_size_t),
        ("scratch_zeroed", C.c_int),
        ("split_len", C.c_int),
        ("out_q8", C.c_void_p),
        ("out_q8_scale", C.c_void_p),
        ("out_peers", C.c_void_p * FLB_MAX_PEERS),
        ("n_out_peers", C.c_int),
        ("out_head_total", C.c_int),
        ("out_head_offset", C.c_int),
        ("early_start", C.c_int),
        ("qkv_row_stride", C.c_int),
    ]


class FlbPeerExchange(C.Structure):
    """struct flb_peer_exchange, field for field."""

    _fields_ = [
        ("rank", C.c_int),
        ("size", C.c_int),
        ("epoch", C.c_uint),
        ("flags_local", C.c_void_p),
        ("flags_peer", C.c_void_p * FLB_MAX_PEERS),
        ("recv", C.c_void_p),
        ("dst", C.c_void_p),
        ("bytes", C.c_size_t),
        ("status", C.c_void_p),
        ("timeout_ms", C.c_uint),
        ("out_q8", C.c_void_p),
        ("out_q8_scale", C.c_void_p),
        ("q8_rows", C.c_int),
        ("q8_row_elems", C.c_int),
    ]


# every symbol include/flb_attn.h declares: name -> (restype, argtypes)
_PP = C.POINTER(FlbAttnParams)
EXPORTS = {
    "flb_attn_abi_version": (C.c_int, []),
    "flb_status_string": (C.c_char_p, [C.c_int]),
    "flb_attn_workspace_bytes": (C.c_int, [_PP, C.POINTER(C.c_size_t)]),
    "flb_attn_counter_bytes": (C.c_int, [_PP, C.POINTER(C.c_size_t)]),
    "flb_attn_validate": (C.c_int, [_PP]),
    "flb_attn_decode": (C.c_int, [_PP, C.c_void_p]),
    "flb_attn_prefill": (C.c_int, [_PP, C.c_void_p]),
    "flb_attn_forward": (C.c_int, [_PP, C.c_void_p]),
    "flb_attn_classify_mask": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_int), C.c_void_p]),
    "flb_attn_scratch_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint), C.c_void_p]),
    "flb_attn_decode_static_scratch": (C.c_int, [_PP, C.c_void_p]),
    "flb_attn_static_scratch_status": (C.c_int, [C.POINTER(C.c_uint), C.c_void_p]),
    "flb_attn_peer_exchange": (C.c_int, [C.POINTER(FlbPeerExchange), C.c_void_p]),
    "flb_attn_quantize": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
}

_lib = None


class FlbError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"flb_attn status {status}: {text}")
        self.status = status


def load_library(path: str | None = None) -> C.CDLL:
    """Loads libflb_attn.so and types its entry points.  Raises if the library is absent or a
    declared symbol is missing; nothing else can serve the calls."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise FileNotFoundError(
            f"{p} is missing: build it with `python -m fasterllama_b200.build` (nvcc, sm_100a). "
            "There is no CPU or PyTorch fallback for the attention path."
        )
    lib = C.CDLL(p)
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    if lib.flb_attn_abi_version() != 4:
        raise RuntimeError("libflb_attn.so has an unexpected ABI version")
    if path is None:
        _lib = lib
    return lib


def check(status: int) -> None:
    if status != FLB_OK:
        raise FlbError(status, load_library().flb_status_string(status).decode())
