"""ctypes binding of oracle/_ref/libflb_ref.so — the REFERENCE's own attention kernels and cuBLAS
calls (built by oracle/build_ref.sh from the reference checkout).  TEST / BASELINE
INFRASTRUCTURE: used to pin the oracle, by the live parity tests and by the benchmark's reference
arm; never by the product path."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_ref", "libflb_ref.so")


class RefAttnArgs(C.Structure):
    _fields_ = [
        ("batch_size", C.c_int), ("head_num", C.c_int), ("size_per_head", C.c_int),
        ("seq_len", C.c_int), ("start_pos", C.c_int), ("total_len", C.c_int),
        ("Q", C.c_void_p), ("K", C.c_void_p), ("V", C.c_void_p),
        ("act_scale", C.c_void_p),
        ("q_w_scale", C.c_void_p), ("k_w_scale", C.c_void_p), ("v_w_scale", C.c_void_p),
        ("freq_cis", C.c_void_p),
        ("attn_mask", C.c_void_p),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("q_out", C.c_void_p), ("k_out", C.c_void_p), ("v_out", C.c_void_p),
        ("qk_buf", C.c_void_p),
        ("out", C.c_void_p),
        ("as_written", C.c_int),
    ]


def available() -> bool:
    return os.path.exists(LIB)


class RefRunner:
    """Owns one cuBLAS handle; `attention` enqueues the reference's seven-step attention chain."""

    def __init__(self):
        if not available():
            raise FileNotFoundError(f"{LIB} is missing (oracle/build_ref.sh builds it where the reference checkout exists)")
        self.lib = C.CDLL(LIB)
        self.lib.ref_create.restype = C.c_void_p
        self.lib.ref_destroy.argtypes = [C.c_void_p]
        self.lib.ref_attention.restype = C.c_int
        self.lib.ref_attention.argtypes = [C.c_void_p, C.POINTER(RefAttnArgs), C.c_void_p]
        self.lib.ref_freq_cis.restype = C.c_int
        self.lib.ref_freq_cis.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        if hasattr(self.lib, "ref_attn_quant"):
            self.lib.ref_attn_quant.restype = C.c_int
            self.lib.ref_attn_quant.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        self.handle = self.lib.ref_create()
        if not self.handle:
            raise RuntimeError("cublasCreate failed")

    def close(self):
        if self.handle:
            self.lib.ref_destroy(self.handle)
            self.handle = None

    def make_args(self, t: dict, *, start_pos: int, rope_row: int = 0, as_written: bool = False) -> RefAttnArgs:
        """`t` maps names to torch CUDA tensors: q,k,v int32 [B,S,H,d]; act_scale; *_w_scale;
        freq_cis [rows,d]; attn_mask [T,T] or absent; k_cache,v_cache fp32 [B,H,T,d];
        out fp32 [B,H,S,d]; work buffers are allocated here (set-up, not timed)."""
        import torch

        B, S, H, d = t["q"].shape
        T = t["k_cache"].shape[2]
        L = S + start_pos
        if "_buffers" not in t:
            dev = t["q"].device
            t["_buffers"] = {
                "q_out": torch.empty(B * H * S * d, dtype=torch.float32, device=dev),
                "k_out": torch.empty(B * H * S * d, dtype=torch.float32, device=dev),
                "v_out": torch.empty(B * H * S * d, dtype=torch.float32, device=dev),
                "qk_buf": torch.zeros(B * H * S * max(T, d), dtype=torch.float32, device=dev),
            }
        w = t["_buffers"]
        a = RefAttnArgs()
        a.batch_size, a.head_num, a.size_per_head, a.seq_len, a.start_pos, a.total_len = B, H, d, S, start_pos, T
        a.Q, a.K, a.V = t["q"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr()
        a.act_scale = t["act_scale"].data_ptr()
        a.q_w_scale, a.k_w_scale, a.v_w_scale = t["q_w_scale"].data_ptr(), t["k_w_scale"].data_ptr(), t["v_w_scale"].data_ptr()
        # the reference rotates token s with row s of the pointer it is handed: offset the pointer
        a.freq_cis = t["freq_cis"].data_ptr() + rope_row * d * 4
        a.attn_mask = t["attn_mask"].data_ptr() if t.get("attn_mask") is not None else None
        a.k_cache, a.v_cache = t["k_cache"].data_ptr(), t["v_cache"].data_ptr()
        a.q_out, a.k_out, a.v_out, a.qk_buf = (w[n].data_ptr() for n in ("q_out", "k_out", "v_out", "qk_buf"))
        a.out = t["out"].data_ptr()
        a.as_written = int(as_written)
        a._keep = (t, w)
        assert L <= T
        return a

    def attention(self, args: RefAttnArgs, stream=None) -> int:
        import torch

        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        return int(self.lib.ref_attention(self.handle, C.byref(args), s))

    def attn_quant(self, attn):
        """The reference's launchAttnQuantizedTransposeKernel on a [B,H,S,d] fp32 CUDA tensor."""
        import torch

        B, H, S, d = attn.shape
        q8 = torch.empty((B, S, H * d), dtype=torch.int8, device=attn.device)
        sc = torch.empty((B * S,), dtype=torch.float32, device=attn.device)
        st = self.lib.ref_attn_quant(q8.data_ptr(), attn.data_ptr(), sc.data_ptr(), B, H, S, d, torch.cuda.current_stream().cuda_stream)
        if st != 0:
            raise RuntimeError(f"ref_attn_quant status {st}")
        return q8, sc

    def freq_cis(self, rows: int, d: int = 128):
        import torch

        t = torch.empty((rows, d), dtype=torch.float32, device="cuda")
        st = self.lib.ref_freq_cis(t.data_ptr(), d, rows, torch.cuda.current_stream().cuda_stream)
        if st != 0:
            raise RuntimeError(f"ref_freq_cis status {st}")
        return t
