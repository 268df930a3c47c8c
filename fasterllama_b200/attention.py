"""Host-side entry to the attention path: builds the `flb_attn_params` block from tensors and calls
the C ABI.  The argument names follow the reference's attention section of
`OpenDecoder::forward` (fasterLlama/cuda/open_decoder.cu:138-239): q/k/v are what the QKV GEMMs
leave in `query_buf_/key_buf_/value_buf_` ([B, S, H, d]), the caches are `key_cache_/value_cache_`
([B, H, T, d]), `out` is `qkv_buf_` ([B, H, S, d]), `scratch` stands in for `qk_buf_`.

Tensors may be torch CUDA tensors (the product path) or numpy arrays (host memory — only the
test oracle consumes those; the CUDA entry points are never given host pointers)."""
from __future__ import annotations

import ctypes as C
import math
from typing import Any

from . import _lib
from ._lib import (  # noqa: F401  (re-exported)
    FLB_F16,
    FLB_F32,
    FLB_IN_F16,
    FLB_IN_F32,
    FLB_IN_INT32,
    FLB_MASK_CAUSAL_INCLUSIVE,
    FLB_MASK_CAUSAL_STRICT,
    FLB_MASK_GENERIC,
    FLB_MASK_NONE,
    FlbAttnParams,
    FlbError,
)


def _ptr(t: Any) -> int | None:
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data  # numpy


def _dtype_name(t: Any) -> str:
    return str(t.dtype).replace("torch.", "")


def _is_contiguous(t: Any) -> bool:
    if hasattr(t, "is_contiguous"):
        return t.is_contiguous()
    return bool(t.flags["C_CONTIGUOUS"])


_IN_MODE = {"int32": FLB_IN_INT32, "float32": FLB_IN_F32, "float16": FLB_IN_F16}
_DT = {"float32": FLB_F32, "float16": FLB_F16}


def _token_row_stride(t: Any, B: int, S: int, H: int, d: int) -> int:
    """Elements between the rows of two consecutive tokens of a q/k/v tensor shaped [B,S,H,d]: H*d when it is dense,
    more when it is a column block of a wider [B*S, row] buffer (the output of one merged QKV projection).  Raises
    for any other layout."""
    if hasattr(t, "stride") and callable(t.stride):
        st = tuple(int(x) for x in t.stride())
    else:
        st = tuple(int(x) // t.itemsize for x in t.strides)
    row = st[1] if S > 1 else (st[0] if B > 1 else H * d)
    ok = (d == 1 or st[3] == 1) and (H == 1 or st[2] == d) and (S == 1 or st[1] == row) and (B == 1 or st[0] == S * row) and row >= H * d
    if not ok:
        raise ValueError("q, k and v must be [B,S,H,d] with unit element stride, head stride d and one common token-row stride")
    return row


def make_params(
    *,
    q,
    k,
    v,
    k_cache,
    v_cache,
    out,
    scratch=None,
    start_pos: int = 0,
    past_lens=None,
    max_past_len: int = 0,
    act_scale=None,
    q_w_scale=None,
    k_w_scale=None,
    v_w_scale=None,
    freq_cis=None,
    rope_pos0: int = 0,
    rope_add_past: bool = False,
    mask_mode: int = FLB_MASK_CAUSAL_INCLUSIVE,
    attn_mask=None,
    mask_row_stride: int = 0,
    softmax_scale: float | None = None,
    scratch_zeroed: bool = False,
    split_len: int = 0,
    out_q8=None,
    out_q8_scale=None,
    out_peers=None,
    out_head_total: int = 0,
    out_head_offset: int = 0,
    out_dtype: str | None = None,
    early_start: int = 0,
) -> FlbAttnParams:
    """Fills a `flb_attn_params`.  Shapes: q/k/v [B,S,H,d]; caches [B,H,T,d]; out [B,H,S,d];
    past_lens int32 [B]; freq_cis float32 [rows,d]; attn_mask float32 [*, mask_row_stride]."""
    B, S, H, d = (int(x) for x in q.shape)
    if tuple(k.shape) != (B, S, H, d) or tuple(v.shape) != (B, S, H, d):
        raise ValueError("q, k and v must share the shape [B, S, H, d]")
    if tuple(k_cache.shape) != tuple(v_cache.shape) or k_cache.shape[0] != B or k_cache.shape[1] != H or k_cache.shape[3] != d:
        raise ValueError("caches must be [B, H, T, d]")
    if out_peers is None and tuple(out.shape) != (B, H, S, d):
        raise ValueError("out must be [B, H, S, d]")
    for name, t in (("k_cache", k_cache), ("v_cache", v_cache), ("out", out)):
        if t is not None and not _is_contiguous(t):
            raise ValueError(f"{name} must be contiguous")
    rows = {_token_row_stride(t, B, S, H, d) for t in (q, k, v)}
    if len(rows) != 1:
        raise ValueError("q, k and v must share one token-row stride")
    row_stride = rows.pop()
    T = int(k_cache.shape[2])
    p = FlbAttnParams()
    p.batch_size, p.head_num, p.size_per_head, p.seq_len = B, H, d, S
    p.start_pos, p.total_len = int(start_pos), T
    p.past_lens = _ptr(past_lens)
    p.max_past_len = int(max_past_len)
    p.input_mode = _IN_MODE[_dtype_name(q)]
    p.q, p.k, p.v = _ptr(q), _ptr(k), _ptr(v)
    p.qkv_row_stride = 0 if row_stride == H * d else row_stride
    p.act_scale, p.q_w_scale, p.k_w_scale, p.v_w_scale = _ptr(act_scale), _ptr(q_w_scale), _ptr(k_w_scale), _ptr(v_w_scale)
    p.freq_cis = _ptr(freq_cis)
    p.rope_pos0, p.rope_add_past = int(rope_pos0), int(bool(rope_add_past))
    p.mask_mode = int(mask_mode)
    p.attn_mask = _ptr(attn_mask)
    if attn_mask is not None and not mask_row_stride:
        mask_row_stride = int(attn_mask.shape[-1])
    p.mask_row_stride = int(mask_row_stride)
    p.k_cache, p.v_cache = _ptr(k_cache), _ptr(v_cache)
    p.cache_dtype = _DT[_dtype_name(k_cache)]
    p.out = _ptr(out)
    p.out_dtype = _DT[_dtype_name(out)] if out is not None else _DT[out_dtype or "float32"]  # push form: the peers' element type
    if out_peers is not None:
        # head-split push: device addresses (ints) of every rank's [B, out_head_total, 1, d] buffer
        if len(out_peers) > _lib.FLB_MAX_PEERS:
            raise ValueError("too many peers")
        for i, addr in enumerate(out_peers):
            p.out_peers[i] = int(addr)
        p.n_out_peers = len(out_peers)
        p.out_head_total, p.out_head_offset = int(out_head_total), int(out_head_offset)
    p.softmax_scale = float(softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d))
    p.scratch = _ptr(scratch)
    p.scratch_bytes = int(scratch.numel() * scratch.element_size()) if hasattr(scratch, "numel") else (int(scratch.nbytes) if scratch is not None else 0)
    p.scratch_zeroed = int(bool(scratch_zeroed))
    p.split_len = int(split_len)
    p.early_start = int(early_start)  # 0 off, 1 or 2: see flb_attn_params.early_start
    p.out_q8, p.out_q8_scale = _ptr(out_q8), _ptr(out_q8_scale)
    # keep the tensors alive as long as the block
    p._keep = (q, k, v, k_cache, v_cache, out, scratch, past_lens, act_scale, q_w_scale, k_w_scale, v_w_scale, freq_cis, attn_mask, out_q8, out_q8_scale)
    return p


def workspace_bytes(batch_size: int, head_num: int, total_len: int, seq_len: int = 1, split_len: int = 0,
                    size_per_head: int = 128) -> int:
    """Scratch bytes for every call these dimensions allow (decode on a full cache, prefill of
    `seq_len` tokens)."""
    p = FlbAttnParams()
    p.batch_size, p.head_num, p.size_per_head = batch_size, head_num, size_per_head
    p.total_len, p.seq_len, p.split_len = total_len, seq_len, split_len
    n = C.c_size_t(0)
    _lib.check(_lib.load_library().flb_attn_workspace_bytes(C.byref(p), C.byref(n)))
    return int(n.value)


def counter_bytes(batch_size: int, head_num: int) -> int:
    p = FlbAttnParams()
    p.batch_size, p.head_num = batch_size, head_num
    n = C.c_size_t(0)
    _lib.check(_lib.load_library().flb_attn_counter_bytes(C.byref(p), C.byref(n)))
    return int(n.value)


def _stream_handle(stream) -> int | None:
    if stream is None:
        import torch

        return torch.cuda.current_stream().cuda_stream
    if hasattr(stream, "cuda_stream"):
        return stream.cuda_stream
    return int(stream)


def validate(p: FlbAttnParams) -> int:
    return int(_lib.load_library().flb_attn_validate(C.byref(p)))


def forward(p: FlbAttnParams, stream=None) -> None:
    """Decode when seq_len == 1, prefill otherwise — the switch of open_decoder.cu:179."""
    _lib.check(_lib.load_library().flb_attn_forward(C.byref(p), _stream_handle(stream)))


def decode(p: FlbAttnParams, stream=None) -> None:
    _lib.check(_lib.load_library().flb_attn_decode(C.byref(p), _stream_handle(stream)))


def decode_static_scratch(p: FlbAttnParams, stream=None) -> None:
    """Decode with the library's own fixed scratch block (for callers that cannot provide any):
    `p.scratch` is ignored.  One block per GPU — keep these calls on one stream."""
    _lib.check(_lib.load_library().flb_attn_decode_static_scratch(C.byref(p), _stream_handle(stream)))


def static_scratch_status(stream=None) -> int:
    """Error word of the calls made through `decode_static_scratch` on the current GPU (0 = clean)."""
    st = C.c_uint(0)
    _lib.check(_lib.load_library().flb_attn_static_scratch_status(C.byref(st), _stream_handle(stream)))
    return int(st.value)


def quantize(attn, q8, scale, stream=None) -> None:
    """The reference's attention-output quantisation as a call of its own: attn fp32 [B,H,S,d] -> q8 int8 [B,S,H*d],
    scale fp32 [B*S]."""
    B, H, S, d = (int(v) for v in attn.shape)
    _lib.check(_lib.load_library().flb_attn_quantize(attn.data_ptr(), q8.data_ptr(), scale.data_ptr(), B, H, S, d, _stream_handle(stream)))


def peer_exchange(*, rank: int, size: int, epoch: int, flags_local: int, flags_peer, recv: int = 0, dst: int = 0,
                  nbytes: int = 0, status: int = 0, timeout_ms: int = 0, out_q8: int = 0, out_q8_scale: int = 0,
                  q8_rows: int = 0, q8_row_elems: int = 0, stream=None) -> None:
    """The hand-shake that follows a pushing decode call (see `flb_peer_exchange`): all pointers are device
    addresses; `flags_peer[r]` is rank r's flag array as mapped into this process."""
    x = _lib.FlbPeerExchange()
    x.rank, x.size, x.epoch = int(rank), int(size), int(epoch)
    x.flags_local = int(flags_local)
    for r, addr in enumerate(flags_peer):
        x.flags_peer[r] = int(addr) if addr else None
    x.recv, x.dst, x.bytes = (int(recv) or None), (int(dst) or None), int(nbytes)
    x.status = int(status) or None
    x.timeout_ms = int(timeout_ms)
    x.out_q8, x.out_q8_scale = (int(out_q8) or None), (int(out_q8_scale) or None)
    x.q8_rows, x.q8_row_elems = int(q8_rows), int(q8_row_elems)
    _lib.check(_lib.load_library().flb_attn_peer_exchange(C.byref(x), _stream_handle(stream)))


def prefill(p: FlbAttnParams, stream=None) -> None:
    _lib.check(_lib.load_library().flb_attn_prefill(C.byref(p), _stream_handle(stream)))


def classify_mask(attn_mask, rows: int | None = None, stream=None) -> int:
    """Which mask mode reproduces a caller-built additive [T, T] mask.  Set-up time only."""
    import torch

    rows = int(rows if rows is not None else attn_mask.shape[0])
    tmp = torch.empty(4, dtype=torch.int32, device=attn_mask.device)
    mode = C.c_int(-1)
    _lib.check(
        _lib.load_library().flb_attn_classify_mask(
            attn_mask.data_ptr(), rows, int(attn_mask.shape[-1]), tmp.data_ptr(), C.byref(mode), _stream_handle(stream)
        )
    )
    return int(mode.value)


def scratch_status(scratch, stream=None) -> int:
    """Error word the kernels leave at the head of `scratch` (0 = clean)."""
    st = C.c_uint(0)
    _lib.check(_lib.load_library().flb_attn_scratch_status(scratch.data_ptr(), C.byref(st), _stream_handle(stream)))
    return int(st.value)
