"""Host-side tests of the C ABI: the library loads, exports every declared symbol, and the
argument checks answer with the documented status codes.  No compute call is made (no GPU)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from fasterllama_b200 import _lib
from fasterllama_b200 import attention as A
from fasterllama_b200 import workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load_library()
    header = open(os.path.join(ROOT, "include", "flb_attn.h")).read()
    declared = set(re.findall(r"^(?:int|const char \*)\s*(flb_\w+)\s*\(", header, flags=re.M))
    assert declared, "no declarations found in the header"
    assert declared == set(_lib.EXPORTS), (declared ^ set(_lib.EXPORTS))
    for name in declared:
        assert hasattr(lib, name)
    assert lib.flb_attn_abi_version() == 4


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(FileNotFoundError):
        _lib.load_library(str(tmp_path / "nope.so"))


def test_struct_layout_matches_the_header(tmp_path):
    # a C compiler's view of the struct: compile a tiny probe against the header
    import subprocess
    probe = str(tmp_path / "abi_probe.c")
    exe = str(tmp_path / "abi_probe")
    with open(probe, "w") as f:
        f.write('#include <stdio.h>\n#include "flb_attn.h"\nint main(void){printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(flb_attn_params),'
                ' offsetof(flb_attn_params, past_lens), offsetof(flb_attn_params, softmax_scale), offsetof(flb_attn_params, out_q8_scale),'
                ' offsetof(flb_attn_params, out_peers), offsetof(flb_attn_params, out_head_offset), sizeof(flb_peer_exchange),'
                ' offsetof(flb_peer_exchange, flags_peer), offsetof(flb_peer_exchange, timeout_ms));return 0;}\n')
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), probe, "-o", exe], check=True)
    got = [int(x) for x in subprocess.run([exe], check=True, capture_output=True, text=True).stdout.split()]
    P = _lib.FlbAttnParams
    X = _lib.FlbPeerExchange
    assert got == [C.sizeof(P), P.past_lens.offset, P.softmax_scale.offset, P.out_q8_scale.offset, P.out_peers.offset,
                   P.out_head_offset.offset, C.sizeof(X), X.flags_peer.offset, X.timeout_ms.offset]


def _valid_case():
    c = W.host_case("v", 1, 2, 4, 64, past=10)
    c.arrays["scratch"] = np.zeros(A.workspace_bytes(2, 4, 64), dtype=np.uint8)
    return c


def test_validate_accepts_a_good_block_and_names_each_fault():
    c = _valid_case()
    assert A.validate(c.params()) == _lib.FLB_OK

    p = c.params(); p.q = None
    assert A.validate(p) == _lib.FLB_ERR_NULL_POINTER
    p = c.params(); p.scratch = None
    assert A.validate(p) == _lib.FLB_ERR_NULL_POINTER
    p = c.params(); p.size_per_head = 96  # decode takes 64, 128 and 256
    assert A.validate(p) == _lib.FLB_ERR_UNSUPPORTED
    p = c.params(); p.batch_size = 0
    assert A.validate(p) == _lib.FLB_ERR_BAD_SHAPE
    p = c.params(); p.start_pos = 64  # start_pos + 1 > total_len
    assert A.validate(p) == _lib.FLB_ERR_BAD_SHAPE
    p = c.params(); p.mask_mode = 9
    assert A.validate(p) == _lib.FLB_ERR_BAD_ENUM
    p = c.params(); p.cache_dtype = 5
    assert A.validate(p) == _lib.FLB_ERR_BAD_ENUM
    p = c.params(); p.k_cache = p.k_cache + 4
    assert A.validate(p) == _lib.FLB_ERR_MISALIGNED
    p = c.params(); p.scratch_bytes = 16
    assert A.validate(p) == _lib.FLB_ERR_SCRATCH_TOO_SMALL
    p = c.params(); p.mask_mode = A.FLB_MASK_GENERIC  # no mask pointer
    assert A.validate(p) == _lib.FLB_ERR_NULL_POINTER
    p = c.params(); p.split_len = 100  # not a multiple of 32
    assert A.validate(p) == _lib.FLB_ERR_BAD_SHAPE
    p = c.params(); p.input_mode = A.FLB_IN_INT32  # scales missing
    assert A.validate(p) == _lib.FLB_ERR_NULL_POINTER
    # head-split push: destinations, head window and mode are checked; `out` is not needed then
    p = c.params(); p.n_out_peers = 2; p.out_head_total = 8; p.out_head_offset = 4
    p.out_peers[0] = p.out; p.out_peers[1] = p.out; p.out = None
    assert A.validate(p) == _lib.FLB_OK
    p.out_head_offset = 6  # 6 + 4 local heads > 8
    assert A.validate(p) == _lib.FLB_ERR_BAD_SHAPE
    p.out_head_offset = 4; p.out_peers[1] = None
    assert A.validate(p) == _lib.FLB_ERR_NULL_POINTER
    p = c.params(); p.n_out_peers = 9
    assert A.validate(p) == _lib.FLB_ERR_BAD_SHAPE
    p = c.params(); p.early_start = 3  # levels are 0, 1, 2
    assert A.validate(p) == _lib.FLB_ERR_BAD_ENUM
    p = c.params(); p.early_start = 2
    assert A.validate(p) == _lib.FLB_OK
    assert _lib.load_library().flb_attn_validate(None) == _lib.FLB_ERR_NULL_POINTER


def test_launch_entry_points_refuse_bad_blocks_without_touching_cuda():
    lib = _lib.load_library()
    c = _valid_case()
    p = c.params(); p.q = None
    assert lib.flb_attn_decode(C.byref(p), None) == _lib.FLB_ERR_NULL_POINTER
    assert lib.flb_attn_forward(None, None) == _lib.FLB_ERR_NULL_POINTER
    p = c.params(); p.seq_len = 4
    assert lib.flb_attn_decode(C.byref(p), None) == _lib.FLB_ERR_BAD_SHAPE
    p = c.params()
    assert lib.flb_attn_prefill(C.byref(p), None) == _lib.FLB_ERR_BAD_SHAPE  # seq_len == 1
    # prefill over a non-empty cache does not exist in the reference
    pc = W.host_case("p", 1, 1, 4, 64, S=8, past=0)
    pc.arrays["scratch"] = np.zeros(A.workspace_bytes(1, 4, 64, 8), dtype=np.uint8)
    p = pc.params(); p.start_pos = 3
    assert lib.flb_attn_prefill(C.byref(p), None) == _lib.FLB_ERR_UNSUPPORTED


def test_workspace_grows_with_cache_capacity_and_covers_the_counters():
    small = A.workspace_bytes(2, 4, 257)
    big = A.workspace_bytes(2, 4, 4097)
    assert big > small > A.counter_bytes(2, 4) >= 16 + 4 * 8
    assert A.workspace_bytes(2, 4, 4097, split_len=1024) < big < A.workspace_bytes(2, 4, 4097, split_len=256)


def test_status_strings():
    lib = _lib.load_library()
    seen = {lib.flb_status_string(s) for s in range(0, -10, -1)}
    assert len(seen) == 10 and all(seen)
    assert lib.flb_status_string(-77) == b"unknown status"


def test_exchange_and_quantize_argument_checks_need_no_gpu():
    """Both calls answer bad arguments before they touch the CUDA runtime."""
    lib = _lib.load_library()
    x = _lib.FlbPeerExchange()
    assert lib.flb_attn_peer_exchange(None, None) == _lib.FLB_ERR_NULL_POINTER
    assert lib.flb_attn_peer_exchange(C.byref(x), None) == _lib.FLB_ERR_NULL_POINTER  # no flag words
    x.flags_local = 4096
    x.rank, x.size, x.epoch = 0, 9, 1
    assert lib.flb_attn_peer_exchange(C.byref(x), None) == _lib.FLB_ERR_BAD_SHAPE  # more ranks than FLB_MAX_PEERS
    x.size, x.epoch = 2, 0
    assert lib.flb_attn_peer_exchange(C.byref(x), None) == _lib.FLB_ERR_BAD_SHAPE  # epochs start at 1
    x.epoch = 1
    x.out_q8 = 4096  # codes without a place for the scales
    assert lib.flb_attn_peer_exchange(C.byref(x), None) == _lib.FLB_ERR_NULL_POINTER
    x.out_q8 = None
    assert lib.flb_attn_peer_exchange(C.byref(x), None) == _lib.FLB_ERR_NULL_POINTER  # rank 1's flag words missing
    assert lib.flb_attn_quantize(None, None, None, 1, 1, 1, 128, None) == _lib.FLB_ERR_NULL_POINTER
    assert lib.flb_attn_quantize(4096, 4096, 4096, 1, 1, 1, 96, None) == _lib.FLB_ERR_UNSUPPORTED
    assert lib.flb_attn_quantize(4096, 4096, 4096, 0, 1, 1, 128, None) == _lib.FLB_ERR_BAD_SHAPE
