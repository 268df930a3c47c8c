"""Parity of the CUDA decode attention (through the C ABI) against the host oracle."""
import numpy as np
import pytest

from fasterllama_b200 import attention as A
from fasterllama_b200 import workloads as W

from util import FP16_ABS, assert_abs_close, assert_fp32_close, run_cuda, run_oracle

pytestmark = pytest.mark.gpu

# every tile (16/32 rows) and split (512 rows) boundary, +-1
LENGTHS = [0, 1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 255, 256, 257, 511, 512, 513, 700, 1024, 1025]


def _check(case, cuda, orc, fp16):
    assert cuda["status"] == 0, f"kernel status word {cuda['status']:#x}"
    if fp16:
        assert_abs_close(cuda["out"], orc["out"].astype(np.float32), FP16_ABS, case.name + " out")
    else:
        assert_fp32_close(cuda["out"], orc["out"], what=case.name + " out")
    # the appended rows are bit-exact (same dequant/RoPE arithmetic up to fma contraction -> 1e-6),
    # every other cache row is untouched
    kc, ko = cuda["k_cache"], orc["k_cache"].astype(np.float32)
    vc, vo = cuda["v_cache"], orc["v_cache"].astype(np.float32)
    tol = 2e-3 if fp16 else 1e-5
    assert np.abs(kc - ko).max() <= tol * max(1.0, np.abs(ko).max())
    assert np.array_equal(vc, vo), "V cache differs (append is a pure copy/round)"


@pytest.mark.parametrize("past", LENGTHS)
def test_fp32_decode_lengths(cuda_device, past):
    case = W.host_case(f"fp32-L{past}", 100 + past, 1, 4, 1100, past=past)
    _check(case, run_cuda(case), run_oracle(case), fp16=False)


@pytest.mark.parametrize("past", LENGTHS)
def test_fp16_decode_lengths(cuda_device, past):
    case = W.host_case(f"fp16-L{past}", 200 + past, 2, 4, 1100, past=past, in_dtype="float16",
                       cache_dtype="float16", out_dtype="float16")
    _check(case, run_cuda(case), run_oracle(case), fp16=True)


@pytest.mark.parametrize("mask_mode", [A.FLB_MASK_NONE, A.FLB_MASK_GENERIC, A.FLB_MASK_CAUSAL_INCLUSIVE, A.FLB_MASK_CAUSAL_STRICT])
@pytest.mark.parametrize("past", [0, 5, 300])
def test_mask_modes(cuda_device, mask_mode, past):
    case = W.host_case(f"mask{mask_mode}-L{past}", 300 + past, 2, 4, 400, past=past, mask_mode=mask_mode)
    cuda, orc = run_cuda(case), run_oracle(case)
    _check(case, cuda, orc, fp16=False)
    if mask_mode == A.FLB_MASK_CAUSAL_STRICT and past == 0:
        # the only key is the token itself and it is masked: the row is fully masked -> zeros
        assert not cuda["out"].any()


def test_int32_inputs_with_scales(cuda_device):
    """The reference's post-GEMM form: int32 accumulators, per-token and per-channel scales."""
    case = W.host_case("int32", 7, 3, 8, 600, past=411, in_dtype="int32")
    _check(case, run_cuda(case), run_oracle(case), fp16=False)


def test_reference_rope_row(cuda_device):
    """The reference rotates a decode token with table row 0 of the pointer it is given."""
    case = W.host_case("rope-ref", 8, 2, 4, 300, past=200, rope="reference")
    _check(case, run_cuda(case), run_oracle(case), fp16=False)
    case = W.host_case("rope-none", 9, 2, 4, 300, past=200, rope="none")
    _check(case, run_cuda(case), run_oracle(case), fp16=False)


def test_per_sequence_lengths(cuda_device):
    lens = np.array([0, 1, 255, 256, 257, 1000, 513, 31], dtype=np.int32)
    case = W.host_case("ragged", 11, 8, 4, 1100, past=lens, in_dtype="float16", cache_dtype="float16", out_dtype="float32")
    _check(case, run_cuda(case), run_oracle(case), fp16=True)


def test_config1_fp32_llama7b_layer(cuda_device):
    """fp32, batch 1, 32 heads x 128, cache 256, RoPE at position 256, seed 0."""
    case = W.host_case("config1", 0, 1, 32, 512, past=256)
    cuda, orc = run_cuda(case), run_oracle(case)
    _check(case, cuda, orc, fp16=False)


def test_config2_fp16_llama7b_full_size(cuda_device):
    """fp16, batch 16, 32 heads x 128, lengths uniform in [1024, 2048], seed 1 — full size."""
    lens = W.draw_lengths(1, 16, 1024, 2048)
    case = W.host_case("config2", 1, 16, 32, 2049, past=lens, in_dtype="float16", cache_dtype="float16", out_dtype="float16")
    _check(case, run_cuda(case), run_oracle(case), fp16=True)


def test_split_len_and_repeat_calls(cuda_device):
    """Other split sizes give results within tolerance of each other; repeating the call on the
    same scratch (counters must have been left at zero) is bit-identical."""
    base = W.host_case("split", 21, 2, 4, 1200, past=1100)
    orc = run_oracle(base)
    outs = []
    for sl in (64, 128, 256, 512):
        case = W.host_case("split", 21, 2, 4, 1200, past=1100, split_len=sl)
        cuda = run_cuda(case)
        _check(case, cuda, orc, fp16=False)
        outs.append(cuda["out"])
    import torch
    case = W.host_case("split", 21, 2, 4, 1200, past=1100)
    r = run_cuda(case, calls=1)
    dev = r["dev"]
    p = case.params(dev)
    first = dev["out"].clone()
    for _ in range(3):
        A.forward(p)
    torch.cuda.synchronize()
    assert torch.equal(first, dev["out"])
    case.scratch_zeroed = True  # counters were left at zero by the calls above
    A.forward(case.params(dev))
    torch.cuda.synchronize()
    assert torch.equal(first, dev["out"])


def test_head_sharding_is_bit_identical(cuda_device):
    """Running a subset of the (b,h) units alone gives the same bits as running them in the full
    batch: the split partition depends on each sequence's length only."""
    import torch
    lens = np.array([700, 300, 1024, 77], dtype=np.int32)
    full = W.host_case("shard-full", 31, 4, 8, 1100, past=lens)
    out_full = run_cuda(full)["out"]
    for hs in (slice(0, 4), slice(4, 8)):
        part = W.host_case("shard-full", 31, 4, 8, 1100, past=lens)
        a = part.arrays
        for n in ("q", "k", "v"):
            a[n] = np.ascontiguousarray(a[n][:, :, hs])
        for n in ("k_cache", "v_cache", "out"):
            a[n] = np.ascontiguousarray(a[n][:, hs])
        part.H = 4
        got = run_cuda(part)["out"]
        assert np.array_equal(got, out_full[:, hs])


def test_out_of_range_length_is_flagged_not_followed(cuda_device):
    """A per-sequence length outside [0, total_len - 1] (a caller bug) must not make the kernel read or
    write outside the cache slab: the length is clamped, the call completes, and the status word at the
    head of the scratch reports it (bit 4) for the host to read."""
    import torch
    lens = np.array([100, 50], dtype=np.int32)
    case = W.host_case("badlen", 51, 2, 4, 256, past=lens)
    dev = W.to_device(case)
    guard = 0xA5
    # canaries either side of the caches: the clamped kernel must leave them alone
    for n in ("k_cache", "v_cache"):
        buf = torch.full((dev[n].numel() + 4096,), float("nan"), device="cuda")
        buf[2048:2048 + dev[n].numel()] = dev[n].flatten()
        dev[n + "_buf"] = buf
        dev[n] = buf[2048:2048 + dev[n].numel()].view(dev[n].shape)
    dev["past_lens"] = torch.tensor([100, 100000], dtype=torch.int32, device="cuda")  # second entry is nonsense
    case.max_past_len = 255
    p = case.params(dev)
    A.forward(p)
    torch.cuda.synchronize()
    assert A.scratch_status(dev["scratch"]) & 4, "the bad length was not reported"
    for n in ("k_cache_buf", "v_cache_buf"):
        assert torch.isnan(dev[n][:2048]).all() and torch.isnan(dev[n][-2048:]).all(), "write outside the cache slab"
    # the well-formed sequence is still right
    good = W.host_case("badlen", 51, 2, 4, 256, past=lens)
    orc = run_oracle(good)
    assert_fp32_close(dev["out"][0].cpu().numpy(), orc["out"][0], what="sequence with a valid length")
    # and the next, well-formed call on the same scratch is clean again
    dev["past_lens"] = torch.from_numpy(lens).cuda()
    A.forward(case.params(dev))
    torch.cuda.synchronize()
    assert A.scratch_status(dev["scratch"]) == 0


@pytest.mark.parametrize("in_dtype,cache_dtype,out_dtype", [("float16", "float16", "float16"), ("int32", "float32", "float32")])
def test_pinned_host_inputs_and_output(cuda_device, in_dtype, cache_dtype, out_dtype):
    """q, k, v (and the scales) and the output may live in pinned host memory: the kernel reads and writes them
    over the bus, the caches and the scratch stay on the device.  Same results, bit for bit, as with device
    buffers."""
    import torch

    past = np.array([1200, 3, 513], dtype=np.int32)
    case = W.host_case("pinned", 77, 3, 8, 1300, past=past, in_dtype=in_dtype, cache_dtype=cache_dtype, out_dtype=out_dtype)
    want = run_cuda(case)
    assert want["status"] == 0
    dev = W.to_device(case, cuda_device)
    host_names = ("q", "k", "v", "act_scale", "q_w_scale", "k_w_scale", "v_w_scale")
    arrays = dict(dev)
    for n in host_names:
        if n in arrays and arrays[n] is not None:
            arrays[n] = arrays[n].cpu().pin_memory()
    arrays["out"] = torch.full_like(dev["out"], float("nan"), device="cpu").pin_memory()
    A.forward(case.params(arrays))
    torch.cuda.synchronize()
    assert A.scratch_status(dev["scratch"]) == 0
    assert np.array_equal(arrays["out"].float().numpy(), want["out"])
    assert np.array_equal(dev["k_cache"].float().cpu().numpy(), want["k_cache"])
    assert np.array_equal(dev["v_cache"].float().cpu().numpy(), want["v_cache"])


def test_early_start_calls_back_to_back(cuda_device):
    """Programmatic dependent launch (both levels): a chain of decode calls that may each start while the one before
    drains gives the same bits as ordinary launches — on rotating buffer sets and on one set reused by every call."""
    import torch

    from fasterllama_b200 import workloads as W2

    lens = W2.draw_lengths(5, 6, 200, 1500)
    outs = {}
    for early in (0, 1, 2):
        sets = []
        for j in range(3):
            c = W2.device_case("early", 50 + j, 6, 8, 1501, lens, device=cuda_device)
            c.scratch_zeroed = True
            c.early_start = early
            sets.append((c, c.params()))
        for i in range(12):
            A.decode(sets[i % 3][1])
        for _ in range(4):
            A.decode(sets[0][1])  # the same buffers, scratch and counters in consecutive launches
        torch.cuda.synchronize()
        assert all(A.scratch_status(c.arrays["scratch"]) == 0 for c, _ in sets)
        outs[early] = ([c.arrays["out"].clone() for c, _ in sets] + [c.arrays["k_cache"].clone() for c, _ in sets]
                       + [c.arrays["v_cache"].clone() for c, _ in sets])
    for level in (1, 2):
        for a, b in zip(outs[0], outs[level]):
            assert torch.equal(a, b)


def test_early_start_level1_behind_a_slow_writer(cuda_device):
    """Level 1 promises only that the cached rows are settled; q, k and v may still be on their way.  Here they are
    produced by a copy that sits behind a slow matrix product, TWO launches in front of the call under test, with
    another early-started decode call between them (a kernel that lets its successor start before it has finished
    itself).  The call must still see the finished inputs: it reads them only after the kernel in front has
    completed, and that kernel completes only after everything in front of it."""
    import torch

    from fasterllama_b200 import workloads as W2

    lens = W2.draw_lengths(9, 4, 100, 900)
    mk = lambda seed: W2.device_case("slow-writer", seed, 4, 8, 901, lens, device=cuda_device)  # noqa: E731
    ref = mk(71)
    A.decode(ref.params())
    torch.cuda.synchronize()
    want = ref.arrays["out"].clone()

    between, late = mk(72), mk(71)  # `late` has the reference's caches; its q, k, v arrive late
    final = {n: late.arrays[n].clone() for n in ("q", "k", "v")}
    for n in ("q", "k", "v"):
        late.arrays[n].zero_()
    for c in (between, late):
        c.scratch_zeroed = True
        c.early_start = 1
    big = torch.randn((6144, 6144), device=cuda_device)
    p_between, p_late = between.params(), late.params()
    torch.cuda.synchronize()
    torch.mm(big, big)                       # milliseconds of work in front of the writer
    for n in ("q", "k", "v"):
        late.arrays[n].copy_(final[n])       # the writer of the late call's inputs
    A.decode(p_between)                      # early-started, unrelated buffers
    A.decode(p_late)                         # early-started: may be resident long before its inputs exist
    torch.cuda.synchronize()
    assert A.scratch_status(late.arrays["scratch"]) == 0 and A.scratch_status(between.arrays["scratch"]) == 0
    assert torch.equal(late.arrays["out"], want)


def test_config4_fp16_13b_full_size_properties(cuda_device):
    """fp16, batch 64, 40 heads x 128, lengths uniform in [2048, 4096], seed 3 — full size (5.4 GB of cache drawn
    on the GPU).  The oracle checks a sample of (batch, head) units; size-independent properties cover the rest:
    every output is finite, a contiguous shard of the units run alone gives the same bits as inside the full
    batch, and a second call on the same buffers repeats the first."""
    import torch

    B, H, T = 64, 40, 4097
    lens = W.draw_lengths(3, B, 2048, 4096)
    case = W.device_case("config4", 3, B, H, T, lens, device=cuda_device)
    a = case.arrays
    A.decode(case.params())
    torch.cuda.synchronize()
    assert A.scratch_status(a["scratch"]) == 0
    out = a["out"].clone()
    assert torch.isfinite(out.float()).all()

    # sampled units against the host oracle (each on its own [1, 1, T, d] slab)
    rng = np.random.default_rng(4)
    for b, h in zip(rng.integers(0, B, 6), rng.integers(0, H, 6)):
        b, h = int(b), int(h)
        one = {
            "q": a["q"][b:b + 1, :, h:h + 1].cpu().numpy(), "k": a["k"][b:b + 1, :, h:h + 1].cpu().numpy(),
            "v": a["v"][b:b + 1, :, h:h + 1].cpu().numpy(),
            "k_cache": a["k_cache"][b:b + 1, h:h + 1].cpu().numpy(), "v_cache": a["v_cache"][b:b + 1, h:h + 1].cpu().numpy(),
            "out": np.zeros((1, 1, 1, 128), dtype=np.float16), "freq_cis": a["freq_cis"].cpu().numpy(),
            "past_lens": np.array([lens[b]], dtype=np.int32),
        }
        # the cache row the call appended is an output: the oracle gets the slab as it was before (row cleared)
        one["k_cache"][0, 0, lens[b]] = 0
        one["v_cache"][0, 0, lens[b]] = 0
        unit = W.Case(name=f"c4-unit-{b}-{h}", B=1, H=1, S=1, T=T, start_pos=0, arrays=one, rope_add_past=case.rope_add_past,
                      mask_mode=case.mask_mode, max_past_len=int(lens[b]))
        orc = run_oracle(unit)
        assert_abs_close(out[b, h].float().cpu().numpy(), orc["out"][0, 0].astype(np.float32), FP16_ABS, f"unit ({b},{h})")
        k_new, k_want = a["k_cache"][b, h, lens[b]].float().cpu().numpy(), orc["k_cache"][0, 0, lens[b]].astype(np.float32)
        assert np.abs(k_new - k_want).max() <= 2e-3 * max(1.0, np.abs(k_want).max())  # rotated, rounded to fp16
        assert np.array_equal(a["v_cache"][b, h, lens[b]].float().cpu().numpy(), orc["v_cache"][0, 0, lens[b]].astype(np.float32))

    # a second call repeats the first (counters were left at zero, the appended row is rewritten with the same bits)
    A.decode(case.params())
    torch.cuda.synchronize()
    assert torch.equal(out, a["out"])

    # one eighth of the batch alone (what one of 8 GPUs would run): same bits
    sl = slice(8, 16)
    part = dict(a)
    for n in ("q", "k", "v", "k_cache", "v_cache"):
        part[n] = a[n][sl].contiguous()
    part["out"] = torch.zeros_like(a["out"][sl])
    part["past_lens"] = a["past_lens"][sl].contiguous()
    part["scratch"] = torch.zeros(A.workspace_bytes(8, H, T), dtype=torch.uint8, device=cuda_device)
    sub = W.Case(name="c4-shard", B=8, H=H, S=1, T=T, start_pos=0, arrays=part, rope_add_past=case.rope_add_past,
                 mask_mode=case.mask_mode, max_past_len=case.max_past_len)
    A.decode(sub.params())
    torch.cuda.synchronize()
    assert torch.equal(part["out"], out[sl])


@pytest.mark.parametrize("cache_dtype", ["float32", "float16"])
def test_cache_at_the_reference_softmax_limit(cuda_device, cache_dtype):
    """12288 keys is where the reference's softmax kernel runs out of shared memory (4 bytes per key); here it is
    24 partitions of 512 rows per (batch, head) unit and one merge.  Ragged neighbours: 12287, 12288 and 1 keys."""
    lens = np.array([12286, 12287, 0], dtype=np.int32)
    fp16 = cache_dtype == "float16"
    case = W.host_case("long-cache", 88, 3, 2, 12288, past=lens, in_dtype="float16" if fp16 else "float32", cache_dtype=cache_dtype,
                       out_dtype="float32")
    _check(case, run_cuda(case), run_oracle(case), fp16=fp16)


@pytest.mark.parametrize("early", [0, 1, 2])
def test_decode_calls_can_be_captured_in_a_graph(cuda_device, early):
    """The call allocates nothing and never synchronises, so a run of decode calls can be recorded once and
    replayed as one graph launch (ordinary launches and early-start launches alike); replays repeat the bits."""
    import torch

    lens = W.draw_lengths(9, 4, 100, 900)
    sets = []
    for j in range(2):
        c = W.device_case("graph", 70 + j, 4, 8, 901, lens, device=cuda_device)
        c.scratch_zeroed = True
        c.early_start = early
        sets.append((c, c.params()))
    for c, p in sets:
        A.decode(p)
    torch.cuda.synchronize()
    want = [c.arrays["out"].clone() for c, _ in sets]
    for c, _ in sets:
        c.arrays["out"].zero_()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for i in range(6):
                A.decode(sets[i % 2][1], torch.cuda.current_stream())
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert all(A.scratch_status(c.arrays["scratch"]) == 0 for c, _ in sets)
    for (c, _), w in zip(sets, want):
        assert torch.equal(c.arrays["out"], w)
