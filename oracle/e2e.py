"""End-to-end run of the reference's DecodingSampling<FP16> (random-init LLaMA-2-shaped weights, INT8
per-channel GEMMs) through one of the two libraries built by make_e2e_variants.py:

    python oracle/e2e.py --variant ref|flb --config small|c5 --out ids.npz [--cache-f16] [--mask strict|inclusive]

`ref` = the reference's own attention (gemv arguments corrected), `flb` = the same classes with the
attention section replaced by the drop-in adaptor.  TEST / BASELINE INFRASTRUCTURE.  Weights are
drawn here with torch (seeded), quantised per output channel, and handed to the reference as device
pointers; the reference does everything else."""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CONFIGS = {
    # the reference's sample sizes (samples/llama_fp16.cu:348-357), top-k instead of top-p
    "small": dict(batch=4, head_num=8, size_per_head=128, vocab=200, max_prompt_len=16, max_gen_len=16, layers=4, ffn=256, topk=4, seed=4),
    "medium": dict(batch=8, head_num=32, size_per_head=128, vocab=2000, max_prompt_len=160, max_gen_len=48, layers=4, ffn=1024, topk=4, seed=4),
    # LLaMA-2-7B: 32 layers, hidden 4096, 32 heads, FFN 11008, vocab 32000; batch 32, prompt 512, 256 new tokens, top-k 4, seed 4
    "c5": dict(batch=32, head_num=32, size_per_head=128, vocab=32000, max_prompt_len=512, max_gen_len=256, layers=32, ffn=11008, topk=4, seed=4),
}


class Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attn_gamma", "wq", "wk", "wv", "wo", "sq", "sk", "sv", "so", "ffn_gamma", "w1", "w2", "w3", "s1", "s2", "s3")]


class Args(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("batch", "max_prompt_len", "max_gen_len", "head_num", "size_per_head", "vocab", "layers", "end_id", "ffn", "topk")] + [
        ("topp", C.c_float), ("device", C.c_int), ("layer", C.POINTER(Layer)), ("attn_mask", C.c_void_p), ("embedding", C.c_void_p),
        ("freq_cis", C.c_void_p), ("prompt_seq_len", C.c_void_p), ("min_prompt", C.c_int), ("max_prompt", C.c_int),
        ("prompt_tokens", C.c_void_p), ("prompt_mask", C.c_void_p), ("final_gamma", C.c_void_p), ("lm_head", C.c_void_p),
        ("output_ids", C.c_void_p), ("seq_len", C.c_void_p)]


def quantise(w: torch.Tensor):
    """Symmetric per-output-channel INT8 of a row-major [in, out] matrix: scale[n] = absmax_k / 127."""
    scale = (w.abs().amax(dim=0) / 127.0).clamp_min(1e-12)
    q = torch.round(w / scale).clamp_(-127, 127).to(torch.int8)
    return q.contiguous(), scale.float().contiguous()


_LIBS: dict = {}


def load(variant: str):
    if variant not in _LIBS:
        lib = C.CDLL(os.path.join(HERE, "_ref", f"libe2e_{variant}.so"))
        lib.e2e_run.restype = C.c_int
        lib.e2e_run.argtypes = [C.POINTER(Args), C.POINTER(C.c_float)]
        _LIBS[variant] = lib
    return _LIBS[variant]


def tp_init(variant: str):
    """Under torchrun with the `tp` library: rank 0 makes an NCCL id, every rank joins the communicator the
    patched OpenDecoder::forward uses for its one all-gather per layer.  Returns (rank, world, local_rank)."""
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    if variant != "tp" or world == 1:
        return rank, world, local
    import torch.distributed as dist

    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    lib = load(variant)
    buf = C.create_string_buffer(128)
    if rank == 0:
        assert lib.e2e_tp_unique_id(buf) == 0
    box = [bytes(buf.raw)]
    dist.broadcast_object_list(box, src=0)
    lib.e2e_tp_init.argtypes = [C.c_int, C.c_int, C.c_int, C.c_char_p]
    assert lib.e2e_tp_init(rank, world, local, box[0]) == 0, "ncclCommInitRank failed"
    return rank, world, local


def run(variant: str, cfg: dict, mask: str = "inclusive", device: int = 0, forced_ids=None, want_logits: bool = False):
    """One generation run.  forced_ids: int32 [steps, batch] on the device — every step's sampled ids are replaced by
    these (teacher forcing with another run's ids).  want_logits: also returns every step's logits row as the sampler
    read it, float32 [steps, batch, vocab] on the device (else None)."""
    lib = load(variant)
    dev = f"cuda:{device}"
    g = torch.Generator(device=dev)
    g.manual_seed(cfg["seed"])
    hidden = cfg["head_num"] * cfg["size_per_head"]
    T = cfg["max_prompt_len"] + cfg["max_gen_len"]
    keep = []

    def dense(i, o):
        w = torch.randn((i, o), generator=g, device=dev) * 0.02
        q, s = quantise(w)
        keep.extend([q, s])
        return q.data_ptr(), s.data_ptr()

    layers = (Layer * cfg["layers"])()
    for l in range(cfg["layers"]):
        ga = torch.ones(hidden, dtype=torch.float16, device=dev)
        gf = torch.ones(hidden, dtype=torch.float16, device=dev)
        keep.extend([ga, gf])
        layers[l].attn_gamma, layers[l].ffn_gamma = ga.data_ptr(), gf.data_ptr()
        layers[l].wq, layers[l].sq = dense(hidden, hidden)
        layers[l].wk, layers[l].sk = dense(hidden, hidden)
        layers[l].wv, layers[l].sv = dense(hidden, hidden)
        layers[l].wo, layers[l].so = dense(hidden, hidden)
        layers[l].w1, layers[l].s1 = dense(hidden, cfg["ffn"])
        layers[l].w3, layers[l].s3 = dense(hidden, cfg["ffn"])
        layers[l].w2, layers[l].s2 = dense(cfg["ffn"], hidden)
    emb = (torch.randn((cfg["vocab"], hidden), generator=g, device=dev) * 0.02).half()
    head = (torch.randn((hidden, cfg["vocab"]), generator=g, device=dev) * 0.02).half()
    fg = torch.ones(hidden, dtype=torch.float16, device=dev)
    B, P = cfg["batch"], cfg["max_prompt_len"]
    prompts = torch.randint(3, cfg["vocab"], (B, P), generator=g, device=dev, dtype=torch.int32)
    pmask = torch.ones((B, P), dtype=torch.bool, device=dev)
    plen = torch.full((B,), P, dtype=torch.int32, device=dev)
    r = torch.arange(T, device=dev)
    vis = (r[None, :] < r[:, None]) if mask == "strict" else (r[None, :] <= r[:, None])
    amask = torch.where(vis, 0.0, -torch.finfo(torch.float32).max).float().contiguous()
    freq = torch.zeros((T, cfg["size_per_head"]), dtype=torch.float32, device=dev)
    out_ids = torch.zeros((B, T), dtype=torch.int32, device=dev)
    seq_len = torch.zeros((B,), dtype=torch.int32, device=dev)
    torch.cuda.synchronize()

    a = Args()
    for n in ("batch", "max_prompt_len", "max_gen_len", "head_num", "size_per_head", "vocab", "layers", "ffn", "topk"):
        setattr(a, n, cfg[n])
    a.end_id, a.topp, a.device = 2, 0.0, device
    a.layer = layers
    a.attn_mask, a.embedding, a.freq_cis = amask.data_ptr(), emb.data_ptr(), freq.data_ptr()
    a.prompt_seq_len, a.min_prompt, a.max_prompt = plen.data_ptr(), P, P
    a.prompt_tokens, a.prompt_mask = prompts.data_ptr(), pmask.data_ptr()
    a.final_gamma, a.lm_head = fg.data_ptr(), head.data_ptr()
    a.output_ids, a.seq_len = out_ids.data_ptr(), seq_len.data_ptr()
    steps = cfg["max_gen_len"]
    logits = torch.zeros((steps, B, cfg["vocab"]), dtype=torch.float32, device=dev) if want_logits else None
    lib.e2e_set_probe.argtypes = [C.c_void_p, C.c_void_p]
    lib.e2e_set_probe.restype = None
    lib.e2e_set_probe(logits.data_ptr() if want_logits else None, forced_ids.data_ptr() if forced_ids is not None else None)
    ms = C.c_float(0)
    st = lib.e2e_run(C.byref(a), C.byref(ms))
    torch.cuda.synchronize()
    lib.e2e_set_probe(None, None)
    if st != 0:
        raise RuntimeError(f"e2e_run status {st}")
    if want_logits:
        return out_ids.cpu().numpy(), seq_len.cpu().numpy(), float(ms.value), logits
    return out_ids.cpu().numpy(), seq_len.cpu().numpy(), float(ms.value)


def compare_logits(variants: list[str], cfg: dict, mask: str = "inclusive", device: int = 0) -> dict:
    """Teacher-forced comparison at the level of the sampler's input: the first variant runs freely; every other variant is
    fed the first one's ids at every step, so all of them see the same token history, and each step's logits row is
    compared with the first variant's.  Per variant: the largest |difference| of a logit, the fraction of (step, sequence)
    pairs whose top-4 SET (what top-k = 4 sampling draws from) and whose arg-max are the same, and the largest difference
    relative to the spread of the row's top-4 values."""
    dev = f"cuda:{device}"
    ids0, sl0, _, base = run(variants[0], cfg, mask, device, want_logits=True)
    steps, B = cfg["max_gen_len"], cfg["batch"]
    forced = torch.from_numpy(np.ascontiguousarray(ids0[:, :steps].T)).to(dev)  # word_ids rows are [step][batch]
    top0 = base.topk(4, dim=-1)
    out = {"reference_variant": variants[0], "steps": steps, "batch": B, "max_abs_logit": float(base[torch.isfinite(base) & (base.abs() < 1e30)].abs().max())}
    for v in variants[1:]:
        _, _, _, lg = run(v, cfg, mask, device, forced_ids=forced, want_logits=True)
        ok = (base.abs() < 1e30) & (lg.abs() < 1e30)  # finished sequences carry +-FLT_MAX rows
        diff = torch.where(ok, (lg - base).abs(), torch.zeros_like(lg))
        top = lg.topk(4, dim=-1)
        same_set = (top.indices.sort(dim=-1).values == top0.indices.sort(dim=-1).values).all(dim=-1)
        same_arg = top.indices[..., 0] == top0.indices[..., 0]
        gap = (top0.values[..., 3] - base.topk(5, dim=-1).values[..., 4]).clamp_min(1e-12)  # what separates the 4th from the 5th candidate
        per_step = diff.amax(dim=(1, 2))
        out[v] = {"max_abs_diff": float(diff.max()), "mean_abs_diff": float(diff.mean()),
                  "max_abs_diff_first_step": float(per_step[0]), "max_abs_diff_last_step": float(per_step[-1]),
                  "top4_set_same": float(same_set.float().mean()), "argmax_same": float(same_arg.float().mean()),
                  "steps_with_all_top4_sets_same": float(same_set.all(dim=1).float().mean()),
                  "median_4th_to_5th_gap": float(gap[torch.isfinite(gap)].median()) if bool(torch.isfinite(gap).any()) else None}
        del lg
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--variant", required=True, choices=["ref", "flb", "ref32", "mix", "tp", "opt"])
    ap.add_argument("--compare-logits", default="", help="comma-separated variants: run --variant freely, feed its ids to these and compare every step's logits with it")
    ap.add_argument("--config", default="small", choices=sorted(CONFIGS))
    ap.add_argument("--out", required=True)
    ap.add_argument("--mask", default="inclusive", choices=["inclusive", "strict"])
    ap.add_argument("--cache-f16", action="store_true")
    ap.add_argument("--fuse-quant", action="store_true", help="adaptor also does the attention-output quantisation")
    ap.add_argument("--merged-qkv", action="store_true", help="opt: one INT8 GEMM for the Q, K and V projections")
    ap.add_argument("--no-push", action="store_true", help="tp: decode steps use ncclAllGather instead of peer stores")
    ap.add_argument("--repeat", type=int, default=1, help="runs; the time of the last one is reported")
    args = ap.parse_args()
    if args.cache_f16:
        os.environ["FLB_CACHE_F16"] = "1"
    if args.fuse_quant:
        os.environ["FLB_FUSE_QUANT"] = "1"
    if args.no_push:
        os.environ["FLB_TP_PUSH"] = "0"
    if args.merged_qkv:
        os.environ["FLB_MERGED_QKV"] = "1"
    cfg = CONFIGS[args.config]
    if args.compare_logits:
        res = compare_logits([args.variant] + [v for v in args.compare_logits.split(",") if v], cfg, mask=args.mask)
        res["config"] = args.config
        print(json.dumps(res))
        return
    rank, world, local = tp_init(args.variant)
    for _ in range(args.repeat):
        ids, sl, ms = run(args.variant, cfg, mask=args.mask, device=local)
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # the slowest rank's time
        ms = float(t.item())
        push_used = bool(load(args.variant).e2e_tp_push_in_use()) if args.variant == "tp" else False
        if args.variant == "tp":
            load(args.variant).e2e_tp_finalize()  # unmaps the peers' exchange blocks, meets the other ranks, frees this rank's
        dist.barrier()
    if rank != 0:
        return
    np.savez(args.out, ids=ids, seq_len=sl, ms=ms)
    if args.variant == "mix":
        lib = load("mix")
        mx = (C.c_double * 4).in_dll(lib, "flb_e2e_mix_max")
        calls = (C.c_long * 3).in_dll(lib, "flb_e2e_mix_calls")
        print(json.dumps({"mix": {"decode_calls": calls[0], "prefill_calls": calls[1], "nan_rows_not_zero": calls[2],
                                  "decode_max_abs_diff": mx[0], "prefill_max_abs_diff": mx[1], "decode_max_abs_ref": mx[2],
                                  "prefill_max_abs_ref": mx[3]}}))
    toks = cfg["batch"] * cfg["max_gen_len"]
    push = push_used if (args.variant == "tp" and world > 1) else False
    print(json.dumps({"variant": args.variant, "tp": world, "tp_decode_exchange": ("peer stores" if push else ("nccl" if world > 1 else None)),
                      "config": args.config, "mask": args.mask, "cache_f16": bool(args.cache_f16),
                      "ms": round(ms, 2), "tokens_per_s": round(toks / ms * 1e3, 1), "first_ids": ids[0, :8].tolist(),
                      "seq_len": sl[:4].tolist()}))


if __name__ == "__main__":
    main()
