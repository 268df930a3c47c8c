"""Builds two end-to-end libraries from a PATCHED COPY of the reference checkout (nothing of the
reference is committed here; the copy lives under oracle/_ref/, which is git-ignored):

  oracle/_ref/libe2e_ref.so   the reference's DecodingSampling + OpenDecoder with
        (1) size_t instead of int for the buffer sizes that overflow 32 bits at LLaMA-2-7B sizes
            (decoding_sampling.cu: cache/workspace/slab sizes; open_decoder.{h,cu}: getWorkspaceSize), and
        (2) the two decode gemv calls given the arguments the code intends (as written they are
            rejected by cuBLAS for L > size_per_head): OP_T m=d n=L, score stride L.
  oracle/_ref/libe2e_flb.so   the same with (1) and, instead of (2), lines 138-239 of open_decoder.cu
        (the whole attention section) replaced by one call of flb_open_decoder_attention()
        (include/flb_open_decoder.h) — the drop-in adaptor.

  oracle/_ref/libe2e_opt.so   libe2e_flb.so plus the steps either side of the attention call (patch_opt): one merged QKV GEMM
        read in place, the LM head over the last rows only, an asynchronous finished check, an fp16-sized cache slab.
  oracle/_ref/libe2e_tp.so    the tensor-parallel layer: like libe2e_flb.so, plus the Q/K/V GEMMs restricted to the rank's
        column slice of the weights and flb_open_decoder_attention_tp() (head-sharded attention + one NCCL all-gather).
  oracle/_ref/libe2e_ref32.so like libe2e_ref.so, but with the prefill GEMMs computing in true fp32
        (CUBLAS_COMPUTE_32F instead of CUBLAS_COMPUTE_32F_FAST_16F in common.h) — used only to measure how far
        the reference's own fp16 tensor-core rounding moves its sampled tokens.

All are linked with oracle/e2e_runner.cu.  TEST / BASELINE INFRASTRUCTURE.
usage: python oracle/make_e2e_variants.py <reference-root> [variants...]   (FLB_REFERENCE_ROOT also names the root)"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref")


def _sub(text: str, pattern: str, repl: str, count: int, what: str) -> str:
    new, n = re.subn(pattern, repl, text, flags=re.S)
    if n != count:
        raise RuntimeError(f"patch '{what}': expected {count} match(es), found {n}")
    return new


def patch_sizes(src: str) -> None:
    p = os.path.join(src, "open_decoder.h")
    t = open(p).read()
    t = _sub(t, r"int getWorkspaceSize\(\);", "size_t getWorkspaceSize();", 1, "header return type")
    open(p, "w").write(t)
    p = os.path.join(src, "cuda", "open_decoder.cu")
    t = open(p).read()
    t = _sub(t, r"\n    int OpenDecoder<OpType_, QuantizationType>::getWorkspaceSize\(\)", "\n    size_t OpenDecoder<OpType_, QuantizationType>::getWorkspaceSize()", 1, "definition return type")
    t = _sub(t, r"int work_space_size =", "size_t work_space_size =", 1, "work_space_size")
    open(p, "w").write(t)
    p = os.path.join(src, "cuda", "decoding_sampling.cu")
    t = open(p).read()
    for name, cnt in (("decoder_workspace_size", 1), ("cache_size", 2), ("datatype_buf_size", 1), ("float_buf_size", 1), ("int_buf_size", 1)):
        t = _sub(t, rf"\bint {name} =", f"size_t {name} =", cnt, name)
    open(p, "w").write(t)


def attention_section(lines: list[str]) -> tuple[int, int]:
    """0-based [start, end) of open_decoder.cu:138-239, checked against its anchors."""
    start, end = 137, 239
    if "Quantized-rope" not in lines[start + 1] or lines[end - 1].strip() != "}" or "quantized qkv to int8" not in lines[end + 2]:
        raise RuntimeError("open_decoder.cu does not look like the expected revision (attention section anchors moved)")
    return start, end


def patch_gemv(src: str) -> None:
    p = os.path.join(src, "cuda", "open_decoder.cu")
    t = open(p).read()
    t = _sub(t, r"CUBLAS_OP_T,\s*seq_len \+ start_pos, size_per_head_,", "CUBLAS_OP_T,\n size_per_head_, seq_len + start_pos,", 1, "gemv-1 m/n")
    t = _sub(t, r"qk_buf_, 1, size_per_head_,(\s*)batch_size_ \* head_num_\)\);", r"qk_buf_, 1, seq_len + start_pos,\1batch_size_ * head_num_));", 1, "gemv-1 score stride")
    t = _sub(t, r"qk_buf_, 1, size_per_head_,(\s*)&qkv_beta,", r"qk_buf_, 1, seq_len + start_pos,\1&qkv_beta,", 1, "gemv-2 score stride")
    open(p, "w").write(t)


def patch_probe(src: str) -> None:
    """Test hooks in the generation loop (every variant): when the runner has set them, each step's logits row
    [batch, vocab] (what the sampling kernels read) is copied out, and the sampled ids are overwritten with forced ones
    (teacher forcing with another run's ids).  Both pointers live in e2e_runner.cu and are NULL by default."""
    p = os.path.join(src, "cuda", "decoding_sampling.cu")
    t = open(p).read()
    t = _sub(t, r'(#include "decoding_sampling.h"\n)', r'\1extern "C" {\nextern float *flb_e2e_logits_out;\nextern const int *flb_e2e_forced_ids;\n}\n', 1, "probe externs")
    t = _sub(t, r"(launchUpdateLogitsWithoutSoftmax\(step_logits_buf_, logits_buf_, args_\.end_id_, finished_buf_, args_\.batch_size_,[^;]*;)",
             r"""\1
                if (flb_e2e_logits_out)
                    cudaMemcpyAsync(flb_e2e_logits_out + (size_t)(step - 1) * args_.batch_size_ * args_.vocab_size_, step_logits_buf_,
                                    sizeof(float) * args_.batch_size_ * args_.vocab_size_, cudaMemcpyDeviceToDevice, decoding_params.stream);""", 1, "logits probe")
    t = _sub(t, r"(launchTopKSamplingKernel\(step_logits_buf_, topk_ids_buf_, topk_val_buf_,[^;]*;)",
             r"""\1
                if (flb_e2e_forced_ids)
                    cudaMemcpyAsync(word_ids_buf_ + (step - 1) * args_.batch_size_, flb_e2e_forced_ids + (size_t)(step - 1) * args_.batch_size_,
                                    sizeof(int) * args_.batch_size_, cudaMemcpyDeviceToDevice, decoding_params.stream);""", 1, "forced ids")
    open(p, "w").write(t)


def patch_ctx(src: str) -> None:
    """The binding's per-object state: a flb_open_decoder_ctx member of OpenDecoder, initialised in its constructor."""
    p = os.path.join(src, "open_decoder.h")
    t = open(p).read()
    t = _sub(t, r'#include "common.h"\n', '#include "common.h"\n#include "flb_open_decoder.h"\n', 1, "binding include")
    t = _sub(t, r"(float \*ffn_inter_scale_buf_;[^\n]*\n)", r"\1        flb_open_decoder_ctx flb_ctx_;\n", 1, "ctx member")
    open(p, "w").write(t)
    p = os.path.join(src, "cuda", "open_decoder.cu")
    t = open(p).read()
    t = _sub(t, r"(\n        hidden_units_ = head_num_ \* size_per_head_;\n)", r"\1        flb_open_decoder_ctx_init(&flb_ctx_);\n", 1, "ctx init")
    open(p, "w").write(t)


def patch_opt(src: str) -> None:
    """On top of the adaptor: the rows of the scope table that lie either side of the attention call.
    (1) One INT8 GEMM for the Q, K and V projections when the binding has a packed weight matrix (FLB_MERGED_QKV=1);
        q, k and v are then column blocks of one buffer and reach the attention call with their row stride.
    (2) The LM head over the last row of each sequence only: nothing else is ever read from the logits
        (decoding_kernels.cu:255-275 takes row seq_len - 1), the reference computes all batch x prompt rows.
    (3) The "is everybody finished" copy of every step made asynchronous and looked at one step later: the loop may run
        one step longer, which cannot change an output (a finished sequence keeps its length and emits end_id).
    (4) With FLB_CACHE_F16=1 the cache slab is allocated at the size fp16 needs."""
    p = os.path.join(src, "cuda", "open_decoder.cu")
    t = open(p).read()
    t = _sub(t, r"(int k = hidden_units_;\n)(\s*)(CHECK_CUBLAS_STATUS\(cublasGemmEx\(param_\.cublas_handle,)",
             r"""\1\2const int8_t *flb_wqkv = flb_open_decoder_packed_qkv(&flb_ctx_, (const int8_t *)param_.attention.query_weight.kernel,
\2        (const int8_t *)param_.attention.key_weight.kernel, (const int8_t *)param_.attention.value_weight.kernel, n, param_.stream);
\2if (flb_wqkv) {
\2CHECK_CUBLAS_STATUS(cublasGemmEx(param_.cublas_handle, CUBLAS_OP_N, CUBLAS_OP_N, 3 * n, m, k, &weight_alpha,
\2        (const weight_DataType_ *)flb_wqkv, weight_Traits_::AType, 3 * n, from_tensor_int8_buf_, weight_Traits_::BType, k, &weight_beta,
\2        query_buf_, weight_Traits_::CType, 3 * n, weight_Traits_::computeType, static_cast<cublasGemmAlgo_t>(cublasAlgo_[0])));
\2} else {
\2\3""", 1, "merged QKV GEMM")
    t = _sub(t, r"(\n\s*)(flb_open_decoder_attention\(&flb_ctx_, batch_size_, head_num_, size_per_head_, max_prompt_len_, total_len_, seq_len, start_pos,\n\s*)query_buf_, key_buf_, value_buf_, hidden_units_,",
             r"\1}\1\2query_buf_, flb_wqkv ? query_buf_ + n : key_buf_, flb_wqkv ? query_buf_ + 2 * n : value_buf_, flb_wqkv ? 3 * n : n,", 1, "strided q/k/v")
    t = _sub(t, r"(OpenDecoder<OpType_, QuantizationType>::~OpenDecoder\(\)\n\s*\{\n)", r"\1        flb_open_decoder_ctx_destroy(&flb_ctx_);\n", 1, "ctx destroy")
    open(p, "w").write(t)

    p = os.path.join(src, "cuda", "decoding_sampling.cu")
    t = open(p).read()
    # (2) LM head on the last rows: B columns of k elements, cur_seq_len * k apart
    t = _sub(t, r"int m = args_\.batch_size_ \* cur_seq_len;", "int m = args_.batch_size_;", 1, "lm head rows")
    t = _sub(t, r"decoder_normed_result_buf_, BType_, k,", "decoder_normed_result_buf_ + (size_t)(cur_seq_len - 1) * k, BType_, k * cur_seq_len,", 1, "lm head operand")
    t = _sub(t, r"(launchUpdateLogitsWithoutSoftmax\(step_logits_buf_, logits_buf_, args_\.end_id_, finished_buf_, args_\.batch_size_,\s*)cur_seq_len,", r"\g<1>1,", 1, "top-k logits row")
    t = _sub(t, r"(launchUpdateLogitsKernelWithoutLog\(step_logits_buf_, logits_buf_, finished_buf_, )cur_seq_len,", r"\g<1>1,", 1, "top-p logits row")
    # (3) lagged, asynchronous finished check
    t = _sub(t, r"(\n\s*)int prev_pos = 0;\n", r"""\1int prev_pos = 0;
\1bool *flb_fin_host = nullptr;
\1cudaEvent_t flb_fin_event;
\1bool flb_fin_pending = false;
\1CHECK_CUDA_ERROR(cudaHostAlloc((void **)&flb_fin_host, sizeof(bool) * args_.batch_size_, cudaHostAllocDefault));
\1CHECK_CUDA_ERROR(cudaEventCreateWithFlags(&flb_fin_event, cudaEventDisableTiming));
""", 1, "finished-check set-up")
    t = _sub(t, r"cudaMemcpy\(h_finished_buf_, finished_buf_, sizeof\(bool\) \* args_\.batch_size_, cudaMemcpyDeviceToHost\);\n(\s*)int sum = 0;\n\s*for \(int i = 0; i < args_\.batch_size_; i\+\+\)\n\s*\{\n\s*sum \+= h_finished_buf_\[i\] \? 1 : 0;\n\s*\}",
             r"""int sum = 0;
\1if (flb_fin_pending && cudaEventQuery(flb_fin_event) == cudaSuccess)
\1{
\1    for (int i = 0; i < args_.batch_size_; i++) sum += flb_fin_host[i] ? 1 : 0;
\1    flb_fin_pending = false;
\1}
\1if (!flb_fin_pending && sum != args_.batch_size_)
\1{
\1    cudaMemcpyAsync(flb_fin_host, finished_buf_, sizeof(bool) * args_.batch_size_, cudaMemcpyDeviceToHost, decoding_params.stream);
\1    cudaEventRecord(flb_fin_event, decoding_params.stream);
\1    flb_fin_pending = true;
\1}""", 1, "finished check")
    t = _sub(t, r"(\n\s*)(launchRemovePromptTokenKernel\(decoding_params\.output_ids,)", r"""\1cudaStreamSynchronize(decoding_params.stream);
\1cudaEventDestroy(flb_fin_event);
\1cudaFreeHost(flb_fin_host);
\1\2""", 1, "finished-check tear-down")
    # (4) fp16 cache slab
    t = _sub(t, r"(size_t cache_size = args_\.batch_size_ \* \(args_\.max_prompt_len_ \+ args_\.max_gen_len_\) \* args_\.hidden_units_;)",
             'size_t cache_size = (size_t)args_.batch_size_ * (args_.max_prompt_len_ + args_.max_gen_len_) * args_.hidden_units_ / (flb_open_decoder_env_int("FLB_CACHE_F16", 0) ? 2 : 1);', 2, "fp16 slab")
    open(p, "w").write(t)


def patch_quant_call(text: str) -> str:
    """The reference's own attention-output quantisation launch is skipped when the adaptor has done it."""
    return _sub(text, r"(\n\s*)launchAttnQuantizedTransposeKernel\(from_tensor_int8_buf_, qkv_buf_,",
                r"\1if (!flb_open_decoder_fused_quant(&flb_ctx_)) launchAttnQuantizedTransposeKernel(from_tensor_int8_buf_, qkv_buf_,", 1,
                "optional fused quantisation")


def patch_adaptor(src: str) -> None:
    p = os.path.join(src, "cuda", "open_decoder.cu")
    lines = open(p).read().split("\n")
    s, e = attention_section(lines)
    call = """            flb_open_decoder_attention(&flb_ctx_, batch_size_, head_num_, size_per_head_, max_prompt_len_, total_len_, seq_len, start_pos,
                                       query_buf_, key_buf_, value_buf_, hidden_units_, from_tensor_scale_buf_,
                                       param_.attention.query_weight.weight_scale, param_.attention.key_weight.weight_scale,
                                       param_.attention.value_weight.weight_scale, freq_cis, param_.attn_mask,
                                       key_cache_, value_cache_, query_out_buf_, qk_buf_, qkv_buf_, from_tensor_int8_buf_, from_tensor_scale_buf_, param_.stream);"""
    lines[s:e] = call.split("\n")
    text = patch_quant_call("\n".join(lines))
    open(p, "w").write(text)


def patch_mix(src: str) -> None:
    """Diagnostic variant: the corrected reference section is kept and the adaptor call is added in front of
    it; the environment variable FLB_E2E_USE picks per call which one runs (bit 0: decode calls use the
    adaptor, bit 1: prefill calls use the adaptor)."""
    patch_gemv(src)
    p = os.path.join(src, "cuda", "open_decoder.cu")
    lines = open(p).read().split("\n")
    s, e = attention_section(lines)
    head = """            static const int flb_use = getenv("FLB_E2E_USE") ? atoi(getenv("FLB_E2E_USE")) : 3;
            if ((seq_len > 1) ? (flb_use & 2) : (flb_use & 1)) {
            flb_open_decoder_attention(&flb_ctx_, batch_size_, head_num_, size_per_head_, max_prompt_len_, total_len_, seq_len, start_pos,
                                       query_buf_, key_buf_, value_buf_, hidden_units_, from_tensor_scale_buf_,
                                       param_.attention.query_weight.weight_scale, param_.attention.key_weight.weight_scale,
                                       param_.attention.value_weight.weight_scale, freq_cis, param_.attn_mask,
                                       key_cache_, value_cache_, query_out_buf_, qk_buf_, qkv_buf_, from_tensor_int8_buf_, from_tensor_scale_buf_, param_.stream);
            } else {"""
    tail = """            }
            if (flb_use & 4) {
                // diagnostic: run the adaptor on the same inputs after the reference section and record the difference
                // (every decode call and every prefill call; the reference's result is kept, so the run stays on the
                // reference's own trajectory: teacher forcing at the level of one attention call)
                const int ph = seq_len > 1 ? 1 : 0;
                const size_t n = (size_t)batch_size_ * head_num_ * seq_len * size_per_head_;
                std::vector<float> h_ref(n), h_flb(n);
                cudaStreamSynchronize(param_.stream);
                cudaMemcpy(h_ref.data(), qkv_buf_, n * sizeof(float), cudaMemcpyDeviceToHost);
                flb_open_decoder_attention(&flb_ctx_, batch_size_, head_num_, size_per_head_, max_prompt_len_, total_len_, seq_len, start_pos,
                                       query_buf_, key_buf_, value_buf_, hidden_units_, from_tensor_scale_buf_,
                                       param_.attention.query_weight.weight_scale, param_.attention.key_weight.weight_scale,
                                       param_.attention.value_weight.weight_scale, freq_cis, param_.attn_mask,
                                       key_cache_, value_cache_, query_out_buf_, qk_buf_, qkv_buf_, from_tensor_int8_buf_, from_tensor_scale_buf_, param_.stream);
                cudaStreamSynchronize(param_.stream);
                cudaMemcpy(h_flb.data(), qkv_buf_, n * sizeof(float), cudaMemcpyDeviceToHost);
                cudaMemcpy(qkv_buf_, h_ref.data(), n * sizeof(float), cudaMemcpyHostToDevice);
                double mx = 0, amax = 0; size_t at = 0, bad = 0;
                for (size_t i = 0; i < n; ++i) {
                    if (std::isnan(h_ref[i])) { if (h_flb[i] != 0.0f) ++bad; continue; } // the reference's 0/0 on a fully masked row: ours is 0
                    double d = fabs((double)h_ref[i] - h_flb[i]); if (d > mx) { mx = d; at = i; } amax = fmax(amax, fabs((double)h_ref[i]));
                }
                flb_e2e_mix_calls[ph] += 1;
                flb_e2e_mix_max[ph] = fmax(flb_e2e_mix_max[ph], mx);
                flb_e2e_mix_max[2 + ph] = fmax(flb_e2e_mix_max[2 + ph], amax);
                flb_e2e_mix_calls[2] += (long)bad;
                if (flb_e2e_mix_calls[ph] <= 8) printf("[cmp %s %ld] start_pos %d seq_len %d max|ref-flb| %.3e at %zu (ref %.6f flb %.6f) max|ref| %.3f\\n", ph ? "prefill" : "decode", flb_e2e_mix_calls[ph], start_pos, seq_len, mx, at, h_ref[at], h_flb[at], amax);
            }"""
    lines[s:e] = head.split("\n") + lines[s:e] + tail.split("\n")
    text = "\n".join(lines)
    text = text.replace('#include "open_decoder.h"', '#include <vector>\n#include <cmath>\n#include "open_decoder.h"\nextern "C" {\nextern double flb_e2e_mix_max[4];\nextern long flb_e2e_mix_calls[3];\n}', 1)
    open(p, "w").write(text)


def patch_tp(src: str) -> None:
    """Tensor-parallel layer: Q/K/V projections on this rank's column slice of the weights, attention on its heads
    through flb_open_decoder_attention_tp (which all-gathers the head outputs); the rest of the layer is untouched."""
    p = os.path.join(src, "cuda", "open_decoder.cu")
    text = open(p).read()
    text = _sub(text, r"(int k = hidden_units_;\n)", r"\1            const int n_tp = n / flb_tp_size(&flb_ctx_);\n            const int tp_col0 = flb_tp_rank(&flb_ctx_) * n_tp;\n", 1, "tp slice")
    for x in ("query", "key", "value"):
        text = _sub(text,
                    rf"n, m, k,(\s*)&weight_alpha,(\s*)param_\.attention\.{x}_weight\.kernel, weight_Traits_::AType, n,(\s*)from_tensor_int8_buf_, weight_Traits_::BType, k,(\s*)&weight_beta,(\s*){x}_buf_, weight_Traits_::CType, n,",
                    rf"n_tp, m, k,\1&weight_alpha,\2param_.attention.{x}_weight.kernel + tp_col0, weight_Traits_::AType, n,\3from_tensor_int8_buf_, weight_Traits_::BType, k,\4&weight_beta,\5{x}_buf_, weight_Traits_::CType, n_tp,",
                    1, f"{x} projection slice")
    lines = text.split("\n")
    s, e = None, None
    for i, l in enumerate(lines):
        if "Quantized-rope" in l and s is None:
            s = i - 1
        if "quantized qkv to int8" in l:
            e = i - 2
    if s is None or e is None or lines[s].strip() != "/**" or lines[e - 1].strip() != "}":
        raise RuntimeError("attention section anchors not found")
    call = """            flb_open_decoder_attention_tp(&flb_ctx_, batch_size_, head_num_, size_per_head_, max_prompt_len_, total_len_, seq_len, start_pos,
                                          query_buf_, key_buf_, value_buf_, from_tensor_scale_buf_,
                                          param_.attention.query_weight.weight_scale, param_.attention.key_weight.weight_scale,
                                          param_.attention.value_weight.weight_scale, freq_cis, param_.attn_mask,
                                          key_cache_, value_cache_, query_out_buf_, qk_buf_, qkv_buf_, from_tensor_int8_buf_, from_tensor_scale_buf_,
                                          param_.stream);"""
    lines[s:e] = call.split("\n")
    text = patch_quant_call("\n".join(lines))
    open(p, "w").write(text)


def build(name: str, ref_root: str) -> str:
    vdir = os.path.join(OUT, "variants", name)
    if os.path.isdir(vdir):
        shutil.rmtree(vdir)
    src = os.path.join(vdir, "fasterLlama")
    shutil.copytree(os.path.join(ref_root, "fasterLlama"), src, ignore=shutil.ignore_patterns("lib", "*.so"))
    os.chmod(src, 0o755)
    for r, ds, fs in os.walk(src):
        for x in ds + fs:
            os.chmod(os.path.join(r, x), 0o755 if x in ds else 0o644)
    patch_sizes(src)
    patch_probe(src)
    if name in ("ref", "ref32"):
        patch_gemv(src)
    elif name == "mix":
        patch_mix(src)
    elif name == "tp":
        patch_tp(src)
    else:
        patch_adaptor(src)
    if name in ("flb", "mix", "tp", "opt"):
        patch_ctx(src)  # after the section patches: those address open_decoder.cu by line number
    if name == "opt":
        patch_opt(src)
    if name == "ref32":
        p = os.path.join(src, "cuda", "common.h")
        t = open(p).read()
        t = _sub(t, r"CUBLAS_COMPUTE_32F_FAST_16F", "CUBLAS_COMPUTE_32F", 1, "fp32 prefill math")
        open(p, "w").write(t)
    lib = os.path.join(OUT, f"libe2e_{name}.so")
    cu = [os.path.join(src, "cuda", f) for f in ("decoder_kernels.cu", "decoding_kernels.cu", "open_decoder.cu", "decoding_sampling.cu")]
    cmd = ["nvcc", "-std=c++17", "-O3", "-DNDEBUG", "-w", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
           "-shared", "-cudart", "shared", "-I", src, "-I", os.path.join(src, "cuda"), "-I", os.path.join(ROOT, "include"),
           *cu, os.path.join(HERE, "e2e_runner.cu"), "-lcublas", "-lcurand", "-o", lib]
    if name in ("flb", "mix", "tp", "opt"):
        pkg = os.path.join(ROOT, "fasterllama_b200")
        cmd += ["-L", pkg, "-lflb_attn", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../fasterllama_b200"]
    if name == "mix":
        cmd += ["-DFLB_OPEN_DECODER_NO_EARLY_START"]  # the reference's own section shares the scratch buffers there
    if name == "tp":
        import torch  # the NCCL this process will already have loaded: link against the same library
        nccl_dir = os.path.join(os.path.dirname(os.path.dirname(torch.__file__)), "nvidia", "nccl")
        cmd += ["-DFLB_WITH_NCCL", "-I", os.path.join(nccl_dir, "include"), "-L", os.path.join(nccl_dir, "lib"), "-l:libnccl.so.2"]
    subprocess.run(cmd, check=True)
    if not os.environ.get("FLB_KEEP_VARIANT_SOURCES"):
        shutil.rmtree(vdir)  # the patched copy of the reference's sources is only needed for the compile
    return lib


def main(ref_root: str | None = None) -> None:
    ref_root = ref_root or os.environ.get("FLB_REFERENCE_ROOT")
    if not ref_root or not os.path.isdir(os.path.join(ref_root, "fasterLlama")):
        raise SystemExit("usage: make_e2e_variants.py <reference checkout> [variants...]  (or set FLB_REFERENCE_ROOT)")
    os.makedirs(OUT, exist_ok=True)
    names = sys.argv[2:] or ["ref", "flb", "ref32", "mix", "tp", "opt"]
    # every variant has its own copy of the sources and its own output: the compiles run side by side
    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(max_workers=min(len(names), os.cpu_count() or 1)) as pool:
        for lib in pool.map(lambda n: build(n, ref_root), names):
            print("built", lib)


if __name__ == "__main__":
    main(*sys.argv[1:2])
