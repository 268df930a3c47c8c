// ref_runner.cu — drives the REFERENCE's own attention kernels and cuBLAS calls.
//
// TEST / BASELINE INFRASTRUCTURE ONLY.  This file holds no attention arithmetic of its own: it
// calls the launchers the reference defines in fasterLlama/cuda/decoder_kernels.cu (compiled from
// the reference checkout, never copied into this repository; see build_ref.sh) in the order of
// OpenDecoder::forward, fasterLlama/cuda/open_decoder.cu:138-239, on caller-provided device
// buffers.  It exists so that (a) the host oracle can be pinned against outputs of the reference
// itself and (b) the benchmark has the reference's kernels to time on the same box.
//
// Two modes for the decode (seq_len == 1) contractions:
//   fixed      the gemv arguments the code intends (K slab is column-major d x L): OP_T m=d n=L
//              lda=d, scores at stride L; P.V with P at stride L.
//   as_written the arguments exactly as open_decoder.cu:194-201 and :231-238 pass them (m and n
//              exchanged, score stride d) — self-consistent only when L == d; for L > d cuBLAS
//              rejects lda < m and the status is returned instead of exit(1).
#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "decoder_kernels.cuh"
#include "decoding_kernels.cuh"

extern "C" {

typedef struct ref_attn_args {
    int batch_size, head_num, size_per_head, seq_len, start_pos, total_len;
    const int32_t *Q, *K, *V;   // [B,S,H*d] int32 accumulators
    const float *act_scale;     // [B*S]
    const float *q_w_scale, *k_w_scale, *v_w_scale; // [H*d]
    const float *freq_cis;      // row 0 is used for token 0 of the chunk (the reference's rule)
    const float *attn_mask;     // [T,T] additive, row 0 (may be NULL)
    float *k_cache, *v_cache;   // [B,H,T,d]
    float *q_out, *k_out, *v_out; // work [B,H,S,d]
    float *qk_buf;              // work [B,H,S,max(L,d)]
    float *out;                 // [B,H,S,d]
    int as_written;
} ref_attn_args;

void *ref_create(void) {
    cublasHandle_t h = nullptr;
    if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) return nullptr;
    return h;
}

void ref_destroy(void *handle) {
    if (handle) cublasDestroy(static_cast<cublasHandle_t>(handle));
}

// returns 0, or 1000 + cublasStatus, or 2000 + cudaError
int ref_attention(void *handle, const ref_attn_args *a, void *cuda_stream) {
    using namespace FasterLLaMA;
    cublasHandle_t h = static_cast<cublasHandle_t>(handle);
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    if (cublasSetStream(h, st) != CUBLAS_STATUS_SUCCESS) return 1001;
    const int B = a->batch_size, H = a->head_num, d = a->size_per_head, S = a->seq_len, T = a->total_len;
    const int sp = a->start_pos, L = S + sp;
    const float one = 1.0f, zero = 0.0f;
    cublasStatus_t cs = CUBLAS_STATUS_SUCCESS;

    launchQKRoteEmbeddingTranspose(a->q_out, a->k_out, a->Q, a->K, a->act_scale, a->act_scale, a->q_w_scale, a->k_w_scale,
                                   a->freq_cis, B, S, sp, T, H, d, st);
    launchDequantizedVTransposeKernel(a->v_out, a->V, a->act_scale, a->v_w_scale, B, S, H, d, st);
    launchStoreKVcacheKernel(a->k_cache, a->v_cache, a->k_out, a->v_out, sp, S, B, H, T, d, st);

    if (S > 1) {
        cs = cublasGemmStridedBatchedEx(h, CUBLAS_OP_T, CUBLAS_OP_N, S, S, d, &one, a->k_out, CUDA_R_32F, d, (long long)S * d,
                                        a->q_out, CUDA_R_32F, d, (long long)S * d, &zero, a->qk_buf, CUDA_R_32F, S,
                                        (long long)S * S, B * H, CUBLAS_COMPUTE_32F_FAST_16F, CUBLAS_GEMM_DEFAULT);
    } else if (a->as_written) {
        cs = cublasSgemvStridedBatched(h, CUBLAS_OP_T, L, d, &one, a->k_cache, d, (long long)T * d, a->q_out, 1, d, &zero,
                                       a->qk_buf, 1, d, B * H);
    } else {
        cs = cublasSgemvStridedBatched(h, CUBLAS_OP_T, d, L, &one, a->k_cache, d, (long long)T * d, a->q_out, 1, d, &zero,
                                       a->qk_buf, 1, L, B * H);
    }
    if (cs != CUBLAS_STATUS_SUCCESS) return 1000 + (int)cs;

    launchBlockSoftmaxKernel(a->qk_buf, a->attn_mask ? a->attn_mask + (size_t)sp * T : nullptr, B, H, S, L, T,
                             rsqrtf((float)d), st);

    if (S > 1) {
        cs = cublasGemmStridedBatchedEx(h, CUBLAS_OP_N, CUBLAS_OP_N, d, S, S, &one, a->v_out, CUDA_R_32F, d, (long long)S * d,
                                        a->qk_buf, CUDA_R_32F, S, (long long)S * S, &zero, a->out, CUDA_R_32F, d,
                                        (long long)S * d, B * H, CUBLAS_COMPUTE_32F_FAST_16F, CUBLAS_GEMM_DEFAULT);
    } else {
        cs = cublasSgemvStridedBatched(h, CUBLAS_OP_N, d, L, &one, a->v_cache, d, (long long)T * d, a->qk_buf, 1,
                                       a->as_written ? d : L, &zero, a->out, 1, d, B * H);
    }
    if (cs != CUBLAS_STATUS_SUCCESS) return 1000 + (int)cs;
    const cudaError_t ce = cudaGetLastError();
    return ce == cudaSuccess ? 0 : 2000 + (int)ce;
}

// The reference's attention-output quantisation + transpose (fasterLlama/cuda/decoder_kernels.cu:1179-1300).
int ref_attn_quant(int8_t *attn_buf, const float *attn, float *scale, int batch_size, int head_num, int seq_len,
                   int size_per_head, void *cuda_stream) {
    FasterLLaMA::launchAttnQuantizedTransposeKernel(attn_buf, attn, scale, batch_size, head_num, seq_len, size_per_head,
                                                    static_cast<cudaStream_t>(cuda_stream));
    const cudaError_t ce = cudaGetLastError();
    return ce == cudaSuccess ? 0 : 2000 + (int)ce;
}

// The reference's RoPE table generator (fasterLlama/cuda/decoding_kernels.cu:85-135).
int ref_freq_cis(float *freq_cis, int size_per_head, int rows, void *cuda_stream) {
    FasterLLaMA::launchPrecomputeFreqsCis(freq_cis, size_per_head, rows, static_cast<cudaStream_t>(cuda_stream));
    const cudaError_t ce = cudaGetLastError();
    return ce == cudaSuccess ? 0 : 2000 + (int)ce;
}

} // extern "C"
