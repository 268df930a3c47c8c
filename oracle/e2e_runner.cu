// e2e_runner.cu — drives the REFERENCE's DecodingSampling<FP16> class on caller-provided weights.
//
// TEST / BASELINE INFRASTRUCTURE.  No model code lives here: the file only marshals device pointers
// into the reference's own parameter structs (fasterLlama/open_decoder.h:8-23,
// fasterLlama/decoding_sampling.h:9-33), constructs the reference's DecodingSampling and calls its
// forward().  It is compiled together with the reference's four translation units, taken from a
// patched copy of the reference checkout made by make_e2e_variants.py (which see for the patches).
#ifdef FLB_WITH_NCCL
#define FLB_OPEN_DECODER_TP_STATE // this translation unit holds the registration pointer of include/flb_open_decoder.h
#endif
#include <cublas_v2.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "decoding_sampling.h"
#ifdef FLB_WITH_NCCL
#include "flb_open_decoder.h"
static flb_tp_ctx g_tp; // this rank's communicator block: owned by the program, registered before the decoder is built
#endif

extern "C" {

// Test hooks read by the patched generation loop (make_e2e_variants.py: patch_probe) and by the `mix` variant's
// side-by-side comparison (patch_mix).  NULL / zero: no effect.
float *flb_e2e_logits_out = nullptr;       // device [steps, batch, vocab]: every step's logits row, as the sampler read it
const int *flb_e2e_forced_ids = nullptr;   // device [steps, batch]: ids that replace the sampled ones (teacher forcing)
double flb_e2e_mix_max[4] = {0, 0, 0, 0};  // max |ref - flb| over decode / prefill calls, max |ref| over decode / prefill
long flb_e2e_mix_calls[3] = {0, 0, 0};     // decode calls compared, prefill calls compared, rows the reference left NaN and ours not 0
void e2e_set_probe(float *logits_out, const int *forced_ids) {
    flb_e2e_logits_out = logits_out;
    flb_e2e_forced_ids = forced_ids;
}

typedef struct e2e_layer {
    void *attn_gamma;
    int8_t *wq, *wk, *wv, *wo;
    float *sq, *sk, *sv, *so;
    void *ffn_gamma;
    int8_t *w1, *w2, *w3;
    float *s1, *s2, *s3;
} e2e_layer;

typedef struct e2e_args {
    int batch, max_prompt_len, max_gen_len, head_num, size_per_head, vocab, layers, end_id, ffn, topk;
    float topp;
    int device;
    const e2e_layer *layer; // host array [layers]
    float *attn_mask;       // [T,T]
    void *embedding;        // half [vocab, hidden]
    float *freq_cis;        // [T, d] (filled by the reference)
    int *prompt_seq_len;    // [B]
    int min_prompt, max_prompt;
    int *prompt_tokens;     // [B, max_prompt]
    bool *prompt_mask;      // [B, max_prompt]
    void *final_gamma;      // half [hidden]
    void *lm_head;          // half [hidden, vocab]
    int *output_ids;        // [B, T]
    int *seq_len;           // [B]
} e2e_args;

#ifdef FLB_WITH_NCCL
// tensor-parallel set-up: rank 0 makes the id, the caller broadcasts its 128 bytes, every rank joins
int e2e_tp_unique_id(char *out128) {
    ncclUniqueId id;
    if (ncclGetUniqueId(&id) != ncclSuccess) return 1;
    memcpy(out128, &id, sizeof(id));
    return 0;
}
// 1 when the decode steps of the last run went through peer stores, 0 when they used ncclAllGather
int e2e_tp_push_in_use(void) { return g_tp.push_ready == 1 ? 1 : 0; }
// gives the exchange block back (every rank calls it, after its last run)
int e2e_tp_finalize(void) {
    if (g_tp.size > 1) flb_tp_push_teardown(&g_tp, 0);
    return 0;
}
int e2e_tp_init(int rank, int size, int device, const char *id128) {
    cudaSetDevice(device);
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclComm_t comm;
    if (ncclCommInitRank(&comm, size, id, rank) != ncclSuccess) return 1;
    flb_tp_ctx_init(&g_tp, comm, rank, size);
    flb_tp_register(&g_tp);
    return 0;
}
#endif

// returns 0; *ms = time of DecodingSampling::forward between two events on its stream
int e2e_run(const e2e_args *a, float *ms) {
    using namespace FasterLLaMA;
    cudaSetDevice(a->device);
    cublasHandle_t handle;
    if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return 1;
    cudaStream_t stream;
    cudaStreamCreate(&stream);
    cublasSetStream(handle, stream);
    Allocator<AllocatorType::CUDA> allocator(a->device);
    DecoderInitParam<half, int8_t> *param = new DecoderInitParam<half, int8_t>[a->layers];
    for (int i = 0; i < a->layers; ++i) {
        const e2e_layer &l = a->layer[i];
        param[i].stream = stream;
        param[i].cublas_handle = handle;
        param[i].attn_resnorm.gamma = (half *)l.attn_gamma;
        param[i].attention.query_weight.kernel = l.wq;
        param[i].attention.query_weight.weight_scale = l.sq;
        param[i].attention.key_weight.kernel = l.wk;
        param[i].attention.key_weight.weight_scale = l.sk;
        param[i].attention.value_weight.kernel = l.wv;
        param[i].attention.value_weight.weight_scale = l.sv;
        param[i].attention.attention_output_weight.kernel = l.wo;
        param[i].attention.attention_output_weight.weight_scale = l.so;
        param[i].attn_mask = a->attn_mask;
        param[i].ffn_resnorm.gamma = (half *)l.ffn_gamma;
        param[i].ffn.w1_weight.kernel = l.w1;
        param[i].ffn.w1_weight.weight_scale = l.s1;
        param[i].ffn.w2_weight.kernel = l.w2;
        param[i].ffn.w2_weight.weight_scale = l.s2;
        param[i].ffn.w3_weight.kernel = l.w3;
        param[i].ffn.w3_weight.weight_scale = l.s3;
    }
    DecodingInitParam<half> dp;
    dp.cublas_handle = handle;
    dp.stream = stream;
    dp.embedding_table = (half *)a->embedding;
    dp.freq_cis = a->freq_cis;
    dp.prompt_sequence_length = a->prompt_seq_len;
    dp.prompt_tokens = a->prompt_tokens;
    dp.prompt_tokens_mask = a->prompt_mask;
    dp.decodingnorm.gamma = (half *)a->final_gamma;
    dp.output_weight.kernel = (half *)a->lm_head;
    dp.output_ids = a->output_ids;
    dp.sequence_length = a->seq_len;
    dp.min_prompt_seq_len = a->min_prompt;
    dp.max_prompt_seq_len = a->max_prompt;

    DecodingSampling<OperationType::FP16> *dec = new DecodingSampling<OperationType::FP16>(
        allocator, a->batch, a->max_prompt_len, a->max_gen_len, a->head_num, a->size_per_head, a->vocab, a->layers, a->end_id,
        a->ffn, a->topk, a->topp);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, stream);
    dec->forward(param, dp);
    cudaEventRecord(e1, stream);
    cudaError_t ce = cudaStreamSynchronize(stream);
#ifdef FLB_WITH_NCCL
    // the decode steps' exchange kernels report a rank that did not show up through a sticky status word
    const unsigned push_status = (ce == cudaSuccess) ? flb_tp_push_status(&g_tp, stream) : 0u;
#else
    const unsigned push_status = 0u;
#endif
    float t = 0.f;
    cudaEventElapsedTime(&t, e0, e1);
    if (ms) *ms = t;
    delete dec;
    delete[] param;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaStreamDestroy(stream);
    cublasDestroy(handle);
    if (ce != cudaSuccess) return 2000 + (int)ce;
    if (push_status) return 3000 + (int)(push_status & 0x3ffu);
    ce = cudaGetLastError();
    return ce == cudaSuccess ? 0 : 2000 + (int)ce;
}

} // extern "C"
