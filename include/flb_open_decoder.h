/*
 * flb_open_decoder.h — the reference-side binding: what OpenDecoder<OpType,INT8>::forward calls where
 * fasterLlama/cuda/open_decoder.cu:138-239 used to be.
 *
 * The calls take OpenDecoder's own members (names as in fasterLlama/open_decoder.h:34-63) and forward()'s
 * arguments, fill one flb_attn_params block and call flb_attn_forward().  Buffers keep the reference's layouts:
 * q/k/v are the int32 outputs of the three INT8 GEMMs (open_decoder.cu:105-136), the result lands in qkv_buf_
 * [B,H,S,d] fp32 for launchAttnQuantizedTransposeKernel (:245), the caches are the caller's [B,H,T,d] slabs.
 * Scratch is the run of workspace buffers the replaced code used and nothing else needs any more:
 * query_out_buf_, key_out_buf_, value_out_fp_buf_ and qk_buf_, which OpenDecoder::initialize carves back to
 * back (open_decoder.cu:39-42).
 *
 * State.  Everything the binding remembers between calls lives in a flb_open_decoder_ctx that the OpenDecoder
 * object owns as a member (one per object: two decoders, two masks, two devices or two streams in one process
 * each keep their own answers), initialised in its constructor:
 *
 *     flb_open_decoder_ctx flb_ctx_;                       // fasterLlama/open_decoder.h, beside the buffers
 *     flb_open_decoder_ctx_init(&flb_ctx_);                // OpenDecoder::OpenDecoder, open_decoder.cu:9-24
 *
 * Errors follow the reference's convention (fasterLlama/cuda/utils.h:50-80): print, then exit(1).
 *
 * Environment switches (read by flb_open_decoder_ctx_init, so that the unchanged DecodingSampling can be
 * steered from outside):
 *   FLB_CACHE_F16=1   keep the caches in fp16 inside the caller's float slabs (first half of each slab)
 *   FLB_MASK_MODE=n   force a flb_mask_mode (default: the caller's additive mask is classified with
 *                     flb_attn_classify_mask the first time a mask pointer is seen)
 *   FLB_EARLY_START=n 0: decode calls keep a counter memset and an ordinary launch each.  1 (default): only the
 *                     first decode call after a prefill clears the counters, the others are launched with
 *                     programmatic stream serialisation and fetch their first cache tiles early.  2: they also
 *                     read q and k and stream the whole cache before the kernel in front has completed — correct
 *                     only if every earlier writer of q, k, the scales and the cache rows has COMPLETED by the
 *                     time the kernel directly in front starts.  Stream order does not imply that when that
 *                     kernel was itself launched with programmatic serialisation (a library GEMM may be), so
 *                     level 2 is opt-in for callers who know their launch chain.
 *   FLB_TP_PUSH=0     tensor-parallel form only: decode steps use ncclAllGather instead of peer stores
 *   FLB_MERGED_QKV=1  one INT8 GEMM for the Q, K and V projections (flb_open_decoder_packed_qkv below); q, k and v are then
 *                     column blocks of one int32 buffer and the attention call reads them in place
 *   FLB_FUSE_QUANT=1  also do the step that follows attention (launchAttnQuantizedTransposeKernel,
 *                     open_decoder.cu:245-246) inside the call; the caller then skips its own launch:
 *                         if (!flb_open_decoder_fused_quant(&flb_ctx_)) launchAttnQuantizedTransposeKernel(...);
 */
#ifndef FLB_OPEN_DECODER_H
#define FLB_OPEN_DECODER_H

#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "flb_attn.h"

struct flb_tp_ctx;

#define FLB_OPEN_DECODER_MAX_LAYERS 128

typedef struct flb_open_decoder_ctx {
    /* switches (environment, read once per object) */
    int cache_f16;
    int forced_mask_mode; /* -1: classify the caller's mask */
    int early_start;      /* 0, 1 or 2 */
    int fused_quant;
    /* what the object has learnt about its caller */
    const float *mask_seen; /* the mask pointer mask_mode was derived from */
    int mask_rows;
    int mask_mode;
    /* scratch whose arrival counters are known to be zero (left so by the last decode call), and the stream
     * that call ran on: another stream or another buffer gets a memset and an ordinary launch again */
    const void *clean_scratch;
    cudaStream_t clean_stream;
    /* tensor-parallel form: the communicator block this decoder uses (NULL: single GPU) */
    struct flb_tp_ctx *tp;
    /* merged QKV projection (FLB_MERGED_QKV=1): per layer, the caller's three [hidden, hidden] INT8 weight matrices
     * packed once into one [hidden, 3*hidden] matrix, found again by the query matrix's address */
    int merged_qkv;
    int n_packed;
    struct {
        const int8_t *wq, *wk, *wv;
        int8_t *packed;
    } packed[FLB_OPEN_DECODER_MAX_LAYERS];
} flb_open_decoder_ctx;

static inline int flb_open_decoder_env_int(const char *name, int fallback) {
    const char *e = getenv(name);
    return e ? atoi(e) : fallback;
}

#ifdef FLB_WITH_NCCL
struct flb_tp_ctx *flb_tp_default(void); /* the block registered with flb_tp_register(), see the tensor-parallel section */
#endif

static inline void flb_open_decoder_ctx_init(flb_open_decoder_ctx *c) {
    memset(c, 0, sizeof(*c));
    c->cache_f16 = flb_open_decoder_env_int("FLB_CACHE_F16", 0);
    c->forced_mask_mode = flb_open_decoder_env_int("FLB_MASK_MODE", -1);
    c->early_start = flb_open_decoder_env_int("FLB_EARLY_START", 1);
    if (c->early_start < 0 || c->early_start > 2) c->early_start = 1;
#ifdef FLB_OPEN_DECODER_NO_EARLY_START /* for builds in which other code may write the scratch between calls */
    c->early_start = 0;
#endif
    c->fused_quant = flb_open_decoder_env_int("FLB_FUSE_QUANT", 0);
    c->merged_qkv = flb_open_decoder_env_int("FLB_MERGED_QKV", 0);
    c->mask_mode = -1;
#ifdef FLB_WITH_NCCL
    c->tp = flb_tp_default();
#endif
}

static inline int flb_open_decoder_fused_quant(const flb_open_decoder_ctx *c) { return c->fused_quant; }

/* Releases what the context owns (the packed weight copies).  OpenDecoder::~OpenDecoder calls it. */
static inline void flb_open_decoder_ctx_destroy(flb_open_decoder_ctx *c) {
    for (int i = 0; i < c->n_packed; ++i) cudaFree(c->packed[i].packed);
    c->n_packed = 0;
}

/* Merged QKV projection (the three cublasGemmEx calls of open_decoder.cu:105-136 as one): returns the layer's
 * [hidden, 3*hidden] INT8 weight matrix — the caller's three row-major [in, out] matrices side by side — packing it on
 * the stream the first time this layer's matrices are seen, or NULL when merging is off or no copy can be made (the
 * caller then issues its three GEMMs as before).  One GEMM  C[m, 3*hidden] = X[m, hidden] . W  then leaves q, k and v
 * as column blocks of ONE int32 buffer, which the attention call reads in place (qkv_row_stride = 3 * hidden).
 * The copies live until flb_open_decoder_ctx_destroy(); the caller's matrices must not change once packed. */
static inline const int8_t *flb_open_decoder_packed_qkv(flb_open_decoder_ctx *c, const int8_t *wq, const int8_t *wk, const int8_t *wv,
                                                        int hidden, cudaStream_t stream) {
    if (!c->merged_qkv) return NULL;
    for (int i = 0; i < c->n_packed; ++i)
        if (c->packed[i].wq == wq && c->packed[i].wk == wk && c->packed[i].wv == wv) return c->packed[i].packed;
    if (c->n_packed >= FLB_OPEN_DECODER_MAX_LAYERS) return NULL;
    int8_t *dst = NULL;
    const size_t n = (size_t)hidden;
    if (cudaMalloc((void **)&dst, 3 * n * n) != cudaSuccess) {
        cudaGetLastError();
        return NULL;
    }
    const int8_t *src[3] = {wq, wk, wv};
    for (int i = 0; i < 3; ++i) {
        if (cudaMemcpy2DAsync(dst + i * n, 3 * n, src[i], n, n, n, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) {
            cudaFree(dst);
            cudaGetLastError();
            return NULL;
        }
    }
    c->packed[c->n_packed].wq = wq;
    c->packed[c->n_packed].wk = wk;
    c->packed[c->n_packed].wv = wv;
    c->packed[c->n_packed].packed = dst;
    ++c->n_packed;
    return dst;
}

/* attn_q8 / attn_q8_scale: from_tensor_int8_buf_ / from_tensor_scale_buf_ (used when FLB_FUSE_QUANT=1; the scale
 * buffer may be the same memory as from_tensor_scale_buf_ passed as the activation scale: every read of a row's
 * activation scale happens before that row's new scale is written).
 * qkv_row_stride: int32 elements between the rows of two tokens in query_buf_/key_buf_/value_buf_ — head_num *
 * size_per_head for the reference's three separate GEMM outputs, 3 * that when they are column blocks of one
 * merged projection's [B*S, 3*hidden] output. */
static inline void flb_open_decoder_fill_params(flb_open_decoder_ctx *c, flb_attn_params *ap, int batch_size_, int head_num_,
                                                int size_per_head_, int total_len_, int seq_len, int start_pos,
                                                const int32_t *query_buf_, const int32_t *key_buf_, const int32_t *value_buf_,
                                                int qkv_row_stride, const float *from_tensor_scale_buf_,
                                                const float *q_weight_scale, const float *k_weight_scale,
                                                const float *v_weight_scale, const float *freq_cis, const float *attn_mask,
                                                float *key_cache_, float *value_cache_, void *scratch, size_t scratch_bytes,
                                                float *out, int8_t *attn_q8, float *attn_q8_scale, cudaStream_t stream) {
    int mask_mode = c->forced_mask_mode;
    if (mask_mode < 0) {
        if (!attn_mask) {
            mask_mode = FLB_MASK_NONE;
        } else {
            if (c->mask_mode < 0 || c->mask_seen != attn_mask || c->mask_rows != total_len_) {
                /* one look at the caller's mask, the first time this pointer is seen (synchronises the stream once;
                 * the check overwrites the head of the scratch, so a decode call after it clears its counters) */
                int m = FLB_MASK_GENERIC;
                if (flb_attn_classify_mask(attn_mask, total_len_, total_len_, scratch, &m, stream) != FLB_OK) m = FLB_MASK_GENERIC;
                c->mask_mode = m;
                c->mask_seen = attn_mask;
                c->mask_rows = total_len_;
                c->clean_scratch = NULL;
            }
            mask_mode = c->mask_mode;
        }
    }
    memset(ap, 0, sizeof(*ap));
    ap->batch_size = batch_size_;
    ap->head_num = head_num_;
    ap->size_per_head = size_per_head_;
    ap->seq_len = seq_len;
    ap->start_pos = start_pos;
    ap->total_len = total_len_;
    ap->input_mode = FLB_IN_INT32;
    ap->q = query_buf_;
    ap->k = key_buf_;
    ap->v = value_buf_;
    ap->qkv_row_stride = qkv_row_stride;
    ap->act_scale = from_tensor_scale_buf_;
    ap->q_w_scale = q_weight_scale;
    ap->k_w_scale = k_weight_scale;
    ap->v_w_scale = v_weight_scale;
    ap->freq_cis = freq_cis; /* row s of this pointer for token s: the reference's rule (decoder_kernels.cu:440) */
    ap->rope_pos0 = 0;
    ap->rope_add_past = 0;
    ap->mask_mode = mask_mode;
    ap->attn_mask = attn_mask;
    ap->mask_row_stride = total_len_;
    ap->k_cache = key_cache_;
    ap->v_cache = value_cache_;
    ap->cache_dtype = c->cache_f16 ? FLB_F16 : FLB_F32;
    ap->out = out;
    ap->out_dtype = FLB_F32;
    ap->softmax_scale = 1.0f / sqrtf((float)size_per_head_);
    ap->scratch = scratch;
    ap->scratch_bytes = scratch_bytes;
    /* The decode kernel leaves its arrival counters at zero, so only the first decode call after something else
     * has used the scratch (a prefill call stages fp16 tiles there, the mask check writes its head) needs them
     * cleared.  Every later decode call on the same scratch and stream skips the memset and may start early. */
    if (seq_len > 1 || !c->early_start) {
        c->clean_scratch = NULL;
        ap->scratch_zeroed = 0;
    } else if (c->clean_scratch != scratch || c->clean_stream != stream) {
        c->clean_scratch = scratch;
        c->clean_stream = stream;
        ap->scratch_zeroed = 0;
    } else {
        ap->scratch_zeroed = 1;
        ap->early_start = c->early_start;
    }
    if (c->fused_quant) {
        ap->out_q8 = attn_q8;
        ap->out_q8_scale = attn_q8_scale;
    }
}

/* Errors follow the reference's convention: print, then exit(1). */
static inline void flb_open_decoder_check(int st, const char *what, int line) {
    if (st != FLB_OK) {
        printf("CUDA Error:\n    File:   %s\n    Line:   %d\n    %s status: %d (%s)\n", __FILE__, line, what, st, flb_status_string(st));
        exit(1);
    }
}

static inline void flb_open_decoder_attention_core(flb_open_decoder_ctx *c, int batch_size_, int head_num_, int size_per_head_,
                                                   int total_len_, int seq_len, int start_pos, const int32_t *query_buf_,
                                                   const int32_t *key_buf_, const int32_t *value_buf_, int qkv_row_stride,
                                                   const float *from_tensor_scale_buf_, const float *q_weight_scale,
                                                   const float *k_weight_scale, const float *v_weight_scale,
                                                   const float *freq_cis, const float *attn_mask, float *key_cache_,
                                                   float *value_cache_, void *scratch, size_t scratch_bytes, float *out,
                                                   int8_t *attn_q8, float *attn_q8_scale, cudaStream_t stream) {
    flb_attn_params ap;
    flb_open_decoder_fill_params(c, &ap, batch_size_, head_num_, size_per_head_, total_len_, seq_len, start_pos, query_buf_, key_buf_,
                                 value_buf_, qkv_row_stride, from_tensor_scale_buf_, q_weight_scale, k_weight_scale, v_weight_scale,
                                 freq_cis, attn_mask, key_cache_, value_cache_, scratch, scratch_bytes, out, attn_q8, attn_q8_scale,
                                 stream);
    flb_open_decoder_check(flb_attn_forward(&ap, stream), "flb_attn", __LINE__);
}

/* The call OpenDecoder::forward makes: scratch = query_out_buf_ .. end of qk_buf_ (3 * buf_size floats + the score
 * buffer, contiguous), output = qkv_buf_.  qkv_row_stride as above (head_num_ * size_per_head_ for the unchanged
 * three projections). */
static inline void flb_open_decoder_attention(flb_open_decoder_ctx *c, int batch_size_, int head_num_, int size_per_head_,
                                              int max_prompt_len_, int total_len_, int seq_len, int start_pos,
                                              const int32_t *query_buf_, const int32_t *key_buf_, const int32_t *value_buf_,
                                              int qkv_row_stride, const float *from_tensor_scale_buf_, const float *q_weight_scale,
                                              const float *k_weight_scale, const float *v_weight_scale, const float *freq_cis,
                                              const float *attn_mask, float *key_cache_, float *value_cache_,
                                              float *query_out_buf_, float *qk_buf_, float *qkv_buf_, int8_t *attn_q8,
                                              float *attn_q8_scale, cudaStream_t stream) {
    const size_t bytes =
        sizeof(float) * ((size_t)(qk_buf_ - query_out_buf_) + (size_t)batch_size_ * head_num_ * max_prompt_len_ * total_len_);
    flb_open_decoder_attention_core(c, batch_size_, head_num_, size_per_head_, total_len_, seq_len, start_pos, query_buf_, key_buf_,
                                    value_buf_, qkv_row_stride, from_tensor_scale_buf_, q_weight_scale, k_weight_scale, v_weight_scale,
                                    freq_cis, attn_mask, key_cache_, value_cache_, query_out_buf_, bytes, qkv_buf_, attn_q8,
                                    attn_q8_scale, stream);
}

/* ---- tensor-parallel form (compiled only with -DFLB_WITH_NCCL) -------------------------------------
 * Each rank owns head_num/size heads: its OpenDecoder::forward computes the Q/K/V projections for its
 * column slice of the weights only (pointer offset rank*hidden/size, leading dimension unchanged),
 * calls flb_open_decoder_attention_tp() on those heads against its own cache shard (the first 1/size of
 * every layer's slab), and gets the full [B,H,S,d] attention output back through ONE exchange: an
 * all-gather of the fp32 head outputs (the next kernel needs the absmax over all heads of a token row).
 * Prefill does it with ncclAllGather; decode steps (small, latency-bound, 32 per token) do it without a
 * collective call: the decode kernel stores its rows into every rank's receive slot as peer stores and
 * flb_attn_peer_exchange() does the flag hand-shake (FLB_TP_PUSH=0 keeps NCCL there too).
 * Everything after that stays replicated.
 *
 * The communicator and everything the exchange remembers live in a flb_tp_ctx that the program owns (one per
 * rank).  OpenDecoder has no notion of ranks and is constructed deep inside DecodingSampling, so the program
 * registers its block once, before it constructs the decoder, with flb_tp_register(); decoders constructed
 * afterwards pick it up in flb_open_decoder_ctx_init().  Exactly one translation unit defines
 * FLB_OPEN_DECODER_TP_STATE before including this header; it holds that one registration pointer. */
#ifdef FLB_WITH_NCCL
#include <nccl.h>

typedef struct flb_tp_ctx {
    ncclComm_t comm;
    int rank, size;
    /* decode steps without NCCL (see flb_tp_push_setup): 0 = not set up yet, 1 = in use, -1 = not available */
    int push_ready;
    unsigned push_epoch;
    size_t push_slot_bytes;
    unsigned char *push_base[FLB_MAX_PEERS]; /* [r]: rank r's block (256 B of flag words + two receive slots) as mapped here */
} flb_tp_ctx;

#ifdef FLB_OPEN_DECODER_TP_STATE
static flb_tp_ctx *flb_tp_registered = NULL;
void flb_tp_register(flb_tp_ctx *tp) { flb_tp_registered = tp; }
flb_tp_ctx *flb_tp_default(void) { return flb_tp_registered; }
#else
void flb_tp_register(flb_tp_ctx *tp);
#endif

static inline void flb_tp_ctx_init(flb_tp_ctx *tp, ncclComm_t comm, int rank, int size) {
    memset(tp, 0, sizeof(*tp));
    tp->comm = comm;
    tp->rank = rank;
    tp->size = size;
}
static inline int flb_tp_size(const flb_open_decoder_ctx *c) { return c->tp ? c->tp->size : 1; }
static inline int flb_tp_rank(const flb_open_decoder_ctx *c) { return c->tp ? c->tp->rank : 0; }

#define FLB_TP_CUDA(call, okvar)                                                                                              \
    do {                                                                                                                      \
        if ((call) != cudaSuccess) (okvar) = 0;                                                                               \
    } while (0)
#define FLB_TP_NCCL(call)                                                                                                     \
    do {                                                                                                                      \
        const ncclResult_t r_ = (call);                                                                                       \
        if (r_ != ncclSuccess) {                                                                                              \
            printf("NCCL Error:\n    File:   %s\n    Line:   %d\n    %s\n", __FILE__, __LINE__, ncclGetErrorString(r_));      \
            exit(1);                                                                                                          \
        }                                                                                                                     \
    } while (0)

/* One-time set-up of the decode exchange that needs no collective call per layer: every rank allocates one block
 * (flag words + two receive slots of slot_bytes), the CUDA IPC handles travel through the communicator once, and
 * every rank maps the others' blocks (which also enables peer access).  All ranks take the same decision: an
 * all-reduce(min) of "it worked here" ends the set-up, so either every rank pushes or every rank keeps NCCL.
 * A failed CUDA call on one rank turns the push path off everywhere; a failed NCCL call ends the program (the ranks
 * could not agree on anything any more).  flb_tp_push_teardown() gives the block back.  FLB_TP_PUSH=0 keeps the
 * NCCL all-gather for decode as well. */
static inline void flb_tp_push_setup(flb_tp_ctx *s, size_t slot_bytes, cudaStream_t stream) {
    const int g = s->size;
    int ok = (g <= FLB_MAX_PEERS) && flb_open_decoder_env_int("FLB_TP_PUSH", 1) != 0;
    unsigned char *own = NULL, *stage = NULL;
    cudaIpcMemHandle_t mine, all[FLB_MAX_PEERS];
    slot_bytes = (slot_bytes + 255) / 256 * 256;
    const size_t total = 256 + 2 * slot_bytes;
    memset(&mine, 0, sizeof(mine));
    memset(all, 0, sizeof(all));
    if (ok) {
        FLB_TP_CUDA(cudaMalloc((void **)&own, total), ok);
        if (ok) FLB_TP_CUDA(cudaMemsetAsync(own, 0, total, stream), ok);
        if (ok) FLB_TP_CUDA(cudaIpcGetMemHandle(&mine, own), ok);
    }
    /* handles (64 bytes each) and the ranks' common decision go through the communicator: the ranks stay in step whatever happened */
    if (cudaMalloc((void **)&stage, (size_t)(g + 1) * 64 + 16) != cudaSuccess) {
        printf("flb_tp_push_setup: cudaMalloc failed\n");
        exit(1);
    }
    FLB_TP_CUDA(cudaMemcpyAsync(stage + (size_t)g * 64, &mine, 64, cudaMemcpyHostToDevice, stream), ok);
    FLB_TP_NCCL(ncclAllGather(stage + (size_t)g * 64, stage, 64, ncclChar, s->comm, stream));
    FLB_TP_CUDA(cudaMemcpyAsync(all, stage, (size_t)g * 64, cudaMemcpyDeviceToHost, stream), ok);
    FLB_TP_CUDA(cudaStreamSynchronize(stream), ok);
    for (int r = 0; r < g; ++r) s->push_base[r] = NULL;
    for (int r = 0; r < g && ok; ++r) {
        if (r == s->rank) {
            s->push_base[r] = own;
        } else if (cudaIpcOpenMemHandle((void **)&s->push_base[r], all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            s->push_base[r] = NULL;
            ok = 0;
        }
    }
    int *decision = (int *)(stage + (size_t)(g + 1) * 64);
    int mine_ok = ok;
    if (cudaMemcpyAsync(decision, &mine_ok, sizeof(int), cudaMemcpyHostToDevice, stream) != cudaSuccess) {
        printf("flb_tp_push_setup: the decision could not be staged\n");
        exit(1);
    }
    FLB_TP_NCCL(ncclAllReduce(decision, decision, 1, ncclInt, ncclMin, s->comm, stream));
    if (cudaMemcpyAsync(&ok, decision, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess) {
        printf("flb_tp_push_setup: the decision could not be read back\n");
        exit(1);
    }
    cudaGetLastError(); /* a failed IPC call above is handled by the common decision, not left as a sticky error text */
    cudaFree(stage);
    s->push_slot_bytes = slot_bytes;
    s->push_epoch = 0;
    s->push_ready = ok ? 1 : -1;
    if (!ok) { /* nobody pushes: give back what this rank had got hold of */
        for (int r = 0; r < g; ++r) {
            if (r != s->rank && s->push_base[r]) cudaIpcCloseMemHandle(s->push_base[r]);
            s->push_base[r] = NULL;
        }
        if (own) cudaFree(own);
    }
}

/* Undoes flb_tp_push_setup(): every rank unmaps the others' blocks, all ranks meet (so that nobody frees memory a
 * peer still has mapped or in flight), then each frees its own.  Call it on every rank, after the last forward(). */
static inline void flb_tp_push_teardown(flb_tp_ctx *s, cudaStream_t stream) {
    if (s->push_ready != 1) {
        s->push_ready = 0;
        return;
    }
    cudaStreamSynchronize(stream);
    for (int r = 0; r < s->size; ++r)
        if (r != s->rank && s->push_base[r]) cudaIpcCloseMemHandle(s->push_base[r]);
    int *token = NULL;
    if (cudaMalloc((void **)&token, sizeof(int)) == cudaSuccess) {
        cudaMemsetAsync(token, 0, sizeof(int), stream);
        FLB_TP_NCCL(ncclAllReduce(token, token, 1, ncclInt, ncclSum, s->comm, stream));
        cudaStreamSynchronize(stream);
        cudaFree(token);
    }
    cudaFree(s->push_base[s->rank]);
    for (int r = 0; r < s->size; ++r) s->push_base[r] = NULL;
    s->push_ready = 0;
}

/* Error bits the exchange kernels have left since set-up (FLB_STATUS_PEER_WAIT: a rank did not show up in time and
 * that step's rows were not delivered).  Synchronises the stream; 0 also when the push path is not in use. */
static inline unsigned flb_tp_push_status(flb_tp_ctx *s, cudaStream_t stream) {
    unsigned v = 0;
    if (s && s->push_ready == 1) {
        cudaMemcpyAsync(&v, s->push_base[s->rank] + 128, sizeof(v), cudaMemcpyDeviceToHost, stream);
        cudaStreamSynchronize(stream);
    }
    return v;
}

static inline void flb_open_decoder_attention_tp(flb_open_decoder_ctx *c, int batch_size_, int head_num_, int size_per_head_,
                                                 int max_prompt_len_, int total_len_, int seq_len, int start_pos,
                                                 const int32_t *query_buf_, const int32_t *key_buf_, const int32_t *value_buf_,
                                                 const float *from_tensor_scale_buf_, const float *q_weight_scale,
                                                 const float *k_weight_scale, const float *v_weight_scale,
                                                 const float *freq_cis, const float *attn_mask, float *key_cache_,
                                                 float *value_cache_, float *query_out_buf_, float *qk_buf_, float *qkv_buf_,
                                                 int8_t *attn_q8, float *attn_q8_scale, cudaStream_t stream) {
    flb_tp_ctx *s = c->tp;
    const int g = s ? s->size : 1, r = s ? s->rank : 0;
    const int fused = flb_open_decoder_fused_quant(c) && attn_q8 && attn_q8_scale; /* FLB_FUSE_QUANT=1: see the header comment */
    const int h_local = head_num_ / g;
    const size_t col0 = (size_t)r * h_local * size_per_head_;
    if (g == 1) {
        flb_open_decoder_attention(c, batch_size_, head_num_, size_per_head_, max_prompt_len_, total_len_, seq_len, start_pos, query_buf_,
                                   key_buf_, value_buf_, head_num_ * size_per_head_, from_tensor_scale_buf_, q_weight_scale,
                                   k_weight_scale, v_weight_scale, freq_cis, attn_mask, key_cache_, value_cache_, query_out_buf_, qk_buf_,
                                   qkv_buf_, attn_q8, attn_q8_scale, stream);
        return;
    }
    /* local heads: q/k/v are [B*S, h_local*d].  query_out_buf_, key_out_buf_, value_out_fp_buf_ are three equal
     * buffers of B*P*hidden floats in front of qk_buf_: the first two are the scratch, the third takes the local
     * output [B,h_local,S,d] (at most half of it with two ranks or more). */
    const size_t buf_size = (size_t)(qk_buf_ - query_out_buf_) / 3;
    float *local_out = query_out_buf_ + 2 * buf_size;
    const int row_stride = h_local * size_per_head_;
    if (seq_len == 1) {
        /* decode: the kernel stores each finished head row into every rank's receive slot (peer stores over NVLink);
         * one small kernel then signals, waits (bounded) and moves the slot into qkv_buf_.  No collective call. */
        const size_t row_bytes = sizeof(float) * (size_t)batch_size_ * head_num_ * size_per_head_;
        if (s->push_ready == 0) flb_tp_push_setup(s, row_bytes, stream);
        if (s->push_ready == 1 && row_bytes <= s->push_slot_bytes) {
            const unsigned epoch = ++s->push_epoch;
            const size_t slot_off = 256 + (size_t)(epoch & 1u) * s->push_slot_bytes;
            flb_attn_params ap;
            flb_open_decoder_fill_params(c, &ap, batch_size_, h_local, size_per_head_, total_len_, seq_len, start_pos, query_buf_, key_buf_,
                                         value_buf_, row_stride, from_tensor_scale_buf_, q_weight_scale + col0, k_weight_scale + col0,
                                         v_weight_scale + col0, freq_cis, attn_mask, key_cache_, value_cache_, query_out_buf_,
                                         sizeof(float) * 2 * buf_size, NULL, NULL, NULL, stream);
            ap.out_q8 = NULL;
            ap.out_q8_scale = NULL;
            ap.n_out_peers = g;
            ap.out_head_total = head_num_;
            ap.out_head_offset = r * h_local;
            for (int i = 0; i < g; ++i) ap.out_peers[i] = s->push_base[i] + slot_off;
            flb_open_decoder_check(flb_attn_decode(&ap, stream), "flb_attn_decode", __LINE__);
            flb_peer_exchange x;
            memset(&x, 0, sizeof(x));
            x.rank = r;
            x.size = g;
            x.epoch = epoch;
            x.flags_local = (unsigned *)s->push_base[r];
            for (int i = 0; i < g; ++i) x.flags_peer[i] = (unsigned *)s->push_base[i];
            x.recv = s->push_base[r] + slot_off;
            x.bytes = row_bytes;
            if (fused) {
                /* the received rows are quantised where they landed (the reference's next kernel, which the caller
                 * then skips); nobody reads the fp32 rows after that, so they are not copied into qkv_buf_ */
                x.dst = NULL;
                x.out_q8 = attn_q8;
                x.out_q8_scale = attn_q8_scale;
                x.q8_rows = batch_size_;
                x.q8_row_elems = head_num_ * size_per_head_;
            } else {
                x.dst = qkv_buf_;
            }
            x.status = (unsigned *)(s->push_base[r] + 128); /* sticky: read it with flb_tp_push_status() */
            x.timeout_ms = 2000;
            flb_open_decoder_check(flb_attn_peer_exchange(&x, stream), "flb_attn_peer_exchange", __LINE__);
            return;
        }
    }
    flb_open_decoder_attention_core(c, batch_size_, h_local, size_per_head_, total_len_, seq_len, start_pos, query_buf_, key_buf_,
                                    value_buf_, row_stride, from_tensor_scale_buf_, q_weight_scale + col0, k_weight_scale + col0,
                                    v_weight_scale + col0, freq_cis, attn_mask, key_cache_, value_cache_, query_out_buf_,
                                    sizeof(float) * 2 * buf_size, local_out, NULL, NULL, stream);
    /* one all-gather of head outputs: per sequence, every rank's [h_local, S, d] block lands in head order */
    const size_t blk = (size_t)h_local * seq_len * size_per_head_;
    FLB_TP_NCCL(ncclGroupStart());
    for (int b = 0; b < batch_size_; ++b)
        FLB_TP_NCCL(ncclAllGather(local_out + (size_t)b * blk, qkv_buf_ + (size_t)b * blk * g, blk, ncclFloat, s->comm, stream));
    FLB_TP_NCCL(ncclGroupEnd());
    if (fused) /* the caller skips its own quantisation launch: do it on the gathered tensor */
        flb_open_decoder_check(flb_attn_quantize(qkv_buf_, attn_q8, attn_q8_scale, batch_size_, head_num_, seq_len, size_per_head_, stream),
                               "flb_attn_quantize", __LINE__);
}
#endif /* FLB_WITH_NCCL */

#endif /* FLB_OPEN_DECODER_H */
