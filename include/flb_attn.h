/*
 * flb_attn.h — C ABI of the B200 (sm_100a) attention path for FasterLLaMA.
 *
 * One call replaces the whole attention section of the reference's decoder layer,
 * OpenDecoder<OpType,INT8>::forward, fasterLlama/cuda/open_decoder.cu:138-239:
 *
 *   launchQKRoteEmbeddingTranspose      fasterLlama/cuda/decoder_kernels.cu:553-590
 *   launchDequantizedVTransposeKernel   fasterLlama/cuda/decoder_kernels.cu:953-986
 *   launchStoreKVcacheKernel            fasterLlama/cuda/decoder_kernels.cu:634-662
 *   cublasSgemvStridedBatched / cublasGemmStridedBatchedEx  (Q.K^T)   open_decoder.cu:181-201
 *   launchBlockSoftmaxKernel            fasterLlama/cuda/decoder_kernels.cu:837-848
 *   cublasSgemvStridedBatched / cublasGemmStridedBatchedEx  (P.V)     open_decoder.cu:218-238
 *
 * Everything is plain C: pointers are device pointers unless said otherwise, sizes are
 * ints / size_t, the stream is a cudaStream_t passed as void*.  The library allocates
 * nothing, never synchronises the device, never exits and never throws: every entry
 * point returns a flb_status.
 */
#ifndef FLB_ATTN_H
#define FLB_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLB_ATTN_ABI_VERSION 4

/* ---- status codes (0 = ok, negative = error) ------------------------------------ */
typedef enum flb_status {
    FLB_OK = 0,
    FLB_ERR_NULL_POINTER = -1,      /* a required pointer is NULL                       */
    FLB_ERR_BAD_SHAPE = -2,         /* a dimension is <= 0 or inconsistent               */
    FLB_ERR_UNSUPPORTED = -3,       /* valid in the reference, not built here            */
    FLB_ERR_MISALIGNED = -4,        /* a pointer or stride breaks the 16-byte rule       */
    FLB_ERR_SCRATCH_TOO_SMALL = -5, /* scratch_bytes < flb_attn_workspace_bytes()        */
    FLB_ERR_LAUNCH = -6,            /* the CUDA runtime refused the launch               */
    FLB_ERR_BAD_ENUM = -7,          /* an enum field holds an unknown value              */
    FLB_ERR_DEVICE = -8,            /* the device is not sm_100 or the driver is missing */
    FLB_ERR_TOO_LARGE = -9          /* beyond a stated fixed maximum                     */
} flb_status;

/* ---- enums ---------------------------------------------------------------------- */

/* Form of q/k/v handed to the call, all laid out [batch, seq_len, head_num, size_per_head]
 * (the row-major output of the QKV GEMMs, open_decoder.cu:105-136). */
typedef enum flb_input_mode {
    FLB_IN_INT32 = 0, /* int32 accumulators; value = float(acc) * act_scale[b*S+s] * w_scale[h*d+i],
                         multiplied in that order (decoder_kernels.cu:449, :875)            */
    FLB_IN_F32 = 1,   /* float values, no scales                                            */
    FLB_IN_F16 = 2    /* half values, no scales                                             */
} flb_input_mode;

typedef enum flb_dtype {
    FLB_F32 = 0,
    FLB_F16 = 1
} flb_dtype;

/* The reference takes an additive fp32 mask [total_len, total_len] from the caller
 * (DecoderInitParam::attn_mask, open_decoder.h:16) and adds mask[start_pos + q][k] to the
 * scaled score (decoder_kernels.cu:807-815).  GENERIC does exactly that.  The CAUSAL modes
 * compute the same thing from indices for the two masks the reference's programs build:
 * strict (key < query position: samples/llama_fp16.cu:73-81) and inclusive
 * (key <= query position).  A query row whose keys are all masked returns zeros. */
typedef enum flb_mask_mode {
    FLB_MASK_NONE = 0,
    FLB_MASK_GENERIC = 1,
    FLB_MASK_CAUSAL_INCLUSIVE = 2,
    FLB_MASK_CAUSAL_STRICT = 3
} flb_mask_mode;

/* ---- the parameter block -------------------------------------------------------- */
#define FLB_MAX_PEERS 8

typedef struct flb_attn_params {
    /* dimensions (names follow OpenDecoder's constructor, open_decoder.h:65) */
    int batch_size;    /* B                                                              */
    int head_num;      /* H                                                              */
    int size_per_head; /* d: 64 or 128; decode calls (seq_len == 1) also take 256          */
    int seq_len;       /* S, tokens of this call per sequence: 1 = decode, >1 = prefill  */
    int start_pos;     /* rows already in the cache, same for every sequence
                          (OpenDecoder::forward's start_pos)                             */
    int total_len;     /* T, row capacity of one (b,h) cache slab                        */

    /* Optional extension the reference lacks: per-sequence cached rows, device int[B].
     * When non-NULL it replaces start_pos (decode only); max_past_len is then the host's
     * upper bound on its entries (0 = total_len - 1) and only sizes the grid. */
    const int *past_lens;
    int max_past_len;

    /* inputs.  Every pointer of this block is a device-addressable address.  For a decode call q, k, v,
     * the scales and `out` may also be PINNED HOST memory (cudaHostAlloc / cudaHostRegister: device-
     * addressable as it is): the kernel then reads the step's inputs and stores its result rows over
     * the bus itself — one launch, no staging copies.  Caches and scratch belong in device memory, and so do the
     * inputs of a prefill call (with half inputs and a half cache the call reads v in 64-row tiles, several times,
     * while its attention kernel runs). */
    int input_mode;         /* flb_input_mode                                            */
    const void *q;          /* [B,S,H,d]                                                 */
    const void *k;          /* [B,S,H,d]                                                 */
    const void *v;          /* [B,S,H,d]                                                 */
    const float *act_scale; /* FLB_IN_INT32: [B*S] per-token activation scale            */
    const float *q_w_scale; /* FLB_IN_INT32: [H*d] per-output-channel weight scales      */
    const float *k_w_scale;
    const float *v_w_scale;

    /* RoPE: table rows of d floats, [2i] = cos, [2i+1] = sin (decoding_kernels.cu:85-114);
     * pairs (2i, 2i+1) are rotated (decoder_kernels.cu:455-458).  Token s of sequence b uses
     * row rope_pos0 + s (+ its cached-row count when rope_add_past != 0).  The reference
     * always uses row s of the pointer it is given (decoder_kernels.cu:440), i.e.
     * rope_pos0 = 0, rope_add_past = 0.  NULL table = no rotation. */
    const float *freq_cis;
    int rope_pos0;
    int rope_add_past;

    /* mask */
    int mask_mode;           /* flb_mask_mode                                            */
    const float *attn_mask;  /* GENERIC: row 0 of the caller's [T,T] mask (NOT offset by
                                start_pos; the call adds the query position itself)      */
    int mask_row_stride;     /* GENERIC: floats between mask rows (the reference: T)     */

    /* KV cache, [B,H,T,d] (open_decoder.h:72-77); rows [past, past+S) are written by the
     * call.  The reference's cache is fp32; fp16 halves the decode traffic and is legal
     * because nothing but attention reads the cache. */
    void *k_cache;
    void *v_cache;
    int cache_dtype;         /* flb_dtype                                                */

    /* output [B,H,S,d] (qkv_buf_, open_decoder.h:61) */
    void *out;
    int out_dtype;           /* flb_dtype; the reference's is fp32                       */

    float softmax_scale;     /* the reference passes rsqrtf(d) (open_decoder.cu:208)     */

    /* Scratch for the split-KV partial results (decode) — the reference's qk_buf_ is free
     * for this.  scratch_zeroed != 0 promises that the first
     * flb_attn_counter_bytes() bytes are zero on entry (they are left zero on exit), which
     * saves one memset node per call. */
    void *scratch;
    size_t scratch_bytes;
    int scratch_zeroed;

    /* rows of one split-KV partition; 0 = default (512; 256 when total_len <= 1024).  Results depend on this
     * value and on each sequence's own length only — never on B, H, the GPU count or the grid. */
    int split_len;

    /* Optional fused epilogue (both NULL = off): the reference's next step,
     * launchAttnQuantizedTransposeKernel (fasterLlama/cuda/decoder_kernels.cu:1179-1300, called at
     * open_decoder.cu:245): per token row, absmax over ALL heads (floor -1e9f as there), scale =
     * absmax / 127 into out_q8_scale[b*S+s], codes cvt.rni.sat.s8(x * 127.0f / absmax) into out_q8
     * laid out [B, S, H*d].  Needs out_dtype == FLB_F32; `out` is still written.  Decode does it in
     * the same launch (the last head to finish a sequence quantises its row); prefill adds one small
     * kernel. */
    int8_t *out_q8;
    float *out_q8_scale;

    /* Optional push of the result to several GPUs (decode only; n_out_peers == 0 = off, `out` is used
     * as above).  For a layer whose heads are split over G GPUs: every rank computes head_num local
     * heads and each finished output row is stored, by the kernel that produced it, straight into
     * out_peers[0..n_out_peers-1] — buffers of [B, out_head_total, 1, d] elements of out_dtype, one per
     * rank (the rank's own included), peer-mapped into this process — at head out_head_offset + h.
     * `out` is ignored then.  The stores are plain peer stores over NVLink; flb_attn_peer_exchange()
     * on the same stream publishes them and waits for the other ranks' rows.  Cannot be combined
     * with out_q8.  No counterpart in the reference (it is single-GPU). */
    void *out_peers[FLB_MAX_PEERS];
    int n_out_peers;
    int out_head_total;
    int out_head_offset;

    /* Decode only, optional: early_start != 0 launches the kernel with programmatic stream
     * serialisation.  Its CTAs may then become resident while the previous kernel on the stream is still
     * draining; what they do before that kernel has completed (griddepcontrol.wait) depends on the level:
     *   1  fetch their first cache tiles.  Promise: the cache rows below each sequence's length and
     *      past_lens were final BEFORE the previous kernel on the stream started (see the note on "final" below).
     *   2  in addition read q and k, rotate them and run the whole pass over the cached rows.  Promise,
     *      on top of level 1: q, k, act_scale, the weight scales and freq_cis were final before the
     *      previous kernel started — only v may still be in flight.  True in the decoder layer, where the
     *      kernel in front is the V projection and the Q and K projections ran before it
     *      (open_decoder.cu:105-136).
     * At both levels the new token's v, the cache append, the scratch and every output are touched only
     * after the previous kernel has completed, and the results are bit-identical to an ordinary launch.
     * Needs scratch_zeroed != 0 (a memset in front would serialise anyway); ignored otherwise.  A decode
     * kernel launched this way also lets the next such call start early.
     * "Final before the previous kernel started" means: every earlier writer of those buffers has COMPLETED.
     * Stream order alone does not give that when the previous kernel was itself launched with programmatic
     * serialisation (it may have started before ITS predecessor finished) — programmatic dependent launch is not
     * transitive.  Level 1 is safe after any kernel that does not write the cache rows below the cached lengths;
     * use level 2 only where the launch chain in front is known. */
    int early_start;

    /* ABI version 4.  Elements between the rows of two consecutive tokens in q, k and v; 0 = head_num *
     * size_per_head (dense [B,S,H,d]).  A larger value lets q, k and v be three column blocks of ONE
     * [B*S, 3*H*d] buffer — the output of a single merged QKV projection in place of the reference's three GEMMs
     * (open_decoder.cu:105-136): q = base, k = base + H*d, v = base + 2*H*d, qkv_row_stride = 3*H*d.  The byte
     * stride must be a multiple of 16. */
    int qkv_row_stride;
} flb_attn_params;

/* One exchange step between the ranks of a head-split layer (see out_peers above).  Every rank
 * calls it on its stream after its flb_attn_decode(): the kernel (1) writes `epoch` into word
 * [rank] of every other rank's flag array (system-scope release: the rows this rank pushed before,
 * in stream order, are visible first), (2) waits, for at most timeout_ms, until every other rank's
 * word in flags_local has reached `epoch`, (3) copies `bytes` from recv to dst (skipped when dst is
 * NULL or equals recv).  A wait that runs out sets FLB_STATUS_PEER_WAIT in *status (a device word,
 * e.g. the head of the scratch) and skips the copy; the context stays usable.
 * Rules for the caller: epoch starts at 1 and grows by one per exchange on every rank (flag words
 * start at 0); the receive buffer has two slots used alternately (slot = epoch & 1), which is
 * enough because no rank can run two exchanges ahead of another. */
typedef struct flb_peer_exchange {
    int rank, size;                       /* size <= FLB_MAX_PEERS                              */
    unsigned epoch;
    unsigned *flags_local;                /* [size] this rank's flag words                      */
    unsigned *flags_peer[FLB_MAX_PEERS];  /* [r] rank r's flag words, peer-mapped ([rank]: unused) */
    const void *recv;                     /* this rank's receive slot for this epoch            */
    void *dst;                            /* e.g. qkv_buf_                                      */
    size_t bytes;                         /* multiple of 16                                     */
    unsigned *status;                     /* device word, error bits are OR-ed in               */
    unsigned timeout_ms;                  /* 0 = default (1000)                                 */
    /* Optional: after the wait, also do the reference's next step on what was received —
     * launchAttnQuantizedTransposeKernel for seq_len == 1 (decoder_kernels.cu:1179-1255): recv is read as
     * q8_rows rows of q8_row_elems fp32 values ([B, H*d]); per row absmax (floor -1e9f), out_q8_scale[row]
     * = absmax / 127, out_q8[row][i] = cvt.rni.sat.s8(x * 127.0f / absmax).  Both NULL = off.  With it,
     * dst may be NULL: nobody needs the fp32 rows any more. */
    int8_t *out_q8;
    float *out_q8_scale;
    int q8_rows;
    int q8_row_elems;                     /* multiple of 4                                      */
} flb_peer_exchange;

#define FLB_STATUS_PEER_WAIT 0x100u

/* ---- entry points --------------------------------------------------------------- */

/* ABI version of the loaded library (== FLB_ATTN_ABI_VERSION it was built with). */
int flb_attn_abi_version(void);

/* Text for a status code; never NULL. */
const char *flb_status_string(int status);

/* Bytes of scratch the decode call needs for these dimensions (host computation only).
 * Replaces the qk_buf_ term of OpenDecoder::getWorkspaceSize (open_decoder.cu:54-68). */
int flb_attn_workspace_bytes(const flb_attn_params *p, size_t *bytes_out);

/* Bytes at the start of scratch that hold the split arrival counters. */
int flb_attn_counter_bytes(const flb_attn_params *p, size_t *bytes_out);

/* Host-side argument check only (no CUDA call); the launch entry points run it first. */
int flb_attn_validate(const flb_attn_params *p);

/* Decode: seq_len == 1.  Replaces open_decoder.cu:142-171 (dequant, RoPE, transpose, cache
 * append) + :194-201 (K.q) + :207-208 (softmax) + :231-238 (P.V) with one kernel launch. */
int flb_attn_decode(const flb_attn_params *p, void *cuda_stream);

/* Prefill: seq_len > 1, start_pos == 0 (the reference attends over the fresh K/V only,
 * open_decoder.cu:181-190, so it is valid for start_pos == 0 only).  Replaces :142-171 +
 * :181-190 + :207-208 + :218-227. */
int flb_attn_prefill(const flb_attn_params *p, void *cuda_stream);

/* Picks decode or prefill from seq_len exactly like open_decoder.cu:179,216. */
int flb_attn_forward(const flb_attn_params *p, void *cuda_stream);

/* Looks at a caller-built additive mask (device fp32 [rows, row_stride]) and reports which
 * flb_mask_mode reproduces it: CAUSAL_STRICT, CAUSAL_INCLUSIVE, NONE (all zero) or GENERIC.
 * A masked entry counts as such only when it is <= -1e30 (the samples use -FLT_MAX), because a
 * milder value such as -1e5 does not drop a key when the whole row is masked.
 * `scratch16` is 16 bytes of device memory the check may overwrite.  Synchronises the stream
 * (it copies the answer to the host): call it once at set-up, never per step. */
int flb_attn_classify_mask(const float *attn_mask, int rows, int row_stride, void *scratch16,
                           int *mode_out, void *cuda_stream);

/* Reads the kernels' error word at the head of `scratch` into *status_out (0 = no kernel gave
 * up on a bounded wait or met a cache length outside [0, total_len-1]).  Synchronises the
 * stream.  The reference has no counterpart: its kernels cannot report anything. */
int flb_attn_scratch_status(const void *scratch, unsigned *status_out, void *cuda_stream);

/* Bytes of device memory the library itself holds, on every GPU that loads it, for
 * flb_attn_decode_static_scratch(). */
#define FLB_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)

/* Decode for callers that have no scratch to give: same work as flb_attn_decode(), but the
 * split-KV scratch is a fixed FLB_STATIC_SCRATCH_BYTES block built into the library, so the call
 * needs nothing beyond the caller's inputs and outputs and never allocates.  The fields scratch,
 * scratch_bytes and scratch_zeroed of `p` are ignored.  This entry point has no counterpart in the
 * reference (whose OpenDecoder is always handed a workspace by its caller).
 *   - Limit: batch_size * head_num * partitions-per-sequence must fit the block (about 520 bytes
 *     per partition: 16 MiB holds e.g. batch 64 x 40 heads x 8 partitions).  Larger calls return
 *     FLB_ERR_TOO_LARGE and launch nothing.
 *   - The first call on each GPU looks the block's address up (not a stream operation): make that
 *     call before starting any stream capture on that GPU.
 *   - One block per GPU, shared by every call: calls that may overlap on a GPU race with each
 *     other; keep them on one stream.
 *   - The arrival counters in the block are cleared by a memset at the head of every call, so the call behaves as
 *     if scratch_zeroed were 0: `early_start` is ignored (every call through this entry point is an ordinary
 *     launch).
 *   - The kernels' error word lives in the block too: read it with flb_attn_static_scratch_status().
 *   - The block's address is looked up once per GPU and kept for the life of the process; a cudaDeviceReset()
 *     invalidates it, so the library must not be used across one. */
int flb_attn_decode_static_scratch(const flb_attn_params *p, void *cuda_stream);

/* Error word of the calls made through flb_attn_decode_static_scratch() on the current GPU (same bits as
 * flb_attn_scratch_status(): a bounded wait that ran out, a cached length outside [0, total_len-1]); 0 when that
 * entry point has not been used on this GPU yet.  Synchronises the stream.  No counterpart in the reference. */
int flb_attn_static_scratch_status(unsigned *status_out, void *cuda_stream);

/* The reference's attention-output quantisation as a call of its own (launchAttnQuantizedTransposeKernel,
 * fasterLlama/cuda/decoder_kernels.cu:1179-1300, called at open_decoder.cu:245): attn fp32 [B,H,S,d] ->
 * q8 int8 [B,S,H*d] + scale fp32 [B*S] (absmax over all heads of a token row / 127, floor -1e9f).  The
 * fused forms (flb_attn_params::out_q8, flb_peer_exchange::out_q8) do the same arithmetic; this entry is
 * for callers that assemble the [B,H,S,d] tensor themselves, e.g. after an all-gather.  d is 64 or 128. */
int flb_attn_quantize(const float *attn, int8_t *q8, float *scale, int batch_size, int head_num, int seq_len,
                      int size_per_head, void *cuda_stream);

/* Signal + bounded wait + copy described at flb_peer_exchange.  One small kernel; no host
 * synchronisation.  No counterpart in the reference. */
int flb_attn_peer_exchange(const flb_peer_exchange *x, void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* FLB_ATTN_H */
