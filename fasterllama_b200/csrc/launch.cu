// launch.cu — the extern "C" layer declared in include/flb_attn.h: argument validation, scratch
// carving and kernel launches.  Stream-ordered, allocation-free, no hidden synchronisation
// (except the two set-up/diagnostic calls that say so), no exit(), no exceptions.
#include "../../include/flb_attn.h"
#include "decode_attn.cuh"
#include "prefill_attn.cuh"

#include <cuda_runtime.h>

namespace flb {
cudaError_t launch_decode(const DecodeArgs &a, bool cache_f16, int head_dim, cudaStream_t stream);
}

namespace {

inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Rows of one split-KV partition.  The default is a function of the slab capacity alone (the same on every GPU that
// holds a shard of the batch, whatever lengths its sequences have), so results stay bit-identical under any sharding:
// short slabs get smaller partitions, whose CTAs fill the tail of a call that is only one or two waves long
// (measured at batch 32 x 32 heads, 640 cached rows: 60.3 us with 256-row partitions against 62.8 us with 512).
inline int split_len_of(const flb_attn_params *p) {
    if (p->split_len > 0) return p->split_len;
    return p->total_len <= flb::kShortSlabRows ? flb::kShortSlabSplitLen : flb::kDefaultSplitLen;
}

// partitions the grid must hold per (b,h) for a cache of `past` rows
inline int nsplit_for(int past, int split_len) { return past <= 0 ? 1 : (past + split_len - 1) / split_len; }

struct ScratchLayout {
    size_t counter_bytes, ml_off, o_off, total;
};
inline ScratchLayout layout_for(int B, int H, int nsplit_max, int head_dim = flb::kHeadDim) {
    ScratchLayout l;
    const size_t units = (size_t)B * H;
    // status words, one arrival counter per (b,h) (partition merge), one per sequence (fused quantisation)
    l.counter_bytes = round_up(sizeof(unsigned) * (flb::kStatusWords + units + (size_t)B), 256);
    l.ml_off = l.counter_bytes;
    l.o_off = l.ml_off + round_up(units * nsplit_max * 2 * sizeof(float), 256);
    l.total = l.o_off + units * nsplit_max * head_dim * sizeof(float);
    return l;
}

int check_common(const flb_attn_params *p) {
    if (!p) return FLB_ERR_NULL_POINTER;
    if (p->batch_size <= 0 || p->head_num <= 0 || p->size_per_head <= 0 || p->seq_len <= 0 || p->total_len <= 0)
        return FLB_ERR_BAD_SHAPE;
    if (p->start_pos < 0) return FLB_ERR_BAD_SHAPE;
    // decode: 64, 128 and 256 of the head sizes that the reference's kernels accept (decoder_kernels.cu:563-589);
    // the tensor-core prefill kernel is built for 64 and 128 (256 would need more accumulator columns than TMEM has
    // beside the scores of two query tiles)
    if (p->size_per_head != 128 && p->size_per_head != 64 && !(p->seq_len == 1 && p->size_per_head == 256))
        return FLB_ERR_UNSUPPORTED;
    if (p->input_mode < FLB_IN_INT32 || p->input_mode > FLB_IN_F16) return FLB_ERR_BAD_ENUM;
    if (p->mask_mode < FLB_MASK_NONE || p->mask_mode > FLB_MASK_CAUSAL_STRICT) return FLB_ERR_BAD_ENUM;
    if (p->cache_dtype != FLB_F32 && p->cache_dtype != FLB_F16) return FLB_ERR_BAD_ENUM;
    if (p->out_dtype != FLB_F32 && p->out_dtype != FLB_F16) return FLB_ERR_BAD_ENUM;
    if (p->split_len < 0 || (p->split_len % 32) != 0) return FLB_ERR_BAD_SHAPE;
    if (!p->q || !p->k || !p->v || !p->k_cache || !p->v_cache) return FLB_ERR_NULL_POINTER;
    if (p->n_out_peers < 0 || p->n_out_peers > FLB_MAX_PEERS) return FLB_ERR_BAD_SHAPE;
    if (p->early_start < 0 || p->early_start > 2) return FLB_ERR_BAD_ENUM;
    if (p->n_out_peers == 0) {
        if (!p->out) return FLB_ERR_NULL_POINTER;
        if (!aligned16(p->out)) return FLB_ERR_MISALIGNED;
    } else {
        // head-split push: decode only, every destination given, the local heads inside the full row
        if (p->seq_len != 1 || p->out_q8) return FLB_ERR_UNSUPPORTED;
        if (p->out_head_offset < 0 || p->out_head_total < p->out_head_offset + p->head_num) return FLB_ERR_BAD_SHAPE;
        for (int i = 0; i < p->n_out_peers; ++i) {
            if (!p->out_peers[i]) return FLB_ERR_NULL_POINTER;
            if (!aligned16(p->out_peers[i])) return FLB_ERR_MISALIGNED;
        }
    }
    if (p->input_mode == FLB_IN_INT32 && (!p->act_scale || !p->q_w_scale || !p->k_w_scale || !p->v_w_scale))
        return FLB_ERR_NULL_POINTER;
    if (p->mask_mode == FLB_MASK_GENERIC) {
        if (!p->attn_mask) return FLB_ERR_NULL_POINTER;
        if (p->mask_row_stride <= 0) return FLB_ERR_BAD_SHAPE;
    }
    if (p->rope_pos0 < 0) return FLB_ERR_BAD_SHAPE;
    if (p->qkv_row_stride != 0) {
        if (p->qkv_row_stride < p->head_num * p->size_per_head) return FLB_ERR_BAD_SHAPE;
        const int esz = (p->input_mode == FLB_IN_F16) ? 2 : 4;
        if (((size_t)p->qkv_row_stride * esz) % 16u) return FLB_ERR_MISALIGNED;
    }
    if (!aligned16(p->k_cache) || !aligned16(p->v_cache) || !aligned16(p->q) || !aligned16(p->k) ||
        !aligned16(p->v))
        return FLB_ERR_MISALIGNED;
    if ((size_t)p->batch_size * p->head_num > (size_t)1 << 24) return FLB_ERR_TOO_LARGE;
    if ((p->out_q8 != nullptr) != (p->out_q8_scale != nullptr)) return FLB_ERR_NULL_POINTER;
    if (p->out_q8 && p->out_dtype != FLB_F32) return FLB_ERR_UNSUPPORTED;
    if (p->out_q8 && !aligned16(p->out_q8)) return FLB_ERR_MISALIGNED;
    return FLB_OK;
}

int max_past_of(const flb_attn_params *p) {
    if (!p->past_lens) return p->start_pos;
    return (p->max_past_len > 0) ? p->max_past_len : p->total_len - 1;
}

} // namespace

extern "C" {

int flb_attn_abi_version(void) { return FLB_ATTN_ABI_VERSION; }

const char *flb_status_string(int status) {
    switch (status) {
    case FLB_OK: return "ok";
    case FLB_ERR_NULL_POINTER: return "a required pointer is NULL";
    case FLB_ERR_BAD_SHAPE: return "a dimension is out of range or inconsistent";
    case FLB_ERR_UNSUPPORTED: return "this shape or mode is not supported by this build";
    case FLB_ERR_MISALIGNED: return "a pointer or stride is not 16-byte aligned";
    case FLB_ERR_SCRATCH_TOO_SMALL: return "scratch is smaller than flb_attn_workspace_bytes()";
    case FLB_ERR_LAUNCH: return "the CUDA runtime refused the launch";
    case FLB_ERR_BAD_ENUM: return "an enum field holds an unknown value";
    case FLB_ERR_DEVICE: return "the device is not sm_100 or a driver entry point is missing";
    case FLB_ERR_TOO_LARGE: return "a size is beyond a fixed maximum of this build";
    default: return "unknown status";
    }
}

int flb_attn_validate(const flb_attn_params *p) {
    int st = check_common(p);
    if (st != FLB_OK) return st;
    if (p->seq_len == 1) {
        const int mp = max_past_of(p);
        if (mp < 0 || mp + 1 > p->total_len) return FLB_ERR_BAD_SHAPE;
        if (p->mask_mode == FLB_MASK_GENERIC && p->mask_row_stride < mp + 1) return FLB_ERR_BAD_SHAPE;
        if (!p->scratch) return FLB_ERR_NULL_POINTER;
        if (!aligned16(p->scratch)) return FLB_ERR_MISALIGNED;
        const int nsm = nsplit_for(mp, split_len_of(p));
        if ((unsigned long long)p->batch_size * p->head_num * nsm > 0x7fffffffull) return FLB_ERR_TOO_LARGE; // grid / int indices
        const ScratchLayout l = layout_for(p->batch_size, p->head_num, nsm, p->size_per_head);
        if (p->scratch_bytes < l.total) return FLB_ERR_SCRATCH_TOO_SMALL;
    } else {
        // the reference's prefill attends over the fresh rows only (open_decoder.cu:181-190)
        if (p->past_lens || p->start_pos != 0) return FLB_ERR_UNSUPPORTED;
        if (p->seq_len > p->total_len) return FLB_ERR_BAD_SHAPE;
        if ((unsigned long long)p->batch_size * p->head_num * ((p->seq_len + 127) / 128) > 0x7fffffffull) return FLB_ERR_TOO_LARGE;
        if (p->mask_mode == FLB_MASK_GENERIC && p->mask_row_stride < p->seq_len) return FLB_ERR_BAD_SHAPE;
        if (!p->scratch) return FLB_ERR_NULL_POINTER;
        if (!aligned16(p->scratch)) return FLB_ERR_MISALIGNED;
        if (p->scratch_bytes < flb::prefill_scratch_bytes(p->batch_size, p->head_num, p->seq_len, p->size_per_head))
            return FLB_ERR_SCRATCH_TOO_SMALL;
    }
    return FLB_OK;
}

int flb_attn_counter_bytes(const flb_attn_params *p, size_t *bytes_out) {
    if (!p || !bytes_out) return FLB_ERR_NULL_POINTER;
    if (p->batch_size <= 0 || p->head_num <= 0) return FLB_ERR_BAD_SHAPE;
    *bytes_out = layout_for(p->batch_size, p->head_num, 1).counter_bytes;
    return FLB_OK;
}

int flb_attn_workspace_bytes(const flb_attn_params *p, size_t *bytes_out) {
    if (!p || !bytes_out) return FLB_ERR_NULL_POINTER;
    if (p->batch_size <= 0 || p->head_num <= 0 || p->total_len <= 0 || p->seq_len <= 0) return FLB_ERR_BAD_SHAPE;
    if (p->split_len < 0 || (p->split_len % 32) != 0) return FLB_ERR_BAD_SHAPE;
    // worst case over every call these dimensions allow: a decode step on a full cache, or a
    // prefill of seq_len tokens
    const size_t dec = layout_for(p->batch_size, p->head_num, nsplit_for(p->total_len - 1, split_len_of(p)), p->size_per_head > 0 ? p->size_per_head : flb::kHeadDim).total;
    const size_t pre = p->seq_len > 1 ? flb::prefill_scratch_bytes(p->batch_size, p->head_num, p->seq_len, p->size_per_head > 0 ? p->size_per_head : flb::kHeadDim) : 0;
    *bytes_out = dec > pre ? dec : pre;
    return FLB_OK;
}

int flb_attn_decode(const flb_attn_params *p, void *cuda_stream) {
    if (p && p->seq_len != 1) return FLB_ERR_BAD_SHAPE;
    const int st = flb_attn_validate(p);
    if (st != FLB_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    const int split_len = split_len_of(p);
    const int nsplit_max = nsplit_for(max_past_of(p), split_len);
    const ScratchLayout l = layout_for(p->batch_size, p->head_num, nsplit_max, p->size_per_head);
    unsigned char *sc = static_cast<unsigned char *>(p->scratch);

    if (!p->scratch_zeroed) {
        if (cudaMemsetAsync(sc, 0, l.counter_bytes, stream) != cudaSuccess) return FLB_ERR_LAUNCH;
    }

    flb::DecodeArgs a;
    a.B = p->batch_size;
    a.H = p->head_num;
    a.T = p->total_len;
    a.start_pos = p->start_pos;
    a.past_lens = p->past_lens;
    a.nsplit_max = nsplit_max;
    a.split_len = split_len;
    a.input_mode = p->input_mode;
    a.q = p->q;
    a.k = p->k;
    a.v = p->v;
    a.row_stride = p->qkv_row_stride ? p->qkv_row_stride : p->head_num * p->size_per_head;
    a.act_scale = p->act_scale;
    a.q_w_scale = p->q_w_scale;
    a.k_w_scale = p->k_w_scale;
    a.v_w_scale = p->v_w_scale;
    a.freq_cis = p->freq_cis;
    a.rope_pos0 = p->rope_pos0;
    a.rope_add_past = p->rope_add_past;
    a.mask_mode = p->mask_mode;
    a.attn_mask = p->attn_mask;
    a.mask_row_stride = p->mask_row_stride;
    a.k_cache = p->k_cache;
    a.v_cache = p->v_cache;
    a.out = p->out;
    a.out_f16 = (p->out_dtype == FLB_F16);
    a.scale_log2e = p->softmax_scale * 1.4426950408889634f;
    a.status = reinterpret_cast<unsigned *>(sc);
    a.counters = reinterpret_cast<unsigned *>(sc) + flb::kStatusWords;
    a.row_counters = a.counters + (size_t)p->batch_size * p->head_num;
    a.out_q8 = p->out_q8;
    a.out_q8_scale = p->out_q8_scale;
    for (int i = 0; i < FLB_MAX_PEERS; ++i) a.out_peers[i] = (i < p->n_out_peers) ? p->out_peers[i] : nullptr;
    a.n_out_peers = p->n_out_peers;
    a.out_head_total = p->out_head_total;
    a.out_head_offset = p->out_head_offset;
    a.early_start = (p->scratch_zeroed != 0) ? p->early_start : 0;
    a.part_ml = reinterpret_cast<float *>(sc + l.ml_off);
    a.part_o = reinterpret_cast<float *>(sc + l.o_off);

    if (flb::launch_decode(a, p->cache_dtype == FLB_F16, p->size_per_head, stream) != cudaSuccess) return FLB_ERR_LAUNCH;
    return FLB_OK;
}

int flb_attn_prefill(const flb_attn_params *p, void *cuda_stream) {
    if (p && p->seq_len <= 1) return FLB_ERR_BAD_SHAPE;
    const int st = flb_attn_validate(p);
    if (st != FLB_OK) return st;
    return flb::launch_prefill(p, static_cast<cudaStream_t>(cuda_stream));
}

int flb_attn_forward(const flb_attn_params *p, void *cuda_stream) {
    if (!p) return FLB_ERR_NULL_POINTER;
    // same switch as open_decoder.cu:179 / :216
    return (p->seq_len > 1) ? flb_attn_prefill(p, cuda_stream) : flb_attn_decode(p, cuda_stream);
}

int flb_attn_quantize(const float *attn, int8_t *q8, float *scale, int batch_size, int head_num, int seq_len, int size_per_head,
                      void *cuda_stream) {
    if (!attn || !q8 || !scale) return FLB_ERR_NULL_POINTER;
    if (batch_size <= 0 || head_num <= 0 || seq_len <= 0) return FLB_ERR_BAD_SHAPE;
    if (size_per_head != 128 && size_per_head != 64) return FLB_ERR_UNSUPPORTED;
    if (batch_size > 65535) return FLB_ERR_TOO_LARGE; // grid.y
    return flb::launch_quantize(attn, q8, scale, batch_size, head_num, seq_len, size_per_head, static_cast<cudaStream_t>(cuda_stream));
}

int flb_attn_scratch_status(const void *scratch, unsigned *status_out, void *cuda_stream) {
    if (!scratch || !status_out) return FLB_ERR_NULL_POINTER;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    if (cudaMemcpyAsync(status_out, scratch, sizeof(unsigned), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
        return FLB_ERR_LAUNCH;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return FLB_ERR_LAUNCH;
    return FLB_OK;
}

} // extern "C"

// ---- mask classification ---------------------------------------------------------------------
namespace {

// maskbits bits: 1 = consistent with strict causal, 2 = with inclusive causal, 4 = all zero
__global__ void classify_mask_kernel(const float *__restrict__ mask, int rows, int stride, unsigned *maskbits) {
    unsigned bad = 0;
    const size_t n = (size_t)rows * rows;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(idx / rows), c = (int)(idx % rows);
        const float m = mask[(size_t)r * stride + c];
        const bool keep = (m == 0.0f), drop = (m <= -1e30f);
        if (!keep) bad |= 4u;
        // strict: keep iff c < r ; inclusive: keep iff c <= r
        if (!((c < r) ? keep : drop)) bad |= 1u;
        if (!((c <= r) ? keep : drop)) bad |= 2u;
    }
    if (bad) atomicAnd(maskbits, ~bad);
}

} // namespace

extern "C" int flb_attn_classify_mask(const float *attn_mask, int rows, int row_stride, void *scratch16, int *mode_out,
                                      void *cuda_stream) {
    if (!attn_mask || !mode_out || !scratch16) return FLB_ERR_NULL_POINTER;
    if (rows <= 0 || row_stride < rows) return FLB_ERR_BAD_SHAPE;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    unsigned *maskbits = static_cast<unsigned *>(scratch16);
    const unsigned all = 7u;
    if (cudaMemcpyAsync(maskbits, &all, sizeof(all), cudaMemcpyHostToDevice, stream) != cudaSuccess) return FLB_ERR_LAUNCH;
    const size_t n = (size_t)rows * rows;
    const int sms = flb::current_device_sm_count();
    if (sms <= 0) return FLB_ERR_DEVICE;
    const size_t cap = (size_t)sms * 8; // a grid-stride loop: eight blocks of 256 threads per SM fill the machine
    const unsigned blocks = (unsigned)((n + 255) / 256 < cap ? (n + 255) / 256 : cap);
    classify_mask_kernel<<<blocks, 256, 0, stream>>>(attn_mask, rows, row_stride, maskbits);
    if (cudaGetLastError() != cudaSuccess) return FLB_ERR_LAUNCH;
    unsigned v = 0;
    if (cudaMemcpyAsync(&v, maskbits, sizeof(v), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return FLB_ERR_LAUNCH;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return FLB_ERR_LAUNCH;
    if (v & 4u)
        *mode_out = FLB_MASK_NONE;
    else if (v & 1u)
        *mode_out = FLB_MASK_CAUSAL_STRICT;
    else if (v & 2u)
        *mode_out = FLB_MASK_CAUSAL_INCLUSIVE;
    else
        *mode_out = FLB_MASK_GENERIC;
    return FLB_OK;
}
