// decode_attn.cuh — device-side argument block shared by the decode kernels and the launch layer.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace flb {

constexpr int kHeadDim = 128;          // size_per_head of the benchmarked models; the default where a call gives none
constexpr int kDefaultSplitLen = 512;  // cache rows per split-KV partition
constexpr int kShortSlabRows = 1024;   // slabs of at most this many rows ...
constexpr int kShortSlabSplitLen = 256; // ... are split into partitions of this many rows
constexpr int kStatusWords = 4;        // status header (16 B) in front of the arrival counters

// Error bits a kernel may set in the status word (scratch[0]).
enum : unsigned {
    kErrProducerWait = 1u,  // the copy-issuing warp gave up waiting for a free stage
    kErrConsumerWait = 2u,  // a compute warp gave up waiting for a stage to land
};

// SMs of the current device (0 when the query fails).  Grid sizes that must stay co-resident, or that are sized in
// waves, are computed from this and not from a constant.
inline int current_device_sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}

struct DecodeArgs {
    int B, H, T;
    int start_pos;
    const int *past_lens;
    int nsplit_max;  // grid holds nsplit_max CTAs per (b,h)
    int split_len;
    int input_mode;
    const void *q, *k, *v;
    int row_stride; // elements between two sequences' rows in q, k, v (H * d when they are dense)
    const float *act_scale, *q_w_scale, *k_w_scale, *v_w_scale;
    const float *freq_cis;
    int rope_pos0, rope_add_past;
    int mask_mode;
    const float *attn_mask;
    int mask_row_stride;
    void *k_cache, *v_cache;
    void *out;
    int out_f16;
    float scale_log2e;  // softmax_scale * log2(e)
    unsigned *status;   // [kStatusWords]
    unsigned *counters; // [B*H] arrivals per (b,h); zero on entry, zero on exit
    unsigned *row_counters; // [B] heads finished per sequence (fused quantisation); zero on entry and exit
    int8_t *out_q8;         // optional [B, H*d] int8 codes of the output row
    float *out_q8_scale;    // optional [B]
    // optional push of every finished row to n_out_peers buffers [B, out_head_total, d] (peer-mapped), at head
    // out_head_offset + h; 0 = store into `out` [B, H, d] only
    void *out_peers[8];
    int n_out_peers, out_head_total, out_head_offset;
    int early_start; // launched with programmatic stream serialisation: cache tiles may be fetched before the wait
    float *part_o;      // [B*H, nsplit_max, d]
    float *part_ml;     // [B*H, nsplit_max, 2]  (running max in the log2 domain, sum)
};

} // namespace flb
