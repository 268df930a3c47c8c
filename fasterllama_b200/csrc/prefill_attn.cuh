// prefill_attn.cuh — host-side interface of the causal prefill attention (seq_len > 1).
#pragma once
#include "../../include/flb_attn.h"
#include <cuda_runtime.h>
#include <stddef.h>

namespace flb {

// Scratch the prefill call needs: a 256-byte status header followed by fp16 staging copies of the
// rotated Q, K and V, each [B,H,S,d] (K and V copies are used only with an fp32 cache; with an
// fp16 cache the tensor-core kernel reads K/V straight from the cache rows it has just written).
inline size_t prefill_scratch_bytes(int B, int H, int S, int d) {
    const size_t one = (size_t)B * H * S * d * 2;
    return 256 + 3 * ((one + 255) / 256 * 256);
}

// Launches prologue + attention on `stream`; returns a flb_status.
int launch_prefill(const flb_attn_params *p, cudaStream_t stream);

// The reference's attention-output quantisation + transpose on a [B,H,S,d] fp32 tensor, d = 64 or 128 (one block per token row).
int launch_quantize(const float *attn, int8_t *q8, float *scale, int B, int H, int S, int d, cudaStream_t stream);

} // namespace flb
