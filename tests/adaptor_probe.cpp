// adaptor_probe.cpp — exercises include/flb_open_decoder.h the way two OpenDecoder objects in one process would:
// two contexts, two different masks, two streams.  Prints one line per check; the test reads them.
// Built and run by tests/test_adaptor_ctx.py (needs a GPU).  TEST INFRASTRUCTURE.
#include <cuda_runtime.h>
#include <float.h>
#include <stdio.h>
#include <vector>

#include "flb_open_decoder.h"

static float *make_mask(int T, bool strict) {
    std::vector<float> h((size_t)T * T);
    for (int r = 0; r < T; ++r)
        for (int c = 0; c < T; ++c) h[(size_t)r * T + c] = (strict ? c < r : c <= r) ? 0.f : -FLT_MAX;
    float *d = nullptr;
    cudaMalloc(&d, h.size() * sizeof(float));
    cudaMemcpy(d, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice);
    return d;
}

int main() {
    const int B = 2, H = 4, d = 128, T = 96;
    float *strict = make_mask(T, true), *inclusive = make_mask(T, false);
    void *scratch_a = nullptr, *scratch_b = nullptr;
    cudaMalloc(&scratch_a, 1 << 20);
    cudaMalloc(&scratch_b, 1 << 20);
    cudaStream_t s1, s2;
    cudaStreamCreate(&s1);
    cudaStreamCreate(&s2);
    // nothing is launched below except the mask classification: fill_params only fills the block
    int32_t *qkv = nullptr;
    float *scale = nullptr, *cache = nullptr, *out = nullptr;
    cudaMalloc(&qkv, sizeof(int32_t) * B * H * d * 3);
    cudaMalloc(&scale, sizeof(float) * H * d);
    cudaMalloc(&cache, sizeof(float) * B * H * T * d);
    cudaMalloc(&out, sizeof(float) * B * H * d);

    flb_open_decoder_ctx a, b;
    flb_open_decoder_ctx_init(&a);
    flb_open_decoder_ctx_init(&b);
    flb_attn_params pa, pb2;
    auto fill = [&](flb_open_decoder_ctx *c, flb_attn_params *p, const float *mask, void *scratch, cudaStream_t st) {
        flb_open_decoder_fill_params(c, p, B, H, d, T, 1, 10, qkv, qkv + B * H * d, qkv + 2 * B * H * d, H * d, scale, scale, scale, scale,
                                     nullptr, mask, cache, cache, scratch, 1 << 20, out, nullptr, nullptr, st);
    };
    fill(&a, &pa, strict, scratch_a, s1);
    fill(&b, &pb2, inclusive, scratch_b, s1);
    printf("mask_a %d\n", pa.mask_mode);
    printf("mask_b %d\n", pb2.mask_mode);
    printf("first_call_zeroed_a %d early_a %d\n", pa.scratch_zeroed, pa.early_start);
    fill(&a, &pa, strict, scratch_a, s1); // same scratch, same stream: counters known to be zero
    printf("second_call_zeroed_a %d early_a %d\n", pa.scratch_zeroed, pa.early_start);
    fill(&a, &pa, strict, scratch_a, s2); // another stream: nothing is known about ordering, start over
    printf("other_stream_zeroed_a %d early_a %d\n", pa.scratch_zeroed, pa.early_start);
    fill(&a, &pa, inclusive, scratch_a, s2); // the caller changed its mask: classified again
    printf("mask_a_changed %d\n", pa.mask_mode);
    fill(&b, &pb2, inclusive, scratch_b, s1);
    printf("b_unaffected %d zeroed_b %d\n", pb2.mask_mode, pb2.scratch_zeroed);
    printf("row_stride %d validate %d\n", pa.qkv_row_stride, flb_attn_validate(&pa));
    cudaDeviceSynchronize();
    printf("cuda %d\n", (int)cudaGetLastError());
    return 0;
}
