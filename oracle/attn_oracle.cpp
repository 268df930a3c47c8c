// attn_oracle.cpp — scalar host restatement of the reference's attention math.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA path: tests, the smoke
// check and the CPU-baseline leg of the benchmark may call it; the product never does.
//
// PARITY PIN.  The reference ships no golden vectors, known-answer tests or fixtures for this
// path (its samples only print), so this restatement is pinned the other way round: the
// reference's own CUDA kernels + cuBLAS calls are compiled from the reference's sources
// (oracle/build_ref.sh -> oracle/_ref/libflb_ref.so), run on a B200 on seeded inputs, and
// their outputs are committed under tests/golden/ (tests/golden/make_ref_golden.py); the CPU
// test-suite checks this oracle against those vectors.
//
// Every function names the reference lines whose arithmetic it restates.  All pointers are
// HOST pointers.  Layout names: B batch, S tokens in this call, H heads, d size_per_head,
// T cache row capacity, L keys attended.
//
// Build: g++ -O2 -std=c++17 -fopenmp -shared -fPIC attn_oracle.cpp -o libflb_oracle.so

#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../include/flb_attn.h"

namespace {

inline float half_round(float x) { return (float)(_Float16)x; }

struct HalfBits {
    static float to_float(uint16_t h) {
        _Float16 f;
        std::memcpy(&f, &h, 2);
        return (float)f;
    }
    static uint16_t from_float(float x) {
        _Float16 f = (_Float16)x;
        uint16_t h;
        std::memcpy(&h, &f, 2);
        return h;
    }
};

// value of element i of token (b,s), head h, of a q/k/v input in any input mode.
// FLB_IN_INT32 restates the dequantisation of decoder_kernels.cu:449-452 and :875-878:
// float(acc) * inp_scale * weight_scale, multiplied left to right in fp32.
inline float load_in(const flb_attn_params *p, const void *base, const float *w_scale, int b, int s,
                     int h, int i) {
    const int S = p->seq_len, H = p->head_num, d = p->size_per_head;
    const size_t row = p->qkv_row_stride ? (size_t)p->qkv_row_stride : (size_t)H * d; // elements between token rows
    const size_t off = ((size_t)b * S + s) * row + (size_t)h * d + i;
    switch (p->input_mode) {
    case FLB_IN_INT32: {
        const float acc = (float)((const int32_t *)base)[off];
        const float a = p->act_scale[(size_t)b * S + s];
        return acc * a * w_scale[(size_t)h * d + i];
    }
    case FLB_IN_F32:
        return ((const float *)base)[off];
    default:
        return HalfBits::to_float(((const uint16_t *)base)[off]);
    }
}

inline int past_of(const flb_attn_params *p, int b) { return p->past_lens ? p->past_lens[b] : p->start_pos; }

} // namespace

extern "C" {

// ---- building blocks, one per reference kernel ------------------------------------------

// Interleaved-pair RoPE on one head vector, in place.
// Restates decoder_kernels.cu:455-458: x' = x*cos - y*sin ; y' = y*cos + x*sin with
// cos = row[2i], sin = row[2i+1], for the pairs (2i, 2i+1).
void orc_rope_row(float *x, const float *freq_row, int d) {
    for (int i = 0; i < d; i += 2) {
        const float c = freq_row[i], s = freq_row[i + 1];
        const float a = x[i], b = x[i + 1];
        x[i] = a * c - b * s;
        x[i + 1] = b * c + a * s;
    }
}

// RoPE table as the reference defines it (decoding_kernels.cu:85-114): row pos, entry 2i = cos,
// 2i+1 = sin of pos * base^(-2i/d).  The reference evaluates this with fast GPU intrinsics; the
// oracle and the CUDA path both take the table as INPUT, so this double-precision version is
// only a generator of test inputs.
void orc_freq_cis(float *table, int rows, int d, double base) {
    for (int r = 0; r < rows; ++r)
        for (int i = 0; i < d; i += 2) {
            const double theta = (double)r * std::pow(base, -(double)i / (double)d);
            table[(size_t)r * d + i] = (float)std::cos(theta);
            table[(size_t)r * d + i + 1] = (float)std::sin(theta);
        }
}

// Row softmax exactly as blockSoftmaxKernel does it (decoder_kernels.cu:800-835):
// v = qk*scaler + mask ; max starts at -1e9f ; e = expf(v - max) ; e / sum.
// `mask_row` may be NULL (the kernel then adds 0, :814).  A zero sum gives NaN there (0/0);
// here the row is returned as zeros and *fully_masked is set.
void orc_softmax_row(float *qk, const float *mask_row, int n, float scaler, int *fully_masked) {
    float mx = -1e9f;
    for (int i = 0; i < n; ++i) {
        const float v = qk[i] * scaler + (mask_row ? mask_row[i] : 0.0f);
        qk[i] = v;
        mx = std::fmax(mx, v);
    }
    double sum = 0.0;
    for (int i = 0; i < n; ++i) {
        const float e = std::exp(qk[i] - mx);
        qk[i] = e;
        sum += (double)e;
    }
    if (fully_masked) *fully_masked = (sum == 0.0);
    if (sum == 0.0) {
        for (int i = 0; i < n; ++i) qk[i] = 0.0f;
        return;
    }
    const float fs = (float)sum;
    for (int i = 0; i < n; ++i) qk[i] = qk[i] / fs;
}

// ---- the whole path -----------------------------------------------------------------------

// Runs the attention section of OpenDecoder::forward (open_decoder.cu:138-239) on the host for
// the parameter block `p` (all pointers host memory):
//   1. dequantise q,k,v and rotate q,k          decoder_kernels.cu:425-464, :858-884
//   2. append k,v to the caches at row past+s   decoder_kernels.cu:597-611
//   3. scores = q . K^T (the contraction open_decoder.cu:181-201 intends; the decode call as
//      written has its m/n exchanged and is only right when L == d)
//   4. softmax(scores*scale + mask)             decoder_kernels.cu:800-835
//   5. out = P . V                              open_decoder.cu:218-238
// Decode (S == 1) attends over cache rows [0, past] (the new row included, subject to the mask);
// prefill (S > 1) attends over the fresh rows only, like the reference, and needs past == 0.
// With an fp16 cache the appended rows are rounded to half first and the rounded values are the
// ones attended over, so that this step and later steps see the same K/V.
// `flags` bit 0: accumulate the two contractions in double (the arbiter); clear = fp32 left-to-right
// sums.  Bit 1: round the prefill operands q, k, v to fp16 before the contractions — the
// reference's prefill GEMMs run fp16 tensor-core math on fp32 storage (CUBLAS_COMPUTE_32F_FAST_16F,
// fasterLlama/cuda/common.h:71), so this is the operand precision of its own prefill; decode
// (cublasSgemv, true fp32) ignores the bit.  The cache always receives the unrounded values.
// Returns 0, or a negative flb_status.
int orc_attention(const flb_attn_params *p, int flags) {
    const int acc_double = flags & 1;
    const bool f16_operands = (flags & 2) != 0 && p->seq_len > 1;
    const int B = p->batch_size, H = p->head_num, d = p->size_per_head, S = p->seq_len, T = p->total_len;
    if (B <= 0 || H <= 0 || d <= 0 || (d & 1) || S <= 0 || T <= 0) return FLB_ERR_BAD_SHAPE;
    if (!p->q || !p->k || !p->v || !p->k_cache || !p->v_cache || !p->out) return FLB_ERR_NULL_POINTER;
    if (S > 1 && (p->past_lens || p->start_pos != 0)) return FLB_ERR_UNSUPPORTED;
    const bool cache16 = p->cache_dtype == FLB_F16;
    const bool out16 = p->out_dtype == FLB_F16;
    int status = 0;

#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < H; ++h) {
            const int past = past_of(p, b);
            if (past < 0 || past + S > T) {
                status = FLB_ERR_BAD_SHAPE;
                continue;
            }
            const int L = past + S;
            std::vector<float> qv((size_t)S * d), kf((size_t)S * d), vf((size_t)S * d);
            // 1. dequant + RoPE
            for (int s = 0; s < S; ++s) {
                for (int i = 0; i < d; ++i) {
                    qv[(size_t)s * d + i] = load_in(p, p->q, p->q_w_scale, b, s, h, i);
                    kf[(size_t)s * d + i] = load_in(p, p->k, p->k_w_scale, b, s, h, i);
                    vf[(size_t)s * d + i] = load_in(p, p->v, p->v_w_scale, b, s, h, i);
                }
                if (p->freq_cis) {
                    const int row = p->rope_pos0 + s + (p->rope_add_past ? past : 0);
                    orc_rope_row(&qv[(size_t)s * d], p->freq_cis + (size_t)row * d, d);
                    orc_rope_row(&kf[(size_t)s * d], p->freq_cis + (size_t)row * d, d);
                }
                if (cache16)
                    for (int i = 0; i < d; ++i) {
                        kf[(size_t)s * d + i] = half_round(kf[(size_t)s * d + i]);
                        vf[(size_t)s * d + i] = half_round(vf[(size_t)s * d + i]);
                    }
            }
            // 2. cache append
            const size_t slab = ((size_t)b * H + h) * (size_t)T * d;
            for (int s = 0; s < S; ++s)
                for (int i = 0; i < d; ++i) {
                    const size_t c = slab + (size_t)(past + s) * d + i;
                    if (cache16) {
                        ((uint16_t *)p->k_cache)[c] = HalfBits::from_float(kf[(size_t)s * d + i]);
                        ((uint16_t *)p->v_cache)[c] = HalfBits::from_float(vf[(size_t)s * d + i]);
                    } else {
                        ((float *)p->k_cache)[c] = kf[(size_t)s * d + i];
                        ((float *)p->v_cache)[c] = vf[(size_t)s * d + i];
                    }
                }
            // keys/values attended over: rows [0, L) of the slab (prefill: past == 0, so these are
            // exactly the fresh rows).
            auto Kat = [&](int r, int i) -> float {
                const size_t c = slab + (size_t)r * d + i;
                const float x = cache16 ? HalfBits::to_float(((const uint16_t *)p->k_cache)[c]) : ((const float *)p->k_cache)[c];
                return f16_operands ? half_round(x) : x;
            };
            auto Vat = [&](int r, int i) -> float {
                const size_t c = slab + (size_t)r * d + i;
                const float x = cache16 ? HalfBits::to_float(((const uint16_t *)p->v_cache)[c]) : ((const float *)p->v_cache)[c];
                return f16_operands ? half_round(x) : x;
            };
            if (f16_operands)
                for (size_t i = 0; i < qv.size(); ++i) qv[i] = half_round(qv[i]);
            std::vector<float> sc(L), mrow(L);
            for (int s = 0; s < S; ++s) {
                const int qpos = past + s;
                // 3. scores
                for (int r = 0; r < L; ++r) {
                    if (acc_double) {
                        double a = 0.0;
                        for (int i = 0; i < d; ++i) a += (double)qv[(size_t)s * d + i] * (double)Kat(r, i);
                        sc[r] = (float)a;
                    } else {
                        float a = 0.0f;
                        for (int i = 0; i < d; ++i) a += qv[(size_t)s * d + i] * Kat(r, i);
                        sc[r] = a;
                    }
                }
                // 4. mask row + softmax
                const float *mptr = nullptr;
                switch (p->mask_mode) {
                case FLB_MASK_GENERIC:
                    mptr = p->attn_mask + (size_t)qpos * p->mask_row_stride;
                    break;
                case FLB_MASK_CAUSAL_INCLUSIVE:
                    for (int r = 0; r < L; ++r) mrow[r] = (r <= qpos) ? 0.0f : -FLT_MAX;
                    mptr = mrow.data();
                    break;
                case FLB_MASK_CAUSAL_STRICT:
                    for (int r = 0; r < L; ++r) mrow[r] = (r < qpos) ? 0.0f : -FLT_MAX;
                    mptr = mrow.data();
                    break;
                default:
                    break;
                }
                orc_softmax_row(sc.data(), mptr, L, p->softmax_scale, nullptr);
                // 5. P.V
                for (int i = 0; i < d; ++i) {
                    float o;
                    if (acc_double) {
                        double a = 0.0;
                        for (int r = 0; r < L; ++r) a += (double)sc[r] * (double)Vat(r, i);
                        o = (float)a;
                    } else {
                        float a = 0.0f;
                        for (int r = 0; r < L; ++r) a += sc[r] * Vat(r, i);
                        o = a;
                    }
                    const size_t oo = (((size_t)b * H + h) * S + s) * d + i;
                    if (out16)
                        ((uint16_t *)p->out)[oo] = HalfBits::from_float(o);
                    else
                        ((float *)p->out)[oo] = o;
                }
            }
        }
    return status;
}

// The step after attention: per token row, absmax over all heads, scale and int8 codes, transposed.
// Restates warpAttnQuantizedTransposeKernel / blockAttnQuantizedTransposeKernel
// (decoder_kernels.cu:1179-1255): absmax starts at -1e9f and ignores NaN (fmaxf), scale = absmax / 127,
// code = round-to-nearest-even, saturated to [-128, 127], of x * 127.0f / absmax (cvt.rni.sat.s8.f32,
// cuda_kernels.cuh:34-41; a NaN input converts to 0).  attn [B,H,S,d] fp32 -> q8 [B,S,H*d], scale [B*S].
void orc_attn_quantize(const float *attn, int8_t *q8, float *scale, int B, int H, int S, int d) {
    for (int b = 0; b < B; ++b)
        for (int s = 0; s < S; ++s) {
            float amax = -1e9f;
            for (int h = 0; h < H; ++h)
                for (int i = 0; i < d; ++i) amax = std::fmax(amax, std::fabs(attn[(((size_t)b * H + h) * S + s) * d + i]));
            scale[(size_t)b * S + s] = amax / 127.0f;
            for (int h = 0; h < H; ++h)
                for (int i = 0; i < d; ++i) {
                    const float x = attn[(((size_t)b * H + h) * S + s) * d + i] * 127.0f / amax;
                    float r = std::nearbyint(x); // default rounding mode: to nearest, ties to even
                    int q = std::isnan(r) ? 0 : (r > 127.f ? 127 : (r < -128.f ? -128 : (int)r));
                    q8[(((size_t)b * S + s) * H + h) * d + i] = (int8_t)q;
                }
        }
}

// Thread control for the timed CPU baseline; returns the thread count that will be used.
int orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

int orc_hw_threads(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}

} // extern "C"
