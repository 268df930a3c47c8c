// decode_attn.cu — masked multi-head decode attention over the KV cache, one launch.
//
// Replaces, for seq_len == 1, the reference's chain
//   warpQKRoteEmbeddingTransposeKernel   fasterLlama/cuda/decoder_kernels.cu:425-464
//   warpDequantizedVTransposeKernel      fasterLlama/cuda/decoder_kernels.cu:858-884
//   storeKVcacheKernel                   fasterLlama/cuda/decoder_kernels.cu:597-611
//   cublasSgemvStridedBatched (K.q)      fasterLlama/cuda/open_decoder.cu:194-201
//   blockSoftmaxKernel                   fasterLlama/cuda/decoder_kernels.cu:800-835
//   cublasSgemvStridedBatched (P.V)      fasterLlama/cuda/open_decoder.cu:231-238
//
// Shape of the kernel (HBM-bound: 1 FMA per 2 cache bytes, so CUDA cores suffice):
//   * grid = (b,h) units x nsplit_max split-KV partitions of `split_len` cache rows; a CTA whose
//     partition lies beyond its sequence's length leaves at once.
//   * one producer warp streams the partition's K rows and V rows (each contiguous in the
//     [B,H,T,d] cache) into a STAGES-deep shared-memory ring with 1-D bulk copies (TMA engine)
//     that complete on mbarriers; NWARPS compute warps consume the ring.
//   * a cache row is d*sizeof(CacheT) bytes = LPR lanes x 16 B; a warp takes 32/LPR rows per
//     step, 16-byte shared loads, fp32 dot product, xor-shuffle reduction, and keeps its own
//     online-softmax state (running max in the log2 domain, sum, d-wide accumulator striped
//     over lanes).  Warps merge through shared memory in warp order.
//   * the new token: every CTA rotates q (RoPE) itself; the CTA that owns the last partition
//     also dequantises/rotates k, rounds k,v to the cache type, appends them at row `past` and
//     folds the new key/value into its partial result from registers, so no CTA ever reads a
//     row that another CTA writes in the same launch.
//   * split merge: partial (max, sum, acc[d]) go to scratch; the CTA that arrives last for a
//     (b,h) (one atomic counter, nobody waits) combines the partitions in partition order, so the
//     result is a function of (sequence length, split_len) only.
#include "decode_attn.cuh"
#include "flb_ptx.cuh"

#include <atomic>

namespace flb {

namespace {

constexpr float kLog2e = 1.4426950408889634f;
// blockSoftmaxKernel starts its running max at -1e9f (decoder_kernels.cu:811); same value in the
// log2 domain.  It keeps fully-masked rows finite: every exp underflows to 0 and the sum is 0.
constexpr float kMaxInit = -1e9f * kLog2e;

template <typename T> struct CacheIO;
template <> struct CacheIO<float> {
    static __device__ __forceinline__ float round(float x) { return x; }
    static __device__ __forceinline__ void store(float *p, float x) { *p = x; }
    // 16 bytes = 4 floats
    static __device__ __forceinline__ void unpack(const uint4 &u, float (&f)[4]) {
        f[0] = __uint_as_float(u.x);
        f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z);
        f[3] = __uint_as_float(u.w);
    }
};
template <> struct CacheIO<__half> {
    static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
    static __device__ __forceinline__ void store(__half *p, float x) { *p = __float2half_rn(x); }
    // 16 bytes = 8 halves
    static __device__ __forceinline__ void unpack(const uint4 &u, float (&f)[8]) {
        const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = __half22float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
};

// One element of q/k/v for sequence b, head h, dim i with seq_len == 1: [B,1,H,d] with row_stride elements
// between sequences (H*d when dense).
// FLB_IN_INT32: float(acc) * act_scale[b] * w_scale[h*d+i], in this order (decoder_kernels.cu:449).
template <int D>
__device__ __forceinline__ float load_input(const DecodeArgs &a, const void *base, const float *w_scale, int unit, int b,
                                            int h, int i) {
    const size_t off = (size_t)b * a.row_stride + (size_t)h * D + i;
    if (a.input_mode == 0) {
        const float acc = (float)__ldg((const int32_t *)base + off);
        return acc * __ldg(a.act_scale + b) * __ldg(w_scale + (size_t)h * D + i);
    } else if (a.input_mode == 1) {
        return __ldg((const float *)base + off);
    }
    return __half2float(((const __half *)base)[off]);
}

} // namespace

// One element of a finished output row: into `out` [B, H, d], or — head-split layer — into every rank's
// [B, out_head_total, d] buffer (plain stores; the remote ones travel over NVLink and are published by the
// exchange kernel that follows on the stream).
template <int D> __device__ __forceinline__ void store_out_element(const DecodeArgs &a, int unit, int col, float r) {
    if (a.n_out_peers == 0) {
        const size_t oo = (size_t)unit * D + col;
        if (a.out_f16)
            ((__half *)a.out)[oo] = __float2half_rn(r);
        else
            ((float *)a.out)[oo] = r;
        return;
    }
    const int b = unit / a.H, h = unit - b * a.H;
    const size_t oo = ((size_t)b * a.out_head_total + a.out_head_offset + h) * D + col;
    if (a.out_f16) {
        const __half hv = __float2half_rn(r);
        for (int p = 0; p < a.n_out_peers; ++p) ((__half *)a.out_peers[p])[oo] = hv;
    } else {
        for (int p = 0; p < a.n_out_peers; ++p) ((float *)a.out_peers[p])[oo] = r;
    }
}

// Fused form of the reference's launchAttnQuantizedTransposeKernel (decoder_kernels.cu:1179-1255) for
// seq_len == 1: called by every CTA that has just written a head's final output.  The one that is last
// for its sequence (an arrival counter per sequence; nobody waits) reads the whole [H, d] fp32 row back,
// takes absmax over all heads with the reference's -1e9f floor, writes absmax / 127 and the codes
// cvt.rni.sat.s8(x * 127.0f / absmax) as [H*d].  All threads of the CTA must call it.
template <int D, int NWARPS>
__device__ __forceinline__ void quantize_row_if_last(const DecodeArgs &a, int b, float *red, int *flag) {
    constexpr int NC = NWARPS * 32; // threads that take part in the row pass: thread t owns dims t, t + NC, ...
    const int tid = threadIdx.x;
    __syncthreads(); // the head's output stores precede the fence of thread 0
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(a.row_counters + b, 1u);
        *flag = (old == (unsigned)(a.H - 1));
    }
    __syncthreads();
    if (!*flag) return;
    __threadfence();
    const float *row = (const float *)a.out + (size_t)b * a.H * D;
    float amax = -1e9f;
    if (tid < NC)
        for (int i = tid; i < D; i += NC)
            for (int h = 0; h < a.H; ++h) amax = fmaxf(amax, fabsf(__ldcg(row + (size_t)h * D + i)));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (tid < NC && (tid & 31) == 0) red[tid >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int w = 1; w < NWARPS; ++w) amax = fmaxf(amax, red[w]);
    if (tid == 0) {
        a.out_q8_scale[b] = amax / 127.0f;
        a.row_counters[b] = 0u; // ready for the next call
    }
    if (tid < NC) {
        int8_t *dst = a.out_q8 + (size_t)b * a.H * D;
        for (int i = tid; i < D; i += NC)
            for (int h = 0; h < a.H; ++h) {
                const float x = __ldcg(row + (size_t)h * D + i) * 127.0f / amax;
                int q;
                asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(x));
                dst[(size_t)h * D + i] = (int8_t)q;
            }
    }
}

template <typename CacheT, int HD, int TILE_ROWS, int STAGES, int NWARPS>
__global__ void __launch_bounds__((NWARPS + 1) * 32) flb_decode_attn_kernel(const __grid_constant__ DecodeArgs a) {
    constexpr int D = HD;
    constexpr int ROW_BYTES = D * (int)sizeof(CacheT);
    constexpr int EPL = 16 / (int)sizeof(CacheT); // elements per 16-byte chunk
    constexpr int CHUNKS = D / EPL;               // chunks per cache row
    constexpr int LPR = CHUNKS < 32 ? CHUNKS : 32; // lanes per cache row
    constexpr int CPL = CHUNKS / LPR;             // chunks per lane: lane c owns chunks c, c + LPR, ...
    constexpr int RPI = 32 / LPR;                 // rows a warp takes per step
    constexpr int ITERS = TILE_ROWS / (NWARPS * RPI);
    constexpr int TILE_BYTES = TILE_ROWS * ROW_BYTES;
    constexpr int NC = NWARPS * 32;               // compute threads
    constexpr int DPT = (D + NC - 1) / NC;        // head dimensions per compute thread: t, t + NC, ...
    static_assert(ITERS * NWARPS * RPI == TILE_ROWS, "tile rows must divide over the compute warps");
    static_assert(LPR * CPL * EPL == D && LPR * RPI == 32, "a row must map onto whole lanes");
    static_assert((NC % 2) == 0, "RoPE pairs sit in neighbouring lanes");

    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + (size_t)STAGES * 2 * TILE_BYTES);
    uint64_t *empty = full + STAGES;
    float *q_s = reinterpret_cast<float *>(empty + STAGES); // [D] rotated q * scale * log2e
    float *wm = q_s + D;                                    // [NWARPS]
    float *wl = wm + NWARPS;                                // [NWARPS]
    float *wo = wl + NWARPS;                                // [NWARPS][D]
    float *red = wo + NWARPS * D;                           // [NWARPS]
    int *flag = reinterpret_cast<int *>(red + NWARPS);

    const int split = blockIdx.x % a.nsplit_max;
    const int unit = blockIdx.x / a.nsplit_max; // b*H + h
    const int b = unit / a.H, h = unit - b * a.H;
    int past = a.past_lens ? __ldg(a.past_lens + b) : a.start_pos;
    // a length outside [0, T-1] or beyond what the grid was sized for is flagged and clamped so
    // that no access leaves the slab
    const int past_cap = min(a.T - 1, a.nsplit_max * a.split_len);
    const bool bad_len = (past < 0 || past > past_cap); // reported by thread 0 once global writes are allowed
    past = max(0, min(past, past_cap));
    const int nsplit = max(1, (past + a.split_len - 1) / a.split_len);
    // Early start (programmatic dependent launch): the call that follows on the stream may begin as soon as
    // every CTA of this grid has got this far; until its own grid_dependency_wait() it only fetches cache rows
    // that are older than this call (and reads past_lens), which the caller has promised are settled.
    if (a.early_start) grid_launch_dependents();
    if (split >= nsplit) return;

    const int row0 = split * a.split_len;
    const int rows = max(0, min(a.split_len, past - row0));
    const int ntiles = (rows + TILE_ROWS - 1) / TILE_ROWS;
    const bool is_last = (split == nsplit - 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], NWARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();

    float vnew[DPT];     // compute thread t of the last partition: new v[t + NC e], rounded to the cache type
#pragma unroll
    for (int e = 0; e < DPT; ++e) vnew[e] = 0.0f;
    float s_new = 0.0f;  // score of the new key in the log2 domain
    bool new_visible = false;

    if (warp == NWARPS) {
        // ---------------- producer warp: one lane issues the bulk copies -------------------
        if (lane == 0) {
            const unsigned char *kb = (const unsigned char *)a.k_cache + ((size_t)unit * a.T + row0) * ROW_BYTES;
            const unsigned char *vb = (const unsigned char *)a.v_cache + ((size_t)unit * a.T + row0) * ROW_BYTES;
            for (int t = 0; t < ntiles; ++t) {
                const int s = t % STAGES;
                const uint32_t use = (uint32_t)(t / STAGES);
                // Level 1: the compute warps sit in griddepcontrol.wait until the kernel in front has completed and
                // free no stage before that, so once the ring is full this lane waits for the same event instead
                // of spending its bounded spin on a stage that cannot become free yet.
                if (a.early_start == 1 && t == STAGES) grid_dependency_wait();
                if (!mbar_wait(&empty[s], (use & 1u) ^ 1u)) {
                    atomicOr(a.status, kErrProducerWait);
                    break;
                }
                const int r = min(TILE_ROWS, rows - t * TILE_ROWS);
                const uint32_t bytes = (uint32_t)r * ROW_BYTES;
                mbar_arrive_expect_tx(&full[s], 2u * bytes);
                bulk_g2s(smem_raw + (size_t)s * 2 * TILE_BYTES, kb + (size_t)t * TILE_BYTES, bytes, &full[s]);
                bulk_g2s(smem_raw + (size_t)s * 2 * TILE_BYTES + TILE_BYTES, vb + (size_t)t * TILE_BYTES, bytes, &full[s]);
            }
        }
        __syncwarp();
    } else {
        // ---------------- compute warps ------------------------------------------------------
        const int tid = threadIdx.x; // < NC
        // Early start, level 1: q, k and v all come from the kernel in front -> wait before any of them is read.
        // Level 2: the caller has promised that q and k (with their scales) were final before that kernel started
        // (in the decoder layer it is the V projection, the Q and K projections ran before it), so the whole
        // streaming pass over the cache runs first and only the new token's v, the cache append and the
        // result/scratch writes wait (after the loop below).
        if (a.early_start == 1) grid_dependency_wait();
        float krot_keep[DPT]; // the new token's rotated k, appended to the cache after the streaming pass
        // -- the new token: dequantise, rotate (a2 of the reference); its v and the append (a3, a4) follow the loop
        {
            float part = 0.f;
#pragma unroll
            for (int e = 0; e < DPT; ++e) {
                const int i = tid + e * NC; // head dimension of this thread
                float qraw = 0.f, kraw = 0.f;
                if (i < D) {
                    qraw = load_input<D>(a, a.q, a.q_w_scale, unit, b, h, i);
                    if (is_last) kraw = load_input<D>(a, a.k, a.k_w_scale, unit, b, h, i);
                }
                float qrot = qraw, krot = kraw;
                if (a.freq_cis) {
                    // pairs (2i, 2i+1) sit in neighbouring lanes of one warp
                    const float qo = __shfl_xor_sync(0xffffffffu, qraw, 1);
                    const float ko = __shfl_xor_sync(0xffffffffu, kraw, 1);
                    if (i < D) {
                        const int row = a.rope_pos0 + (a.rope_add_past ? past : 0);
                        const float *fr = a.freq_cis + (size_t)row * D;
                        const float c = __ldg(fr + (i & ~1)), sn = __ldg(fr + (i | 1));
                        if (i & 1) {
                            qrot = qraw * c + qo * sn;
                            krot = kraw * c + ko * sn;
                        } else {
                            qrot = qraw * c - qo * sn;
                            krot = kraw * c - ko * sn;
                        }
                    }
                }
                krot_keep[e] = 0.f;
                if (i < D) {
                    const float qs = qrot * a.scale_log2e;
                    q_s[i] = qs;
                    if (is_last) {
                        const float kr = CacheIO<CacheT>::round(krot);
                        krot_keep[e] = krot;
                        part += qs * kr;
                    }
                }
            }
            if (is_last) {
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
                if (lane == 0) red[warp] = part;
            }
            named_bar_sync(1, NC);
            if (is_last) {
                float t = 0.f;
#pragma unroll
                for (int w = 0; w < NWARPS; ++w) t += red[w];
                s_new = t;
                switch (a.mask_mode) {
                case 1: // generic additive mask, row = query position, column = key position
                    s_new += __ldg(a.attn_mask + (size_t)past * a.mask_row_stride + past) * kLog2e;
                    new_visible = true;
                    break;
                case 3: // strictly causal: a token does not see itself
                    new_visible = false;
                    break;
                default:
                    new_visible = true;
                    break;
                }
            }
        }

        const int c = lane % LPR;   // first 16-byte chunk of the row this lane owns (then c + LPR, ...)
        const int sub = lane / LPR; // which of the RPI rows of a step
        float qreg[CPL][EPL];
#pragma unroll
        for (int k = 0; k < CPL; ++k)
#pragma unroll
            for (int j = 0; j < EPL; ++j) qreg[k][j] = q_s[(c + k * LPR) * EPL + j];

        float m_run = kMaxInit, l_run = 0.f;
        float o[CPL][EPL];
#pragma unroll
        for (int k = 0; k < CPL; ++k)
#pragma unroll
            for (int j = 0; j < EPL; ++j) o[k][j] = 0.f;

        const float *mask_row = (a.mask_mode == 1) ? a.attn_mask + (size_t)past * a.mask_row_stride + row0 : nullptr;

        bool ok = true;
        for (int t = 0; t < ntiles && ok; ++t) {
            const int s = t % STAGES;
            const uint32_t use = (uint32_t)(t / STAGES);
            if (!mbar_wait(&full[s], use & 1u)) {
                if (lane == 0) atomicOr(a.status, kErrConsumerWait);
                ok = false;
                break;
            }
            const CacheT *Kt = reinterpret_cast<const CacheT *>(smem_raw + (size_t)s * 2 * TILE_BYTES);
            const CacheT *Vt = reinterpret_cast<const CacheT *>(smem_raw + (size_t)s * 2 * TILE_BYTES + TILE_BYTES);
            const int rvalid = min(TILE_ROWS, rows - t * TILE_ROWS);

            float sc[ITERS];
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                const int r = (it * NWARPS + warp) * RPI + sub;
                float acc = 0.f;
#pragma unroll
                for (int k = 0; k < CPL; ++k) {
                    const uint4 kv = *reinterpret_cast<const uint4 *>(Kt + (size_t)r * D + (c + k * LPR) * EPL);
                    float kf[EPL];
                    CacheIO<CacheT>::unpack(kv, kf);
#pragma unroll
                    for (int j = 0; j < EPL; ++j) acc = fmaf(qreg[k][j], kf[j], acc);
                }
                sc[it] = acc;
            }
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
#pragma unroll
                for (int off = LPR / 2; off > 0; off >>= 1) sc[it] += __shfl_xor_sync(0xffffffffu, sc[it], off);
            }
            float mt = kMaxInit;
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                const int r = (it * NWARPS + warp) * RPI + sub;
                if (r >= rvalid) {
                    sc[it] = -INFINITY;
                } else if (mask_row) {
                    sc[it] += __ldg(mask_row + t * TILE_ROWS + r) * kLog2e;
                }
                mt = fmaxf(mt, sc[it]);
            }
#pragma unroll
            for (int off = 16; off >= LPR; off >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, off)); // the warp's RPI rows
            const float m_new = fmaxf(m_run, mt);
            const float corr = ex2(m_run - m_new);
            m_run = m_new;
            l_run *= corr;
#pragma unroll
            for (int k = 0; k < CPL; ++k)
#pragma unroll
                for (int j = 0; j < EPL; ++j) o[k][j] *= corr;
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                const int r = (it * NWARPS + warp) * RPI + sub;
                if (r < rvalid) {
                    const float p = ex2(sc[it] - m_new);
                    l_run += p;
#pragma unroll
                    for (int k = 0; k < CPL; ++k) {
                        const uint4 vv = *reinterpret_cast<const uint4 *>(Vt + (size_t)r * D + (c + k * LPR) * EPL);
                        float vf[EPL];
                        CacheIO<CacheT>::unpack(vv, vf);
#pragma unroll
                        for (int j = 0; j < EPL; ++j) o[k][j] = fmaf(p, vf[j], o[k][j]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }

        // -- from here on the kernel writes global memory and reads the new token's v: the kernel in front of
        //    this one must have completed (a no-op unless the launch was an early-start one)
        if (a.early_start == 2) grid_dependency_wait();
        if (bad_len && tid == 0 && split == 0) atomicOr(a.status, 4u);
        if (is_last) {
            // a3, a4 of the reference: dequantise v, round k and v to the cache type, append row `past`
#pragma unroll
            for (int e = 0; e < DPT; ++e) {
                const int i = tid + e * NC;
                if (i < D) {
                    const float vraw = load_input<D>(a, a.v, a.v_w_scale, unit, b, h, i);
                    vnew[e] = CacheIO<CacheT>::round(vraw);
                    const size_t cidx = ((size_t)unit * a.T + past) * D + i;
                    CacheIO<CacheT>::store((CacheT *)a.k_cache + cidx, krot_keep[e]);
                    CacheIO<CacheT>::store((CacheT *)a.v_cache + cidx, vraw);
                }
            }
        }

        // the warp's RPI rows of a step fold into one partial per chunk
#pragma unroll
        for (int off = 16; off >= LPR; off >>= 1) {
            l_run += __shfl_xor_sync(0xffffffffu, l_run, off);
#pragma unroll
            for (int k = 0; k < CPL; ++k)
#pragma unroll
                for (int j = 0; j < EPL; ++j) o[k][j] += __shfl_xor_sync(0xffffffffu, o[k][j], off);
        }
        if (sub == 0) {
#pragma unroll
            for (int k = 0; k < CPL; ++k)
#pragma unroll
                for (int j = 0; j < EPL; ++j) wo[warp * D + (c + k * LPR) * EPL + j] = o[k][j];
        }
        if (lane == 0) {
            wm[warp] = m_run;
            wl[warp] = l_run;
        }
    }
    __syncthreads();

    // ---------------- merge the compute warps (warp order), add the new token ----------------
    // compute thread t finishes head dimensions t, t + NC, ...
    const int tid = threadIdx.x;
    float acc[DPT], lsum = 0.f, M = kMaxInit;
#pragma unroll
    for (int e = 0; e < DPT; ++e) acc[e] = 0.f;
    if (tid < NC) {
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, wm[w]);
        if (is_last && new_visible) M = fmaxf(M, s_new);
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float e2 = ex2(wm[w] - M);
#pragma unroll
            for (int e = 0; e < DPT; ++e)
                if (tid + e * NC < D) acc[e] = fmaf(wo[w * D + tid + e * NC], e2, acc[e]);
            lsum = fmaf(wl[w], e2, lsum);
        }
        if (is_last && new_visible) {
            const float p = ex2(s_new - M);
#pragma unroll
            for (int e = 0; e < DPT; ++e) acc[e] = fmaf(p, vnew[e], acc[e]);
            lsum += p;
        }
    }

    if (nsplit == 1) {
        if (tid < NC) {
#pragma unroll
            for (int e = 0; e < DPT; ++e)
                if (tid + e * NC < D) store_out_element<D>(a, unit, tid + e * NC, (lsum > 0.f) ? acc[e] / lsum : 0.f);
        }
        if (a.out_q8) quantize_row_if_last<D, NWARPS>(a, b, red, flag);
        return;
    }

    // ---------------- split-KV: publish the partial, the last arriver merges ------------------
    const size_t pbase = (size_t)unit * a.nsplit_max;
    if (tid < NC) {
#pragma unroll
        for (int e = 0; e < DPT; ++e)
            if (tid + e * NC < D) a.part_o[(pbase + split) * D + tid + e * NC] = acc[e];
        if (tid == 0) {
            a.part_ml[(pbase + split) * 2 + 0] = M;
            a.part_ml[(pbase + split) * 2 + 1] = lsum;
        }
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence(); // cumulative: orders the whole CTA's partial (made visible to this thread by the barrier)
        const unsigned old = atomicAdd(a.counters + unit, 1u);
        *flag = (old == (unsigned)(nsplit - 1));
    }
    __syncthreads();
    if (!*flag) return;
    __threadfence();
    if (tid < NC) {
        float M2 = kMaxInit;
        for (int i = 0; i < nsplit; ++i) M2 = fmaxf(M2, __ldcg(a.part_ml + (pbase + i) * 2));
        float acc2[DPT], l2 = 0.f;
#pragma unroll
        for (int e = 0; e < DPT; ++e) acc2[e] = 0.f;
        for (int i = 0; i < nsplit; ++i) {
            const float e2 = ex2(__ldcg(a.part_ml + (pbase + i) * 2) - M2);
#pragma unroll
            for (int e = 0; e < DPT; ++e)
                if (tid + e * NC < D) acc2[e] = fmaf(__ldcg(a.part_o + (pbase + i) * D + tid + e * NC), e2, acc2[e]);
            l2 = fmaf(__ldcg(a.part_ml + (pbase + i) * 2 + 1), e2, l2);
        }
#pragma unroll
        for (int e = 0; e < DPT; ++e)
            if (tid + e * NC < D) store_out_element<D>(a, unit, tid + e * NC, (l2 > 0.f) ? acc2[e] / l2 : 0.f);
        if (tid == 0) a.counters[unit] = 0u; // ready for the next call
    }
    if (a.out_q8) quantize_row_if_last<D, NWARPS>(a, b, red, flag);
}

// ---- host-side launcher ------------------------------------------------------------------

template <typename CacheT, int HD, int TILE_ROWS, int STAGES, int NWARPS>
static cudaError_t launch_decode_t(const DecodeArgs &a, cudaStream_t stream) {
    constexpr int TILE_BYTES = TILE_ROWS * HD * (int)sizeof(CacheT);
    constexpr size_t smem = (size_t)STAGES * 2 * TILE_BYTES + 2 * STAGES * sizeof(uint64_t) +
                            sizeof(float) * (HD + 2 * NWARPS + NWARPS * HD + NWARPS) + 16;
    auto kern = flb_decode_attn_kernel<CacheT, HD, TILE_ROWS, STAGES, NWARPS>;
    // the shared-memory opt-in is a property of (kernel, device): set once per device, not on every call (it costs about
    // a microsecond of host time, which an isolated call sees in full)
    static std::atomic<unsigned long long> opted_in{0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const unsigned long long bit = (dev >= 0 && dev < 64) ? (1ull << dev) : 0ull;
    if (!(opted_in.load(std::memory_order_acquire) & bit)) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (bit) opted_in.fetch_or(bit, std::memory_order_release);
    }
    const unsigned grid = (unsigned)a.B * (unsigned)a.H * (unsigned)a.nsplit_max;
    if (!a.early_start) {
        kern<<<grid, (NWARPS + 1) * 32, smem, stream>>>(a);
        return cudaGetLastError();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((NWARPS + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, a);
}

cudaError_t launch_decode(const DecodeArgs &a, bool cache_f16, int head_dim, cudaStream_t stream) {
    // Two stages of 8 KB K + 8 KB V tiles (32 rows of 128 halves, 16 rows of 128 floats, ...) = 32 KB of ring per
    // CTA, so that 6 CTAs share an SM: measured on B200 at head size 128, many small rings beat few deep ones
    // (each CTA's prologue and merge overlap the other CTAs' streaming); deeper rings (4, 6 stages) lost 15-40 %
    // of the bandwidth.  The other head sizes the reference's kernels accept up to 256
    // (decoder_kernels.cu:563-589) keep the tile's byte size.
    if (cache_f16) {
        if (head_dim == 64) return launch_decode_t<__half, 64, 64, 2, 4>(a, stream);
        if (head_dim == 256) return launch_decode_t<__half, 256, 16, 2, 4>(a, stream);
        return launch_decode_t<__half, 128, 32, 2, 4>(a, stream);
    }
    if (head_dim == 64) return launch_decode_t<float, 64, 32, 2, 4>(a, stream);
    if (head_dim == 256) return launch_decode_t<float, 256, 8, 2, 4>(a, stream);
    return launch_decode_t<float, 128, 16, 2, 4>(a, stream);
}

} // namespace flb
