// prefill_attn.cu — causal prefill attention (seq_len > 1, empty cache) for sm_100a.
//
// Replaces, for seq_len > 1, the reference's chain
//   warpQKRoteEmbeddingTransposeKernel   fasterLlama/cuda/decoder_kernels.cu:425-464
//   warpDequantizedVTransposeKernel      fasterLlama/cuda/decoder_kernels.cu:858-884
//   storeKVcacheKernel                   fasterLlama/cuda/decoder_kernels.cu:597-611
//   cublasGemmStridedBatchedEx (Q.K^T)   fasterLlama/cuda/open_decoder.cu:181-190
//   blockSoftmaxKernel                   fasterLlama/cuda/decoder_kernels.cu:800-835
//   cublasGemmStridedBatchedEx (P.V)     fasterLlama/cuda/open_decoder.cu:218-227
// with two launches:
//
// 1. flb_prefill_prologue_kernel — one streaming pass: dequantise q,k,v, rotate q,k (RoPE),
//    transpose [B,S,H,d] -> [B,H,S,d], append k,v to the caches (rows 0..S-1) and leave fp16
//    copies of Q (and of K,V when the cache is fp32) for the tensor cores.
//
// 2. flb_prefill_attn_kernel — flash attention on the 5th-generation tensor cores, one persistent CTA of 16
//    warps per SM.  A work item is 256 query rows of one (b,h) (two 128-row query tiles); items are handed out through
//    an atomic counter, heavy (late) query blocks first, in groups of heads whose K/V stay in L2.  Key tiles hold 64
//    keys.  TMEM (512 columns): per query tile two score buffers of 64 columns (fp32 scores; P overwrites them as
//    fp16 pairs) and one column of fp32 accumulator O per head dimension (128 or 64).  Warp roles:
//      warp 0      work scheduler + K/V loader: TMA boxes (128-byte swizzle) into a ring of K tiles and a ring of V
//                  tiles (64 keys each); the tensor maps carry the 64-dim block of a row as a dimension of its own,
//                  so one instruction brings a whole tile (a single issuing thread pays 100-250 cycles per TMA
//                  instruction).  A K tile goes back to the loader when both query tiles' S over it have
//                  landed, a V tile when both query tiles' P.V over it have retired: K is needed two tiles earlier
//                  than V and is free two tiles earlier, so two rings do in 96-128 KB what one ring needed 160 KB for.
//                  With fp16 inputs and an fp16 cache the V tiles come straight from the caller's v (a rank-5 tensor
//                  map over its [B,S,H,d] rows) and the loader stores them into the cache from the ring (TMA store,
//                  two loader steps after the load, never waited for): the streaming pass in front then moves q and k only
//      warps 1, 3  issue S = Q_t.K_j^T for query tile 0 / 1 (SS form: both operands in shared memory, 128 x 64 x 16
//                  per instruction) and load that tile's query rows.  S runs TWO key tiles ahead of P.V: while
//                  the softmax threads work on S_j, S_{j+1} is already in TMEM, so they never wait for the pipe;
//                  S_{j+2} overwrites the buffer P_j occupied and is issued once P_j.V_j has retired
//      warp 2      issues every O_t += P_j.V_j (P read from TMEM as the A operand, V from shared memory as an
//                  MN-major B operand).  tcgen05.mma is issued by single threads, and one thread cannot issue, wait
//                  and commit fast enough for the pipe: three do it.  The tile stream runs across work items
//                  (the next item's first two S are issued while the current item's last products retire).
//      warps 4-7   softmax of query tile 0, one thread per row: load the 64 scores of a key tile, maximum,
//      warps 8-11  P = 2^(x - m) and the row sum, P stored over the scores, buffer handed to warp 2; O is rescaled
//      (tile 1)    only when a row's maximum grew by more than 2^8 (exact: the final division uses the same
//                  reference maximum).  Masked tiles are first brought into the unmasked form, so that the
//                  arithmetic exists once: the kernel's instruction footprint is a first-order cost here
//      warps 12-15 epilogue: O_t / l from TMEM to global memory while the other warps are on the next item
//    All hand-offs are mbarriers (TMA transaction counts, tcgen05.commit, thread arrivals); every
//    wait is bounded by a wall-clock budget and reports through the status word instead of hanging.
//    Causal modes skip the key tiles above the diagonal.  No multicast, no cluster: the same code runs in the
//    head-split layer on several GPUs.
#include "prefill_attn.cuh"

#include "decode_attn.cuh"

#include "flb_ptx.cuh"

#include <cuda_fp16.h>

#include <atomic>

namespace flb {

namespace {

// The head size is a template parameter (128, or 64): a tile is made of [rows x 64 dims] blocks in the 128-byte-swizzled
// operand layout, one block per 64 head dimensions.
constexpr int BM = 128;      // query rows per tile (two tiles per work item)
constexpr int BN = 64;       // keys per K/V tile
constexpr int HALF_BYTES = BM * 64 * 2;    // one [128 x 64] block of a query tile: 16 KB
constexpr int KV_HALF_BYTES = BN * 64 * 2; // one [64 x 64] block of a K or V tile: 8 KB
constexpr int tile_bytes(int d) { return BM * d * 2; }    // query tile: 128 rows of fp16 (32 KB at d = 128)
constexpr int kv_tile_bytes(int d) { return BN * d * 2; } // K or V tile: 64 keys (16 KB at d = 128)
#ifndef FLB_PF_K_STAGES
#define FLB_PF_K_STAGES 4
#endif
#ifndef FLB_PF_V_STAGES
#define FLB_PF_V_STAGES 4
#endif
#ifndef FLB_PF_EMUL
#define FLB_PF_EMUL 0
#endif
// Two rings of 64-key tiles.  A K tile is needed two tiles earlier than the V tile of the same keys (S runs two tiles
// ahead of P.V) and is free again as soon as both query tiles' S over it have landed; a V tile is free once both query
// tiles' P.V over it have retired.  Three stages each already match one ring of five K+V stages; four each leave room for
// the V tiles' way into the cache (below) and for the longer latency of V tiles read from the caller's strided rows.
constexpr int K_STAGES = FLB_PF_K_STAGES;
constexpr int V_STAGES = FLB_PF_V_STAGES;
constexpr int kExpOnFmaEvery = FLB_PF_EMUL; // every n-th exponential of a row on the FMA pipe (0 = none)
constexpr int NUM_THREADS = 512;          // warps: 0 scheduler + K/V loads, 1 and 3 S issue + Q loads, 2 P.V issue, 4-11 softmax, 12-15 epilogue
constexpr uint32_t TMEM_COLS = 512;       // per query tile: two score buffers of 64 columns + 128 columns of O
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f; // log2 domain: P stays below 2^8, exact in fp16 range
constexpr int kWorkCounterWord = 4;       // word of the status header the work scheduler counts in (cleared by the prologue)

enum : unsigned { kErrPrefillWait = 8u, kErrPrefillAlign = 16u };

struct PrefillArgs {
    int B, H, S, T;
    int input_mode;
    const void *q, *k, *v;
    int row_stride; // elements between two tokens' rows in q, k, v (H * d when they are dense)
    const float *act_scale, *q_w_scale, *k_w_scale, *v_w_scale;
    const float *freq_cis;
    int rope_pos0;
    void *k_cache, *v_cache;
    int cache_f16;
    __half *qh, *kh, *vh; // fp16 staging [B,H,S,d]; kh/vh only with an fp32 cache
    int mask_mode;
    const float *attn_mask;
    int mask_row_stride;
    void *out;
    int out_f16;
    float scale_log2e;
    unsigned *status;
    int heads_per_group; // work list: groups of this many (b,h) units, heavy query blocks first inside a group
    int v_direct; // fp16 v into an fp16 cache: nothing to convert, so the attention kernel takes the V tiles straight from the
                  // caller's v and stores them into the cache itself; the streaming pass leaves v alone
};

// ------------------------------------------------------------------------------------------------
// prologue
// ------------------------------------------------------------------------------------------------
// Raw 8-element load (no use of the data: the conversion comes after every load of the thread has
// been issued).  MODE: 0 = int32 accumulators, 1 = fp32, 2 = fp16.
struct Raw8 {
    uint4 lo, hi; // fp16 uses lo only
};
template <int MODE> __device__ __forceinline__ Raw8 load_raw8(const void *base, size_t off) {
    Raw8 r;
    if (MODE == 2) {
        r.lo = __ldg(reinterpret_cast<const uint4 *>((const __half *)base + off));
        r.hi = make_uint4(0, 0, 0, 0);
    } else {
        const uint4 *p = reinterpret_cast<const uint4 *>((const uint32_t *)base + off);
        r.lo = __ldg(p);
        r.hi = __ldg(p + 1);
    }
    return r;
}
template <int MODE>
__device__ __forceinline__ void convert8(const Raw8 &r, float as, const float4 &w0, const float4 &w1, float (&x)[8]) {
    if (MODE == 0) {
        // float(acc) * act_scale * w_scale, in this order (decoder_kernels.cu:449, :875)
        x[0] = (float)(int)r.lo.x * as * w0.x;
        x[1] = (float)(int)r.lo.y * as * w0.y;
        x[2] = (float)(int)r.lo.z * as * w0.z;
        x[3] = (float)(int)r.lo.w * as * w0.w;
        x[4] = (float)(int)r.hi.x * as * w1.x;
        x[5] = (float)(int)r.hi.y * as * w1.y;
        x[6] = (float)(int)r.hi.z * as * w1.z;
        x[7] = (float)(int)r.hi.w * as * w1.w;
    } else if (MODE == 1) {
        x[0] = __uint_as_float(r.lo.x); x[1] = __uint_as_float(r.lo.y); x[2] = __uint_as_float(r.lo.z); x[3] = __uint_as_float(r.lo.w);
        x[4] = __uint_as_float(r.hi.x); x[5] = __uint_as_float(r.hi.y); x[6] = __uint_as_float(r.hi.z); x[7] = __uint_as_float(r.hi.w);
    } else {
        const __half2 *hp = reinterpret_cast<const __half2 *>(&r.lo);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = __half22float2(hp[i]);
            x[2 * i] = t.x;
            x[2 * i + 1] = t.y;
        }
    }
}

__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
    uint4 u;
    __half2 *hp = reinterpret_cast<__half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) hp[i] = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
    return u;
}

__device__ __forceinline__ void store_cache8(const PrefillArgs &a, void *cache, size_t off, const float (&x)[8]) {
    if (a.cache_f16) {
        *reinterpret_cast<uint4 *>((__half *)cache + off) = pack8(x);
    } else {
        float4 *p = reinterpret_cast<float4 *>((float *)cache + off);
        p[0] = make_float4(x[0], x[1], x[2], x[3]);
        p[1] = make_float4(x[4], x[5], x[6], x[7]);
    }
}

// Each thread takes 8 consecutive head dimensions of kRowsPerThread tokens of one (b, h); a block of
// 256 threads covers 16 * kRowsPerThread consecutive tokens: it reads 256-byte segments (token stride
// H*d) and writes 4 KB runs into each of the [B,H,*,d] destinations.  All loads of a thread are
// issued before the first use, so that enough bytes are in flight to cover the DRAM latency.
constexpr int kRowsPerThread = 2;

__device__ __forceinline__ void rope8(const float4 &f0, const float4 &f1, float (&x)[8]) {
    // pairs (2i, 2i+1): x' = x cos - y sin ; y' = y cos + x sin (decoder_kernels.cu:455-458)
    const float cs[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        const float co = cs[i], sn = cs[i + 1];
        const float a0 = x[i], a1 = x[i + 1];
        x[i] = a0 * co - a1 * sn;
        x[i + 1] = a1 * co + a0 * sn;
    }
}

template <int MODE, int HD> __global__ void __launch_bounds__(256) flb_prefill_prologue_kernel(const PrefillArgs a) {
    constexpr int R = kRowsPerThread;
    constexpr int D = HD;
    constexpr int TPR = D / 8;    // threads per token row
    constexpr int RPP = 256 / TPR; // token rows a block covers per pass
    const int sblocks = (a.S + RPP * R - 1) / (RPP * R);
    const int c = threadIdx.x % TPR;
    const int s0 = (int)(blockIdx.x % sblocks) * (RPP * R) + (threadIdx.x / TPR);
    const int h = (int)((blockIdx.x / sblocks) % a.H);
    const int b = (int)(blockIdx.x / ((size_t)sblocks * a.H));
    Raw8 rq[R], rk[R], rv[R];
    float4 f0[R], f1[R];
    float as[R];
    // lets the attention kernel behind it (launched with programmatic stream serialisation) become resident and
    // set itself up while this kernel drains
    grid_launch_dependents();
    if (blockIdx.x == 0 && threadIdx.x < 8) a.status[threadIdx.x] = 0u; // the call's error word and the work counter start clean
    // ---- every load first
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int s = min(s0 + RPP * r, a.S - 1); // rows past the end load a valid row and are not stored
        const size_t in_off = ((size_t)b * a.S + s) * a.row_stride + (size_t)h * D + c * 8;
        rq[r] = load_raw8<MODE>(a.q, in_off);
        rk[r] = load_raw8<MODE>(a.k, in_off);
        if (!(MODE == 2 && a.v_direct)) rv[r] = load_raw8<MODE>(a.v, in_off);
        as[r] = (MODE == 0) ? __ldg(a.act_scale + (size_t)b * a.S + s) : 1.0f;
        if (a.freq_cis) {
            const float4 *fr = reinterpret_cast<const float4 *>(a.freq_cis + (size_t)(a.rope_pos0 + s) * D + c * 8);
            f0[r] = __ldg(fr);
            f1[r] = __ldg(fr + 1);
        }
    }
    float4 wq0, wq1, wk0, wk1, wv0, wv1;
    wq0 = wq1 = wk0 = wk1 = wv0 = wv1 = make_float4(1.f, 1.f, 1.f, 1.f);
    if (MODE == 0) {
        const size_t wo = (size_t)h * D + c * 8;
        wq0 = __ldg(reinterpret_cast<const float4 *>(a.q_w_scale + wo));
        wq1 = __ldg(reinterpret_cast<const float4 *>(a.q_w_scale + wo) + 1);
        wk0 = __ldg(reinterpret_cast<const float4 *>(a.k_w_scale + wo));
        wk1 = __ldg(reinterpret_cast<const float4 *>(a.k_w_scale + wo) + 1);
        wv0 = __ldg(reinterpret_cast<const float4 *>(a.v_w_scale + wo));
        wv1 = __ldg(reinterpret_cast<const float4 *>(a.v_w_scale + wo) + 1);
    }
    // ---- then convert, rotate, store
    const size_t bh = (size_t)b * a.H + h;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int s = s0 + RPP * r;
        if (s < a.S) {
            float q[8], k[8], v[8];
            convert8<MODE>(rq[r], as[r], wq0, wq1, q);
            convert8<MODE>(rk[r], as[r], wk0, wk1, k);
            if (!(MODE == 2 && a.v_direct)) convert8<MODE>(rv[r], as[r], wv0, wv1, v);
            if (a.freq_cis) {
                rope8(f0[r], f1[r], q);
                rope8(f0[r], f1[r], k);
            }
            const size_t st_off = (bh * a.S + s) * D + c * 8; // [B,H,S,d]
            const size_t ca_off = (bh * a.T + s) * D + c * 8; // [B,H,T,d]
            *reinterpret_cast<uint4 *>(a.qh + st_off) = pack8(q);
            store_cache8(a, a.k_cache, ca_off, k);
            if (!(MODE == 2 && a.v_direct)) store_cache8(a, a.v_cache, ca_off, v);
            if (!a.cache_f16) {
                *reinterpret_cast<uint4 *>(a.kh + st_off) = pack8(k);
                *reinterpret_cast<uint4 *>(a.vh + st_off) = pack8(v);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// attention
// ------------------------------------------------------------------------------------------------
constexpr int SCHED_DEPTH = 4;        // work items the scheduler may publish ahead
constexpr int kSchedConsumers = 15;   // two S issuers, the P.V issuer, 8 softmax warps, 4 epilogue warps
constexpr size_t kGroupBytes = 64u << 20; // work list: groups of (b,h) units whose K and V rows stay in L2 while the group is worked on

struct __align__(8) PrefillBarriers {
    uint64_t q_full[2], q_empty[2];   // per query tile of the item
    uint64_t k_full[K_STAGES], k_empty[K_STAGES]; // K tile landed / S of both query tiles over it has landed (2 arrivals)
    uint64_t v_full[V_STAGES], v_empty[V_STAGES]; // V tile landed / P.V of both query tiles over it has retired
    uint64_t s_full[2][2];            // [t][buffer] S = Q_t.K_j^T landed in score buffer j & 1 of query tile t
    uint64_t p_full[2][2];            // [t][buffer] P_j written over the scores by the 128 softmax threads of query tile t
    uint64_t pv_done[2][2];           // [t][buffer] O_t += P_j.V_j retired: score buffer j & 1 may take S_{j+2}
    uint64_t o_full[2], o_empty[2];   // last P.V of an item retired / the epilogue has read O_t out of TMEM
    uint64_t l_full[2], l_empty[2];   // row sums of an item in shared memory / read by the epilogue
    uint64_t sched_full[SCHED_DEPTH], sched_empty[SCHED_DEPTH];
    int sched_bh[SCHED_DEPTH], sched_qb[SCHED_DEPTH]; // the published items; bh < 0 = no more work
    int v_store_bh[V_STAGES], v_store_j[V_STAGES];    // loader's notes: the V tile in stage s still has to go into the cache (bh < 0: not)
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int kBarrierSlot = 512;
constexpr size_t prefill_smem(int d) {
    return 2 * (size_t)tile_bytes(d) + (size_t)(K_STAGES + V_STAGES) * kv_tile_bytes(d) + 2 * BM * sizeof(float) + kBarrierSlot;
}
static_assert(sizeof(PrefillBarriers) <= kBarrierSlot, "barrier block must fit its slot");
static_assert(prefill_smem(128) <= 232448, "exceeds the 227 KB a CTA may use");

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait (0.2 s of wall clock).  On failure raises the CTA's abort flag and the status bit.  The slow part is
// kept out of line: the common case (the phase has completed, or completes within one try_wait, which itself
// suspends the thread for a while) is two instructions at the call site.
__device__ __noinline__ bool wait_bar_slow(uint64_t *bar, uint32_t parity, PrefillBarriers *pb, unsigned *status) {
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0) {
            if (*reinterpret_cast<volatile int *>(&pb->abort_flag)) return false;
            if (globaltimer_ns() - t0 > 200000000ull) break;
        }
    }
    *reinterpret_cast<volatile int *>(&pb->abort_flag) = 1;
    atomicOr(status, kErrPrefillWait);
    return false;
}
__device__ __forceinline__ bool wait_bar(uint64_t *bar, uint32_t parity, PrefillBarriers *pb, unsigned *status) {
    if (mbar_try_wait(bar, parity)) return true;
    return wait_bar_slow(bar, parity, pb, status);
}


// A work item is 256 query rows of one (b,h): two 128-row tiles, each with its own S/P and O columns in TMEM.
struct ItemGeom {
    int q0[2];   // first query row of tile t
    int n[2];    // key tiles query tile t attends over (n[0] <= n[1])
    int nmax;
};
__device__ __forceinline__ ItemGeom item_geom(int qb, int S, bool causal) {
    ItemGeom g;
    const int n_all = (S + BN - 1) / BN;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        g.q0[t] = qb * (2 * BM) + t * BM;
        // causal modes skip the key tiles above the diagonal: query tile t ends at row q0 + 127.  A query tile that
        // lies beyond the prompt (the second tile of a ragged last block) is worked on like any other: its rows are
        // zero-filled by the loads and never stored, and every role keeps the same step pattern for every item.
        g.n[t] = causal ? min(n_all, (g.q0[t] + BM - 1) / BN + 1) : n_all;
    }
    g.nmax = max(g.n[0], g.n[1]);
    return g;
}

// Next published item for a consumer role (`count` = items this role has taken so far).  Single-thread roles
// release the slot themselves; warp roles read on every lane and let lane 0 release after a __syncwarp().
__device__ __forceinline__ bool sched_read(PrefillBarriers *pb, unsigned *status, uint32_t count, int &bh, int &qb) {
    const uint32_t slot = count % SCHED_DEPTH;
    if (!wait_bar(&pb->sched_full[slot], (count / SCHED_DEPTH) & 1u, pb, status)) return false;
    bh = *reinterpret_cast<volatile int *>(&pb->sched_bh[slot]);
    qb = *reinterpret_cast<volatile int *>(&pb->sched_qb[slot]);
    return true;
}
__device__ __forceinline__ void sched_release(PrefillBarriers *pb, uint32_t count) { mbar_arrive(&pb->sched_empty[count % SCHED_DEPTH]); }

// Softmax arithmetic on 32 scores of one query row held in registers.  A tile that needs masking is brought into the
// common form first (mask_chunk: the scaled score plus the mask value, or -inf, written back over the raw score, and
// the scale set to 1), so that the maximum and the exponentials exist once in the kernel: what the sixteen warps'
// different roles execute has to fit the SM's instruction cache together (measured: the same kernel with each masked
// form expanded separately, 83 KB of code instead of 52 KB, ran 12 % slower).
// GENERIC: the caller's additive mask row; otherwise keys [0, lim) are visible (causal diagonal / end of the prompt).
template <bool GENERIC> __device__ __forceinline__ void mask_chunk(uint32_t (&r)[32], int base, int lim, float scale, const float *mrow) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        float x = -INFINITY;
        if (base + i < lim) x = GENERIC ? fmaf(__ldg(mrow + base + i), kLog2e, __uint_as_float(r[i]) * scale) : __uint_as_float(r[i]) * scale;
        r[i] = __float_as_uint(x);
    }
}
__device__ __forceinline__ float chunk_max(const uint32_t (&r)[32], float m) {
#pragma unroll
    for (int i = 0; i < 32; i += 2) m = max3(m, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
    return m;
}
// P = 2^(x * scale - m) as fp16 pairs, row sum.  EMUL > 0: every EMUL-th exponential on the FMA pipe instead of the
// special-function unit.
template <int EMUL>
__device__ __forceinline__ void chunk_exp(const uint32_t (&r)[32], float scale, float neg_m, float2 &l2, uint32_t (&packed)[16]) {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        const float2 y = __ffma2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), make_float2(scale, scale),
                                    make_float2(neg_m, neg_m));
        constexpr int E = EMUL > 0 ? EMUL : 1;
        float2 p;
        p.x = (EMUL > 0 && (i % E) == E - 1) ? ex2_fma(y.x) : ex2(y.x);
        p.y = (EMUL > 0 && ((i + 1) % E) == E - 1) ? ex2_fma(y.y) : ex2(y.y);
        l2 = __fadd2_rn(l2, p);
        const __half2 h2 = __floats2half2_rn(p.x, p.y);
        packed[i >> 1] = *reinterpret_cast<const uint32_t *>(&h2);
    }
}

// GENERIC_MASK: the caller's additive mask is read (mask_mode GENERIC); OUT_F16: the output element type.  Compile-time so
// that each form carries only its own code: what the sixteen warps execute has to share the instruction cache.
template <int EMUL, bool GENERIC_MASK, bool OUT_F16, int HD>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    flb_prefill_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmVin, const PrefillArgs a,
                            const int num_items) {
    // The 128-byte swizzle pattern is a function of address bits [4,10): tiles must start on 1 KB.
    constexpr int D = HD;
    constexpr int TILE_BYTES = BM * D * 2;
    constexpr int KV_TILE_BYTES = BN * D * 2;
    static_assert(D == 64 || D == 128, "O_t takes D TMEM columns per query tile beside the 256 columns of scores");
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char *sQ = smem;                                  // two query tiles
    unsigned char *sK = sQ + 2 * TILE_BYTES;                   // K ring
    unsigned char *sV = sK + K_STAGES * KV_TILE_BYTES;         // V ring
    float *l_buf = reinterpret_cast<float *>(sV + V_STAGES * KV_TILE_BYTES); // [2][128] row sums of the item being finished
    PrefillBarriers *pb = reinterpret_cast<PrefillBarriers *>(l_buf + 2 * BM);
    if (smem_u32(smem) & 1023u) { // never observed; without it the MMAs would read scrambled tiles
        grid_dependency_wait();
        if (threadIdx.x == 0) atomicOr(a.status, kErrPrefillAlign);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool causal = (a.mask_mode == 2 || a.mask_mode == 3);
    const int nqb = (a.S + 2 * BM - 1) / (2 * BM); // 256-row query blocks per (b,h)

    if (threadIdx.x == 0) {
        for (int t = 0; t < 2; ++t) {
            mbar_init(&pb->q_full[t], 1);
            mbar_init(&pb->q_empty[t], 1);
            mbar_init(&pb->s_full[t][0], 1);
            mbar_init(&pb->s_full[t][1], 1);
            mbar_init(&pb->p_full[t][0], BM);
            mbar_init(&pb->p_full[t][1], BM);
            mbar_init(&pb->pv_done[t][0], 1);
            mbar_init(&pb->pv_done[t][1], 1);
            mbar_init(&pb->o_full[t], 1);
            mbar_init(&pb->o_empty[t], BM);
            mbar_init(&pb->l_full[t], BM);
            mbar_init(&pb->l_empty[t], BM);
        }
        for (int s = 0; s < K_STAGES; ++s) {
            mbar_init(&pb->k_full[s], 1);
            mbar_init(&pb->k_empty[s], 2); // per query tile: its softmax warps once S has landed, or its S issuer for a tile it skips
        }
        for (int s = 0; s < V_STAGES; ++s) {
            mbar_init(&pb->v_full[s], 1);
            mbar_init(&pb->v_empty[s], 1); // the P.V issuer: both query tiles' products over it have retired
        }
        for (int s = 0; s < SCHED_DEPTH; ++s) {
            mbar_init(&pb->sched_full[s], 1);
            mbar_init(&pb->sched_empty[s], kSchedConsumers);
        }
        pb->abort_flag = 0;
        for (int s = 0; s < V_STAGES; ++s) pb->v_store_bh[s] = -1;
        mbar_fence_init();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        if (a.v_direct) tma_prefetch_desc(&tmVin);
    }
    if (warp == 1) {
        tmem_alloc(&pb->tmem_base, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Programmatic dependent launch: everything above ran while the prologue kernel was draining; its output (the
    // staged Q, the cache rows, the cleared status words and work counter) is touched only from here on.  The
    // kernel behind this one is let go only after that wait, so "the kernel in front of it has completed" keeps
    // meaning "everything before that has completed as well".
    grid_dependency_wait();
    grid_launch_dependents();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(&pb->tmem_base);
    // TMEM columns: query tile t has its two score buffers at 128 t and 128 t + 64, its accumulator O_t at 256 + 128 t
    const uint32_t tO[2] = {tmem + 256u, tmem + 256u + (uint32_t)D};

    if (warp == 0) {
        // ======================= work scheduler + K/V loader =======================
        if (lane == 0) {
            unsigned *counter = a.status + kWorkCounterWord;
            const int BH = a.B * a.H;
            const int hpg = a.heads_per_group;
            const int per_group = hpg * nqb, full_groups = BH / hpg;
            uint32_t published = 0, kt = 0;
            bool ok = true;
            // item k of the list -> (b,h) unit and query block: groups of 32 units (their K/V stay in L2 while the
            // group is worked on), late = heavy query blocks first inside a group
            auto decode = [&](int k, int &bh, int &qb) {
                if (k < 0) { bh = -1; qb = 0; return; }
                const int g = k / per_group;
                if (g < full_groups) {
                    const int r = k - g * per_group;
                    qb = nqb - 1 - r / hpg;
                    bh = g * hpg + r % hpg;
                } else {
                    const int rem = BH - full_groups * hpg, r = k - full_groups * per_group;
                    qb = nqb - 1 - r / rem;
                    bh = full_groups * hpg + r % rem;
                }
            };
            auto publish = [&](int k) -> bool {
                const uint32_t slot = published % SCHED_DEPTH;
                if (!wait_bar(&pb->sched_empty[slot], ((published / SCHED_DEPTH) & 1u) ^ 1u, pb, a.status)) return false;
                int bh, qb;
                decode(k, bh, qb);
                pb->sched_bh[slot] = bh;
                pb->sched_qb[slot] = qb;
                mbar_arrive(&pb->sched_full[slot]); // release: the two words above are visible to whoever sees the phase
                ++published;
                return true;
            };
            // the first gridDim.x items are taken by block index (no round trip before the first load); the rest
            // through the counter, which the prologue kernel left at zero
            auto fetch = [&]() -> int {
                const unsigned k = gridDim.x + atomicAdd(counter, 1u);
                return k < (unsigned)num_items ? (int)k : -1;
            };
            // V tiles that come straight from the caller's v (fp16 into an fp16 cache) also have to be appended to the cache:
            // the item that covers every key tile of its unit (the last query block) sends each of its V tiles on with a
            // TMA store out of the stage.  The store of tile n is issued two loader steps after its load (it has landed by
            // then: the wait returns at once) and every step closes a bulk group, so that "at most the two newest groups
            // still read shared memory" covers the stage that is about to be overwritten (tile n - 4) without the loader
            // ever standing still for a store (measured: waiting for the store right before the reload cost the loader
            // 1100 cycles per key tile against 490 without a store, and the kernel 11 us at batch 8 x 1024 tokens).
            auto store_tile = [&](uint32_t st) -> bool {
                const uint32_t ss = st % V_STAGES;
                const int sbh = pb->v_store_bh[ss];
                if (sbh < 0) return true;
                if (!wait_bar(&pb->v_full[ss], (st / V_STAGES) & 1u, pb, a.status)) return false;
                const int sj = pb->v_store_j[ss];
                unsigned char *dv = sV + ss * KV_TILE_BYTES;
                tma_store_4d(&tmV, dv, 0, sj * BN, 0, sbh);
                pb->v_store_bh[ss] = -1;
                return true;
            };
            // The V tile of a key tile is wanted two tiles later than its K tile, so the loader issues it one step late:
            // K_j, then V_{j-1} (across items as well).  Whatever the V stage costs on its way to reuse — the wait for
            // both P.V products, the store into the cache — then never sits in front of a K load.
            int late_bh = -1, late_j = 0;
            bool late_keeper = false;
            uint32_t vt = 0;
            auto load_v_late = [&]() -> bool {
                if (late_bh < 0) return true;
                const uint32_t vs = vt % V_STAGES;
                if (a.v_direct) {
                    if (vt >= 2 && !store_tile(vt - 2)) return false;
                    bulk_commit_group();
                    bulk_wait_group_read<2>();
                }
                if (!wait_bar(&pb->v_empty[vs], ((vt / V_STAGES) & 1u) ^ 1u, pb, a.status)) return false;
                unsigned char *dv = sV + vs * KV_TILE_BYTES;
                if (a.v_direct) {
                    if (late_keeper) {
                        pb->v_store_bh[vs] = late_bh;
                        pb->v_store_j[vs] = late_j;
                    }
                    const int b = late_bh / a.H, h = late_bh - b * a.H;
                    mbar_arrive_expect_tx(&pb->v_full[vs], KV_TILE_BYTES);
                    tma_load_5d(dv, &tmVin, 0, late_j * BN, 0, h, b, &pb->v_full[vs]);
                } else {
                    mbar_arrive_expect_tx(&pb->v_full[vs], KV_TILE_BYTES);
                    tma_load_4d(dv, &tmV, 0, late_j * BN, 0, late_bh, &pb->v_full[vs]);
                }
                ++vt;
                late_bh = -1;
                return true;
            };
            auto load_k = [&](int bh, int j, bool keeper) -> bool {
                const uint32_t ks = kt % K_STAGES;
                if (!wait_bar(&pb->k_empty[ks], ((kt / K_STAGES) & 1u) ^ 1u, pb, a.status)) return false;
                unsigned char *dk = sK + ks * KV_TILE_BYTES;
                mbar_arrive_expect_tx(&pb->k_full[ks], KV_TILE_BYTES);
                tma_load_4d(dk, &tmK, 0, j * BN, 0, bh, &pb->k_full[ks]);
                ++kt;
                if (!load_v_late()) return false;
                late_bh = bh;
                late_j = j;
                late_keeper = keeper;
                return true;
            };
            int cur = (int)blockIdx.x; // < num_items: the grid never exceeds the item count
            ok = publish(cur);
            while (cur >= 0 && ok) {
                const int nxt = fetch(); // in flight while the first tile of `cur` is issued
                int bh, qb;
                decode(cur, bh, qb);
                const ItemGeom g = item_geom(qb, a.S, causal);
                const bool keeper = (qb == nqb - 1); // its query rows see every key tile of the unit
                ok = load_k(bh, 0, keeper);
                if (ok) ok = publish(nxt); // one item of look-ahead for the other roles
                for (int j = 1; j < g.nmax && ok; ++j) ok = load_k(bh, j, keeper);
                cur = nxt;
            }
            if (ok) ok = load_v_late(); // the last V tile
            if (a.v_direct) {
                // the last two tiles, and everything sent has to have arrived before the kernel ends
                for (uint32_t st = vt >= 2 ? vt - 2 : 0; st < vt && ok; ++st) ok = store_tile(st);
                bulk_commit_group();
                bulk_wait_group_all();
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 3) {
        // ======================= S issuers: warp 1 for query tile 0, warp 3 for query tile 1 =======================
        // tcgen05.mma is issued by single threads, and one thread cannot issue (and wait, and commit) fast enough for the
        // pipe: three do it.  These two issue S = Q_t.K_j^T, each for its query tile, and load that tile's query rows;
        // warp 2 issues every P.V.  A query tile has two score buffers, and its S runs two key tiles ahead of its P.V:
        // while the softmax threads work on S_j, S_{j+1} is already in TMEM and P_{j-1}.V_{j-1} is running, so the
        // softmax warps never wait for the tensor pipe.  S_{j+2} overwrites score buffer j & 1, which P_j occupied: it is
        // issued once P_j.V_j has retired (pv_done).  The stream of key tiles runs across work items.  Every descriptor is
        // a constant plus a start address computed once: the loop is a few dozen instructions.
        if (lane == 0) {
            const int t = warp >> 1;
            // A (Q) and B (K) both K-major, 128-byte swizzle, 8-row groups 1024 B apart
            constexpr uint32_t idesc_qk = umma_idesc_f16(BM, BN, false, false);
            const uint32_t tS_t = tmem + (uint32_t)(t * 128);
            // descriptor start addresses count 16-byte units
            const uint64_t dq0 = umma_desc_sw128(smem_u32(sQ) + t * TILE_BYTES, 16, 1024);
            const uint64_t dk0 = umma_desc_sw128(smem_u32(sK), 16, 1024);
            uint64_t *const q_full = &pb->q_full[t], *const q_empty = &pb->q_empty[t], *const s_full = &pb->s_full[t][0],
                            *const pv_done = &pb->pv_done[t][0];
            unsigned char *const sQ_t = sQ + t * TILE_BYTES;
            uint32_t taken = 0, kt = 0, gs = 0, nq = 0; // items read, ring tiles passed, S issued, query tiles loaded
            int nmax = 0, n_t = 0, j = 0;
            bool ok = true, valid = true;
            while (ok && valid) {
                if (j == nmax) {
                    // ---- next work item: its query rows go into the tile's buffer as soon as the previous item's
                    // last S has retired.  The two key tiles of lead hide the load's latency from the softmax warps.
                    int bh, qb;
                    ok = sched_read(pb, a.status, taken, bh, qb);
                    if (!ok) break;
                    sched_release(pb, taken++);
                    valid = bh >= 0;
                    if (!valid) break;
                    const ItemGeom g = item_geom(qb, a.S, causal);
                    nmax = g.nmax;
                    n_t = t ? g.n[1] : g.n[0];
                    j = 0;
                    if (nq > 0) {
                        ok = wait_bar(q_empty, (nq - 1u) & 1u, pb, a.status);
                        if (!ok) break;
                    }
                    mbar_arrive_expect_tx(q_full, TILE_BYTES);
                    tma_load_4d(sQ_t, &tmQ, 0, t ? g.q0[1] : g.q0[0], 0, bh, q_full);
                    ++nq;
                    continue;
                }
                const uint32_t ks = kt % K_STAGES;
                ok = wait_bar(&pb->k_full[ks], (kt / K_STAGES) & 1u, pb, a.status);
                if (!ok) break;
                ++kt;
                if (j >= n_t) { // above this query tile's diagonal: nothing of this tile is read on its behalf
                    mbar_arrive(&pb->k_empty[ks]);
                    ++j;
                    continue;
                }
                if (j == 0) ok = wait_bar(q_full, (nq - 1u) & 1u, pb, a.status);
                const uint32_t buf = gs & 1u;
                if (ok && gs >= 2) ok = wait_bar(pv_done + buf, ((gs - 2u) >> 1) & 1u, pb, a.status); // P_{j-2}.V_{j-2} has read this buffer
                if (!ok) break;
                tc_fence_after();
                const uint64_t dk = dk0 + (uint64_t)(ks * (uint32_t)(KV_TILE_BYTES >> 4));
                const uint32_t ts = tS_t + buf * (uint32_t)BN;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) { // dims 16 kk .. 16 kk + 15
                    const uint32_t oq = (uint32_t)((kk >> 2) * (HALF_BYTES >> 4) + (kk & 3) * 2);
                    const uint32_t okk = (uint32_t)((kk >> 2) * (KV_HALF_BYTES >> 4) + (kk & 3) * 2);
                    umma_f16_ss(ts, dq0 + oq, dk + okk, idesc_qk, kk > 0 ? 1u : 0u);
                }
                umma_commit(s_full + buf);
                if (j == n_t - 1) umma_commit(q_empty); // the query tile's buffer may take the next item's rows
                ++gs;
                ++j;
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        // ======================= P.V issuer (both query tiles) =======================
        // O_t (+)= P_j.V_j for t = 0, 1 over every ring tile: P read from TMEM as the A operand (fp16 pairs in the
        // columns S came from), V from shared memory as an MN-major B operand (the two 64-dim blocks KV_HALF_BYTES
        // apart (LBO), 8-key groups 1024 B apart (SBO)).  The V stage goes back to the loader when both have retired.
        if (lane == 0) {
            constexpr uint32_t idesc_pv = umma_idesc_f16(BM, D, false, true);
            const uint64_t dv0 = umma_desc_sw128(smem_u32(sV), KV_HALF_BYTES, 1024);
            uint32_t taken = 0, vt = 0, gp[2] = {0, 0}, ci[2] = {0, 0};
            int nmax = 0, n[2] = {0, 0}, j = 0;
            bool ok = true;
            for (;;) {
                if (j == nmax) {
                    int bh, qb;
                    ok = sched_read(pb, a.status, taken, bh, qb);
                    if (!ok) break;
                    sched_release(pb, taken++);
                    if (bh < 0) break;
                    const ItemGeom g = item_geom(qb, a.S, causal);
                    nmax = g.nmax;
                    n[0] = g.n[0];
                    n[1] = g.n[1];
                    j = 0;
                    continue;
                }
                const uint32_t vs = vt % V_STAGES;
                ok = wait_bar(&pb->v_full[vs], (vt / V_STAGES) & 1u, pb, a.status);
                if (!ok) break;
                const uint64_t dv = dv0 + (uint64_t)(vs * (uint32_t)(KV_TILE_BYTES >> 4));
                ++vt;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (j >= n[t] || !ok) continue; // above this query tile's diagonal
                    if (j == 0) { // the epilogue has read the previous item's O_t
                        ok = wait_bar(&pb->o_empty[t], (ci[t] & 1u) ^ 1u, pb, a.status);
                        if (!ok) continue;
                    }
                    const uint32_t buf = gp[t] & 1u;
                    ok = wait_bar(&pb->p_full[t][buf], (gp[t] >> 1) & 1u, pb, a.status);
                    if (!ok) continue;
                    tc_fence_after();
                    const uint32_t tp = tmem + (uint32_t)(t * 128) + buf * (uint32_t)BN;
#pragma unroll
                    for (int kk = 0; kk < BN / 16; ++kk) // 16 keys = 2048 bytes of the tile per step
                        umma_f16_ts(tO[t], tp + kk * 8, dv + (uint32_t)(kk * (2048 >> 4)), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(&pb->pv_done[t][buf]);
                    if (j == n[t] - 1) {
                        umma_commit(&pb->o_full[t]);
                        ++ci[t];
                    }
                    ++gp[t];
                }
                if (!ok) break;
                umma_commit(&pb->v_empty[vs]);
                ++j;
            }
        }
        __syncwarp();
    } else if (warp < 12) {
        // ======================= softmax: warps 4-7 query tile 0, warps 8-11 query tile 1 =======================
        const int t = (warp - 4) >> 2;
        const int quarter = warp & 3;                  // TMEM lane quarter this warp may access
        const int lrow = quarter * 32 + lane;          // query row inside the tile
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint32_t tS_t = tmem + (uint32_t)(t * 128), tO_t = tmem + 256u + (uint32_t)(t * D);
        uint64_t *const s_full = &pb->s_full[t][0], *const pv_done = &pb->pv_done[t][0], *const l_full = &pb->l_full[t],
                        *const l_empty = &pb->l_empty[t], *const p_full = &pb->p_full[t][0];
        uint32_t taken = 0, ct = 0, ci = 0, kbase = 0; // kbase: K-ring tiles of the items before this one
        const bool k_releaser = (quarter == 0 && lane == 0); // one thread per query tile hands K tiles back to the loader
        bool ok = true;
        for (;;) {
            int bh, qb;
            ok = sched_read(pb, a.status, taken, bh, qb);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            __syncwarp();
            if (lane == 0) sched_release(pb, taken);
            ++taken;
            if (bh < 0) break;
            const ItemGeom g = item_geom(qb, a.S, causal);
            const int n_t = t ? g.n[1] : g.n[0];
            const int q0 = t ? g.q0[1] : g.q0[0], row = q0 + lrow;
            float m_used = -1e30f;
            float2 l2 = make_float2(0.f, 0.f);
            uint32_t ra[32], rb[32];
            for (int j = 0; j < n_t; ++j) {
                // One key tile = one step of the online softmax: load the 64 scores of this row, maximum, (rarely)
                // rescale, P = 2^(x - m) stored over the scores as fp16 pairs, hand the buffer to the tensor core.
                const int k0 = j * BN;
                const uint32_t buf = ct & 1u;
                ok = wait_bar(s_full + buf, (ct >> 1) & 1u, pb, a.status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                // S_j has landed, so this query tile's product has finished reading K_j (the issuer hands back the tiles
                // it skips itself; the other query tile's share comes from its own softmax warps)
                if (k_releaser) mbar_arrive(&pb->k_empty[(kbase + (uint32_t)j) % K_STAGES]);
                const uint32_t ts = tS_t + buf * (uint32_t)BN + lane_addr;
                tmem_ld32(ts, ra);
                tmem_ld32(ts + 32, rb);
                // a warp whose 32 rows all lie at or below the tile's last key needs no diagonal test (k0 + 63 is never a
                // multiple of 32, so the comparison is the same for the inclusive and the strict form)
                const int mode = GENERIC_MASK ? 2 : (((causal && k0 + BN - 1 > q0 + quarter * 32) || (k0 + BN > a.S)) ? 1 : 0);
                // keys this row may see inside the tile: [0, lim)
                int lim = min(BN, a.S - k0);
                if (a.mask_mode == 2) lim = min(lim, row - k0 + 1);
                if (a.mask_mode == 3) lim = min(lim, row - k0);
                if (GENERIC_MASK && row >= a.S) lim = 0; // rows beyond the prompt: no mask row to read
                const float *mrow = GENERIC_MASK ? a.attn_mask + (size_t)min(row, a.S - 1) * a.mask_row_stride + k0 : nullptr;
                tmem_wait_ld(ra, rb);
                float sc = a.scale_log2e;
                if (mode != 0) { // rare: the causal diagonal, the end of the prompt, or a caller-supplied mask
                    mask_chunk<GENERIC_MASK>(ra, 0, lim, sc, mrow);
                    mask_chunk<GENERIC_MASK>(rb, 32, lim, sc, mrow);
                    sc = 1.0f;
                }
                // two independent chains: the maximum is a latency chain, not a throughput one; scale > 0 commutes with max
                const float m_tile = fmaxf(chunk_max(ra, -INFINITY), chunk_max(rb, -INFINITY)) * sc;
                if (j == 0) {
                    m_used = fmaxf(m_tile, -1e30f);
                } else {
                    const bool grow = m_tile > m_used + kRescaleThreshold;
                    if (__any_sync(0xffffffffu, grow)) {
                        // O_t must hold every product up to tile j-1 before it is rescaled
                        ok = wait_bar(pv_done + ((ct - 1u) & 1u), ((ct - 1u) >> 1) & 1u, pb, a.status);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tc_fence_after();
                        const float m_new = fmaxf(m_used, m_tile);
                        const float alpha = ex2(m_used - m_new);
                        m_used = m_new;
                        l2.x *= alpha;
                        l2.y *= alpha;
                        uint32_t o[32];
#pragma unroll 1
                        for (int ch = 0; ch < D / 32; ++ch) {
                            tmem_ld32(tO_t + lane_addr + ch * 32, o);
                            tmem_wait_ld(o);
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st32(tO_t + lane_addr + ch * 32, o);
                        }
                        tmem_wait_st();
                    }
                }
                const float neg_m = -m_used;
                uint32_t packed[16];
                chunk_exp<EMUL>(ra, sc, neg_m, l2, packed);
                tmem_st16(ts, packed);
                chunk_exp<EMUL>(rb, sc, neg_m, l2, packed);
                tmem_st16(ts + 16, packed);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(p_full + buf);
                ++ct;
            }
            if (!ok) break;
            // ---- the item's row sums go to the epilogue warps through shared memory
            if (ci > 0) {
                ok = wait_bar(l_empty, (ci - 1u) & 1u, pb, a.status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            l_buf[t * BM + lrow] = l2.x + l2.y;
            mbar_arrive(l_full);
            ++ci;
            kbase += (uint32_t)g.nmax;
        }
    } else {
        // ======================= epilogue: warps 12-15, O_t / l -> global =======================
        const int quarter = warp & 3;
        const int lrow = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        constexpr int esz = OUT_F16 ? 2 : 4;
        uint32_t taken = 0, ci[2] = {0, 0};
        bool ok = true;
        for (;;) {
            int bh, qb;
            ok = sched_read(pb, a.status, taken, bh, qb);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            __syncwarp();
            if (lane == 0) sched_release(pb, taken);
            ++taken;
            if (bh < 0) break;
            const ItemGeom g = item_geom(qb, a.S, causal);
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                if (g.n[t] == 0) continue;
                ok = wait_bar(&pb->l_full[t], ci[t] & 1u, pb, a.status) && wait_bar(&pb->o_full[t], ci[t] & 1u, pb, a.status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const float l_sum = l_buf[t * BM + lrow];
                mbar_arrive(&pb->l_empty[t]);
                const float inv = (l_sum > 0.f) ? 1.0f / l_sum : 0.f; // fully masked row -> zeros
                const int row = g.q0[t] + lrow;
                unsigned char *gout = (unsigned char *)a.out + ((size_t)bh * a.S + row) * D * esz;
                uint32_t o[32];
#pragma unroll 1
                for (int ch = 0; ch < D / 32; ++ch) {
                    tmem_ld32(tO[t] + lane_addr + ch * 32, o);
                    tmem_wait_ld(o);
                    if (ch == D / 32 - 1) { // O_t is in registers: the next item may overwrite it
                        tc_fence_before();
                        mbar_arrive(&pb->o_empty[t]);
                    }
                    if (row < a.S) {
                        if (OUT_F16) {
                            uint4 *dst = reinterpret_cast<uint4 *>(gout + ch * 32 * 2);
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint32_t w[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const __half2 h2 = __floats2half2_rn(__uint_as_float(o[8 * q + 2 * e]) * inv,
                                                                         __uint_as_float(o[8 * q + 2 * e + 1]) * inv);
                                    w[e] = *reinterpret_cast<const uint32_t *>(&h2);
                                }
                                dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        } else {
                            float4 *dst = reinterpret_cast<float4 *>(gout + ch * 32 * 4);
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                dst[q] = make_float4(__uint_as_float(o[4 * q]) * inv, __uint_as_float(o[4 * q + 1]) * inv,
                                                     __uint_as_float(o[4 * q + 2]) * inv, __uint_as_float(o[4 * q + 3]) * inv);
                        }
                    }
                }
                ++ci[t];
            }
            if (!ok) break;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// optional epilogue: the reference's attention-output quantisation + transpose
// ------------------------------------------------------------------------------------------------
// launchAttnQuantizedTransposeKernel (decoder_kernels.cu:1179-1300) restated: one block per token row
// (b, s); absmax over all heads (floor -1e9f), scale = absmax / 127, codes cvt.rni.sat.s8(x*127/absmax),
// [B,H,S,d] fp32 -> [B,S,H*d] int8.
// One thread per head dimension (blockDim.x = head size: 64 or 128).
__global__ void __launch_bounds__(128) flb_attn_quant_transpose_kernel(const float *__restrict__ attn, int8_t *__restrict__ q8,
                                                                      float *__restrict__ scale, int H, int S) {
    __shared__ float red[4];
    const int s = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, D = (int)blockDim.x;
    if (tid < 4) red[tid] = -1e9f;
    __syncthreads();
    float amax = -1e9f;
    for (int h = 0; h < H; ++h) amax = fmaxf(amax, fabsf(attn[(((size_t)b * H + h) * S + s) * D + tid]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((tid & 31) == 0) red[tid >> 5] = amax;
    __syncthreads();
    amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    if (tid == 0) scale[(size_t)b * S + s] = amax / 127.0f;
    for (int h = 0; h < H; ++h) {
        const float x = attn[(((size_t)b * H + h) * S + s) * D + tid] * 127.0f / amax;
        int q;
        asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(x));
        q8[(((size_t)b * S + s) * H + h) * D + tid] = (int8_t)q;
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    // the driver entry point does not change during the life of the process: looked up once
    static std::atomic<void *> cached{nullptr};
    void *fn = cached.load(std::memory_order_acquire);
    if (fn) return reinterpret_cast<EncodeTiledFn>(fn);
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
    if (qres != cudaDriverEntryPointSuccess || !fn) return nullptr;
    cached.store(fn, std::memory_order_release);
    return reinterpret_cast<EncodeTiledFn>(fn);
}

// fp16 tensor [bh][rows_valid of rows_stride][D] seen as [bh][D/64 blocks][rows][64]: one box = box_rows rows of every
// 64-dim block, which lands in shared memory block after block, each [box_rows x 64] in the 128-byte-swizzled operand
// layout — a whole tile with one instruction.  Rows at or beyond rows_valid read as zeros.
bool make_map(EncodeTiledFn enc, CUtensorMap *tm, const void *base, int BH, int rows_valid, int rows_stride, int box_rows, int D) {
    const cuuint64_t dims[4] = {64, (cuuint64_t)rows_valid, (cuuint64_t)(D / 64), (cuuint64_t)BH};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, 128, (cuuint64_t)rows_stride * D * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, (cuuint32_t)(D / 64), 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D> int launch_prefill_hd(const flb_attn_params *p, cudaStream_t stream) {
    if (p->freq_cis && (reinterpret_cast<uintptr_t>(p->freq_cis) & 15u)) return FLB_ERR_MISALIGNED;
    if (p->input_mode == FLB_IN_INT32 &&
        ((reinterpret_cast<uintptr_t>(p->q_w_scale) | reinterpret_cast<uintptr_t>(p->k_w_scale) |
          reinterpret_cast<uintptr_t>(p->v_w_scale)) & 15u))
        return FLB_ERR_MISALIGNED;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return FLB_ERR_DEVICE;

    const int B = p->batch_size, H = p->head_num, S = p->seq_len, T = p->total_len;
    const size_t one = ((size_t)B * H * S * D * 2 + 255) / 256 * 256;
    unsigned char *sc = static_cast<unsigned char *>(p->scratch);

    PrefillArgs a;
    a.B = B; a.H = H; a.S = S; a.T = T;
    a.input_mode = p->input_mode;
    a.q = p->q; a.k = p->k; a.v = p->v;
    a.row_stride = p->qkv_row_stride ? p->qkv_row_stride : H * D;
    a.act_scale = p->act_scale; a.q_w_scale = p->q_w_scale; a.k_w_scale = p->k_w_scale; a.v_w_scale = p->v_w_scale;
    a.freq_cis = p->freq_cis;
    a.rope_pos0 = p->rope_pos0;
    a.k_cache = p->k_cache; a.v_cache = p->v_cache;
    a.cache_f16 = (p->cache_dtype == FLB_F16);
    a.qh = reinterpret_cast<__half *>(sc + 256);
    a.kh = reinterpret_cast<__half *>(sc + 256 + one);
    a.vh = reinterpret_cast<__half *>(sc + 256 + 2 * one);
    a.mask_mode = p->mask_mode;
    a.attn_mask = p->attn_mask;
    a.mask_row_stride = p->mask_row_stride;
    a.out = p->out;
    a.out_f16 = (p->out_dtype == FLB_F16);
    a.scale_log2e = p->softmax_scale * kLog2e;
    a.status = reinterpret_cast<unsigned *>(sc);
    a.v_direct = (a.input_mode == FLB_IN_F16 && a.cache_f16) ? 1 : 0;
    // The larger the group, the closer the list is to heaviest-first over everything (measured at batch 8 x 32 heads x 1024
    // tokens: 142 us with groups of 32 units, 138 us with 64, 139 us with 128, 141 us with all 256 in one group; at
    // batch 32 x 512 tokens 210 us with 32 or 64, 214 us with 256); the limit is what a group's K and V rows (fp16) take in
    // the 126 MB L2 beside everything else: 64 MB (batch 2 x 4096 tokens: 305 us with groups of 32 units = 64 MB, 313 us
    // with 64).  A power of two between 8 and 64.
    {
        const size_t per_unit = (size_t)S * D * 2 * 2;
        int hpg = 8;
        while (hpg < 64 && (size_t)hpg * 2 * per_unit <= kGroupBytes && hpg * 2 <= B * H) hpg *= 2;
        a.heads_per_group = hpg;
    }

    CUtensorMap tmQ, tmK, tmV;
    bool ok = make_map(enc, &tmQ, a.qh, B * H, S, S, BM, D);
    if (a.cache_f16) {
        ok = ok && make_map(enc, &tmK, p->k_cache, B * H, S, T, BN, D) && make_map(enc, &tmV, p->v_cache, B * H, S, T, BN, D);
    } else {
        ok = ok && make_map(enc, &tmK, a.kh, B * H, S, S, BN, D) && make_map(enc, &tmV, a.vh, B * H, S, S, BN, D);
    }
    // the caller's v as a [batch][head][token][128] view of its [B,S,H,d] rows, for the V tiles taken from it directly
    CUtensorMap tmVin = tmV;
    if (ok && a.v_direct) {
        const cuuint64_t dims[5] = {64, (cuuint64_t)S, (cuuint64_t)(D / 64), (cuuint64_t)H, (cuuint64_t)B};
        const cuuint64_t strides[4] = {(cuuint64_t)a.row_stride * 2, 128, (cuuint64_t)D * 2, (cuuint64_t)S * a.row_stride * 2};
        const cuuint32_t box[5] = {64, (cuuint32_t)BN, (cuuint32_t)(D / 64), 1, 1};
        const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        ok = enc(&tmVin, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void *>(a.v), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    if (!ok) return FLB_ERR_LAUNCH;
    const int sms = current_device_sm_count();
    if (sms <= 0) return FLB_ERR_DEVICE;

    cudaLaunchConfig_t cfg = {};
    cfg.stream = stream;
    constexpr int pro_rows = (256 / (D / 8)) * kRowsPerThread; // token rows per block of the streaming pass
    const size_t pro_blocks = (size_t)B * H * ((S + pro_rows - 1) / pro_rows);
    cfg.numAttrs = 0; // the prologue is launched the ordinary way (measured: starting it early costs 25 us)
    cfg.gridDim = dim3((unsigned)pro_blocks);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    cudaError_t le;
    if (a.input_mode == 0)
        le = cudaLaunchKernelEx(&cfg, flb_prefill_prologue_kernel<0, D>, a);
    else if (a.input_mode == 1)
        le = cudaLaunchKernelEx(&cfg, flb_prefill_prologue_kernel<1, D>, a);
    else
        le = cudaLaunchKernelEx(&cfg, flb_prefill_prologue_kernel<2, D>, a);
    if (le != cudaSuccess) return FLB_ERR_LAUNCH;

    // The attention kernel is launched with programmatic stream serialisation: its CTAs set themselves up
    // (barriers, descriptors, TMEM) while the prologue drains and wait for it before they touch memory.  The
    // prologue clears the status words and the work counter itself, so no memset node sits between the two.
    // One persistent CTA per SM; the CTAs pull their work items from the counter.
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    const bool generic_mask = (a.mask_mode == FLB_MASK_GENERIC);
    auto kern = generic_mask ? (a.out_f16 ? flb_prefill_attn_kernel<kExpOnFmaEvery, true, true, D> : flb_prefill_attn_kernel<kExpOnFmaEvery, true, false, D>)
                             : (a.out_f16 ? flb_prefill_attn_kernel<kExpOnFmaEvery, false, true, D> : flb_prefill_attn_kernel<kExpOnFmaEvery, false, false, D>);
    constexpr size_t smem_bytes = prefill_smem(D);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes) != cudaSuccess) return FLB_ERR_LAUNCH;
    const long long num_items = (long long)B * H * ((S + 2 * BM - 1) / (2 * BM));
    cfg.attrs = pdl;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3((unsigned)(num_items < sms ? num_items : sms));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem_bytes;
    if (cudaLaunchKernelEx(&cfg, kern, tmQ, tmK, tmV, tmVin, a, (int)num_items) != cudaSuccess) return FLB_ERR_LAUNCH;
    if (p->out_q8) {
        flb_attn_quant_transpose_kernel<<<dim3((unsigned)S, (unsigned)B), D, 0, stream>>>((const float *)p->out, p->out_q8,
                                                                                         p->out_q8_scale, H, S);
        if (cudaGetLastError() != cudaSuccess) return FLB_ERR_LAUNCH;
    }
    return FLB_OK;
}

} // namespace

int launch_prefill(const flb_attn_params *p, cudaStream_t stream) {
    if (p->size_per_head == 128) return launch_prefill_hd<128>(p, stream);
    if (p->size_per_head == 64) return launch_prefill_hd<64>(p, stream);
    return FLB_ERR_UNSUPPORTED;
}

int launch_quantize(const float *attn, int8_t *q8, float *scale, int B, int H, int S, int d, cudaStream_t stream) {
    if (d != 64 && d != 128) return FLB_ERR_UNSUPPORTED;
    flb_attn_quant_transpose_kernel<<<dim3((unsigned)S, (unsigned)B), (unsigned)d, 0, stream>>>(attn, q8, scale, H, S);
    return cudaGetLastError() == cudaSuccess ? FLB_OK : FLB_ERR_LAUNCH;
}

} // namespace flb
