// peer_exchange.cu — the exchange step of a head-split (tensor-parallel) decode layer.
//
// The decode kernel of every rank stores its finished rows straight into every rank's receive slot
// (plain peer stores, flb_attn_params::out_peers).  What remains of the all-gather is a hand-shake:
// tell the others "my rows for this step are in your memory" and learn the same from them.  One small
// kernel per rank does that, stream-ordered behind the rank's decode kernel:
//
//   signal  thread r of block 0 stores `epoch` into word [rank] of rank r's flag array, as a
//           system-scope release after a system-scope fence: everything this GPU wrote before in
//           stream order (the pushed rows) is visible to whoever acquires the flag;
//   wait    threads 0..size-1 of EVERY block poll this rank's own flag words (system-scope acquire)
//           until word r has reached `epoch`, for at most timeout_ms of wall clock; a wait that runs
//           out ORs FLB_STATUS_PEER_WAIT into *status and the block skips its copy — nothing spins for
//           ever, the context stays usable;
//   copy    the receive slot goes to its final place (16-byte vectors, grid-strided);
//   quant   optionally, the reference's attention-output quantisation of the received rows (its next kernel).
//
// Blocks do not depend on each other, only on flags written by OTHER GPUs, and each rank signals
// before it waits, so the ranks cannot dead-lock each other however their kernels are scheduled.
// Flag words only grow; comparison is by signed difference, so the 32-bit epoch may wrap.
#include "../../include/flb_attn.h"
#include "decode_attn.cuh"

#include <cuda_runtime.h>
#include <stdint.h>

namespace {

struct ExchangeArgs {
    int rank, size;
    unsigned epoch;
    unsigned *flags_local;
    unsigned *flags_peer[FLB_MAX_PEERS];
    const uint4 *recv;
    uint4 *dst;
    size_t n_vec;
    unsigned *status;
    unsigned long long timeout_ns;
    int8_t *out_q8;
    float *out_q8_scale;
    int q8_rows, q8_row_elems;
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) flb_peer_exchange_kernel(const ExchangeArgs x) {
    __shared__ int failed;
    const int tid = threadIdx.x;
    if (tid == 0) failed = 0;
    __syncthreads();

    if (blockIdx.x == 0 && tid < x.size && tid != x.rank) {
        __threadfence_system();
        st_release_sys(x.flags_peer[tid] + x.rank, x.epoch);
    }
    if (tid < x.size && tid != x.rank) {
        const unsigned *w = x.flags_local + tid;
        bool ok = (int)(ld_acquire_sys(w) - x.epoch) >= 0;
        if (!ok) {
            const unsigned long long t0 = globaltimer_ns();
            for (unsigned i = 1; !ok; ++i) {
                ok = (int)(ld_acquire_sys(w) - x.epoch) >= 0;
                if (!ok && (i & 15u) == 0) {
                    if (globaltimer_ns() - t0 > x.timeout_ns) break;
                    __nanosleep(64);
                }
            }
        }
        if (!ok) {
            failed = 1;
            if (x.status) atomicOr(x.status, FLB_STATUS_PEER_WAIT);
        }
    }
    __syncthreads();
    if (failed) return;
    if (x.dst)
        for (size_t i = blockIdx.x * (size_t)blockDim.x + tid; i < x.n_vec; i += (size_t)gridDim.x * blockDim.x) x.dst[i] = x.recv[i];
    if (!x.out_q8) return;
    // the reference's attention-output quantisation for one-token rows (decoder_kernels.cu:1179-1255): absmax over
    // the whole row with the -1e9f floor, scale = absmax / 127, codes cvt.rni.sat.s8(x * 127.0f / absmax)
    __shared__ float red[8];
    const float *src = reinterpret_cast<const float *>(x.recv);
    for (int row = blockIdx.x; row < x.q8_rows; row += gridDim.x) {
        const float4 *r4 = reinterpret_cast<const float4 *>(src + (size_t)row * x.q8_row_elems);
        const int n4 = x.q8_row_elems / 4;
        float amax = -1e9f;
        for (int i = tid; i < n4; i += blockDim.x) {
            const float4 v = r4[i];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        __syncthreads(); // red[] of the previous row has been read by everybody
        if ((tid & 31) == 0) red[tid >> 5] = amax;
        __syncthreads();
        amax = red[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
        if (tid == 0) x.out_q8_scale[row] = amax / 127.0f;
        char4 *d4 = reinterpret_cast<char4 *>(x.out_q8 + (size_t)row * x.q8_row_elems);
        for (int i = tid; i < n4; i += blockDim.x) {
            const float4 v = r4[i];
            int q0, q1, q2, q3;
            asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q0) : "f"(v.x * 127.0f / amax));
            asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q1) : "f"(v.y * 127.0f / amax));
            asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q2) : "f"(v.z * 127.0f / amax));
            asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q3) : "f"(v.w * 127.0f / amax));
            d4[i] = make_char4((signed char)q0, (signed char)q1, (signed char)q2, (signed char)q3);
        }
    }
}

} // namespace

extern "C" int flb_attn_peer_exchange(const flb_peer_exchange *x, void *cuda_stream) {
    if (!x || !x->flags_local) return FLB_ERR_NULL_POINTER;
    if (x->size < 1 || x->size > FLB_MAX_PEERS || x->rank < 0 || x->rank >= x->size) return FLB_ERR_BAD_SHAPE;
    if (x->epoch == 0) return FLB_ERR_BAD_SHAPE;
    const bool copy = x->dst && x->dst != x->recv && x->bytes > 0;
    const bool quant = x->out_q8 != nullptr || x->out_q8_scale != nullptr;
    if (quant) {
        if (!x->out_q8 || !x->out_q8_scale || !x->recv) return FLB_ERR_NULL_POINTER;
        if (x->q8_rows <= 0 || x->q8_row_elems <= 0 || (x->q8_row_elems & 3)) return FLB_ERR_BAD_SHAPE;
        if ((reinterpret_cast<uintptr_t>(x->recv) & 15u) || (reinterpret_cast<uintptr_t>(x->out_q8) & 3u)) return FLB_ERR_MISALIGNED;
    }
    if (copy) {
        if (!x->recv) return FLB_ERR_NULL_POINTER;
        if ((x->bytes & 15u) || (reinterpret_cast<uintptr_t>(x->recv) & 15u) || (reinterpret_cast<uintptr_t>(x->dst) & 15u))
            return FLB_ERR_MISALIGNED;
    }
    ExchangeArgs a;
    a.rank = x->rank;
    a.size = x->size;
    a.epoch = x->epoch;
    a.flags_local = x->flags_local;
    for (int r = 0; r < FLB_MAX_PEERS; ++r) {
        a.flags_peer[r] = (r < x->size) ? x->flags_peer[r] : nullptr;
        if (r < x->size && r != x->rank && !a.flags_peer[r]) return FLB_ERR_NULL_POINTER;
    }
    a.recv = static_cast<const uint4 *>(x->recv);
    a.dst = copy ? static_cast<uint4 *>(x->dst) : nullptr;
    a.n_vec = copy ? x->bytes / 16 : 0;
    a.status = x->status;
    a.timeout_ns = (unsigned long long)(x->timeout_ms ? x->timeout_ms : 1000u) * 1000000ull;
    a.out_q8 = quant ? x->out_q8 : nullptr;
    a.out_q8_scale = quant ? x->out_q8_scale : nullptr;
    a.q8_rows = quant ? x->q8_rows : 0;
    a.q8_row_elems = quant ? x->q8_row_elems : 0;
    // enough blocks to move a decode step's rows (a few hundred KB) in one wave, never more than one per SM
    size_t blocks = copy ? (a.n_vec + 256 * 4 - 1) / (256 * 4) : 1;
    if (quant && blocks < (size_t)x->q8_rows) blocks = (size_t)x->q8_rows;
    if (blocks < 1) blocks = 1;
    const int sms = flb::current_device_sm_count();
    if (sms <= 0) return FLB_ERR_DEVICE;
    if (blocks > (size_t)sms) blocks = (size_t)sms;
    flb_peer_exchange_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(a);
    return cudaGetLastError() == cudaSuccess ? FLB_OK : FLB_ERR_LAUNCH;
}
