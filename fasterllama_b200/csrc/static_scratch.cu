// static_scratch.cu — decode attention for callers that cannot hand over scratch memory.
//
// Who needs this: code that runs where device allocation is off the table — inside a memory-pool
// that has already been carved up, in a plugin whose host gives it only its input and output
// tensors, or in a serving loop that must not touch the allocator while requests are in flight.
// Such a caller has nowhere to get the split-KV scratch that flb_attn_decode() asks for, so this
// file keeps one fixed block of device memory inside the library image itself and lends it to
// the decode kernel.
//
// The block is a file-scope __device__ array: the CUDA runtime places it in every GPU's memory when
// the library's code is loaded on that GPU and it stays there until the process exits (it costs
// FLB_STATIC_SCRATCH_BYTES per GPU whether or not this entry point is ever called).  Host code may
// not use the array's name as a pointer — on the host that name is only a handle; the device
// address is looked up with cudaGetSymbolAddress(), once per GPU, with that GPU current, the first
// time the entry point runs there.  Do that first call outside any stream capture (the lookup is
// not a stream operation).
//
// There is one block per GPU and every call uses it: two calls whose kernels may overlap on the
// same GPU (different streams, different host threads) would trample each other's partial results.
// Issue calls to this entry point on one stream at a time per GPU.  The block keeps whatever the
// previous call left; the part that has to start at zero (the arrival counters and the status
// word) is cleared by a memset node at the head of each call — which also means that such a call is always an
// ordinary launch: the early-start levels need counters that are already zero without a memset in front.
#include "../../include/flb_attn.h"

#include <cuda_runtime.h>

#include <mutex>

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[FLB_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void *g_scratch_ptr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the block on the current GPU; looked up on first use.
int static_scratch_for_current_device(void **out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FLB_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return FLB_ERR_DEVICE;
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return FLB_OK;
}

} // namespace

extern "C" int flb_attn_decode_static_scratch(const flb_attn_params *p, void *cuda_stream) {
    if (!p) return FLB_ERR_NULL_POINTER;
    if (p->seq_len != 1) return FLB_ERR_BAD_SHAPE;
    flb_attn_params q = *p;
    // size check first, on the host, against the fixed block: a placeholder non-null, aligned
    // pointer stands in until the real address is known
    q.scratch = reinterpret_cast<void *>(static_cast<uintptr_t>(256));
    q.scratch_bytes = FLB_STATIC_SCRATCH_BYTES;
    q.scratch_zeroed = 0; // the counters are cleared on every call
    int st = flb_attn_validate(&q);
    if (st == FLB_ERR_SCRATCH_TOO_SMALL) return FLB_ERR_TOO_LARGE; // batch x heads x partitions beyond the fixed block
    if (st != FLB_OK) return st;
    void *ptr = nullptr;
    st = static_scratch_for_current_device(&ptr);
    if (st != FLB_OK) return st;
    q.scratch = ptr;
    return flb_attn_decode(&q, cuda_stream);
}

extern "C" int flb_attn_static_scratch_status(unsigned *status_out, void *cuda_stream) {
    if (!status_out) return FLB_ERR_NULL_POINTER;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FLB_ERR_DEVICE;
    void *ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_scratch_mutex);
        ptr = g_scratch_ptr[dev];
    }
    if (!ptr) { // the entry point has not run on this GPU: nothing can have been reported
        *status_out = 0u;
        return FLB_OK;
    }
    return flb_attn_scratch_status(ptr, status_out, cuda_stream);
}
