// prefill_attn.cu — causal prefill attention (placeholder until the tensor-core kernel lands).
#include "prefill_attn.cuh"
namespace flb {
int launch_prefill(const flb_attn_params *, cudaStream_t) { return FLB_ERR_UNSUPPORTED; }
} // namespace flb
