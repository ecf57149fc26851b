#include "kernels.cuh"
namespace nf4 {
bool prefill_supported(const nf4_linear_args &) { return false; }
uint64_t prefill_workspace_bytes(uint64_t, uint32_t) { return 0; }
int32_t prefill_forward(const nf4_linear_args &, cudaStream_t) { return fail(NF4_ERR_UNSUPPORTED, "prefill: not built"); }
}
