// placeholder so the library links before the tensor-core path lands
#include "ringrnn_common.cuh"
namespace ringrnn {
bool bf16_supported(const RingRnnProblem&) { return false; }
size_t bf16_fwd_workspace_bytes(const RingRnnProblem&) { return 0; }
size_t bf16_saved_bytes(const RingRnnProblem&) { return 0; }
size_t bf16_bwd_workspace_bytes(const RingRnnProblem&) { return 0; }
int bf16_forward(const RingRnnFwdArgs&, const DevProblem&, cudaStream_t) { return RINGRNN_ERR_UNSUPPORTED; }
int bf16_backward(const RingRnnBwdArgs&, const DevProblem&, cudaStream_t) { return RINGRNN_ERR_UNSUPPORTED; }
}
