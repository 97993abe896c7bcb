#include "common.cuh"
namespace mgpt {
int tc_experts_forward(mgpt_moe_layer*, const Workspace&, char*, cudaStream_t) { return fail(MGPT_MOE_ESTATE, "tcgen05 path not built"); }
int tc_experts_backward(mgpt_moe_layer*, const Workspace&, char*, cudaStream_t) { return fail(MGPT_MOE_ESTATE, "tcgen05 path not built"); }
void tc_destroy(mgpt_moe_layer*) {}
}
