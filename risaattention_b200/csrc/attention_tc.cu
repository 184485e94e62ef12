// placeholder replaced below by the tensor-core kernel
#include "attention_common.cuh"
namespace risa_b200 {
bool attention_tc_supported(const AttentionArgs&) { return false; }
int attention_tc(const AttentionArgs&, cudaStream_t) { return fail(RISA_B200_INVALID, "tc kernel absent"); }
}
