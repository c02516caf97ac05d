// tcgen05 grouped GEMM back end (placeholder until the tensor-core kernels land).
#include "common.cuh"
#include "gemm.h"
namespace fmoe {
bool tc_forward_supported(const LinearArgs&) { return false; }
bool tc_backward_supported(const LinearBwdArgs&) { return false; }
int tc_linear_forward(const LinearArgs&, cudaStream_t) { return fail(FMOE_ERR_UNSUPPORTED, "tcgen05 path not built"); }
int tc_linear_backward(const LinearBwdArgs&, cudaStream_t) { return fail(FMOE_ERR_UNSUPPORTED, "tcgen05 path not built"); }
size_t tc_backward_scratch_bytes(int64_t, int64_t, int64_t, int, int) { return 0; }
}  // namespace fmoe
