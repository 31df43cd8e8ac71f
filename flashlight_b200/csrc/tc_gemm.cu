// Placeholder translation unit for the tcgen05 contraction: reports "not covered"
// for every shape, so TF32 mode currently runs the fp32 kernel.
#include "tc_gemm.cuh"

namespace flb200 {
bool tc_gemm_supported(const flb200_matmul_desc*, const void*, const void*, const void*) {
  return false;
}
size_t tc_gemm_workspace_bytes(const flb200_matmul_desc*) { return 0; }
int tc_gemm_run(const flb200_matmul_desc*, const void*, const void*, void*, void*, size_t,
                cudaStream_t) {
  return fail(FLB200_UNSUPPORTED, "tc_gemm: not built");
}
}  // namespace flb200

extern "C" int flb200_has_tensor_core_path(void) { return 0; }
