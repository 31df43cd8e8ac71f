// Placeholder translation unit for the tcgen05 convolution: reports "not covered"
// for every shape, so TF32 mode currently runs the fp32 kernel.
#include "tc_conv.cuh"

namespace flb200 {
bool tc_conv_supported(const ConvGeo&, int, size_t) { return false; }
size_t tc_conv_workspace_bytes(const ConvGeo&, int) { return 0; }
int tc_conv_forward(const ConvGeo&, const float*, const float*, const float*, float*, void*, size_t,
                    cudaStream_t) {
  return fail(FLB200_UNSUPPORTED, "tc_conv: not built");
}
int tc_conv_backward_data(const ConvGeo&, const float*, const float*, float*, void*, size_t,
                          cudaStream_t) {
  return fail(FLB200_UNSUPPORTED, "tc_conv: not built");
}
int tc_conv_backward_filter(const ConvGeo&, const float*, const float*, float*, void*, size_t,
                            cudaStream_t) {
  return fail(FLB200_UNSUPPORTED, "tc_conv: not built");
}
}  // namespace flb200
