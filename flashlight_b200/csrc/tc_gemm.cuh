// Interface of the tcgen05 (tensor-core) contraction used by TF32 mode.
#pragma once
#include "common.cuh"

namespace flb200 {

// True when the tensor-core kernel covers this problem (layout, alignment, size).
bool tc_gemm_supported(const flb200_matmul_desc* d, const void* a, const void* b, const void* c);
size_t tc_gemm_workspace_bytes(const flb200_matmul_desc* d);
int tc_gemm_run(const flb200_matmul_desc* d, const void* a, const void* b, void* c, void* ws,
                size_t ws_bytes, cudaStream_t st);

}  // namespace flb200
