// Fused LSTM time step (rnn_step.cu): recurrent GEMM on tcgen05, split-K reduction over a
// thread-block cluster's shared memories, cell update in the epilogue.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace flb200 {

// TF32 mode on sm_100, batch <= 32, hidden size a multiple of 256 up to 2048.
bool lstm_step_supported(int math_mode, int B, int H);
// Tensor map of W_hh [4H][H]; made once per (layer, direction).
int lstm_step_weight_map(CUtensorMap* map, const float* w_hh, int H);
// gates [B][4H] holds the input projection plus both biases on entry and the activated gates
// on return; c_out [B][H]; h_prev / c_prev / h_out rows have the given strides (elements).
int lstm_step_forward(const CUtensorMap& map_w, const float* h_prev, long long hp_stride,
                      float* gates, const float* c_prev, long long cp_stride, float* c_out,
                      float* h_out, long long ho_stride, int B, int H, cudaStream_t st);

}  // namespace flb200
