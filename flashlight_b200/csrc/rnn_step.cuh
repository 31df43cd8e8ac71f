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
int lstm_step_weight_map(CUtensorMap* map, const float* w_hh, int H, int G = 4);
// gates [B][4H] holds the input projection plus both biases on entry and the activated gates
// on return; c_out [B][H]; h_prev / c_prev / h_out rows have the given strides (elements).
int lstm_step_forward(const CUtensorMap& map_w, const float* h_prev, long long hp_stride,
                      float* gates, const float* c_prev, long long cp_stride, float* c_out,
                      float* h_out, long long ho_stride, int B, int H, cudaStream_t st);

// G = 4: LSTM.  G = 3: GRU — `cells` then holds q = U_n h + b_hn per step (what its gradient
// needs), c0 is unused, b_hn is the candidate gate's recurrent bias; backward: c0 = h0, `out` =
// the forward output, dgh = the second gate-gradient tensor (the recurrent side's), dc0 / dc_out
// unused.  G = 1: the plain cells (act 0 relu, 1 tanh): gates holds h, no cell tensors.
// The whole recurrence of one (layer, direction) in one persistent kernel (W_hh resident in
// shared memory, a grid-wide barrier per step).  Supported where lstm_step_forward is and the
// device can hold every cluster of the launch at once.  gates [T][B][4H] (input projections
// plus biases in, activated gates out), cells [T][B][H], out = this direction's first column
// of the layer output (rows of out_stride floats, row t * B + b), h0 / c0 [B][H] (never null),
// sync = 4 bytes of scratch.  wait_budget: clocks a CTA waits at the barrier before it gives
// up (0 = the library's default of about two seconds); absent_cta >= 0 makes that CTA never
// arrive (used by the bounded-wait test only).
bool lstm_sequence_supported(int math_mode, int B, int H, int G = 4);
int lstm_sequence_forward(const CUtensorMap& map_w, float* gates, float* cells, float* out,
                          long long out_stride, const float* h0, const float* c0, unsigned* sync,
                          int T, int B, int H, int reverse, long long wait_budget, int absent_cta,
                          cudaStream_t st, int G = 4, const float* b_hn = nullptr, int act = 0);

// The backward recurrence of one (layer, direction) in one persistent kernel: cell gradients
// and dh_{t-1} = dgates_t * W_hh for all T steps, W_hh resident in shared memory (read from the
// forward weights as an MN-major operand).  TF32 mode, batch <= 32, H of 256, 512 or 1024, and
// a device that holds all H / 128 * H / 64 CTAs at once.  xbuf: lstm_sequence_backward_scratch_bytes
// of 16-byte aligned scratch (the per-step exchange of partial sums).  gates / cells: the forward pass's
// reserve tensors; dy: this direction's first column of the output gradient (rows of dy_stride
// floats) or null; dh0 / dc0 [B][H] or null; dgates [T][B][4H], dh_out / dc_out [B][H] out.
bool lstm_sequence_backward_supported(int math_mode, int B, int H, int G = 4);
int lstm_sequence_weight_map_transposed(CUtensorMap* map, const float* w_hh, int H, int G = 4);
int lstm_sequence_backward(const CUtensorMap& map_wt, const float* gates, const float* cells,
                           const float* c0, const float* dy, long long dy_stride,
                           const float* dh0, const float* dc0, float* dgates, float* dh_out,
                           float* dc_out, float* xbuf, unsigned* sync, int T, int B, int H,
                           int reverse, cudaStream_t st, int G = 4, float* dgh = nullptr,
                           const float* out = nullptr, long long out_stride = 0, int act = 0);
size_t lstm_sequence_backward_scratch_bytes(int H);

}  // namespace flb200
