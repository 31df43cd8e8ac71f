// softmax over the rows of attention scores with the scale and the causal mask folded in:
//   y[r][c] = softmax_c(scale * x[r][c] + mask(r, c)),  mask = -inf for c > (r mod period)
// (fl::softmax, flashlight/fl/autograd/Functions.cpp:1021-1042, on scores masked as in
// flashlight/fl/contrib/modules/Transformer.cpp:112-119), and its gradient
//   dx = scale * y * (dy - sum_c dy * y).
// One warp per row, the row held in registers (up to 32 x kPerLane columns), warp-shuffle
// reductions, one read and one write of each tensor.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "common.cuh"

namespace flb200 {
namespace {

constexpr int kPerLane = 64;  // rows of up to 2048 columns

template <typename T, int PER>
__global__ void __launch_bounds__(256)
softmax_forward_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int cols,
                       float scale, int period, float* __restrict__ lse) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int limit = period > 0 ? (int)(r % period) : cols - 1;  // last unmasked column
  const T* xr = x + r * cols;
  float v[PER];
  float m = -CUDART_INF_F;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = j * 32 + lane;
    v[j] = (c < cols && c <= limit) ? scale * Num<T>::to_f(xr[c]) : -CUDART_INF_F;
    m = fmaxf(m, v[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    v[j] = v[j] == -CUDART_INF_F ? 0.f : expf(v[j] - m);
    s += v[j];
  }
  s = warp_sum(s);
  const float inv = 1.f / s;
  if (lse && lane == 0) lse[r] = m + logf(s);  // log of the sum of exp(scale * x) over the row
  T* yr = y + r * cols;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = j * 32 + lane;
    if (c < cols) yr[c] = Num<T>::from_f(v[j] * inv);
  }
}

template <typename T, int PER>
__global__ void __launch_bounds__(256)
softmax_backward_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
                        long long rows, int cols, float scale) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const T* yr = y + r * cols;
  const T* gr = dy + r * cols;
  float p[PER], g[PER];
  float dot = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = j * 32 + lane;
    p[j] = c < cols ? Num<T>::to_f(yr[c]) : 0.f;
    g[j] = c < cols ? Num<T>::to_f(gr[c]) : 0.f;
    dot += p[j] * g[j];
  }
  dot = warp_sum(dot);
  T* xr = dx + r * cols;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = j * 32 + lane;
    if (c < cols) xr[c] = Num<T>::from_f(scale * p[j] * (g[j] - dot));  // masked columns: p = 0
  }
}

template <typename T>
int launch(bool backward, const void* a, const void* b, void* out, long long rows, int cols,
           float scale, int period, cudaStream_t st, float* lse) {
  const unsigned grid = (unsigned)((rows + 7) / 8);
#define FLB200_SOFTMAX_CASE(PER)                                                              \
  if (cols <= 32 * PER) {                                                                     \
    if (backward)                                                                             \
      softmax_backward_kernel<T, PER><<<grid, 256, 0, st>>>(                                  \
          static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), rows,     \
          cols, scale);                                                                       \
    else                                                                                      \
      softmax_forward_kernel<T, PER><<<grid, 256, 0, st>>>(                                   \
          static_cast<const T*>(a), static_cast<T*>(out), rows, cols, scale, period, lse);    \
    return FLB200_OK;                                                                         \
  }
  FLB200_SOFTMAX_CASE(4)
  FLB200_SOFTMAX_CASE(16)
  FLB200_SOFTMAX_CASE(32)
  FLB200_SOFTMAX_CASE(kPerLane)
#undef FLB200_SOFTMAX_CASE
  return fail(FLB200_UNSUPPORTED, "softmax: rows of more than %d columns", 32 * kPerLane);
}

int dispatch(bool backward, const void* a, const void* b, void* out, long long rows, long long cols,
             float scale, long long period, int dtype, void* stream, float* lse = nullptr) {
  const char* name = backward ? "softmax_backward" : "softmax_forward";
  FLB200_REQUIRE(rows >= 0 && cols >= 1 && period >= 0, "%s: bad extents", name);
  FLB200_REQUIRE(cols <= 32 * kPerLane, "%s: rows of more than %d columns", name, 32 * kPerLane);
  FLB200_REQUIRE(rows < (1LL << 34), "%s: too many rows", name);
  if (rows == 0) return FLB200_OK;
  FLB200_REQUIRE(a && out && (!backward || b), "%s: null tensor", name);
  cudaStream_t st = as_stream(stream);
  int rc;
  switch (dtype) {
    case FLB200_F32: rc = launch<float>(backward, a, b, out, rows, (int)cols, scale, (int)period, st, lse); break;
    case FLB200_F16: rc = launch<__half>(backward, a, b, out, rows, (int)cols, scale, (int)period, st, lse); break;
    case FLB200_BF16:
      rc = launch<__nv_bfloat16>(backward, a, b, out, rows, (int)cols, scale, (int)period, st, lse);
      break;
    default: return fail(FLB200_UNSUPPORTED, "%s: unknown dtype %d", name, dtype);
  }
  if (rc) return rc;
  FLB200_AFTER_LAUNCH(name);
  return FLB200_OK;
}

}  // namespace
}  // namespace flb200

extern "C" {

int flb200_softmax_forward(const void* x, void* y, int64_t cols, int64_t rows, float scale,
                           int64_t causal_period, int dtype, void* stream) {
  return flb200::dispatch(false, x, nullptr, y, rows, cols, scale, causal_period, dtype, stream);
}

int flb200_softmax_forward_lse(const void* x, void* y, float* lse, int64_t cols, int64_t rows,
                               float scale, int64_t causal_period, int dtype, void* stream) {
  return flb200::dispatch(false, x, nullptr, y, rows, cols, scale, causal_period, dtype, stream,
                          lse);
}

int flb200_softmax_backward(const void* y, const void* grad_y, void* grad_x, int64_t cols,
                            int64_t rows, float scale, int dtype, void* stream) {
  return flb200::dispatch(true, y, grad_y, grad_x, rows, cols, scale, 0, dtype, stream);
}

}  // extern "C"
