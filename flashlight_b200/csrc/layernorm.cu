// fl::LayerNorm over the rows of a [rows][features] matrix as one operator each way.
//
// The reference builds it from batchnorm over the normalised axes followed by
// tileAs(weight) * x_hat + tileAs(bias) (flashlight/fl/nn/modules/LayerNorm.cpp:66-128), five
// passes over the tensor forward and eight backward through this library's own stand-alone
// kernels.  Here a warp owns a row:
//   forward  : one read of x (kept in registers for rows of up to 2048 features, re-read from L1
//              beyond), mean and variance by warp shuffles, one write each of y and x_hat
//              (12 B / element instead of 20);
//   backward : dx = invstd * (g - mean(g) - x_hat * mean(g * x_hat)), g = dy * weight, from one
//              read of dy and x_hat (12 B / element), and the parameter gradients
//              dweight = sum_rows dy * x_hat, dbias = sum_rows dy from the column-sum kernels of
//              batchnorm.cu over the same two tensors (8 B / element): 20 instead of 32.
// Statistics are computed in fp32 around the row's mean (two sweeps over registers), which is
// as well conditioned as the shifted sums of the batch-norm kernels.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "flb200.h"

namespace flb200 {
namespace {

constexpr int kLnMaxPerLane = 64;  // rows of up to 32 * 64 = 2048 features live in registers

template <typename T, int PER>
__global__ void __launch_bounds__(256)
layernorm_forward_kernel(const T* __restrict__ x, const float* __restrict__ weight,
                         const float* __restrict__ bias, T* __restrict__ y,
                         T* __restrict__ xhat, float* __restrict__ mean_out,
                         float* __restrict__ invstd_out, long long rows, int features, float eps) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const T* xr = x + r * features;
  float v[PER];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = j * 32 + lane;
    v[j] = c < features ? Num<T>::to_f(xr[c]) : 0.f;
    s += v[j];
  }
  const float mean = warp_sum(s) / (float)features;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = j * 32 + lane;
    const float d = c < features ? v[j] - mean : 0.f;
    q += d * d;
  }
  const float invstd = rsqrtf(warp_sum(q) / (float)features + eps);
  if (lane == 0) {
    if (mean_out) mean_out[r] = mean;
    if (invstd_out) invstd_out[r] = invstd;
  }
  T* yr = y + r * features;
  T* hr = xhat ? xhat + r * features : nullptr;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = j * 32 + lane;
    if (c < features) {
      const float h = (v[j] - mean) * invstd;
      if (hr) hr[c] = Num<T>::from_f(h);
      yr[c] = Num<T>::from_f(weight ? fmaf(h, weight[c], bias ? bias[c] : 0.f)
                                    : h + (bias ? bias[c] : 0.f));
    }
  }
}

template <typename T, int PER>
__global__ void __launch_bounds__(256)
layernorm_backward_kernel(const T* __restrict__ dy, const T* __restrict__ xhat,
                          const float* __restrict__ weight, const float* __restrict__ invstd,
                          T* __restrict__ dx, long long rows, int features) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const T* gr = dy + r * features;
  const T* hr = xhat + r * features;
  float g[PER], h[PER];
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = j * 32 + lane;
    const bool in = c < features;
    g[j] = in ? Num<T>::to_f(gr[c]) * (weight ? weight[c] : 1.f) : 0.f;
    h[j] = in ? Num<T>::to_f(hr[c]) : 0.f;
    s0 += g[j];
    s1 += g[j] * h[j];
  }
  const float m0 = warp_sum(s0) / (float)features;
  const float m1 = warp_sum(s1) / (float)features;
  const float is = invstd[r];
  T* xr = dx + r * features;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = j * 32 + lane;
    if (c < features) xr[c] = Num<T>::from_f(is * (g[j] - m0 - h[j] * m1));
  }
}

// 16-byte variants for rows of a multiple of V = 16 / sizeof(T) features (row starts are then
// 16-byte aligned with the tensors): lane l owns vectors l, l + 32, ... of the row, PERV of them.
template <typename T, int V>
__device__ __forceinline__ void ln_load(const T* p, float* f) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int k = 0; k < V; ++k) f[k] = Num<T>::to_f(e[k]);
}
template <typename T, int V>
__device__ __forceinline__ void ln_store(T* p, const float* f) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int k = 0; k < V; ++k) e[k] = Num<T>::from_f(f[k]);
  *reinterpret_cast<uint4*>(p) = raw;
}

template <typename T, int PERV>
__global__ void __launch_bounds__(256)
layernorm_forward_vec_kernel(const T* __restrict__ x, const float* __restrict__ weight,
                             const float* __restrict__ bias, T* __restrict__ y,
                             T* __restrict__ xhat, float* __restrict__ mean_out,
                             float* __restrict__ invstd_out, long long rows, int features,
                             float eps) {
  constexpr int V = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const T* xr = x + r * features;
  float v[PERV][V];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < PERV; ++j) {
    const int c = (j * 32 + lane) * V;
    if (c < features) {
      ln_load<T, V>(xr + c, v[j]);
#pragma unroll
      for (int k = 0; k < V; ++k) s += v[j][k];
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) v[j][k] = 0.f;
    }
  }
  const float mean = warp_sum(s) / (float)features;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < PERV; ++j) {
    const int c = (j * 32 + lane) * V;
    if (c < features) {
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float d = v[j][k] - mean;
        q += d * d;
      }
    }
  }
  const float invstd = rsqrtf(warp_sum(q) / (float)features + eps);
  if (lane == 0) {
    if (mean_out) mean_out[r] = mean;
    if (invstd_out) invstd_out[r] = invstd;
  }
  T* yr = y + r * features;
  T* hr = xhat ? xhat + r * features : nullptr;
#pragma unroll
  for (int j = 0; j < PERV; ++j) {
    const int c = (j * 32 + lane) * V;
    if (c >= features) continue;
    float h[V], o[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
      h[k] = (v[j][k] - mean) * invstd;
      const float b = bias ? bias[c + k] : 0.f;
      o[k] = weight ? fmaf(h[k], weight[c + k], b) : h[k] + b;
    }
    if (hr) ln_store<T, V>(hr + c, h);
    ln_store<T, V>(yr + c, o);
  }
}

template <typename T, int PERV>
__global__ void __launch_bounds__(256)
layernorm_backward_vec_kernel(const T* __restrict__ dy, const T* __restrict__ xhat,
                              const float* __restrict__ weight, const float* __restrict__ invstd,
                              T* __restrict__ dx, long long rows, int features) {
  constexpr int V = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const T* gr = dy + r * features;
  const T* hr = xhat + r * features;
  float g[PERV][V], h[PERV][V];
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int j = 0; j < PERV; ++j) {
    const int c = (j * 32 + lane) * V;
    if (c < features) {
      ln_load<T, V>(gr + c, g[j]);
      ln_load<T, V>(hr + c, h[j]);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        g[j][k] *= weight ? weight[c + k] : 1.f;
        s0 += g[j][k];
        s1 += g[j][k] * h[j][k];
      }
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) g[j][k] = h[j][k] = 0.f;
    }
  }
  const float m0 = warp_sum(s0) / (float)features;
  const float m1 = warp_sum(s1) / (float)features;
  const float is = invstd[r];
  T* xr = dx + r * features;
#pragma unroll
  for (int j = 0; j < PERV; ++j) {
    const int c = (j * 32 + lane) * V;
    if (c >= features) continue;
    float o[V];
#pragma unroll
    for (int k = 0; k < V; ++k) o[k] = is * (g[j][k] - m0 - h[j][k] * m1);
    ln_store<T, V>(xr + c, o);
  }
}

template <typename T>
bool ln_vec_ok(const void* a, const void* b, const void* c, int features) {
  constexpr int V = 16 / sizeof(T);
  return features % V == 0 && features <= 32 * V * 8 && aligned16(a) && aligned16(b) &&
         (!c || aligned16(c));
}

template <typename T>
int launch_forward(const void* x, const float* w, const float* b, void* y, void* xhat, float* mean,
                   float* invstd, long long rows, int features, float eps, cudaStream_t st) {
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (ln_vec_ok<T>(x, y, xhat, features)) {
    constexpr int V = 16 / sizeof(T);
#define FLB200_LN_VEC(PERV)                                                                       \
  if (features <= 32 * V * PERV) {                                                                \
    layernorm_forward_vec_kernel<T, PERV><<<grid, 256, 0, st>>>(                                  \
        static_cast<const T*>(x), w, b, static_cast<T*>(y), static_cast<T*>(xhat), mean, invstd,  \
        rows, features, eps);                                                                     \
    return FLB200_OK;                                                                             \
  }
    FLB200_LN_VEC(1)
    FLB200_LN_VEC(2)
    FLB200_LN_VEC(3)
    FLB200_LN_VEC(4)
    FLB200_LN_VEC(6)
    FLB200_LN_VEC(8)
#undef FLB200_LN_VEC
  }
#define FLB200_LN_CASE(PER)                                                                       \
  if (features <= 32 * PER) {                                                                     \
    layernorm_forward_kernel<T, PER><<<grid, 256, 0, st>>>(                                       \
        static_cast<const T*>(x), w, b, static_cast<T*>(y), static_cast<T*>(xhat), mean, invstd,  \
        rows, features, eps);                                                                     \
    return FLB200_OK;                                                                             \
  }
  FLB200_LN_CASE(4)
  FLB200_LN_CASE(8)
  FLB200_LN_CASE(24)
  FLB200_LN_CASE(32)
  FLB200_LN_CASE(kLnMaxPerLane)
#undef FLB200_LN_CASE
  return fail(FLB200_UNSUPPORTED, "layernorm_forward: rows of more than %d features",
              32 * kLnMaxPerLane);
}

template <typename T>
int launch_backward(const void* dy, const void* xhat, const float* w, const float* invstd,
                    void* dx, long long rows, int features, cudaStream_t st) {
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (ln_vec_ok<T>(dy, xhat, dx, features)) {
    constexpr int V = 16 / sizeof(T);
#define FLB200_LN_VEC(PERV)                                                                   \
  if (features <= 32 * V * PERV) {                                                            \
    layernorm_backward_vec_kernel<T, PERV><<<grid, 256, 0, st>>>(                             \
        static_cast<const T*>(dy), static_cast<const T*>(xhat), w, invstd, static_cast<T*>(dx), \
        rows, features);                                                                      \
    return FLB200_OK;                                                                         \
  }
    FLB200_LN_VEC(1)
    FLB200_LN_VEC(2)
    FLB200_LN_VEC(3)
    FLB200_LN_VEC(4)
    FLB200_LN_VEC(6)
    FLB200_LN_VEC(8)
#undef FLB200_LN_VEC
  }
#define FLB200_LN_CASE(PER)                                                                   \
  if (features <= 32 * PER) {                                                                 \
    layernorm_backward_kernel<T, PER><<<grid, 256, 0, st>>>(                                  \
        static_cast<const T*>(dy), static_cast<const T*>(xhat), w, invstd, static_cast<T*>(dx), \
        rows, features);                                                                      \
    return FLB200_OK;                                                                         \
  }
  FLB200_LN_CASE(4)
  FLB200_LN_CASE(8)
  FLB200_LN_CASE(24)
  FLB200_LN_CASE(32)
  FLB200_LN_CASE(kLnMaxPerLane)
#undef FLB200_LN_CASE
  return fail(FLB200_UNSUPPORTED, "layernorm_backward: rows of more than %d features",
              32 * kLnMaxPerLane);
}

}  // namespace
}  // namespace flb200

using namespace flb200;

extern "C" {

int flb200_layernorm_forward(const void* x, const float* weight, const float* bias, void* y,
                             void* xhat, float* mean, float* invstd, int64_t rows,
                             int64_t features, double epsilon, int dtype, void* stream) {
  FLB200_REQUIRE(rows >= 0 && features >= 1, "layernorm_forward: bad extents");
  FLB200_REQUIRE(features <= 32 * kLnMaxPerLane, "layernorm_forward: rows of more than %d features",
                 32 * kLnMaxPerLane);
  if (rows == 0) return FLB200_OK;
  FLB200_REQUIRE(x && y, "layernorm_forward: null tensor");
  cudaStream_t st = as_stream(stream);
  int rc;
  switch (dtype) {
    case FLB200_F32:
      rc = launch_forward<float>(x, weight, bias, y, xhat, mean, invstd, rows, (int)features,
                                 (float)epsilon, st);
      break;
    case FLB200_F16:
      rc = launch_forward<__half>(x, weight, bias, y, xhat, mean, invstd, rows, (int)features,
                                  (float)epsilon, st);
      break;
    case FLB200_BF16:
      rc = launch_forward<__nv_bfloat16>(x, weight, bias, y, xhat, mean, invstd, rows,
                                         (int)features, (float)epsilon, st);
      break;
    default:
      return fail(FLB200_UNSUPPORTED, "layernorm_forward: unknown dtype %d", dtype);
  }
  if (rc) return rc;
  FLB200_AFTER_LAUNCH("layernorm_forward");
  return FLB200_OK;
}

size_t flb200_layernorm_backward_workspace_bytes(int64_t rows, int64_t features) {
  return flb200_layernorm_affine_workspace_bytes(rows, features);
}

int flb200_layernorm_backward(const void* grad_y, const void* xhat, const float* weight,
                              const float* invstd, void* grad_x, float* grad_weight,
                              float* grad_bias, int64_t rows, int64_t features, int dtype,
                              void* workspace, size_t workspace_bytes, void* stream) {
  FLB200_REQUIRE(rows >= 0 && features >= 1, "layernorm_backward: bad extents");
  FLB200_REQUIRE(features <= 32 * kLnMaxPerLane,
                 "layernorm_backward: rows of more than %d features", 32 * kLnMaxPerLane);
  if (rows == 0) return FLB200_OK;
  FLB200_REQUIRE(grad_y && xhat && invstd, "layernorm_backward: null tensor");
  cudaStream_t st = as_stream(stream);
  if (grad_x) {
    int rc;
    switch (dtype) {
      case FLB200_F32:
        rc = launch_backward<float>(grad_y, xhat, weight, invstd, grad_x, rows, (int)features, st);
        break;
      case FLB200_F16:
        rc = launch_backward<__half>(grad_y, xhat, weight, invstd, grad_x, rows, (int)features, st);
        break;
      case FLB200_BF16:
        rc = launch_backward<__nv_bfloat16>(grad_y, xhat, weight, invstd, grad_x, rows,
                                            (int)features, st);
        break;
      default:
        return fail(FLB200_UNSUPPORTED, "layernorm_backward: unknown dtype %d", dtype);
    }
    if (rc) return rc;
    FLB200_AFTER_LAUNCH("layernorm_backward");
  }
  if (grad_weight || grad_bias)  // column sums of dy and dy * x_hat; writes no dx_hat
    return flb200_layernorm_affine_backward(grad_y, xhat, weight, nullptr, grad_weight, grad_bias,
                                            rows, features, dtype, workspace, workspace_bytes,
                                            stream);
  return FLB200_OK;
}

}  // extern "C"
