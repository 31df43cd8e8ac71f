// logSoftmax and categoricalCrossEntropy, forward and gradient
// (flashlight/fl/autograd/Functions.cpp:1044-1070, 1078-1154).  The reference
// builds these from tile / sum / exp tensor ops and a dense [C,X] one-hot mask;
// here each is one pass over the [C,X] array, plus a fused
// logSoftmax+crossEntropy gradient that never materialises the mask.
//
// Layout: column-major [C, X] = X contiguous rows of C classes.  Rows of up to
// 1024 classes are owned by one warp (8 rows per CTA), longer rows by a CTA.
// Algorithmic bytes per element: forward 8, logSoftmax gradient 12, fused
// gradient 8, crossEntropy gradient 4.
#include <type_traits>

#include "common.cuh"

namespace flb200 {
namespace {

constexpr int kRowThreads = 256;

// Group-wide reductions for GROUP = 32 (a warp) or kRowThreads (the CTA).
template <int GROUP>
__device__ __forceinline__ float group_sum(float v, float* scratch) {
  if (GROUP == 32) return warp_sum(v);
  return block_sum(v, scratch);
}
template <int GROUP>
__device__ __forceinline__ float group_max(float v, float* scratch) {
  v = warp_max(v);
  if (GROUP == 32) return v;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < (kRowThreads / 32) ? scratch[lane] : -INFINITY;
  return warp_max(r);
}

// y = x - (max + log sum exp(x - max))
template <typename T, int GROUP>
__global__ void __launch_bounds__(kRowThreads)
log_softmax_forward_kernel(const T* __restrict__ x, T* __restrict__ y, long long C, long long X) {
  __shared__ float scratch[32];
  const int rows_per_cta = kRowThreads / GROUP;
  const int lane = threadIdx.x % GROUP;
  const int sub = threadIdx.x / GROUP;
  // Every thread of a CTA runs the same number of iterations so that the CTA-wide
  // barriers of the GROUP == CTA case stay matched.
  for (long long row0 = (long long)blockIdx.x * rows_per_cta; row0 < X;
       row0 += (long long)gridDim.x * rows_per_cta) {
    const long long row = row0 + sub;
    const bool live = row < X;
    const T* xr = x + (live ? row : 0) * C;
    float m = -INFINITY;
    if (live)
      for (long long c = lane; c < C; c += GROUP) m = fmaxf(m, Num<T>::to_f(xr[c]));
    m = group_max<GROUP>(m, scratch);
    float s = 0.f;
    if (live)
      for (long long c = lane; c < C; c += GROUP) s += expf(Num<T>::to_f(xr[c]) - m);
    s = group_sum<GROUP>(s, scratch);
    const float lse = m + logf(s);
    if (live) {
      T* yr = y + row * C;
      for (long long c = lane; c < C; c += GROUP) yr[c] = Num<T>::from_f(Num<T>::to_f(xr[c]) - lse);
    }
  }
}

// Long fp32 rows (C a multiple of 4, 16-byte aligned): a CTA per row, 16-byte accesses, the
// maximum and the sum of exponentials taken in ONE sweep (a running maximum, the sum rescaled
// whenever it moves), then the sweep that writes y: two reads of the row instead of three, the
// second one out of cache.
__global__ void __launch_bounds__(kRowThreads)
log_softmax_forward_vec_kernel(const float* __restrict__ x, float* __restrict__ y, long long C4,
                               long long X) {
  __shared__ float scratch[32];
  for (long long row = blockIdx.x; row < X; row += gridDim.x) {
    const float4* xr = reinterpret_cast<const float4*>(x) + row * C4;
    float m = -INFINITY, s = 0.f;
    for (long long c = threadIdx.x; c < C4; c += kRowThreads) {
      const float4 v = xr[c];
      const float vm = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
      if (vm > m) {
        s *= expf(m - vm);  // m = -inf: s is 0 and stays 0
        m = vm;
      }
      s += expf(v.x - m) + expf(v.y - m) + expf(v.z - m) + expf(v.w - m);
    }
    const float row_max = group_max<kRowThreads>(m, scratch);
    // a thread that saw nothing (m = -inf) contributes 0; rows whose maximum is -inf or NaN
    // give NaN, as the three-sweep kernel does
    const float mine = m == -INFINITY ? 0.f : s * expf(m - row_max);
    const float total = group_sum<kRowThreads>(mine, scratch);
    const float lse = row_max + logf(total);
    float4* yr = reinterpret_cast<float4*>(y) + row * C4;
    for (long long c = threadIdx.x; c < C4; c += kRowThreads) {
      const float4 v = xr[c];
      yr[c] = make_float4(v.x - lse, v.y - lse, v.z - lse, v.w - lse);
    }
  }
}

// dx = dy - exp(y) * sum_c dy
template <typename T, int GROUP>
__global__ void __launch_bounds__(kRowThreads)
log_softmax_backward_kernel(const T* __restrict__ y, const T* __restrict__ dy,
                            T* __restrict__ dx, long long C, long long X) {
  __shared__ float scratch[32];
  const int rows_per_cta = kRowThreads / GROUP;
  const int lane = threadIdx.x % GROUP;
  const int sub = threadIdx.x / GROUP;
  for (long long row0 = (long long)blockIdx.x * rows_per_cta; row0 < X;
       row0 += (long long)gridDim.x * rows_per_cta) {
    const long long row = row0 + sub;
    const bool live = row < X;
    const long long base = (live ? row : 0) * C;
    float s = 0.f;
    if (live)
      for (long long c = lane; c < C; c += GROUP) s += Num<T>::to_f(dy[base + c]);
    s = group_sum<GROUP>(s, scratch);
    if (live)
      for (long long c = lane; c < C; c += GROUP)
        dx[base + c] =
            Num<T>::from_f(Num<T>::to_f(dy[base + c]) - expf(Num<T>::to_f(y[base + c])) * s);
  }
}

// Per-target gradient weight g(x) of the crossEntropy gradFunc.
__device__ __forceinline__ float cce_weight(const float* grad_loss, const int32_t* count,
                                            long long xcol, int reduction) {
  if (reduction == FLB200_REDUCE_NONE) return grad_loss[xcol];
  if (reduction == FLB200_REDUCE_MEAN) return grad_loss[0] / (float)(*count);
  return grad_loss[0];
}

// partial[blockIdx] = (sum of -logp[target], number of targets kept)
template <typename T>
__global__ void __launch_bounds__(256)
cce_forward_kernel(const T* __restrict__ logp, const int32_t* __restrict__ targets,
                   float* __restrict__ loss_none, float2* __restrict__ partial,
                   int32_t* __restrict__ bad_flag, long long C, long long X, int ignore_index) {
  __shared__ float scratch[32];
  float s = 0.f, n = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < X; i += stride) {
    const int t = targets[i];
    float v = 0.f;
    if (t == ignore_index) {
      // contributes nothing (Functions.cpp:1119-1121)
    } else if (t < 0 || t >= C) {
      if (bad_flag) atomicOr(bad_flag, 1);
    } else {
      v = -Num<T>::to_f(logp[i * C + t]);
      n += 1.f;
    }
    if (loss_none) loss_none[i] = v;
    s += v;
  }
  s = block_sum(s, scratch);
  n = block_sum(n, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = make_float2(s, n);
}

__global__ void cce_finalize_kernel(const float2* __restrict__ partial, int nparts,
                                    float* __restrict__ loss, int32_t* __restrict__ count_out,
                                    int reduction) {
  double s = 0.0, n = 0.0;
  for (int i = threadIdx.x; i < nparts; i += 32) {
    s += (double)partial[i].x;
    n += (double)partial[i].y;
  }
  s = warp_sum(s);
  n = warp_sum(n);
  if (threadIdx.x == 0) {
    if (count_out) *count_out = (int32_t)(n + 0.5);
    if (reduction == FLB200_REDUCE_MEAN) loss[0] = (float)(s / n);
    else if (reduction == FLB200_REDUCE_SUM) loss[0] = (float)s;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
cce_backward_kernel(const float* __restrict__ grad_loss, const int32_t* __restrict__ targets,
                    const int32_t* __restrict__ count, T* __restrict__ grad_logp, long long C,
                    long long X, int reduction, int ignore_index) {
  const long long total = C * X;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long xcol = i / C;
    const int c = (int)(i - xcol * C);
    const int t = targets[xcol];
    float v = 0.f;
    if (t == c && t != ignore_index) v = -cce_weight(grad_loss, count, xcol, reduction);
    grad_logp[i] = Num<T>::from_f(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
lsm_cce_backward_kernel(const T* __restrict__ y, const float* __restrict__ grad_loss,
                        const int32_t* __restrict__ targets, const int32_t* __restrict__ count,
                        T* __restrict__ dx, long long C, long long X, int reduction,
                        int ignore_index) {
  const long long total = C * X;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long xcol = i / C;
    const int c = (int)(i - xcol * C);
    const int t = targets[xcol];
    float v = 0.f;
    if (t != ignore_index && t >= 0 && t < C) {
      const float g = cce_weight(grad_loss, count, xcol, reduction);
      v = g * (expf(Num<T>::to_f(y[i])) - (t == c ? 1.f : 0.f));
    }
    dx[i] = Num<T>::from_f(v);
  }
}

// The same for fp32 rows of a multiple of 4 classes (16-byte aligned): blockIdx.y = row, four
// classes per thread, the row's target and weight read once per thread, no division.
__global__ void __launch_bounds__(256)
lsm_cce_backward_vec_kernel(const float* __restrict__ y, const float* __restrict__ grad_loss,
                            const int32_t* __restrict__ targets,
                            const int32_t* __restrict__ count, float* __restrict__ dx,
                            long long C4, int reduction, int ignore_index) {
  const long long row = blockIdx.y;
  const int t = targets[row];
  const bool live = t != ignore_index && t >= 0 && t < 4 * C4;
  const float g = live ? cce_weight(grad_loss, count, row, reduction) : 0.f;
  const float4* yr = reinterpret_cast<const float4*>(y) + row * C4;
  float4* dr = reinterpret_cast<float4*>(dx) + row * C4;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < C4;
       c += (long long)gridDim.x * blockDim.x) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
      const float4 l = yr[c];
      v = make_float4(g * expf(l.x), g * expf(l.y), g * expf(l.z), g * expf(l.w));
      if ((t >> 2) == c) {  // the one class that also gets the -1 of the one-hot target
        const int k = t & 3;
        const float e = k == 0 ? l.x : (k == 1 ? l.y : (k == 2 ? l.z : l.w));
        const float fixed = g * (expf(e) - 1.f);
        if (k == 0) v.x = fixed; else if (k == 1) v.y = fixed; else if (k == 2) v.z = fixed; else v.w = fixed;
      }
    }
    dr[c] = v;
  }
}

constexpr int kCceParts = 1024;

template <typename T>
int lsm_launch(bool backward, const void* a, const void* b, void* out, long long C, long long X,
               cudaStream_t st) {
  if (C <= 1024) {
    const int grid = grid_for(X, kRowThreads / 32);
    if (backward)
      log_softmax_backward_kernel<T, 32><<<grid, kRowThreads, 0, st>>>(
          static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), C, X);
    else
      log_softmax_forward_kernel<T, 32><<<grid, kRowThreads, 0, st>>>(
          static_cast<const T*>(a), static_cast<T*>(out), C, X);
  } else {
    const int grid = grid_for(X, 1);
    if constexpr (std::is_same<T, float>::value) {
      if (!backward && C % 4 == 0 && aligned16(a) && aligned16(out)) {
        log_softmax_forward_vec_kernel<<<grid, kRowThreads, 0, st>>>(
            static_cast<const float*>(a), static_cast<float*>(out), C / 4, X);
        FLB200_AFTER_LAUNCH("log_softmax_forward");
        return FLB200_OK;
      }
    }
    if (backward)
      log_softmax_backward_kernel<T, kRowThreads><<<grid, kRowThreads, 0, st>>>(
          static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), C, X);
    else
      log_softmax_forward_kernel<T, kRowThreads><<<grid, kRowThreads, 0, st>>>(
          static_cast<const T*>(a), static_cast<T*>(out), C, X);
  }
  FLB200_AFTER_LAUNCH(backward ? "log_softmax_backward" : "log_softmax_forward");
  return FLB200_OK;
}

int lsm_dispatch(bool backward, const void* a, const void* b, void* out, long long C, long long X,
                 int dtype, void* stream) {
  const char* name = backward ? "log_softmax_backward" : "log_softmax_forward";
  FLB200_REQUIRE(C >= 1 && X >= 0, "%s: bad extents", name);
  if (X == 0) return FLB200_OK;
  FLB200_REQUIRE(a && out && (!backward || b), "%s: null tensor", name);
  cudaStream_t st = as_stream(stream);
  switch (dtype) {
    case FLB200_F32: return lsm_launch<float>(backward, a, b, out, C, X, st);
    case FLB200_F16: return lsm_launch<__half>(backward, a, b, out, C, X, st);
    case FLB200_BF16: return lsm_launch<__nv_bfloat16>(backward, a, b, out, C, X, st);
    default: return fail(FLB200_UNSUPPORTED, "%s: unknown dtype %d", name, dtype);
  }
}

int check_reduction(const char* name, int reduction) {
  FLB200_REQUIRE(reduction >= FLB200_REDUCE_NONE && reduction <= FLB200_REDUCE_SUM,
                 "unknown reduction method for categorical cross entropy (%s: %d)", name,
                 reduction);
  return FLB200_OK;
}

}  // namespace
}  // namespace flb200

using namespace flb200;

extern "C" {

int flb200_log_softmax_forward(const void* x, void* y, int64_t C, int64_t X, int dtype,
                               void* stream) {
  return lsm_dispatch(false, x, nullptr, y, C, X, dtype, stream);
}

int flb200_log_softmax_backward(const void* y, const void* grad_y, void* grad_x, int64_t C,
                                int64_t X, int dtype, void* stream) {
  return lsm_dispatch(true, y, grad_y, grad_x, C, X, dtype, stream);
}

size_t flb200_cce_workspace_bytes(int64_t X) {
  (void)X;
  return (size_t)kCceParts * sizeof(float2);
}

int flb200_cce_forward(const void* logp, const int32_t* targets, float* loss, int32_t* count_out,
                       int32_t* bad_target_flag, int64_t C, int64_t X, int reduction,
                       int ignore_index, int dtype, void* workspace, size_t workspace_bytes,
                       void* stream) {
  if (int st = check_reduction("cce_forward", reduction)) return st;
  FLB200_REQUIRE(C >= 1 && X >= 1, "cce_forward: bad extents");
  FLB200_REQUIRE(logp && targets && loss, "cce_forward: null tensor");
  if (!workspace || workspace_bytes < flb200_cce_workspace_bytes(X))
    return fail(FLB200_WORKSPACE_TOO_SMALL, "cce_forward: workspace too small");
  cudaStream_t st = as_stream(stream);
  int grid = grid_for(X, 256);
  if (grid > kCceParts) grid = kCceParts;
  float2* partial = static_cast<float2*>(workspace);
  float* loss_none = reduction == FLB200_REDUCE_NONE ? loss : nullptr;
  switch (dtype) {
    case FLB200_F32:
      cce_forward_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(logp), targets,
                                                      loss_none, partial, bad_target_flag, C, X,
                                                      ignore_index);
      break;
    case FLB200_F16:
      cce_forward_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(logp), targets,
                                                       loss_none, partial, bad_target_flag, C, X,
                                                       ignore_index);
      break;
    case FLB200_BF16:
      cce_forward_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          static_cast<const __nv_bfloat16*>(logp), targets, loss_none, partial, bad_target_flag, C,
          X, ignore_index);
      break;
    default:
      return fail(FLB200_UNSUPPORTED, "cce_forward: unknown dtype %d", dtype);
  }
  FLB200_AFTER_LAUNCH("cce_forward");
  cce_finalize_kernel<<<1, 32, 0, st>>>(partial, grid, loss, count_out, reduction);
  FLB200_AFTER_LAUNCH("cce_finalize");
  return FLB200_OK;
}

int flb200_cce_backward(const float* grad_loss, const int32_t* targets, const int32_t* count,
                        void* grad_logp, int64_t C, int64_t X, int reduction, int ignore_index,
                        int dtype, void* stream) {
  if (int st = check_reduction("cce_backward", reduction)) return st;
  FLB200_REQUIRE(C >= 1 && X >= 1, "cce_backward: bad extents");
  FLB200_REQUIRE(grad_loss && targets && grad_logp, "cce_backward: null tensor");
  FLB200_REQUIRE(reduction != FLB200_REDUCE_MEAN || count, "cce_backward: MEAN needs count");
  cudaStream_t st = as_stream(stream);
  const int grid = grid_for(C * X, 256 * 4);
  switch (dtype) {
    case FLB200_F32:
      cce_backward_kernel<float><<<grid, 256, 0, st>>>(grad_loss, targets, count,
                                                       static_cast<float*>(grad_logp), C, X,
                                                       reduction, ignore_index);
      break;
    case FLB200_F16:
      cce_backward_kernel<__half><<<grid, 256, 0, st>>>(grad_loss, targets, count,
                                                        static_cast<__half*>(grad_logp), C, X,
                                                        reduction, ignore_index);
      break;
    case FLB200_BF16:
      cce_backward_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          grad_loss, targets, count, static_cast<__nv_bfloat16*>(grad_logp), C, X, reduction,
          ignore_index);
      break;
    default:
      return fail(FLB200_UNSUPPORTED, "cce_backward: unknown dtype %d", dtype);
  }
  FLB200_AFTER_LAUNCH("cce_backward");
  return FLB200_OK;
}

int flb200_log_softmax_cce_backward(const void* y, const float* grad_loss, const int32_t* targets,
                                    const int32_t* count, void* grad_x, int64_t C, int64_t X,
                                    int reduction, int ignore_index, int dtype, void* stream) {
  if (int st = check_reduction("log_softmax_cce_backward", reduction)) return st;
  FLB200_REQUIRE(C >= 1 && X >= 1, "log_softmax_cce_backward: bad extents");
  FLB200_REQUIRE(y && grad_loss && targets && grad_x, "log_softmax_cce_backward: null tensor");
  FLB200_REQUIRE(reduction != FLB200_REDUCE_MEAN || count,
                 "log_softmax_cce_backward: MEAN needs count");
  cudaStream_t st = as_stream(stream);
  const int grid = grid_for(C * X, 256 * 4);
  if (dtype == FLB200_F32 && C % 4 == 0 && X <= 65535 && aligned16(y) && aligned16(grad_x)) {
    long long bx = (C / 4 + 255) / 256;
    if (bx > 64) bx = 64;
    lsm_cce_backward_vec_kernel<<<dim3((unsigned)bx, (unsigned)X), 256, 0, st>>>(
        static_cast<const float*>(y), grad_loss, targets, count, static_cast<float*>(grad_x),
        C / 4, reduction, ignore_index);
    FLB200_AFTER_LAUNCH("log_softmax_cce_backward");
    return FLB200_OK;
  }
  switch (dtype) {
    case FLB200_F32:
      lsm_cce_backward_kernel<float><<<grid, 256, 0, st>>>(
          static_cast<const float*>(y), grad_loss, targets, count, static_cast<float*>(grad_x), C,
          X, reduction, ignore_index);
      break;
    case FLB200_F16:
      lsm_cce_backward_kernel<__half><<<grid, 256, 0, st>>>(
          static_cast<const __half*>(y), grad_loss, targets, count, static_cast<__half*>(grad_x),
          C, X, reduction, ignore_index);
      break;
    case FLB200_BF16:
      lsm_cce_backward_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          static_cast<const __nv_bfloat16*>(y), grad_loss, targets, count,
          static_cast<__nv_bfloat16*>(grad_x), C, X, reduction, ignore_index);
      break;
    default:
      return fail(FLB200_UNSUPPORTED, "log_softmax_cce_backward: unknown dtype %d", dtype);
  }
  FLB200_AFTER_LAUNCH("log_softmax_cce_backward");
  return FLB200_OK;
}

}  // extern "C"
