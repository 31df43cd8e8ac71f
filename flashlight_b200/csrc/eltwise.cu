// Bandwidth-bound gradient functions of Flashlight's autograd tape, each as ONE
// fused pass (the reference runs them as chains of tensor ops with temporaries:
// flashlight/fl/autograd/Functions.cpp:329-338, 454-463, 1777-1796;
// flashlight/fl/autograd/Variable.cpp:205-211).
//
// Layout: flat arrays, 128-bit accesses, four independent vectors in flight per
// thread, grid = a few full waves of 148 SMs with a grid-stride loop.
// Algorithmic bytes per element: 12 for the binary gradients (two reads, one
// write), 8 for the unary forwards.
#include "common.cuh"

namespace flb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

template <typename T, typename Op>
__global__ void __launch_bounds__(kThreads) unary_vec_kernel(const T* __restrict__ a,
                                                             T* __restrict__ out, int64_t n,
                                                             Op op) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = n / V;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
    Vec16<T> va[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) va[u] = load16(a + (i + u * stride) * V);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      Vec16<T> vo;
#pragma unroll
      for (int j = 0; j < V; ++j) vo.v[j] = Num<T>::from_f(op(Num<T>::to_f(va[u].v[j])));
      store16(out + (i + u * stride) * V, vo);
    }
  }
  for (; i < nvec; i += stride) {
    Vec16<T> va = load16(a + i * V), vo;
#pragma unroll
    for (int j = 0; j < V; ++j) vo.v[j] = Num<T>::from_f(op(Num<T>::to_f(va.v[j])));
    store16(out + i * V, vo);
  }
  for (int64_t t = nvec * V + (int64_t)blockIdx.x * kThreads + threadIdx.x; t < n; t += stride)
    out[t] = Num<T>::from_f(op(Num<T>::to_f(a[t])));
}

template <typename T, typename Op>
__global__ void __launch_bounds__(kThreads) unary_scalar_kernel(const T* __restrict__ a,
                                                                T* __restrict__ out, int64_t n,
                                                                Op op) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < n; t += stride)
    out[t] = Num<T>::from_f(op(Num<T>::to_f(a[t])));
}

template <typename T, typename Op>
__global__ void __launch_bounds__(kThreads) binary_vec_kernel(const T* __restrict__ a,
                                                              const T* __restrict__ b,
                                                              T* __restrict__ out, int64_t n,
                                                              Op op) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = n / V;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
    Vec16<T> va[kUnroll], vb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      va[u] = load16(a + (i + u * stride) * V);
      vb[u] = load16(b + (i + u * stride) * V);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      Vec16<T> vo;
#pragma unroll
      for (int j = 0; j < V; ++j)
        vo.v[j] = Num<T>::from_f(op(Num<T>::to_f(va[u].v[j]), Num<T>::to_f(vb[u].v[j])));
      store16(out + (i + u * stride) * V, vo);
    }
  }
  for (; i < nvec; i += stride) {
    Vec16<T> va = load16(a + i * V), vb = load16(b + i * V), vo;
#pragma unroll
    for (int j = 0; j < V; ++j)
      vo.v[j] = Num<T>::from_f(op(Num<T>::to_f(va.v[j]), Num<T>::to_f(vb.v[j])));
    store16(out + i * V, vo);
  }
  for (int64_t t = nvec * V + (int64_t)blockIdx.x * kThreads + threadIdx.x; t < n; t += stride)
    out[t] = Num<T>::from_f(op(Num<T>::to_f(a[t]), Num<T>::to_f(b[t])));
}

template <typename T, typename Op>
__global__ void __launch_bounds__(kThreads) binary_scalar_kernel(const T* __restrict__ a,
                                                                 const T* __restrict__ b,
                                                                 T* __restrict__ out, int64_t n,
                                                                 Op op) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < n; t += stride)
    out[t] = Num<T>::from_f(op(Num<T>::to_f(a[t]), Num<T>::to_f(b[t])));
}

template <typename T, typename Op>
int launch_unary(const char* name, const void* a, void* out, int64_t n, Op op, void* stream) {
  if (n == 0) return FLB200_OK;
  const bool vec = aligned16(a) && aligned16(out);
  const int grid = grid_for(n, kThreads * Vec16<T>::N * kUnroll);
  if (vec)
    unary_vec_kernel<T, Op><<<grid, kThreads, 0, as_stream(stream)>>>(
        static_cast<const T*>(a), static_cast<T*>(out), n, op);
  else
    unary_scalar_kernel<T, Op><<<grid, kThreads, 0, as_stream(stream)>>>(
        static_cast<const T*>(a), static_cast<T*>(out), n, op);
  FLB200_AFTER_LAUNCH(name);
  return FLB200_OK;
}

template <typename T, typename Op>
int launch_binary(const char* name, const void* a, const void* b, void* out, int64_t n, Op op,
                  void* stream) {
  if (n == 0) return FLB200_OK;
  const bool vec = aligned16(a) && aligned16(b) && aligned16(out);
  const int grid = grid_for(n, kThreads * Vec16<T>::N * kUnroll);
  if (vec)
    binary_vec_kernel<T, Op><<<grid, kThreads, 0, as_stream(stream)>>>(
        static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), n, op);
  else
    binary_scalar_kernel<T, Op><<<grid, kThreads, 0, as_stream(stream)>>>(
        static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), n, op);
  FLB200_AFTER_LAUNCH(name);
  return FLB200_OK;
}

template <typename Op>
int dispatch_unary(const char* name, const void* a, void* out, int64_t n, int dtype, Op op,
                   void* stream) {
  FLB200_REQUIRE(n >= 0, "%s: negative element count", name);
  FLB200_REQUIRE(n == 0 || (a && out), "%s: null pointer", name);
  switch (dtype) {
    case FLB200_F32: return launch_unary<float>(name, a, out, n, op, stream);
    case FLB200_F16: return launch_unary<__half>(name, a, out, n, op, stream);
    case FLB200_BF16: return launch_unary<__nv_bfloat16>(name, a, out, n, op, stream);
    default: return fail(FLB200_UNSUPPORTED, "%s: unknown dtype %d", name, dtype);
  }
}

template <typename Op>
int dispatch_binary(const char* name, const void* a, const void* b, void* out, int64_t n,
                    int dtype, Op op, void* stream) {
  FLB200_REQUIRE(n >= 0, "%s: negative element count", name);
  FLB200_REQUIRE(n == 0 || (a && b && out), "%s: null pointer", name);
  switch (dtype) {
    case FLB200_F32: return launch_binary<float>(name, a, b, out, n, op, stream);
    case FLB200_F16: return launch_binary<__half>(name, a, b, out, n, op, stream);
    case FLB200_BF16: return launch_binary<__nv_bfloat16>(name, a, b, out, n, op, stream);
    default: return fail(FLB200_UNSUPPORTED, "%s: unknown dtype %d", name, dtype);
  }
}

// ---- the functors -----------------------------------------------------
struct ReluFwd {
  // fl::max(x, 0.0): NaN compares false and falls to the second operand's
  // branch in ArrayFire's max; keep x for NaN so that it propagates like torch.
  __device__ float operator()(float x) const { return x > 0.f ? x : (x != x ? x : 0.f); }
};
struct ReluBwd {  // (x > 0) * dy
  __device__ float operator()(float x, float dy) const { return x > 0.f ? dy : 0.f; }
};
constexpr float kGeluA = 0.7978845608f;
constexpr float kGeluB = 0.044715f;
struct GeluFwd {
  __device__ float operator()(float x) const {
    const float u = kGeluA * (x + kGeluB * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
  }
};
struct GeluBwd {
  // d/dx [0.5 x (1 + tanh u)], u = a (x + b x^3)
  __device__ float operator()(float x, float dy) const {
    const float x2 = x * x;
    const float u = kGeluA * (x + kGeluB * x * x2);
    const float t = tanhf(u);
    const float du = kGeluA * (1.f + 3.f * kGeluB * x2);
    return dy * (0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du);
  }
};
struct TanhFwd {
  __device__ float operator()(float x) const { return tanhf(x); }
};
struct TanhBwd {  // (1 - y^2) * dy
  __device__ float operator()(float y, float dy) const { return (1.f - y * y) * dy; }
};
struct MaskScale {
  float scale;
  __device__ float operator()(float x, float m) const { return x * m * scale; }
};
struct Add {
  __device__ float operator()(float a, float b) const { return a + b; }
};

}  // namespace
}  // namespace flb200

using namespace flb200;

extern "C" {

int flb200_relu_forward(const void* x, void* y, int64_t n, int dtype, void* stream) {
  return dispatch_unary("relu_forward", x, y, n, dtype, ReluFwd{}, stream);
}
int flb200_relu_backward(const void* x, const void* grad_y, void* grad_x, int64_t n, int dtype,
                         void* stream) {
  return dispatch_binary("relu_backward", x, grad_y, grad_x, n, dtype, ReluBwd{}, stream);
}
int flb200_gelu_forward(const void* x, void* y, int64_t n, int dtype, void* stream) {
  return dispatch_unary("gelu_forward", x, y, n, dtype, GeluFwd{}, stream);
}
int flb200_gelu_backward(const void* x, const void* grad_y, void* grad_x, int64_t n, int dtype,
                         void* stream) {
  return dispatch_binary("gelu_backward", x, grad_y, grad_x, n, dtype, GeluBwd{}, stream);
}
int flb200_tanh_forward(const void* x, void* y, int64_t n, int dtype, void* stream) {
  return dispatch_unary("tanh_forward", x, y, n, dtype, TanhFwd{}, stream);
}
int flb200_tanh_backward(const void* y, const void* grad_y, void* grad_x, int64_t n, int dtype,
                         void* stream) {
  return dispatch_binary("tanh_backward", y, grad_y, grad_x, n, dtype, TanhBwd{}, stream);
}
int flb200_dropout_apply(const void* in, const void* mask, void* out, float scale, int64_t n,
                         int dtype, void* stream) {
  return dispatch_binary("dropout_apply", in, mask, out, n, dtype, MaskScale{scale}, stream);
}
int flb200_add(const void* a, const void* b, void* out, int64_t n, int dtype, void* stream) {
  return dispatch_binary("add", a, b, out, n, dtype, Add{}, stream);
}

}  // extern "C"
