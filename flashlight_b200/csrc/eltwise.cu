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

// ---- relu with a bit mask ----------------------------------------------------------------
// Forward writes, next to y, one bit per element (x > 0); backward then reads dy and the mask
// (4.125 bytes per element) instead of dy and y (8).  A thread owns groups of 8 elements: two
// 16-byte vectors and one mask byte, two groups in flight per iteration.
__device__ __forceinline__ unsigned relu8(const float4& a, const float4& b, float4& ya, float4& yb) {
  const ReluFwd f{};
  ya = make_float4(f(a.x), f(a.y), f(a.z), f(a.w));
  yb = make_float4(f(b.x), f(b.y), f(b.z), f(b.w));
  return (a.x > 0.f ? 1u : 0u) | (a.y > 0.f ? 2u : 0u) | (a.z > 0.f ? 4u : 0u) |
         (a.w > 0.f ? 8u : 0u) | (b.x > 0.f ? 16u : 0u) | (b.y > 0.f ? 32u : 0u) |
         (b.z > 0.f ? 64u : 0u) | (b.w > 0.f ? 128u : 0u);
}

__device__ __forceinline__ float4 add4(const float4& a, const float4& b) {
  return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}

// ADD: the input is the sum x + x2 (a residual join fused with its relu), else x alone.
template <bool ADD>
__global__ void __launch_bounds__(256)
relu_forward_mask_kernel(const float* __restrict__ x, const float* __restrict__ x2,
                         float* __restrict__ y, uint8_t* __restrict__ mask, long long n) {
  const long long full = n >> 3;  // complete groups of 8
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float4* xv = reinterpret_cast<const float4*>(x);
  const float4* x2v = reinterpret_cast<const float4*>(x2);
  float4* yv = reinterpret_cast<float4*>(y);
  long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; g + stride < full; g += 2 * stride) {
    const long long g2 = g + stride;
    float4 a0 = xv[2 * g], b0 = xv[2 * g + 1], a1 = xv[2 * g2], b1 = xv[2 * g2 + 1];
    if (ADD) {
      const float4 c0 = x2v[2 * g], d0 = x2v[2 * g + 1], c1 = x2v[2 * g2], d1 = x2v[2 * g2 + 1];
      a0 = add4(a0, c0); b0 = add4(b0, d0); a1 = add4(a1, c1); b1 = add4(b1, d1);
    }
    float4 ya, yb;
    mask[g] = (uint8_t)relu8(a0, b0, ya, yb);
    yv[2 * g] = ya; yv[2 * g + 1] = yb;
    mask[g2] = (uint8_t)relu8(a1, b1, ya, yb);
    yv[2 * g2] = ya; yv[2 * g2 + 1] = yb;
  }
  if (g < full) {
    float4 a0 = xv[2 * g], b0 = xv[2 * g + 1];
    if (ADD) { a0 = add4(a0, x2v[2 * g]); b0 = add4(b0, x2v[2 * g + 1]); }
    float4 ya, yb;
    mask[g] = (uint8_t)relu8(a0, b0, ya, yb);
    yv[2 * g] = ya; yv[2 * g + 1] = yb;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0 && (n & 7)) {  // ragged tail
    unsigned bits = 0;
    for (long long i = full * 8; i < n; ++i) {
      const float v = ADD ? x[i] + x2[i] : x[i];
      y[i] = ReluFwd{}(v);
      bits |= (v > 0.f ? 1u : 0u) << (i - full * 8);
    }
    mask[full] = (uint8_t)bits;
  }
}

__device__ __forceinline__ void relu_bwd8(unsigned m, const float4& a, const float4& b, float4& da,
                                          float4& db) {
  da = make_float4(m & 1u ? a.x : 0.f, m & 2u ? a.y : 0.f, m & 4u ? a.z : 0.f, m & 8u ? a.w : 0.f);
  db = make_float4(m & 16u ? b.x : 0.f, m & 32u ? b.y : 0.f, m & 64u ? b.z : 0.f,
                   m & 128u ? b.w : 0.f);
}

// ADD: the gradient is the sum dy + dy2 (two consumers of the relu's output, summed on the fly
// instead of by a separate accumulation pass), else dy alone.
template <bool ADD>
__global__ void __launch_bounds__(256)
relu_backward_mask_kernel(const uint8_t* __restrict__ mask, const float* __restrict__ dy,
                          const float* __restrict__ dy2, float* __restrict__ dx, long long n) {
  const long long full = n >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float4* gv = reinterpret_cast<const float4*>(dy);
  const float4* g2v = reinterpret_cast<const float4*>(dy2);
  float4* ov = reinterpret_cast<float4*>(dx);
  long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; g + stride < full; g += 2 * stride) {
    const long long g2 = g + stride;
    const unsigned m0 = mask[g], m1 = mask[g2];
    float4 a0 = gv[2 * g], b0 = gv[2 * g + 1], a1 = gv[2 * g2], b1 = gv[2 * g2 + 1];
    if (ADD) {
      const float4 c0 = g2v[2 * g], d0 = g2v[2 * g + 1], c1 = g2v[2 * g2], d1 = g2v[2 * g2 + 1];
      a0 = add4(a0, c0); b0 = add4(b0, d0); a1 = add4(a1, c1); b1 = add4(b1, d1);
    }
    float4 da, db;
    relu_bwd8(m0, a0, b0, da, db);
    ov[2 * g] = da; ov[2 * g + 1] = db;
    relu_bwd8(m1, a1, b1, da, db);
    ov[2 * g2] = da; ov[2 * g2 + 1] = db;
  }
  if (g < full) {
    float4 a0 = gv[2 * g], b0 = gv[2 * g + 1];
    if (ADD) { a0 = add4(a0, g2v[2 * g]); b0 = add4(b0, g2v[2 * g + 1]); }
    float4 da, db;
    relu_bwd8(mask[g], a0, b0, da, db);
    ov[2 * g] = da; ov[2 * g + 1] = db;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0 && (n & 7)) {
    const unsigned bits = mask[full];
    for (long long i = full * 8; i < n; ++i)
      dx[i] = (bits >> (i - full * 8)) & 1u ? (ADD ? dy[i] + dy2[i] : dy[i]) : 0.f;
  }
}

// ---- SGD step --------------------------------------------------------------------------------
// One pass over a parameter: reads p, g, v, writes p and v (20 bytes per element; the reference's
// chain of whole-tensor operations moves about three times that).
__global__ void __launch_bounds__(256)
sgd_step_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ v, long long n,
                float lr, float mu, float wd, int nesterov, float grad_scale, int grad_mode) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                     (v ? reinterpret_cast<uintptr_t>(v) : 0)) & 15) == 0;
  auto one = [&](float pp, float gg, float& vv) {
    gg = gg * grad_scale + wd * pp;
    if (mu != 0.f) {
      vv = mu * vv + gg;
      gg = nesterov ? gg + mu * vv : vv;
    }
    return pp - lr * gg;
  };
  const long long nv = vec ? n >> 2 : 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float4 vv = v ? reinterpret_cast<float4*>(v)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    pp.x = one(pp.x, gg.x, vv.x); pp.y = one(pp.y, gg.y, vv.y);
    pp.z = one(pp.z, gg.z, vv.z); pp.w = one(pp.w, gg.w, vv.w);
    reinterpret_cast<float4*>(p)[i] = pp;
    if (v) reinterpret_cast<float4*>(v)[i] = vv;
    if (grad_mode == 1) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (long long i = nv * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float vv = v ? v[i] : 0.f;
    p[i] = one(p[i], g[i], vv);
    if (v) v[i] = vv;
    if (grad_mode == 1) g[i] = 0.f;
  }
}

extern "C" {

int flb200_sgd_step(void* param, void* grad, void* velocity, int64_t n, float lr, float momentum,
                    float weight_decay, int nesterov, float grad_scale, int zero_grad, int dtype,
                    void* stream) {
  FLB200_REQUIRE(n >= 0, "sgd_step: negative size");
  if (n == 0) return FLB200_OK;
  FLB200_REQUIRE(param && grad, "sgd_step: null tensor");
  FLB200_REQUIRE(momentum == 0.f || velocity, "sgd_step: momentum needs a velocity buffer");
  if (dtype != FLB200_F32) return fail(FLB200_UNSUPPORTED, "sgd_step: f32 parameters only");
  const int grid = grid_for((n + 3) / 4, 256);
  sgd_step_kernel<<<grid, 256, 0, as_stream(stream)>>>(
      static_cast<float*>(param), static_cast<float*>(grad),
      momentum != 0.f ? static_cast<float*>(velocity) : nullptr, n, lr, momentum, weight_decay,
      nesterov ? 1 : 0, grad_scale, zero_grad ? 1 : 0);
  FLB200_AFTER_LAUNCH("sgd_step");
  return FLB200_OK;
}

namespace {
int relu_mask_forward(const char* name, const void* x, const void* x2, void* y, uint8_t* mask,
                      int64_t n, int dtype, void* stream) {
  FLB200_REQUIRE(n >= 0, "%s: negative size", name);
  if (n == 0) return FLB200_OK;
  FLB200_REQUIRE(x && y && mask, "%s: null tensor", name);
  if (dtype != FLB200_F32 || !aligned16(x) || !aligned16(y) || (x2 && !aligned16(x2)))
    return fail(FLB200_UNSUPPORTED, "%s: f32 tensors aligned to 16 bytes only", name);
  const int grid = grid_for((n + 7) / 8, 256 * 2);
  if (x2)
    relu_forward_mask_kernel<true><<<grid, 256, 0, as_stream(stream)>>>(
        static_cast<const float*>(x), static_cast<const float*>(x2), static_cast<float*>(y), mask, n);
  else
    relu_forward_mask_kernel<false><<<grid, 256, 0, as_stream(stream)>>>(
        static_cast<const float*>(x), nullptr, static_cast<float*>(y), mask, n);
  FLB200_AFTER_LAUNCH(name);
  return FLB200_OK;
}
int relu_mask_backward(const char* name, const uint8_t* mask, const void* g1, const void* g2,
                       void* grad_x, int64_t n, int dtype, void* stream) {
  FLB200_REQUIRE(n >= 0, "%s: negative size", name);
  if (n == 0) return FLB200_OK;
  FLB200_REQUIRE(mask && g1 && grad_x, "%s: null tensor", name);
  if (dtype != FLB200_F32 || !aligned16(g1) || !aligned16(grad_x) || (g2 && !aligned16(g2)))
    return fail(FLB200_UNSUPPORTED, "%s: f32 tensors aligned to 16 bytes only", name);
  const int grid = grid_for((n + 7) / 8, 256 * 2);
  if (g2)
    relu_backward_mask_kernel<true><<<grid, 256, 0, as_stream(stream)>>>(
        mask, static_cast<const float*>(g1), static_cast<const float*>(g2),
        static_cast<float*>(grad_x), n);
  else
    relu_backward_mask_kernel<false><<<grid, 256, 0, as_stream(stream)>>>(
        mask, static_cast<const float*>(g1), nullptr, static_cast<float*>(grad_x), n);
  FLB200_AFTER_LAUNCH(name);
  return FLB200_OK;
}
}  // namespace

int flb200_relu_forward_mask(const void* x, void* y, uint8_t* mask, int64_t n, int dtype,
                             void* stream) {
  return relu_mask_forward("relu_forward_mask", x, nullptr, y, mask, n, dtype, stream);
}
int flb200_add_relu_forward_mask(const void* a, const void* b, void* y, uint8_t* mask, int64_t n,
                                 int dtype, void* stream) {
  FLB200_REQUIRE(b != nullptr || n == 0, "add_relu_forward_mask: null tensor");
  return relu_mask_forward("add_relu_forward_mask", a, b, y, mask, n, dtype, stream);
}
int flb200_relu_backward_mask(const uint8_t* mask, const void* grad_y, void* grad_x, int64_t n,
                              int dtype, void* stream) {
  return relu_mask_backward("relu_backward_mask", mask, grad_y, nullptr, grad_x, n, dtype, stream);
}
int flb200_relu_backward_mask_sum(const uint8_t* mask, const void* grad_y_a, const void* grad_y_b,
                                  void* grad_x, int64_t n, int dtype, void* stream) {
  return relu_mask_backward("relu_backward_mask_sum", mask, grad_y_a, grad_y_b, grad_x, n, dtype,
                            stream);
}

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

// ---- Bernoulli masks -------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11), a
// counter-based generator: element block i of the stream (seed, offset) is a pure function of
// (seed, offset + i), so a mask is reproducible whatever the grid that wrote it.
namespace flb200 {
namespace {

__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  constexpr uint32_t kM0 = 0xD2511F53u, kM1 = 0xCD9E8D57u, kW0 = 0x9E3779B9u, kW1 = 0xBB67AE85u;
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(kM0, ctr.x), lo0 = kM0 * ctr.x;
    const uint32_t hi1 = __umulhi(kM1, ctr.z), lo1 = kM1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += kW0;
    key.y += kW1;
  }
  return ctr;
}

template <typename T>
__global__ void bernoulli_mask_kernel(T* out, long long n, float keep, unsigned long long seed,
                                      unsigned long long offset) {
  const long long blocks = (n + 3) / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < blocks;
       i += (long long)gridDim.x * blockDim.x) {
    const unsigned long long c = offset + (unsigned long long)i;
    const uint4 r = philox4x32_10(make_uint4((uint32_t)c, (uint32_t)(c >> 32), 0u, 0u),
                                  make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long e = 4 * i + j;
      // 24 random bits -> a uniform value in [0, 1) that fp32 holds exactly
      if (e < n) out[e] = Num<T>::from_f(((w[j] >> 8) * (1.0f / 16777216.0f)) < keep ? 1.f : 0.f);
    }
  }
}

}  // namespace
}  // namespace flb200

extern "C" int flb200_bernoulli_mask(void* out, int64_t n, float keep_prob, uint64_t seed,
                                     uint64_t offset, int dtype, void* stream) {
  using namespace flb200;
  FLB200_REQUIRE(n >= 0, "bernoulli_mask: negative size");
  FLB200_REQUIRE(keep_prob >= 0.f && keep_prob <= 1.f, "bernoulli_mask: probability outside [0, 1]");
  if (n == 0) return FLB200_OK;
  FLB200_REQUIRE(out, "bernoulli_mask: null tensor");
  const long long blocks = (n + 3) / 4;
  const unsigned grid = (unsigned)std::min<long long>((blocks + 255) / 256, 148 * 8);
  cudaStream_t st = as_stream(stream);
  switch (dtype) {
    case FLB200_F32:
      bernoulli_mask_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(out), n, keep_prob,
                                                         seed, offset);
      break;
    case FLB200_F16:
      bernoulli_mask_kernel<__half><<<grid, 256, 0, st>>>(static_cast<__half*>(out), n, keep_prob,
                                                          seed, offset);
      break;
    case FLB200_BF16:
      bernoulli_mask_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          static_cast<__nv_bfloat16*>(out), n, keep_prob, seed, offset);
      break;
    default:
      return fail(FLB200_UNSUPPORTED, "bernoulli_mask: unsupported dtype %d", dtype);
  }
  FLB200_AFTER_LAUNCH("bernoulli_mask");
  return FLB200_OK;
}

// ---- reorder -----------------------------------------------------------------------------------
// fl::reorder (flashlight/fl/autograd/Functions.cpp:513-535) for the case every head split / merge
// of an attention block is: up to four outer indices permuted, the innermost run of `inner`
// elements contiguous on both sides.  A group of lanes copies one run with 16-byte accesses.
namespace flb200 {
namespace {

struct ReorderGeo {
  long long d[4];   // outer extents in OUTPUT order (the output is contiguous)
  long long is[4];  // input strides of those indices, in 16-byte units
  int lanes_shift;  // log2 of the lanes per run
  int vecs;         // 16-byte vectors per run
};

__global__ void __launch_bounds__(256)
reorder_runs_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, ReorderGeo g,
                    long long runs) {
  const int lanes = 1 << g.lanes_shift;
  const int sub = threadIdx.x & (lanes - 1);
  const long long per_cta = 256 >> g.lanes_shift;
  for (long long r = (long long)blockIdx.x * per_cta + (threadIdx.x >> g.lanes_shift); r < runs;
       r += (long long)gridDim.x * per_cta) {
    long long t = r;
    const long long i3 = t % g.d[3]; t /= g.d[3];
    const long long i2 = t % g.d[2]; t /= g.d[2];
    const long long i1 = t % g.d[1]; t /= g.d[1];
    const uint4* src = in + t * g.is[0] + i1 * g.is[1] + i2 * g.is[2] + i3 * g.is[3];
    uint4* dst = out + r * g.vecs;
    for (int v = sub; v < g.vecs; v += lanes) dst[v] = src[v];
  }
}

}  // namespace
}  // namespace flb200

extern "C" int flb200_reorder(const void* in, void* out, const int64_t* dims,
                              const int64_t* in_strides, int64_t inner, int dtype, void* stream) {
  using namespace flb200;
  FLB200_REQUIRE(in && out && dims && in_strides, "reorder: null argument");
  const size_t es = dtype == FLB200_F32 ? 4 : ((dtype == FLB200_F16 || dtype == FLB200_BF16) ? 2 : 0);
  FLB200_REQUIRE(es != 0, "reorder: unknown dtype %d", dtype);
  FLB200_REQUIRE(inner >= 1 && (inner * (int64_t)es) % 16 == 0 && aligned16(in) && aligned16(out),
                 "reorder: runs must be whole 16-byte vectors of 16-byte aligned tensors");
  ReorderGeo g{};
  long long runs = 1;
  const long long per_vec = (long long)(16 / es);
  for (int k = 0; k < 4; ++k) {
    FLB200_REQUIRE(dims[k] >= 0 && in_strides[k] >= 0 && in_strides[k] % per_vec == 0,
                   "reorder: input strides must be whole 16-byte vectors");
    g.d[k] = dims[k];
    g.is[k] = in_strides[k] / per_vec;
    runs *= dims[k];
  }
  if (runs == 0) return FLB200_OK;
  g.vecs = (int)(inner / per_vec);
  g.lanes_shift = 0;
  while ((1 << g.lanes_shift) < g.vecs && g.lanes_shift < 5) ++g.lanes_shift;
  const long long per_cta = 256 >> g.lanes_shift;
  long long grid = (runs + per_cta - 1) / per_cta;
  const long long cap = 32LL * device_info().sm_count;
  if (grid > cap) grid = cap;
  reorder_runs_kernel<<<(unsigned)grid, 256, 0, as_stream(stream)>>>(
      static_cast<const uint4*>(in), static_cast<uint4*>(out), g, runs);
  FLB200_AFTER_LAUNCH("reorder");
  return FLB200_OK;
}
