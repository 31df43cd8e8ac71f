// batchnorm / LayerNorm forward and backward, convolution bias gradient, bias
// tile-add.  Stands behind fl::AutogradExtension::batchnorm and
// ::batchnormBackward (flashlight/fl/autograd/tensor/AutogradExtension.h:82-94,
// 155-164); geometry rule from
// flashlight/fl/autograd/tensor/backend/cudnn/BatchNorm.cpp:22-75 (identical to
// backend/onednn/BatchNorm.cpp:40-71).  fl::LayerNorm runs through the same
// entry points (flashlight/fl/nn/modules/LayerNorm.cpp:88-97).
//
// Forward (training):  pass 1 shifted sums -> finalize (double) -> pass 2 apply.
// Backward:            pass 1 (sum dy, sum dy*(x-mean)) -> finalize -> pass 2.
// Algorithmic bytes per element: forward 8 (+4 for the second read when the
// slab does not stay in L2), backward 12 (+8 likewise).
#include <mutex>
#include <type_traits>

#include "channel_ops.cuh"

namespace flb200 {

namespace {

// ------------------------------------------------------------ functors
struct SumF {
  struct K {};
  __device__ K channel(long long) const { return K{}; }
  __device__ void accumulate(const K&, float a, float, float& s0, float&) const { s0 += a; }
};

// Sums of (x - shift) and (x - shift)^2 with shift = the channel's first
// element: keeps E[d^2] - E[d]^2 well conditioned when |mean| >> std.
struct StatsF {
  const float* x_first;   // base of the tensor (fp32 view used only for the shift)
  long long inner;        // stride between channels in elements
  int dtype;
  struct K { float shift; };
  __device__ K channel(long long c) const {
    float v;
    if (dtype == FLB200_F32) v = x_first[c * inner];
    else if (dtype == FLB200_F16) v = __half2float(reinterpret_cast<const __half*>(x_first)[c * inner]);
    else v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x_first)[c * inner]);
    if (!(fabsf(v) < 3.0e38f)) v = 0.f;  // inf/NaN shift would poison finite data
    return K{v};
  }
  __device__ void accumulate(const K& k, float a, float, float& s0, float& s1) const {
    const float d = a - k.shift;
    s0 += d;
    s1 += d * d;
  }
};

struct BnBwdReduceF {  // a = x, b = dy
  const float* mean;
  struct K { float mean; };
  __device__ K channel(long long c) const { return K{mean[c]}; }
  __device__ void accumulate(const K& k, float a, float b, float& s0, float& s1) const {
    s0 += b;
    s1 += b * (a - k.mean);
  }
};

// The normalised, scaled and shifted value.  One expression for the forward pass and for the
// fused-relu backward passes, which recompute it to get the relu predicate back from x.
__device__ __forceinline__ float bn_value(float x, float mean, float scale, float shift) {
  return __fmaf_rn(x - mean, scale, shift);
}
// scale = invstd * gamma from the SAVED (rounded) invstd, so that backward can rebuild it.
__device__ __forceinline__ float bn_scale(float invstd, const float* weight, long long c) {
  return (float)((double)invstd * (weight ? (double)weight[c] : 1.0));
}

template <bool RELU>
struct BnFwdApplyF {  // y = (x - mean) * scale + shift, then max(., 0) when RELU
  const float* mean;
  const float* scale;  // invstd * gamma
  const float* shift;  // beta
  struct K { float mean, scale, shift; };
  __device__ K channel(long long c) const { return K{mean[c], scale[c], shift ? shift[c] : 0.f}; }
  __device__ float apply(const K& k, float a, float) const {
    const float z = bn_value(a, k.mean, k.scale, k.shift);
    return RELU ? (z > 0.f ? z : (z != z ? z : 0.f)) : z;
  }
};

// Backward of relu(batchnorm(x)): the relu predicate is rebuilt from x (z > 0 with z exactly
// as forward computed it), so neither the output nor a mask is read and the relu gradient
// costs no pass of its own.  a = x, b = dy.
struct BnReluBwdReduceF {
  const float* mean;
  const float* invstd;
  const float* weight;
  const float* shift;
  struct K { float mean, scale, shift; };
  __device__ K channel(long long c) const {
    return K{mean[c], bn_scale(invstd[c], weight, c), shift ? shift[c] : 0.f};
  }
  __device__ void accumulate(const K& k, float a, float b, float& s0, float& s1) const {
    const float g = bn_value(a, k.mean, k.scale, k.shift) > 0.f ? b : 0.f;
    s0 += g;
    s1 += g * (a - k.mean);
  }
};
struct BnReluBwdApplyF {
  const float4* coef;  // (mean, k1, mean_dbeta, k4)
  const float* invstd;
  const float* weight;
  const float* shift;
  struct K { float mean, k1, mb, k4, scale, shift; };
  __device__ K channel(long long c) const {
    const float4 v = coef[c];
    return K{v.x, v.y, v.z, v.w, bn_scale(invstd[c], weight, c), shift ? shift[c] : 0.f};
  }
  __device__ float apply(const K& k, float a, float b) const {
    const float g = bn_value(a, k.mean, k.scale, k.shift) > 0.f ? b : 0.f;
    return k.k1 * (g - k.mb - (a - k.mean) * k.k4);
  }
};

struct BnBwdApplyF {  // a = x, b = dy: dx = k1 * (dy - mb - (x - mean) * k4)
  const float4* coef;  // (mean, k1, mean_dbeta, k4)
  struct K { float mean, k1, mb, k4; };
  __device__ K channel(long long c) const {
    const float4 v = coef[c];
    return K{v.x, v.y, v.z, v.w};
  }
  __device__ float apply(const K& k, float a, float b) const {
    return k.k1 * (b - k.mb - (a - k.mean) * k.k4);
  }
};

// y = relu(batchnorm(x) + addend) and the bit mask of the predicate: the last batchnorm of a
// residual block fused with the block's join.  A thread owns G consecutive elements of one
// channel row (G = 8 when rows are a multiple of 8 elements, else 4) and one mask byte:
// bit j of byte (offset / G) belongs to element offset + j.
template <int G>
__global__ void __launch_bounds__(kChanThreads)
bn_add_relu_apply_kernel(const float* __restrict__ x, const float* __restrict__ addend,
                         float* __restrict__ y, uint8_t* __restrict__ mask, ChannelGeo g,
                         const float* __restrict__ mean, const float* __restrict__ scale,
                         const float* __restrict__ shift) {
  constexpr int NV = G / 4;
  const long long c = blockIdx.x;
  const float m = mean[c], sc = scale[c], sh = shift ? shift[c] : 0.f;
  long long begin = (long long)blockIdx.y * g.chunk;
  long long end = begin + g.chunk;
  if (end > g.per_channel) end = g.per_channel;
  for (long long e = begin + (long long)threadIdx.x * G; e < end; e += (long long)kChanThreads * G) {
    const long long off = channel_elem_offset(g, c, e);
    float4 a[NV], s[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      a[v] = *reinterpret_cast<const float4*>(x + off + 4 * v);
      s[v] = *reinterpret_cast<const float4*>(addend + off + 4 * v);
    }
    unsigned bits = 0;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const float z[4] = {bn_value(a[v].x, m, sc, sh) + s[v].x, bn_value(a[v].y, m, sc, sh) + s[v].y,
                          bn_value(a[v].z, m, sc, sh) + s[v].z, bn_value(a[v].w, m, sc, sh) + s[v].w};
      float r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        r[j] = z[j] > 0.f ? z[j] : (z[j] != z[j] ? z[j] : 0.f);
        bits |= (z[j] > 0.f ? 1u : 0u) << (4 * v + j);
      }
      *reinterpret_cast<float4*>(y + off + 4 * v) = make_float4(r[0], r[1], r[2], r[3]);
    }
    mask[off / G] = (uint8_t)bits;
  }
}

// First pass of the batch-norm gradient at a residual block's tail.  The gradient that reaches
// the batch-norm is the relu gradient of the join, mask ? (ga + gb) : 0, where ga and gb come
// from the join's two consumers (gb may be null).  Instead of a relu-gradient kernel that
// writes that tensor and a reduction pass that reads it back, this pass forms it, writes it
// (it is also the shortcut's gradient and the apply pass's input) and reduces it in one go:
// s0 = sum g, s1 = sum g * (x - mean).  G consecutive elements of a channel row per thread,
// mask layout as above.
template <int G>
__global__ void __launch_bounds__(kChanThreads)
bn_tail_backward_reduce_kernel(const float* __restrict__ x, const float* __restrict__ ga,
                               const float* __restrict__ gb, const uint8_t* __restrict__ mask,
                               float* __restrict__ gz, float2* __restrict__ partial, ChannelGeo g,
                               const float* __restrict__ mean) {
  constexpr int NV = G / 4;
  __shared__ float scratch[32];
  const long long c = blockIdx.x;
  const float m = mean[c];
  long long begin = (long long)blockIdx.y * g.chunk;
  long long end = begin + g.chunk;
  if (end > g.per_channel) end = g.per_channel;
  float s0 = 0.f, s1 = 0.f;
  for (long long e = begin + (long long)threadIdx.x * G; e < end; e += (long long)kChanThreads * G) {
    const long long off = channel_elem_offset(g, c, e);
    float4 xv[NV], av[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      xv[v] = *reinterpret_cast<const float4*>(x + off + 4 * v);
      av[v] = *reinterpret_cast<const float4*>(ga + off + 4 * v);
      if (gb) {
        const float4 b = *reinterpret_cast<const float4*>(gb + off + 4 * v);
        av[v] = make_float4(av[v].x + b.x, av[v].y + b.y, av[v].z + b.z, av[v].w + b.w);
      }
    }
    const unsigned bits = mask[off / G];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const unsigned b4 = bits >> (4 * v);
      const float4 r = make_float4(b4 & 1u ? av[v].x : 0.f, b4 & 2u ? av[v].y : 0.f,
                                   b4 & 4u ? av[v].z : 0.f, b4 & 8u ? av[v].w : 0.f);
      *reinterpret_cast<float4*>(gz + off + 4 * v) = r;
      s0 += (r.x + r.y) + (r.z + r.w);
      s1 += r.x * (xv[v].x - m) + r.y * (xv[v].y - m) + r.z * (xv[v].z - m) + r.w * (xv[v].w - m);
    }
  }
  s0 = block_sum(s0, scratch);
  s1 = block_sum(s1, scratch);
  if (threadIdx.x == 0) partial[c * g.splits + blockIdx.y] = make_float2(s0, s1);
}

// The same two passes for channel rows of any length (one element and one mask byte per
// thread step): the 7 x 7 planes of the last ResNet stage.
__global__ void __launch_bounds__(kChanThreads)
bn_add_relu_apply_scalar_kernel(const float* __restrict__ x, const float* __restrict__ addend,
                                float* __restrict__ y, uint8_t* __restrict__ mask, ChannelGeo g,
                                const float* __restrict__ mean, const float* __restrict__ scale,
                                const float* __restrict__ shift) {
  const long long c = blockIdx.x;
  const float m = mean[c], sc = scale[c], sh = shift ? shift[c] : 0.f;
  long long begin = (long long)blockIdx.y * g.chunk;
  long long end = begin + g.chunk;
  if (end > g.per_channel) end = g.per_channel;
  for (long long e = begin + threadIdx.x; e < end; e += kChanThreads) {
    const long long off = channel_elem_offset(g, c, e);
    const float z = bn_value(x[off], m, sc, sh) + addend[off];
    y[off] = z > 0.f ? z : (z != z ? z : 0.f);
    mask[off] = z > 0.f ? 1 : 0;
  }
}
__global__ void __launch_bounds__(kChanThreads)
bn_tail_backward_reduce_scalar_kernel(const float* __restrict__ x, const float* __restrict__ ga,
                                      const float* __restrict__ gb,
                                      const uint8_t* __restrict__ mask, float* __restrict__ gz,
                                      float2* __restrict__ partial, ChannelGeo g,
                                      const float* __restrict__ mean) {
  __shared__ float scratch[32];
  const long long c = blockIdx.x;
  const float m = mean[c];
  long long begin = (long long)blockIdx.y * g.chunk;
  long long end = begin + g.chunk;
  if (end > g.per_channel) end = g.per_channel;
  float s0 = 0.f, s1 = 0.f;
  for (long long e = begin + threadIdx.x; e < end; e += kChanThreads) {
    const long long off = channel_elem_offset(g, c, e);
    const float r = mask[off] ? (gb ? ga[off] + gb[off] : ga[off]) : 0.f;
    gz[off] = r;
    s0 += r;
    s1 += r * (x[off] - m);
  }
  s0 = block_sum(s0, scratch);
  s1 = block_sum(s1, scratch);
  if (threadIdx.x == 0) partial[c * g.splits + blockIdx.y] = make_float2(s0, s1);
}

// The two passes above for channels-last tensors ([pixels][channels], channels a multiple of 8):
// a thread owns 8 consecutive channels of a pixel = two 16-byte vectors and one mask byte (bit j
// of byte offset / 8 belongs to element offset + j, the layout of flb200_relu_forward_mask).  A
// CTA is CO channel octets x 256 / CO row lanes (CO a power of two <= 32).
struct OctetTiling { int co_shift, col_blocks; };
inline OctetTiling octet_tiling(long long channels) {
  const long long octs = channels / 8;
  int shift = 0;
  while ((2LL << shift) <= octs && shift < 5) ++shift;
  return OctetTiling{shift, (int)((octs + (1LL << shift) - 1) >> shift)};
}

__global__ void __launch_bounds__(256)
bn_add_relu_apply_cl_kernel(const float* __restrict__ x, const float* __restrict__ addend,
                            float* __restrict__ y, uint8_t* __restrict__ mask, long long rows,
                            long long channels, long long rows_per_split, int co_shift,
                            const float* __restrict__ mean, const float* __restrict__ scale,
                            const float* __restrict__ shift) {
  const int co = 1 << co_shift, rl = 256 >> co_shift;
  const int tq = threadIdx.x & (co - 1), tr = threadIdx.x >> co_shift;
  const long long c = ((long long)blockIdx.x * co + tq) * 8;
  if (c >= channels) return;
  float m[8], sc[8], sh[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    m[j] = mean[c + j];
    sc[j] = scale[c + j];
    sh[j] = shift ? shift[c + j] : 0.f;
  }
  const long long r0 = (long long)blockIdx.y * rows_per_split;
  long long r1 = r0 + rows_per_split;
  if (r1 > rows) r1 = rows;
  for (long long r = r0 + tr; r < r1; r += rl) {
    const long long off = r * channels + c;
    float a[8], s[8], z[8];
    *reinterpret_cast<float4*>(a) = *reinterpret_cast<const float4*>(x + off);
    *reinterpret_cast<float4*>(a + 4) = *reinterpret_cast<const float4*>(x + off + 4);
    *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(addend + off);
    *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(addend + off + 4);
    unsigned bits = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float v = bn_value(a[j], m[j], sc[j], sh[j]) + s[j];
      z[j] = v > 0.f ? v : (v != v ? v : 0.f);
      bits |= (v > 0.f ? 1u : 0u) << j;
    }
    *reinterpret_cast<float4*>(y + off) = make_float4(z[0], z[1], z[2], z[3]);
    *reinterpret_cast<float4*>(y + off + 4) = make_float4(z[4], z[5], z[6], z[7]);
    mask[off >> 3] = (uint8_t)bits;
  }
}

__global__ void __launch_bounds__(256)
bn_tail_backward_reduce_cl_kernel(const float* __restrict__ x, const float* __restrict__ ga,
                                  const float* __restrict__ gb, const uint8_t* __restrict__ mask,
                                  float* __restrict__ gz, float2* __restrict__ partial,
                                  long long rows, long long channels, int splits,
                                  long long rows_per_split, int co_shift,
                                  const float* __restrict__ mean) {
  __shared__ float sh0[2048];
  __shared__ float sh1[2048];
  const int co = 1 << co_shift, rl = 256 >> co_shift;
  const int tq = threadIdx.x & (co - 1), tr = threadIdx.x >> co_shift;
  const long long c = ((long long)blockIdx.x * co + tq) * 8;
  float s0[8], s1[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s0[j] = s1[j] = 0.f;
  if (c < channels) {
    float m[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) m[j] = mean[c + j];
    const long long r0 = (long long)blockIdx.y * rows_per_split;
    long long r1 = r0 + rows_per_split;
    if (r1 > rows) r1 = rows;
    for (long long r = r0 + tr; r < r1; r += rl) {
      const long long off = r * channels + c;
      float xv[8], av[8];
      *reinterpret_cast<float4*>(xv) = *reinterpret_cast<const float4*>(x + off);
      *reinterpret_cast<float4*>(xv + 4) = *reinterpret_cast<const float4*>(x + off + 4);
      *reinterpret_cast<float4*>(av) = *reinterpret_cast<const float4*>(ga + off);
      *reinterpret_cast<float4*>(av + 4) = *reinterpret_cast<const float4*>(ga + off + 4);
      if (gb) {
        float bv[8];
        *reinterpret_cast<float4*>(bv) = *reinterpret_cast<const float4*>(gb + off);
        *reinterpret_cast<float4*>(bv + 4) = *reinterpret_cast<const float4*>(gb + off + 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) av[j] += bv[j];
      }
      const unsigned bits = mask[off >> 3];
      float rv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        rv[j] = (bits >> j) & 1u ? av[j] : 0.f;
        s0[j] += rv[j];
        s1[j] += rv[j] * (xv[j] - m[j]);
      }
      *reinterpret_cast<float4*>(gz + off) = make_float4(rv[0], rv[1], rv[2], rv[3]);
      *reinterpret_cast<float4*>(gz + off + 4) = make_float4(rv[4], rv[5], rv[6], rv[7]);
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    sh0[(tr << (co_shift + 3)) + tq * 8 + j] = s0[j];
    sh1[(tr << (co_shift + 3)) + tq * 8 + j] = s1[j];
  }
  __syncthreads();
  if ((int)threadIdx.x < 8 * co) {
    const long long cc = (long long)blockIdx.x * co * 8 + threadIdx.x;
    if (cc < channels) {
      float t0 = 0.f, t1 = 0.f;
      for (int i = 0; i < rl; ++i) {
        t0 += sh0[(i << (co_shift + 3)) + threadIdx.x];
        t1 += sh1[(i << (co_shift + 3)) + threadIdx.x];
      }
      partial[cc * splits + blockIdx.y] = make_float2(t0, t1);
    }
  }
}

// Affine part of fl::LayerNorm over rows of features: y = xhat * gamma + beta, and its gradient
// chain dgamma = sum_rows dy * xhat, dbeta = sum_rows dy, dxhat = dy * gamma.
struct AffineFwdF {
  const float* weight;
  const float* bias;
  struct K { float w, b; };
  __device__ K channel(long long c) const { return K{weight[c], bias ? bias[c] : 0.f}; }
  __device__ float apply(const K& k, float a, float) const { return __fmaf_rn(a, k.w, k.b); }
};
struct AffineBwdReduceF {  // a = dy, b = xhat
  struct K {};
  __device__ K channel(long long) const { return K{}; }
  __device__ void accumulate(const K&, float a, float b, float& s0, float& s1) const {
    s0 += a;
    s1 += a * b;
  }
};
struct ScaleF {  // a = dy
  const float* weight;
  struct K { float w; };
  __device__ K channel(long long c) const { return K{weight[c]}; }
  __device__ float apply(const K& k, float a, float) const { return a * k.w; }
};

struct BiasAddF {
  const float* bias;
  struct K { float b; };
  __device__ K channel(long long c) const { return K{bias[c]}; }
  __device__ float apply(const K& k, float a, float) const { return a + k.b; }
};

// ----------------------------------------------------- finalize kernels
// One warp per channel: the lanes add the channel's per-split partial sums (double), lane 0
// finishes.  kFinThreads threads per CTA = kFinThreads / 32 channels.
constexpr int kFinThreads = 128;
inline unsigned fin_grid(long long channels) {
  return (unsigned)((channels * 32 + kFinThreads - 1) / kFinThreads);
}
__device__ __forceinline__ bool fin_sums(const float2* __restrict__ partial, int splits,
                                         long long channels, long long* c_out, double* s0_out,
                                         double* s1_out) {
  const long long c = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (c >= channels) return false;  // whole warps only: c is uniform across a warp
  double s0 = 0.0, s1 = 0.0;
  for (int i = lane; i < splits; i += 32) {
    const float2 p = partial[c * splits + i];
    s0 += (double)p.x;
    s1 += (double)p.y;
  }
  *s0_out = warp_sum(s0);
  *s1_out = warp_sum(s1);
  *c_out = c;
  return lane == 0;
}

__global__ void sum_finalize_kernel(const float2* __restrict__ partial, int splits,
                                    long long channels, float* __restrict__ out) {
  long long c;
  double s0, s1;
  if (!fin_sums(partial, splits, channels, &c, &s0, &s1)) return;
  out[c] = (float)s0;
}

// Turns the shifted sums into mean / inverse std, updates the running stats and
// prepares the per-channel scale (invstd * gamma) for the apply pass.
__global__ void bn_stats_finalize_kernel(const float2* __restrict__ partial, int splits,
                                         long long channels, double count,
                                         const void* __restrict__ x, long long inner, int dtype,
                                         const float* __restrict__ weight, double eps,
                                         double momentum, float* __restrict__ running_mean,
                                         float* __restrict__ running_var,
                                         float* __restrict__ save_mean,
                                         float* __restrict__ save_invstd,
                                         float* __restrict__ scale) {
  long long c;
  double s0, s1;
  if (!fin_sums(partial, splits, channels, &c, &s0, &s1)) return;
  StatsF sf{reinterpret_cast<const float*>(x), inner, dtype};
  const double shift = (double)sf.channel(c).shift;
  const double md = s0 / count;
  double var = s1 / count - md * md;
  if (var < 0.0) var = 0.0;
  const double mean = md + shift;
  const double invstd = 1.0 / sqrt(var + eps);
  save_mean[c] = (float)mean;
  save_invstd[c] = (float)invstd;
  scale[c] = bn_scale((float)invstd, weight, c);
  if (running_mean) running_mean[c] = (float)((1.0 - momentum) * running_mean[c] + momentum * mean);
  if (running_var) {
    const double unbiased = count > 1.0 ? var * count / (count - 1.0) : var;
    running_var[c] = (float)((1.0 - momentum) * running_var[c] + momentum * unbiased);
  }
}

// The same from the statistics matrix a convolution's epilogue wrote for x (EpiStats,
// tc_kernel.cuh): `partial` holds the column sums of its [groups][2 * channels] rows in the
// making — sums of x in columns [0, channels), sums of x^2 in [channels, 2 * channels).
__global__ void bn_stats_finalize_matrix_kernel(const float2* __restrict__ partial, int splits,
                                                long long channels, double count,
                                                const float* __restrict__ weight, double eps,
                                                double momentum, float* __restrict__ running_mean,
                                                float* __restrict__ running_var,
                                                float* __restrict__ save_mean,
                                                float* __restrict__ save_invstd,
                                                float* __restrict__ scale) {
  const long long c = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (c >= channels) return;  // whole warps only
  double s = 0.0, q = 0.0;
  for (int i = lane; i < splits; i += 32) {
    s += (double)partial[c * splits + i].x;
    q += (double)partial[(channels + c) * splits + i].x;
  }
  s = warp_sum(s);
  q = warp_sum(q);
  if (lane != 0) return;
  const double mean = s / count;
  double var = q / count - mean * mean;
  if (var < 0.0) var = 0.0;
  const double invstd = 1.0 / sqrt(var + eps);
  save_mean[c] = (float)mean;
  save_invstd[c] = (float)invstd;
  scale[c] = bn_scale((float)invstd, weight, c);
  if (running_mean) running_mean[c] = (float)((1.0 - momentum) * running_mean[c] + momentum * mean);
  if (running_var) {
    const double unbiased = count > 1.0 ? var * count / (count - 1.0) : var;
    running_var[c] = (float)((1.0 - momentum) * running_var[c] + momentum * unbiased);
  }
}

__global__ void affine_bwd_finalize_kernel(const float2* __restrict__ partial, int splits,
                                           long long channels, float* __restrict__ grad_weight,
                                           float* __restrict__ grad_bias) {
  long long c;
  double s0, s1;
  if (!fin_sums(partial, splits, channels, &c, &s0, &s1)) return;
  if (grad_bias) grad_bias[c] = (float)s0;
  if (grad_weight) grad_weight[c] = (float)s1;
}

__global__ void bn_infer_prepare_kernel(long long channels, const float* __restrict__ weight,
                                        const float* __restrict__ running_var, double eps,
                                        float* __restrict__ scale) {
  const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const double invstd = 1.0 / sqrt((double)running_var[c] + eps);
  scale[c] = (float)(invstd * (weight ? (double)weight[c] : 1.0));
}

__global__ void bn_bwd_finalize_kernel(const float2* __restrict__ partial, int splits,
                                       long long channels, double count,
                                       const float* __restrict__ weight,
                                       const float* __restrict__ save_mean,
                                       const float* __restrict__ save_invstd,
                                       float* __restrict__ grad_weight,
                                       float* __restrict__ grad_bias,
                                       float4* __restrict__ coef) {
  long long c;
  double s0, s1;
  if (!fin_sums(partial, splits, channels, &c, &s0, &s1)) return;
  const double invstd = (double)save_invstd[c];
  const double gamma = weight ? (double)weight[c] : 1.0;
  grad_bias[c] = (float)s0;
  grad_weight[c] = (float)(s1 * invstd);
  coef[c] = make_float4(save_mean[c], (float)(gamma * invstd), (float)(s0 / count),
                        (float)(invstd * invstd * s1 / count));
}

// ------------------------------------------------------------ launchers
template <typename T, int NIN, typename F>
int launch_reduce(const char* name, const void* a, const void* b, float2* partial,
                  long long outer, long long channels, long long inner, F f, int* splits_out,
                  cudaStream_t st) {
  if (inner == 1) {
    const int splits = column_splits(outer, channels);
    const long long rps = (outer + splits - 1) / splits;
    if constexpr (std::is_same<T, float>::value) {
      if (channels % 4 == 0 && aligned16(a) && (NIN == 1 || aligned16(b))) {
        const ColumnTiling ct = column_tiling(channels);
        dim3 vgrid((unsigned)ct.col_blocks, (unsigned)splits);
        column_reduce_vec_kernel<NIN, F><<<vgrid, 256, 0, st>>>(
            static_cast<const float*>(a), static_cast<const float*>(b), partial, outer, channels,
            splits, rps, ct.cq_shift, f);
        FLB200_AFTER_LAUNCH(name);
        *splits_out = splits;
        return FLB200_OK;
      }
    }
    dim3 grid((unsigned)((channels + 31) / 32), (unsigned)splits);
    column_reduce_kernel<T, NIN, F><<<grid, 256, 0, st>>>(
        static_cast<const T*>(a), static_cast<const T*>(b), partial, outer, channels, splits, rps,
        f);
    FLB200_AFTER_LAUNCH(name);
    *splits_out = splits;
    return FLB200_OK;
  }
  const ChannelGeo g = make_channel_geo(outer, channels, inner);
  const bool vec = inner % Vec16<T>::N == 0 && aligned16(a) && (NIN == 1 || aligned16(b));
  dim3 grid((unsigned)channels, (unsigned)g.splits);
  if (vec)
    channel_reduce_kernel<T, NIN, true, F><<<grid, kChanThreads, 0, st>>>(
        static_cast<const T*>(a), static_cast<const T*>(b), partial, g, f);
  else
    channel_reduce_kernel<T, NIN, false, F><<<grid, kChanThreads, 0, st>>>(
        static_cast<const T*>(a), static_cast<const T*>(b), partial, g, f);
  FLB200_AFTER_LAUNCH(name);
  *splits_out = g.splits;
  return FLB200_OK;
}

template <typename T, int NIN, typename F>
int launch_apply(const char* name, const void* a, const void* b, void* out, long long outer,
                 long long channels, long long inner, F f, cudaStream_t st) {
  if (inner == 1) {
    if constexpr (std::is_same<T, float>::value) {
      if (channels % 4 == 0 && aligned16(a) && aligned16(out) && (NIN == 1 || aligned16(b))) {
        const ColumnTiling ct = column_tiling(channels);
        // about 16 CTAs per SM, at least 32 rows each
        long long splits = (16LL * device_info().sm_count + ct.col_blocks - 1) / ct.col_blocks;
        if (splits > (outer + 31) / 32) splits = (outer + 31) / 32;
        if (splits > 65535) splits = 65535;
        if (splits < 1) splits = 1;
        const long long rps = (outer + splits - 1) / splits;
        dim3 vgrid((unsigned)ct.col_blocks, (unsigned)splits);
        column_apply_vec_kernel<NIN, F><<<vgrid, 256, 0, st>>>(
            static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(out),
            outer, channels, rps, ct.cq_shift, f);
        FLB200_AFTER_LAUNCH(name);
        return FLB200_OK;
      }
    }
    const int grid = grid_for(outer * channels, 256 * 4);
    column_apply_kernel<T, NIN, F><<<grid, 256, 0, st>>>(
        static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), outer, channels,
        f);
    FLB200_AFTER_LAUNCH(name);
    return FLB200_OK;
  }
  const ChannelGeo g = make_channel_geo(outer, channels, inner);
  const bool vec = inner % Vec16<T>::N == 0 && aligned16(a) && aligned16(out) &&
                   (NIN == 1 || aligned16(b));
  dim3 grid((unsigned)channels, (unsigned)g.splits);
  if (vec)
    channel_apply_kernel<T, NIN, true, F><<<grid, kChanThreads, 0, st>>>(
        static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), g, f);
  else
    channel_apply_kernel<T, NIN, false, F><<<grid, kChanThreads, 0, st>>>(
        static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), g, f);
  FLB200_AFTER_LAUNCH(name);
  return FLB200_OK;
}

#define FLB200_DISPATCH_DTYPE(dtype, name, CALL)                                   \
  switch (dtype) {                                                                 \
    case FLB200_F32: { using T = float; CALL; } break;                             \
    case FLB200_F16: { using T = __half; CALL; } break;                            \
    case FLB200_BF16: { using T = __nv_bfloat16; CALL; } break;                    \
    default: return fail(FLB200_UNSUPPORTED, "%s: unknown dtype %d", name, dtype); \
  }

int check_geo(const char* name, long long outer, long long channels, long long inner) {
  FLB200_REQUIRE(outer >= 1 && channels >= 1 && inner >= 1, "%s: empty geometry", name);
  FLB200_REQUIRE(channels < 0x7fffffffLL, "%s: too many channels", name);
  return FLB200_OK;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace
}  // namespace flb200

using namespace flb200;

extern "C" {

size_t flb200_channel_sum_workspace_bytes(int64_t outer, int64_t channels, int64_t inner) {
  if (outer < 1 || channels < 1 || inner < 1) return 0;
  return channel_partial_bytes(outer, channels, inner);
}

int flb200_channel_sum(const void* in, float* out, int64_t outer, int64_t channels, int64_t inner,
                       int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  if (int st = check_geo("channel_sum", outer, channels, inner)) return st;
  FLB200_REQUIRE(in && out, "channel_sum: null pointer");
  if (workspace_bytes < channel_partial_bytes(outer, channels, inner) || !workspace)
    return fail(FLB200_WORKSPACE_TOO_SMALL, "channel_sum: workspace %zu < %zu", workspace_bytes,
                channel_partial_bytes(outer, channels, inner));
  cudaStream_t st = as_stream(stream);
  float2* partial = static_cast<float2*>(workspace);
  int splits = 0;
  int rc = FLB200_OK;
  FLB200_DISPATCH_DTYPE(dtype, "channel_sum",
                        rc = (launch_reduce<T, 1>("channel_sum", in, nullptr, partial, outer,
                                                  channels, inner, SumF{}, &splits, st)));
  if (rc) return rc;
  sum_finalize_kernel<<<fin_grid(channels), kFinThreads, 0, st>>>(partial, splits, channels, out);
  FLB200_AFTER_LAUNCH("channel_sum_finalize");
  return FLB200_OK;
}

// ---- channel sum for callers that cannot hand over scratch memory ------------------------
// The partial sums of flb200_channel_sum normally live in scratch the caller allocates.  Some
// callers have no way to get device memory at the moment of the call: code that runs inside a
// host framework's memory-manager callback (re-entering the allocator there would deadlock or
// recurse), an out-of-memory handler, or a plugin host that handed out its whole device budget at
// start-up and forbids cudaMalloc afterwards.  For them the partials go into this fixed array,
// which every GPU that loads the library holds from load until the process exits.
constexpr size_t kStaticScratchBytes = 1u << 20;  // 1 MiB
static __device__ __align__(256) unsigned char g_channel_sum_scratch[kStaticScratchBytes];

int flb200_channel_sum_static_scratch(const void* in, float* out, int64_t outer, int64_t channels,
                                      int64_t inner, int dtype, void* stream) {
  if (int st = check_geo("channel_sum_static_scratch", outer, channels, inner)) return st;
  const size_t need = channel_partial_bytes(outer, channels, inner);
  if (need > kStaticScratchBytes)
    return fail(FLB200_INVALID_ARG,
                "channel_sum_static_scratch: this shape needs %zu bytes of partial sums, the "
                "built-in scratch holds %zu; use flb200_channel_sum with caller scratch",
                need, (size_t)kStaticScratchBytes);
  // In host code the array's name is only a handle; the device address has to be looked up,
  // once per device, with that device current.  This happens on the first call per device
  // (guarded, so that two host threads making that first call at once do not race); the
  // lookup can make the CUDA runtime load this library's device code, which may allocate, so
  // the no-allocation promise holds from the second call on: callers warm each device up once
  // at start-up.
  static std::once_flag looked_up[64];
  static void* device_addr[64] = {nullptr};
  static cudaError_t lookup_error[64];
  int dev = 0;
  FLB200_CUDA_CHECK(cudaGetDevice(&dev));
  FLB200_REQUIRE(dev >= 0 && dev < 64, "channel_sum_static_scratch: device ordinal %d out of range",
                 dev);
  std::call_once(looked_up[dev], [dev] {
    void* p = nullptr;
    lookup_error[dev] = cudaGetSymbolAddress(&p, g_channel_sum_scratch);
    device_addr[dev] = lookup_error[dev] == cudaSuccess ? p : nullptr;
  });
  if (!device_addr[dev]) {
    (void)cudaGetLastError();
    return fail(FLB200_LAUNCH_FAILURE,
                "channel_sum_static_scratch: cudaGetSymbolAddress failed on device %d: %s", dev,
                cudaGetErrorString(lookup_error[dev]));
  }
  // Every partial is written before it is read, so stale contents of earlier calls do no harm.
  return flb200_channel_sum(in, out, outer, channels, inner, dtype, device_addr[dev],
                            kStaticScratchBytes, stream);
}

int flb200_channel_bias_add(const void* x, const float* bias, void* y, int64_t outer,
                            int64_t channels, int64_t inner, int dtype, void* stream) {
  if (int st = check_geo("channel_bias_add", outer, channels, inner)) return st;
  FLB200_REQUIRE(x && bias && y, "channel_bias_add: null pointer");
  int rc = FLB200_OK;
  FLB200_DISPATCH_DTYPE(dtype, "channel_bias_add",
                        rc = (launch_apply<T, 1>("channel_bias_add", x, nullptr, y, outer, channels,
                                                 inner, BiasAddF{bias}, as_stream(stream))));
  return rc;
}

size_t flb200_layernorm_affine_workspace_bytes(int64_t rows, int64_t features) {
  if (rows < 1 || features < 1) return 0;
  return channel_partial_bytes(rows, features, 1);
}

int flb200_layernorm_affine_forward(const void* xhat, const float* weight, const float* bias,
                                    void* y, int64_t rows, int64_t features, int dtype,
                                    void* stream) {
  if (int st = check_geo("layernorm_affine_forward", rows, features, 1)) return st;
  FLB200_REQUIRE(xhat && weight && y, "layernorm_affine_forward: null pointer");
  int rc = FLB200_OK;
  FLB200_DISPATCH_DTYPE(dtype, "layernorm_affine_forward",
                        rc = (launch_apply<T, 1>("layernorm_affine_forward", xhat, nullptr, y, rows,
                                                 features, 1, AffineFwdF{weight, bias},
                                                 as_stream(stream))));
  return rc;
}

int flb200_layernorm_affine_backward(const void* grad_y, const void* xhat, const float* weight,
                                     void* grad_xhat, float* grad_weight, float* grad_bias,
                                     int64_t rows, int64_t features, int dtype, void* workspace,
                                     size_t workspace_bytes, void* stream) {
  if (int st = check_geo("layernorm_affine_backward", rows, features, 1)) return st;
  FLB200_REQUIRE(grad_y && xhat && (weight || !grad_xhat), "layernorm_affine_backward: null pointer");
  cudaStream_t st = as_stream(stream);
  int rc = FLB200_OK;
  if (grad_weight || grad_bias) {
    const size_t need = channel_partial_bytes(rows, features, 1);
    if (!workspace || workspace_bytes < need)
      return fail(FLB200_WORKSPACE_TOO_SMALL, "layernorm_affine_backward: workspace %zu < %zu",
                  workspace_bytes, need);
    float2* partial = static_cast<float2*>(workspace);
    int splits = 0;
    FLB200_DISPATCH_DTYPE(dtype, "layernorm_affine_backward",
                          rc = (launch_reduce<T, 2>("layernorm_affine_backward_reduce", grad_y, xhat,
                                                    partial, rows, features, 1, AffineBwdReduceF{},
                                                    &splits, st)));
    if (rc) return rc;
    affine_bwd_finalize_kernel<<<fin_grid(features), kFinThreads, 0, st>>>(
        partial, splits, features, grad_weight, grad_bias);
    FLB200_AFTER_LAUNCH("layernorm_affine_backward_finalize");
  }
  if (grad_xhat) {
    FLB200_DISPATCH_DTYPE(dtype, "layernorm_affine_backward",
                          rc = (launch_apply<T, 1>("layernorm_affine_backward_apply", grad_y, nullptr,
                                                   grad_xhat, rows, features, 1, ScaleF{weight},
                                                   st)));
  }
  return rc;
}

int flb200_batchnorm_geometry(const int64_t* shape, int ndim, const int32_t* axes, int naxes,
                              flb200_batchnorm_desc* out) {
  FLB200_REQUIRE(shape && axes && out, "batchnorm_geometry: null pointer");
  FLB200_REQUIRE(ndim >= 1 && ndim <= 8 && naxes >= 1 && naxes <= ndim,
                 "batchnorm_geometry: bad rank (ndim %d, naxes %d)", ndim, naxes);
  int min_axis = axes[0], max_axis = axes[0];
  int64_t nfeatures = 1, elements = 1;
  for (int i = 0; i < ndim; ++i) {
    FLB200_REQUIRE(shape[i] >= 1, "batchnorm_geometry: empty dimension %d", i);
    elements *= shape[i];
  }
  for (int i = 0; i < naxes; ++i) {
    // "batchnorm - passed axes ... exceeds the number of dimensions of the input"
    FLB200_REQUIRE(axes[i] >= 0 && axes[i] <= ndim - 1,
                   "batchnorm - passed axes (axis value %d) exceeds the number of dimensions of "
                   "the input (%d)",
                   axes[i], ndim);
    for (int j = 0; j < i; ++j)
      FLB200_REQUIRE(axes[j] != axes[i], "batchnorm_geometry: duplicate axis %d", axes[i]);
    nfeatures *= shape[axes[i]];
    if (axes[i] < min_axis) min_axis = axes[i];
    if (axes[i] > max_axis) max_axis = axes[i];
  }
  FLB200_REQUIRE(naxes == max_axis - min_axis + 1, "axis array should be continuous");
  if (min_axis == 0) {  // per-activation
    out->outer = elements / nfeatures;
    out->channels = nfeatures;
    out->inner = 1;
  } else {
    int64_t batch = 1;
    for (int i = max_axis + 1; i < ndim; ++i) batch *= shape[i];
    out->outer = batch;
    out->channels = nfeatures;
    out->inner = elements / (nfeatures * batch);
  }
  out->dtype = FLB200_F32;
  return FLB200_OK;
}

// Workspace layout: [partials][scale: C floats][coef: C float4]
size_t flb200_batchnorm_workspace_bytes(const flb200_batchnorm_desc* d) {
  if (!d || d->outer < 1 || d->channels < 1 || d->inner < 1) return 0;
  return align_up(channel_partial_bytes(d->outer, d->channels, d->inner), 256) +
         align_up((size_t)d->channels * sizeof(float), 256) +
         align_up((size_t)d->channels * sizeof(float4), 256);
}

static int batchnorm_forward_impl(bool relu, const void* addend, uint8_t* mask,
                                  const flb200_batchnorm_desc* d, const void* x,
                                  const float* weight, const float* bias, float* running_mean,
                                  float* running_var, float* save_mean, float* save_invstd,
                                  int train, double momentum, double epsilon, void* y,
                                  void* workspace, size_t workspace_bytes, void* stream,
                                  const float* stats = nullptr, long long stat_groups = 0) {
  FLB200_REQUIRE(d, "batchnorm_forward: null descriptor");
  if (int st = check_geo("batchnorm_forward", d->outer, d->channels, d->inner)) return st;
  FLB200_REQUIRE(x && y, "batchnorm_forward: null tensor");
  const size_t base_need = flb200_batchnorm_workspace_bytes(d);
  const size_t need =
      base_need + (stats ? channel_partial_bytes(stat_groups, 2 * d->channels, 1) : 0);
  if (!workspace || workspace_bytes < need)
    return fail(FLB200_WORKSPACE_TOO_SMALL, "batchnorm_forward: workspace %zu < %zu",
                workspace_bytes, need);
  cudaStream_t st = as_stream(stream);
  const long long C = d->channels;
  char* ws = static_cast<char*>(workspace);
  float2* partial = reinterpret_cast<float2*>(ws);
  float* scale =
      reinterpret_cast<float*>(ws + align_up(channel_partial_bytes(d->outer, C, d->inner), 256));
  int rc = FLB200_OK;
  const float* mean_ptr;
  if (train) {
    FLB200_REQUIRE(save_mean && save_invstd, "batchnorm_forward: training needs save_mean/save_invstd");
    if (stats) {
      // the producer of x took the sums in its epilogue: reduce its small matrix instead of x
      float2* p2 = reinterpret_cast<float2*>(ws + base_need);
      int splits = 0;
      rc = launch_reduce<float, 1>("batchnorm_stats_matrix", stats, nullptr, p2, stat_groups,
                                   2 * C, 1, SumF{}, &splits, st);
      if (rc) return rc;
      bn_stats_finalize_matrix_kernel<<<fin_grid(C), kFinThreads, 0, st>>>(
          p2, splits, C, (double)d->outer * (double)d->inner, weight, epsilon, momentum,
          running_mean, running_var, save_mean, save_invstd, scale);
      FLB200_AFTER_LAUNCH("batchnorm_stats_finalize_matrix");
    } else {
      int splits = 0;
      StatsF sf{static_cast<const float*>(x), d->inner, d->dtype};
      FLB200_DISPATCH_DTYPE(d->dtype, "batchnorm_forward",
                            rc = (launch_reduce<T, 1>("batchnorm_stats", x, nullptr, partial,
                                                      d->outer, C, d->inner, sf, &splits, st)));
      if (rc) return rc;
      bn_stats_finalize_kernel<<<fin_grid(C), kFinThreads, 0, st>>>(
          partial, splits, C, (double)d->outer * (double)d->inner, x, d->inner, d->dtype, weight,
          epsilon, momentum, running_mean, running_var, save_mean, save_invstd, scale);
      FLB200_AFTER_LAUNCH("batchnorm_stats_finalize");
    }
    mean_ptr = save_mean;
  } else {
    FLB200_REQUIRE(running_mean && running_var,
                   "batchnorm_forward: inference needs running_mean/running_var");
    bn_infer_prepare_kernel<<<(unsigned)((C + 127) / 128), 128, 0, st>>>(C, weight, running_var,
                                                                         epsilon, scale);
    FLB200_AFTER_LAUNCH("batchnorm_infer_prepare");
    mean_ptr = running_mean;
  }
  if (addend && d->inner == 1) {
    const OctetTiling ot = octet_tiling(C);
    long long splits = (16LL * device_info().sm_count + ot.col_blocks - 1) / ot.col_blocks;
    if (splits > (d->outer + 31) / 32) splits = (d->outer + 31) / 32;
    if (splits > 65535) splits = 65535;
    if (splits < 1) splits = 1;
    const long long rps = (d->outer + splits - 1) / splits;
    bn_add_relu_apply_cl_kernel<<<dim3((unsigned)ot.col_blocks, (unsigned)splits), 256, 0, st>>>(
        static_cast<const float*>(x), static_cast<const float*>(addend), static_cast<float*>(y),
        mask, d->outer, C, rps, ot.co_shift, mean_ptr, scale, bias);
    FLB200_AFTER_LAUNCH("batchnorm_add_relu_apply_channels_last");
  } else if (addend) {
    const ChannelGeo g = make_channel_geo(d->outer, C, d->inner);
    const dim3 grid((unsigned)C, (unsigned)g.splits);
    if (d->inner % 8 == 0)
      bn_add_relu_apply_kernel<8><<<grid, kChanThreads, 0, st>>>(
          static_cast<const float*>(x), static_cast<const float*>(addend), static_cast<float*>(y),
          mask, g, mean_ptr, scale, bias);
    else if (d->inner % 4 != 0)
      bn_add_relu_apply_scalar_kernel<<<grid, kChanThreads, 0, st>>>(
          static_cast<const float*>(x), static_cast<const float*>(addend), static_cast<float*>(y),
          mask, g, mean_ptr, scale, bias);
    else
      bn_add_relu_apply_kernel<4><<<grid, kChanThreads, 0, st>>>(
          static_cast<const float*>(x), static_cast<const float*>(addend), static_cast<float*>(y),
          mask, g, mean_ptr, scale, bias);
    FLB200_AFTER_LAUNCH("batchnorm_add_relu_apply");
  } else if (relu) {
    BnFwdApplyF<true> af{mean_ptr, scale, bias};
    FLB200_DISPATCH_DTYPE(d->dtype, "batchnorm_relu_forward",
                          rc = (launch_apply<T, 1>("batchnorm_relu_apply", x, nullptr, y, d->outer,
                                                   C, d->inner, af, st)));
  } else {
    BnFwdApplyF<false> af{mean_ptr, scale, bias};
    FLB200_DISPATCH_DTYPE(d->dtype, "batchnorm_forward",
                          rc = (launch_apply<T, 1>("batchnorm_apply", x, nullptr, y, d->outer, C,
                                                   d->inner, af, st)));
  }
  return rc;
}

int flb200_batchnorm_forward(const flb200_batchnorm_desc* d, const void* x, const float* weight,
                             const float* bias, float* running_mean, float* running_var,
                             float* save_mean, float* save_invstd, int train, double momentum,
                             double epsilon, void* y, void* workspace, size_t workspace_bytes,
                             void* stream) {
  return batchnorm_forward_impl(false, nullptr, nullptr, d, x, weight, bias, running_mean,
                                running_var, save_mean,
                                save_invstd, train, momentum, epsilon, y, workspace,
                                workspace_bytes, stream);
}
int flb200_batchnorm_relu_forward(const flb200_batchnorm_desc* d, const void* x,
                                  const float* weight, const float* bias, float* running_mean,
                                  float* running_var, float* save_mean, float* save_invstd,
                                  int train, double momentum, double epsilon, void* y,
                                  void* workspace, size_t workspace_bytes, void* stream) {
  return batchnorm_forward_impl(true, nullptr, nullptr, d, x, weight, bias, running_mean,
                                running_var, save_mean,
                                save_invstd, train, momentum, epsilon, y, workspace,
                                workspace_bytes, stream);
}

int flb200_batchnorm_add_relu_forward(const flb200_batchnorm_desc* d, const void* x,
                                      const void* addend, const float* weight, const float* bias,
                                      float* running_mean, float* running_var, float* save_mean,
                                      float* save_invstd, int train, double momentum,
                                      double epsilon, void* y, uint8_t* mask, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  FLB200_REQUIRE(d && addend && mask, "batchnorm_add_relu_forward: null argument");
  if (d->dtype != FLB200_F32 || (d->inner < 2 && d->channels % 8 != 0) || !aligned16(x) ||
      !aligned16(addend) || !aligned16(y))
    return fail(FLB200_UNSUPPORTED,
                "batchnorm_add_relu_forward: f32, 16-byte aligned tensors, in a spatial layout or "
                "channels-last with a multiple of 8 channels, only");
  return batchnorm_forward_impl(true, addend, mask, d, x, weight, bias, running_mean, running_var,
                                save_mean, save_invstd, train, momentum, epsilon, y, workspace,
                                workspace_bytes, stream);
}

size_t flb200_batchnorm_from_stats_workspace_bytes(const flb200_batchnorm_desc* d,
                                                   int64_t groups) {
  if (!d || groups < 1) return 0;
  const size_t base = flb200_batchnorm_workspace_bytes(d);
  return base == 0 ? 0 : base + channel_partial_bytes(groups, 2 * d->channels, 1);
}

int flb200_batchnorm_forward_from_stats(const flb200_batchnorm_desc* d, const void* x,
                                        const void* addend, int relu, const float* stats,
                                        int64_t groups, const float* weight, const float* bias,
                                        float* running_mean, float* running_var,
                                        float* save_mean, float* save_invstd, double momentum,
                                        double epsilon, void* y, uint8_t* mask, void* workspace,
                                        size_t workspace_bytes, void* stream) {
  FLB200_REQUIRE(d && stats && groups >= 1, "batchnorm_forward_from_stats: null argument");
  FLB200_REQUIRE(d->dtype == FLB200_F32 && aligned16(stats) && d->channels % 4 == 0,
                 "batchnorm_forward_from_stats: f32 tensors, channels a multiple of 4");
  if (addend) {
    FLB200_REQUIRE(mask, "batchnorm_forward_from_stats: the add + relu form writes a mask");
    if ((d->inner < 2 && d->channels % 8 != 0) || !aligned16(x) || !aligned16(addend) ||
        !aligned16(y))
      return fail(FLB200_UNSUPPORTED,
                  "batchnorm_forward_from_stats: the add + relu form needs 16-byte aligned "
                  "tensors, in a spatial layout or channels-last with a multiple of 8 channels");
  }
  return batchnorm_forward_impl(addend != nullptr || relu != 0, addend, mask, d, x, weight, bias,
                                running_mean, running_var, save_mean, save_invstd, 1, momentum,
                                epsilon, y, workspace, workspace_bytes, stream, stats, groups);
}

// tail_mask != null: grad_y / tail_gb are the join's two incoming gradients (tail_gb may be
// null), tail_sum receives mask ? grad_y + tail_gb : 0 and is what the batch-norm differentiates.
static int batchnorm_backward_impl(bool relu, const uint8_t* tail_mask, const void* tail_gb,
                                   void* tail_sum, const flb200_batchnorm_desc* d,
                                   const void* grad_y, const void* x, const float* weight,
                                   const float* bias,
                                   const float* save_mean, const float* save_invstd, void* grad_x,
                                   float* grad_weight, float* grad_bias, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  FLB200_REQUIRE(d, "batchnorm_backward: null descriptor");
  if (int st = check_geo("batchnorm_backward", d->outer, d->channels, d->inner)) return st;
  FLB200_REQUIRE(grad_y && x && save_mean && save_invstd && grad_x && grad_weight && grad_bias,
                 "batchnorm_backward: null tensor");
  const size_t need = flb200_batchnorm_workspace_bytes(d);
  if (!workspace || workspace_bytes < need)
    return fail(FLB200_WORKSPACE_TOO_SMALL, "batchnorm_backward: workspace %zu < %zu",
                workspace_bytes, need);
  cudaStream_t st = as_stream(stream);
  const long long C = d->channels;
  char* ws = static_cast<char*>(workspace);
  float2* partial = reinterpret_cast<float2*>(ws);
  size_t off = align_up(channel_partial_bytes(d->outer, C, d->inner), 256);
  off += align_up((size_t)C * sizeof(float), 256);
  float4* coef = reinterpret_cast<float4*>(ws + off);
  int rc = FLB200_OK, splits = 0;
  if (tail_mask && d->inner == 1) {
    const OctetTiling ot = octet_tiling(C);
    splits = column_splits(d->outer, C);
    const long long rps = (d->outer + splits - 1) / splits;
    bn_tail_backward_reduce_cl_kernel<<<dim3((unsigned)ot.col_blocks, (unsigned)splits), 256, 0,
                                        st>>>(
        static_cast<const float*>(x), static_cast<const float*>(grad_y),
        static_cast<const float*>(tail_gb), tail_mask, static_cast<float*>(tail_sum), partial,
        d->outer, C, splits, rps, ot.co_shift, save_mean);
    FLB200_AFTER_LAUNCH("batchnorm_tail_backward_reduce_channels_last");
    grad_y = tail_sum;
  } else if (tail_mask) {
    const ChannelGeo g = make_channel_geo(d->outer, C, d->inner);
    const dim3 grid((unsigned)C, (unsigned)g.splits);
    if (d->inner % 8 == 0)
      bn_tail_backward_reduce_kernel<8><<<grid, kChanThreads, 0, st>>>(
          static_cast<const float*>(x), static_cast<const float*>(grad_y),
          static_cast<const float*>(tail_gb), tail_mask, static_cast<float*>(tail_sum), partial, g,
          save_mean);
    else if (d->inner % 4 != 0)
      bn_tail_backward_reduce_scalar_kernel<<<grid, kChanThreads, 0, st>>>(
          static_cast<const float*>(x), static_cast<const float*>(grad_y),
          static_cast<const float*>(tail_gb), tail_mask, static_cast<float*>(tail_sum), partial, g,
          save_mean);
    else
      bn_tail_backward_reduce_kernel<4><<<grid, kChanThreads, 0, st>>>(
          static_cast<const float*>(x), static_cast<const float*>(grad_y),
          static_cast<const float*>(tail_gb), tail_mask, static_cast<float*>(tail_sum), partial, g,
          save_mean);
    FLB200_AFTER_LAUNCH("batchnorm_tail_backward_reduce");
    splits = g.splits;
    grad_y = tail_sum;
  } else if (relu) {
    BnReluBwdReduceF rf{save_mean, save_invstd, weight, bias};
    FLB200_DISPATCH_DTYPE(d->dtype, "batchnorm_relu_backward",
                          rc = (launch_reduce<T, 2>("batchnorm_relu_backward_reduce", x, grad_y,
                                                    partial, d->outer, C, d->inner, rf, &splits,
                                                    st)));
  } else {
    BnBwdReduceF rf{save_mean};
    FLB200_DISPATCH_DTYPE(d->dtype, "batchnorm_backward",
                          rc = (launch_reduce<T, 2>("batchnorm_backward_reduce", x, grad_y,
                                                    partial, d->outer, C, d->inner, rf, &splits,
                                                    st)));
  }
  if (rc) return rc;
  bn_bwd_finalize_kernel<<<fin_grid(C), kFinThreads, 0, st>>>(
      partial, splits, C, (double)d->outer * (double)d->inner, weight, save_mean, save_invstd,
      grad_weight, grad_bias, coef);
  FLB200_AFTER_LAUNCH("batchnorm_backward_finalize");
  if (relu) {
    BnReluBwdApplyF af{coef, save_invstd, weight, bias};
    FLB200_DISPATCH_DTYPE(d->dtype, "batchnorm_relu_backward",
                          rc = (launch_apply<T, 2>("batchnorm_relu_backward_apply", x, grad_y,
                                                   grad_x, d->outer, C, d->inner, af, st)));
  } else {
    BnBwdApplyF af{coef};
    FLB200_DISPATCH_DTYPE(d->dtype, "batchnorm_backward",
                          rc = (launch_apply<T, 2>("batchnorm_backward_apply", x, grad_y, grad_x,
                                                   d->outer, C, d->inner, af, st)));
  }
  return rc;
}

int flb200_batchnorm_backward(const flb200_batchnorm_desc* d, const void* grad_y, const void* x,
                              const float* weight, const float* save_mean,
                              const float* save_invstd, void* grad_x, float* grad_weight,
                              float* grad_bias, void* workspace, size_t workspace_bytes,
                              void* stream) {
  return batchnorm_backward_impl(false, nullptr, nullptr, nullptr, d, grad_y, x, weight, nullptr,
                                 save_mean, save_invstd,
                                 grad_x, grad_weight, grad_bias, workspace, workspace_bytes,
                                 stream);
}
int flb200_batchnorm_relu_backward(const flb200_batchnorm_desc* d, const void* grad_y,
                                   const void* x, const float* weight, const float* bias,
                                   const float* save_mean, const float* save_invstd,
                                   void* grad_x, float* grad_weight, float* grad_bias,
                                   void* workspace, size_t workspace_bytes, void* stream) {
  return batchnorm_backward_impl(true, nullptr, nullptr, nullptr, d, grad_y, x, weight, bias,
                                 save_mean, save_invstd, grad_x, grad_weight, grad_bias, workspace,
                                 workspace_bytes, stream);
}
int flb200_batchnorm_add_relu_backward(const flb200_batchnorm_desc* d, const uint8_t* mask,
                                       const void* grad_y_a, const void* grad_y_b, const void* x,
                                       const float* weight, const float* save_mean,
                                       const float* save_invstd, void* grad_sum, void* grad_x,
                                       float* grad_weight, float* grad_bias, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  FLB200_REQUIRE(d && mask && grad_y_a && grad_sum, "batchnorm_add_relu_backward: null argument");
  if (d->dtype != FLB200_F32 || (d->inner < 2 && d->channels % 8 != 0) || !aligned16(x) ||
      !aligned16(grad_y_a) || !aligned16(grad_sum) || (grad_y_b && !aligned16(grad_y_b)))
    return fail(FLB200_UNSUPPORTED,
                "batchnorm_add_relu_backward: f32, 16-byte aligned tensors, in a spatial layout or "
                "channels-last with a multiple of 8 channels, only");
  return batchnorm_backward_impl(false, mask, grad_y_b, grad_sum, d, grad_y_a, x, weight, nullptr,
                                 save_mean, save_invstd, grad_x, grad_weight, grad_bias, workspace,
                                 workspace_bytes, stream);
}

}  // extern "C"
