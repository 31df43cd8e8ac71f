// Per-channel reductions and per-channel affine passes over a tensor viewed as
// [outer][channels][inner] (row-major).  This is the one access pattern behind
// batchnorm / LayerNorm forward and backward, the convolution bias gradient and
// sumAs / tile of a bias, so they share these templates.
//
// Work split: grid = (channels, splits).  A CTA owns one channel and a
// contiguous range of that channel's outer*inner elements, walks it with
// 128-bit accesses when inner is a multiple of the vector width, and leaves two
// partial sums per (channel, split) in a small scratch array that a one-thread-
// per-channel kernel finishes in double precision.  The channel is constant per
// CTA, so the per-channel constants live in registers.
#pragma once
#include "common.cuh"

namespace flb200 {

constexpr int kChanThreads = 256;

struct ChannelGeo {
  long long outer, channels, inner;
  long long per_channel;  // outer * inner
  int splits;             // gridDim.y
  long long chunk;        // elements of one channel per split (multiple of 16)
};

// Picks the number of splits so that the grid fills the device a few times but
// a CTA still has at least 8K elements to amortise its reduction.
inline ChannelGeo make_channel_geo(long long outer, long long channels, long long inner) {
  ChannelGeo g;
  g.outer = outer;
  g.channels = channels;
  g.inner = inner;
  g.per_channel = outer * inner;
  const long long target_ctas = 4LL * 8 * device_info().sm_count;
  long long splits = (target_ctas + channels - 1) / channels;
  const long long max_by_work = (g.per_channel + 8191) / 8192;
  if (splits > max_by_work) splits = max_by_work;
  if (splits < 1) splits = 1;
  if (splits > 4096) splits = 4096;
  long long chunk = (g.per_channel + splits - 1) / splits;
  chunk = (chunk + 15) / 16 * 16;
  splits = (g.per_channel + chunk - 1) / chunk;
  if (splits < 1) splits = 1;
  g.splits = static_cast<int>(splits);
  g.chunk = chunk;
  return g;
}

// Address of element e (0 <= e < outer*inner) of channel c.
__device__ __forceinline__ long long channel_elem_offset(const ChannelGeo& g, long long c,
                                                         long long e) {
  // 32-bit division when it fits: it does for every shape of the five workloads.
  long long o, i;
  if (g.per_channel < 0x7fffffffLL) {
    const unsigned eo = static_cast<unsigned>(e) / static_cast<unsigned>(g.inner);
    o = eo;
    i = static_cast<unsigned>(e) - eo * static_cast<unsigned>(g.inner);
  } else {
    o = e / g.inner;
    i = e - o * g.inner;
  }
  return (o * g.channels + c) * g.inner + i;
}

// F: struct with
//   struct K {...};  __device__ K channel(long long c) const;
//   __device__ void accumulate(const K&, float a, float b, float& s0, float& s1) const;
// NIN = number of input tensors (1 or 2).  partial[(c*splits + s)] = (s0, s1).
template <typename T, int NIN, bool VEC, typename F>
__global__ void __launch_bounds__(kChanThreads)
channel_reduce_kernel(const T* __restrict__ a, const T* __restrict__ b,
                      float2* __restrict__ partial, ChannelGeo g, F f) {
  __shared__ float scratch[32];
  const long long c = blockIdx.x;
  const int s = blockIdx.y;
  const typename F::K k = f.channel(c);
  long long begin = (long long)s * g.chunk;
  long long end = begin + g.chunk;
  if (end > g.per_channel) end = g.per_channel;
  float s0 = 0.f, s1 = 0.f;
  if (VEC) {
    constexpr int V = Vec16<T>::N;
    // chunk is a multiple of 16 and inner a multiple of V, so vectors never straddle rows.
    for (long long e = begin + (long long)threadIdx.x * V; e < end;
         e += (long long)kChanThreads * V * 2) {
      const long long e2 = e + (long long)kChanThreads * V;
      const bool two = e2 < end;
      const long long off = channel_elem_offset(g, c, e);
      const long long off2 = two ? channel_elem_offset(g, c, e2) : off;
      Vec16<T> va = load16(a + off), vb, va2, vb2;
      if (NIN == 2) vb = load16(b + off);
      if (two) {
        va2 = load16(a + off2);
        if (NIN == 2) vb2 = load16(b + off2);
      }
#pragma unroll
      for (int j = 0; j < V; ++j)
        f.accumulate(k, Num<T>::to_f(va.v[j]), NIN == 2 ? Num<T>::to_f(vb.v[j]) : 0.f, s0, s1);
      if (two) {
#pragma unroll
        for (int j = 0; j < V; ++j)
          f.accumulate(k, Num<T>::to_f(va2.v[j]), NIN == 2 ? Num<T>::to_f(vb2.v[j]) : 0.f, s0,
                       s1);
      }
    }
  } else {
    for (long long e = begin + threadIdx.x; e < end; e += kChanThreads) {
      const long long off = channel_elem_offset(g, c, e);
      f.accumulate(k, Num<T>::to_f(a[off]), NIN == 2 ? Num<T>::to_f(b[off]) : 0.f, s0, s1);
    }
  }
  s0 = block_sum(s0, scratch);
  s1 = block_sum(s1, scratch);
  if (threadIdx.x == 0) partial[c * g.splits + s] = make_float2(s0, s1);
}

// F: struct with K / channel(c) as above and
//   __device__ float apply(const K&, float a, float b) const;
template <typename T, int NIN, bool VEC, typename F>
__global__ void __launch_bounds__(kChanThreads)
channel_apply_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                     ChannelGeo g, F f) {
  const long long c = blockIdx.x;
  const int s = blockIdx.y;
  const typename F::K k = f.channel(c);
  long long begin = (long long)s * g.chunk;
  long long end = begin + g.chunk;
  if (end > g.per_channel) end = g.per_channel;
  if (VEC) {
    constexpr int V = Vec16<T>::N;
    for (long long e = begin + (long long)threadIdx.x * V; e < end;
         e += (long long)kChanThreads * V * 2) {
      const long long e2 = e + (long long)kChanThreads * V;
      const bool two = e2 < end;
      const long long off = channel_elem_offset(g, c, e);
      const long long off2 = two ? channel_elem_offset(g, c, e2) : off;
      Vec16<T> va = load16(a + off), vb, va2, vb2, vo;
      if (NIN == 2) vb = load16(b + off);
      if (two) {
        va2 = load16(a + off2);
        if (NIN == 2) vb2 = load16(b + off2);
      }
#pragma unroll
      for (int j = 0; j < V; ++j)
        vo.v[j] = Num<T>::from_f(
            f.apply(k, Num<T>::to_f(va.v[j]), NIN == 2 ? Num<T>::to_f(vb.v[j]) : 0.f));
      store16(out + off, vo);
      if (two) {
#pragma unroll
        for (int j = 0; j < V; ++j)
          vo.v[j] = Num<T>::from_f(
              f.apply(k, Num<T>::to_f(va2.v[j]), NIN == 2 ? Num<T>::to_f(vb2.v[j]) : 0.f));
        store16(out + off2, vo);
      }
    }
  } else {
    for (long long e = begin + threadIdx.x; e < end; e += kChanThreads) {
      const long long off = channel_elem_offset(g, c, e);
      out[off] = Num<T>::from_f(
          f.apply(k, Num<T>::to_f(a[off]), NIN == 2 ? Num<T>::to_f(b[off]) : 0.f));
    }
  }
}

// inner == 1 ([rows][channels], channel fastest): a CTA of 32 x 8 threads owns
// 32 adjacent channels and a range of rows; lanes read 128 contiguous bytes.
template <typename T, int NIN, typename F>
__global__ void __launch_bounds__(256)
column_reduce_kernel(const T* __restrict__ a, const T* __restrict__ b,
                     float2* __restrict__ partial, long long rows, long long channels,
                     int splits, long long rows_per_split, F f) {
  __shared__ float sh0[8][33];
  __shared__ float sh1[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long c = (long long)blockIdx.x * 32 + tx;
  const int s = blockIdx.y;
  float s0 = 0.f, s1 = 0.f;
  if (c < channels) {
    const typename F::K k = f.channel(c);
    long long r0 = (long long)s * rows_per_split;
    long long r1 = r0 + rows_per_split;
    if (r1 > rows) r1 = rows;
    for (long long r = r0 + ty; r < r1; r += 8) {
      const long long off = r * channels + c;
      f.accumulate(k, Num<T>::to_f(a[off]), NIN == 2 ? Num<T>::to_f(b[off]) : 0.f, s0, s1);
    }
  }
  sh0[ty][tx] = s0;
  sh1[ty][tx] = s1;
  __syncthreads();
  if (ty == 0 && c < channels) {
#pragma unroll
    for (int j = 1; j < 8; ++j) {
      s0 += sh0[j][tx];
      s1 += sh1[j][tx];
    }
    partial[c * splits + s] = make_float2(s0, s1);
  }
}

template <typename T, int NIN, typename F>
__global__ void __launch_bounds__(256)
column_apply_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                    long long rows, long long channels, F f) {
  const long long total = rows * channels;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const long long c = t % channels;
    const typename F::K k = f.channel(c);
    out[t] = Num<T>::from_f(f.apply(k, Num<T>::to_f(a[t]), NIN == 2 ? Num<T>::to_f(b[t]) : 0.f));
  }
}

// ------------------------------------------------------------------------------------------
// inner == 1 with fp32 data, channels a multiple of 4 and 16-byte aligned tensors (the
// channels-last image tensors, [pixels][channels]): the same column reduction and per-channel
// pass with 16-byte accesses.  A CTA of 256 threads is CQ column quads (4 channels each, CQ a
// power of two <= 64) x 256 / CQ row lanes; a thread keeps the constants of its four channels in
// registers and walks the rows of its split with four independent loads in flight.
struct ColumnTiling {
  int cq_shift;    // log2(CQ)
  int col_blocks;  // ceil(channels / (4 * CQ))
};
inline ColumnTiling column_tiling(long long channels) {
  const long long quads = (channels + 3) / 4;
  int shift = 0;
  while ((2LL << shift) <= quads && shift < 6) ++shift;
  ColumnTiling t;
  t.cq_shift = shift;
  t.col_blocks = (int)((quads + (1LL << shift) - 1) >> shift);
  return t;
}

template <int NIN, typename F>
__global__ void __launch_bounds__(256)
column_reduce_vec_kernel(const float* __restrict__ a, const float* __restrict__ b,
                         float2* __restrict__ partial, long long rows, long long channels,
                         int splits, long long rows_per_split, int cq_shift, F f) {
  __shared__ float sh0[1024];
  __shared__ float sh1[1024];
  const int cq = 1 << cq_shift, rl = 256 >> cq_shift;
  const int tq = threadIdx.x & (cq - 1), tr = threadIdx.x >> cq_shift;
  const long long c = ((long long)blockIdx.x * cq + tq) * 4;
  const int s = blockIdx.y;
  float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
  const bool live = c < channels;
  if (live) {
    typename F::K k[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) k[j] = f.channel(c + j);
    const long long r0 = (long long)s * rows_per_split;
    long long r1 = r0 + rows_per_split;
    if (r1 > rows) r1 = rows;
    long long r = r0 + tr;
    // eight 16-byte loads in flight per thread: 8 rows of one tensor or 4 rows of two
    constexpr int U = NIN == 2 ? 4 : 8;
    for (; r + (long long)(U - 1) * rl < r1; r += (long long)U * rl) {
      float4 va[U], vb[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long off = (r + (long long)u * rl) * channels + c;
        va[u] = *reinterpret_cast<const float4*>(a + off);
        if (NIN == 2) vb[u] = *reinterpret_cast<const float4*>(b + off);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        f.accumulate(k[0], va[u].x, NIN == 2 ? vb[u].x : 0.f, s0[0], s1[0]);
        f.accumulate(k[1], va[u].y, NIN == 2 ? vb[u].y : 0.f, s0[1], s1[1]);
        f.accumulate(k[2], va[u].z, NIN == 2 ? vb[u].z : 0.f, s0[2], s1[2]);
        f.accumulate(k[3], va[u].w, NIN == 2 ? vb[u].w : 0.f, s0[3], s1[3]);
      }
    }
    for (; r < r1; r += rl) {
      const long long off = r * channels + c;
      const float4 va = *reinterpret_cast<const float4*>(a + off);
      float4 vb = make_float4(0.f, 0.f, 0.f, 0.f);
      if (NIN == 2) vb = *reinterpret_cast<const float4*>(b + off);
      f.accumulate(k[0], va.x, vb.x, s0[0], s1[0]);
      f.accumulate(k[1], va.y, vb.y, s0[1], s1[1]);
      f.accumulate(k[2], va.z, vb.z, s0[2], s1[2]);
      f.accumulate(k[3], va.w, vb.w, s0[3], s1[3]);
    }
  }
  // sh[tr][tq * 4 + j]: 256 threads x 4 values
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    sh0[(tr << (cq_shift + 2)) + tq * 4 + j] = s0[j];
    sh1[(tr << (cq_shift + 2)) + tq * 4 + j] = s1[j];
  }
  __syncthreads();
  // thread t < 4 * CQ finishes column t of the block
  if ((int)threadIdx.x < 4 * cq) {
    const long long cc = (long long)blockIdx.x * cq * 4 + threadIdx.x;
    if (cc < channels) {
      float t0 = 0.f, t1 = 0.f;
      for (int i = 0; i < rl; ++i) {
        t0 += sh0[(i << (cq_shift + 2)) + threadIdx.x];
        t1 += sh1[(i << (cq_shift + 2)) + threadIdx.x];
      }
      partial[cc * splits + s] = make_float2(t0, t1);
    }
  }
}

template <int NIN, typename F>
__global__ void __launch_bounds__(256)
column_apply_vec_kernel(const float* __restrict__ a, const float* __restrict__ b,
                        float* __restrict__ out, long long rows, long long channels,
                        long long rows_per_split, int cq_shift, F f) {
  const int cq = 1 << cq_shift, rl = 256 >> cq_shift;
  const int tq = threadIdx.x & (cq - 1), tr = threadIdx.x >> cq_shift;
  const long long c = ((long long)blockIdx.x * cq + tq) * 4;
  if (c >= channels) return;
  typename F::K k[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) k[j] = f.channel(c + j);
  const long long r0 = (long long)blockIdx.y * rows_per_split;
  long long r1 = r0 + rows_per_split;
  if (r1 > rows) r1 = rows;
  long long r = r0 + tr;
  for (; r + 3LL * rl < r1; r += 4LL * rl) {
    float4 va[4], vb[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long off = (r + (long long)u * rl) * channels + c;
      va[u] = *reinterpret_cast<const float4*>(a + off);
      if (NIN == 2) vb[u] = *reinterpret_cast<const float4*>(b + off);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long off = (r + (long long)u * rl) * channels + c;
      *reinterpret_cast<float4*>(out + off) =
          make_float4(f.apply(k[0], va[u].x, NIN == 2 ? vb[u].x : 0.f),
                      f.apply(k[1], va[u].y, NIN == 2 ? vb[u].y : 0.f),
                      f.apply(k[2], va[u].z, NIN == 2 ? vb[u].z : 0.f),
                      f.apply(k[3], va[u].w, NIN == 2 ? vb[u].w : 0.f));
    }
  }
  for (; r < r1; r += rl) {
    const long long off = r * channels + c;
    const float4 va = *reinterpret_cast<const float4*>(a + off);
    float4 vb = make_float4(0.f, 0.f, 0.f, 0.f);
    if (NIN == 2) vb = *reinterpret_cast<const float4*>(b + off);
    *reinterpret_cast<float4*>(out + off) =
        make_float4(f.apply(k[0], va.x, vb.x), f.apply(k[1], va.y, vb.y), f.apply(k[2], va.z, vb.z),
                    f.apply(k[3], va.w, vb.w));
  }
}

// Splits of the column path (rows handled per CTA): about six CTAs per SM over the vector
// tiling's column blocks, at least 64 rows each, at most 512 splits.
inline int column_splits(long long rows, long long channels) {
  const long long col_blocks = column_tiling(channels).col_blocks;
  long long splits = (6LL * device_info().sm_count + col_blocks - 1) / col_blocks;
  const long long max_by_work = (rows + 63) / 64;
  if (splits > max_by_work) splits = max_by_work;
  if (splits > 512) splits = 512;
  if (splits < 1) splits = 1;
  return static_cast<int>(splits);
}

// Scratch bytes for the (channel, split) partial sums of any op built on these.
inline size_t channel_partial_bytes(long long outer, long long channels, long long inner) {
  long long splits;
  if (inner == 1) {
    splits = column_splits(outer, channels);
  } else {
    splits = make_channel_geo(outer, channels, inner).splits;
  }
  return static_cast<size_t>(channels) * static_cast<size_t>(splits) * sizeof(float2);
}

}  // namespace flb200
