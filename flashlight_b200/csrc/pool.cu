// pool2d forward / backward (max, average with and without padding in the
// divisor).  Stands behind fl::AutogradExtension::pool2d / ::pool2dBackward
// (flashlight/fl/autograd/tensor/AutogradExtension.h:71-80, 141-152); output
// extent as flashlight/fl/autograd/tensor/backend/onednn/Pool2D.cpp:100-102.
//
// Layout: x [N][C][H][W] row-major (fl [W,H,C,N]).  Forward: one thread per
// output element, lanes along Wo.  Backward is a GATHER: one thread per input
// element adds up the windows that selected it, so there are no atomics and the
// result does not depend on scheduling.  The forward pass leaves one byte per
// output element (the selected window position) for backward; without it the
// selection is recomputed from x.
// Algorithmic bytes: forward 4*(N_in + N_out); backward 4*(2*N_in + N_out).
#include "common.cuh"

#include <cfloat>
#include <type_traits>

namespace flb200 {
namespace {

struct PoolGeo {
  int W, H, Wo, Ho;
  int wx, wy, sx, sy, px, py;
  int mode;
  long long planes;  // N * C
};

// Selected window position (ky*wx + kx) and value of window (p, q) of one plane.
// First in-bounds element wins ties; a NaN takes over and later NaNs keep moving
// the selection, as in the CPU stand-in this library is checked against.
template <typename T>
__device__ __forceinline__ int window_argmax(const T* __restrict__ plane, const PoolGeo& g, int p,
                                             int q, float* best_out) {
  const int h0 = p * g.sy - g.py, w0 = q * g.sx - g.px;
  float best = -INFINITY;
  int arg = 255;
  for (int ky = 0; ky < g.wy; ++ky) {
    const int h = h0 + ky;
    if (h < 0 || h >= g.H) continue;
    for (int kx = 0; kx < g.wx; ++kx) {
      const int w = w0 + kx;
      if (w < 0 || w >= g.W) continue;
      const float v = Num<T>::to_f(plane[(long long)h * g.W + w]);
      if (arg == 255 || v > best || v != v) {
        best = v;
        arg = ky * g.wx + kx;
      }
    }
  }
  *best_out = best;
  return arg;
}

__device__ __forceinline__ float window_divisor(const PoolGeo& g, int p, int q) {
  if (g.mode == FLB200_POOL_AVG_INCLUDE_PAD) return (float)(g.wx * g.wy);
  const int h0 = p * g.sy - g.py, w0 = q * g.sx - g.px;
  const int h1 = min(h0 + g.wy, g.H), w1 = min(w0 + g.wx, g.W);
  const int cnt = (h1 - max(h0, 0)) * (w1 - max(w0, 0));
  return (float)max(cnt, 1);
}

template <typename T>
__global__ void __launch_bounds__(256) pool_forward_kernel(const T* __restrict__ x,
                                                           T* __restrict__ y,
                                                           uint8_t* __restrict__ argmax,
                                                           PoolGeo g) {
  const long long out_plane = (long long)g.Ho * g.Wo;
  const long long total = g.planes * out_plane;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const long long plane = t / out_plane;
    const int r = (int)(t - plane * out_plane);
    const int p = r / g.Wo, q = r - p * g.Wo;
    const T* xp = x + plane * (long long)g.H * g.W;
    if (g.mode == FLB200_POOL_MAX) {
      float best;
      const int arg = window_argmax(xp, g, p, q, &best);
      y[t] = Num<T>::from_f(best);
      if (argmax) argmax[t] = (uint8_t)arg;
    } else {
      const int h0 = p * g.sy - g.py, w0 = q * g.sx - g.px;
      float acc = 0.f;
      for (int ky = 0; ky < g.wy; ++ky) {
        const int h = h0 + ky;
        if (h < 0 || h >= g.H) continue;
        for (int kx = 0; kx < g.wx; ++kx) {
          const int w = w0 + kx;
          if (w < 0 || w >= g.W) continue;
          acc += Num<T>::to_f(xp[(long long)h * g.W + w]);
        }
      }
      y[t] = Num<T>::from_f(acc / window_divisor(g, p, q));
    }
  }
}

__device__ __forceinline__ int ceil_div_pos(int a, int b) {  // ceil(a / b) for b > 0, any a
  return a >= 0 ? (a + b - 1) / b : -((-a) / b);
}

template <typename T>
__global__ void __launch_bounds__(256) pool_backward_kernel(const T* __restrict__ dy,
                                                            const T* __restrict__ x,
                                                            const uint8_t* __restrict__ argmax,
                                                            T* __restrict__ dx, PoolGeo g) {
  const long long in_plane = (long long)g.H * g.W;
  const long long out_plane = (long long)g.Ho * g.Wo;
  const long long total = g.planes * in_plane;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const long long plane = t / in_plane;
    const int r = (int)(t - plane * in_plane);
    const int h = r / g.W, w = r - h * g.W;
    // windows p with p*sy - py <= h <= p*sy - py + wy - 1
    const int p_lo = max(ceil_div_pos(h + g.py - g.wy + 1, g.sy), 0);
    const int p_hi = min((h + g.py) / g.sy, g.Ho - 1);
    const int q_lo = max(ceil_div_pos(w + g.px - g.wx + 1, g.sx), 0);
    const int q_hi = min((w + g.px) / g.sx, g.Wo - 1);
    const T* dyp = dy + plane * out_plane;
    float acc = 0.f;
    for (int p = p_lo; p <= p_hi; ++p) {
      for (int q = q_lo; q <= q_hi; ++q) {
        const long long o = (long long)p * g.Wo + q;
        if (g.mode == FLB200_POOL_MAX) {
          const int mine = (h + g.py - p * g.sy) * g.wx + (w + g.px - q * g.sx);
          int sel;
          if (argmax) {
            sel = argmax[plane * out_plane + o];
          } else {
            float unused;
            sel = window_argmax(x + plane * in_plane, g, p, q, &unused);
          }
          if (sel == mine) acc += Num<T>::to_f(dyp[o]);
        } else {
          acc += Num<T>::to_f(dyp[o]) / window_divisor(g, p, q);
        }
      }
    }
    dx[t] = Num<T>::from_f(acc);
  }
}

// ------------------------------------------------------------ tiled fp32 max pooling
// The generic kernels above read each input element through the cache once per covering
// window.  For fp32 max pooling (the workloads' hot case) a CTA instead owns a band of
// output rows of one plane: the input rows the band needs are one contiguous range, copied
// to shared memory with 16-byte loads; windows are then scanned out of shared memory.
// band_rows output rows per CTA; tile = ((band_rows - 1) * sy + wy) * W floats of dynamic
// shared memory.  Same selection rule as window_argmax.
// WX, WY, SX, SY: window and stride as compile-time constants for the common cases (0 = take
// them from the geometry), so that the index arithmetic has no runtime divisions.
template <int WX, int WY, int SX, int SY>
__global__ void __launch_bounds__(256)
pool_forward_max_tile_kernel(const float* __restrict__ x, float* __restrict__ y,
                             uint8_t* __restrict__ argmax, PoolGeo g, int band_rows, int nbands) {
  extern __shared__ float tile[];
  const int wx = WX ? WX : g.wx, wy = WY ? WY : g.wy, sx = SX ? SX : g.sx, sy = SY ? SY : g.sy;
  const long long plane = blockIdx.x / nbands;
  const int band = blockIdx.x - (int)(plane * nbands);
  const int p0 = band * band_rows;
  const int p1 = min(p0 + band_rows, g.Ho);
  const int h_lo = max(p0 * sy - g.py, 0);
  const int h_hi = min((p1 - 1) * sy - g.py + wy, g.H);
  const float* src = x + plane * (long long)g.H * g.W + (long long)h_lo * g.W;
  const int n = (h_hi - h_lo) * g.W;
  if ((g.W & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    for (int i = threadIdx.x * 4; i < n; i += 256 * 4)
      *reinterpret_cast<float4*>(tile + i) = *reinterpret_cast<const float4*>(src + i);
  } else {
    for (int i = threadIdx.x; i < n; i += 256) tile[i] = src[i];
  }
  __syncthreads();
  float* yp = y + plane * (long long)g.Ho * g.Wo;
  uint8_t* ap = argmax ? argmax + plane * (long long)g.Ho * g.Wo : nullptr;
  // 64 x 4 threads: columns across the x index, rows across the y index
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int p = p0 + ty; p < p1; p += 4) {
    const int h0 = p * sy - g.py;
    for (int q = tx; q < g.Wo; q += 64) {
      const int w0 = q * sx - g.px;
      float best = -INFINITY;
      int arg = 255;
      if (h0 >= 0 && h0 + wy <= g.H && w0 >= 0 && w0 + wx <= g.W) {
        // window inside the image: no per-element bounds checks
        const float* row = tile + (h0 - h_lo) * g.W + w0;
        best = row[0];
        arg = 0;
#pragma unroll
        for (int ky = 0; ky < wy; ++ky) {
#pragma unroll
          for (int kx = 0; kx < wx; ++kx) {
            const float v = row[ky * g.W + kx];
            if (v > best || v != v) {
              best = v;
              arg = ky * wx + kx;
            }
          }
        }
      } else {
#pragma unroll
        for (int ky = 0; ky < wy; ++ky) {
          const int h = h0 + ky;
          if (h < 0 || h >= g.H) continue;
          const float* row = tile + (h - h_lo) * g.W;
#pragma unroll
          for (int kx = 0; kx < wx; ++kx) {
            const int w = w0 + kx;
            if (w < 0 || w >= g.W) continue;
            const float v = row[w];
            if (arg == 255 || v > best || v != v) {
              best = v;
              arg = ky * wx + kx;
            }
          }
        }
      }
      yp[p * g.Wo + q] = best;
      if (ap) ap[p * g.Wo + q] = (uint8_t)arg;
    }
  }
}

// Gradient: a CTA owns a band of INPUT rows of one plane, copies the dy values and argmax
// bytes of every output row whose windows reach the band into shared memory, and each thread
// then gathers a strip of four input pixels from them in a fixed order (no atomics).
template <int WX, int WY, int SX, int SY>
__global__ void __launch_bounds__(256)
pool_backward_max_tile_kernel(const float* __restrict__ dy, const uint8_t* __restrict__ argmax,
                              float* __restrict__ dx, PoolGeo g, int band_rows, int nbands,
                              int max_out_rows) {
  extern __shared__ float tile[];  // [max_out_rows][Wo] dy, then the argmax bytes
  const int wx = WX ? WX : g.wx, wy = WY ? WY : g.wy, sx = SX ? SX : g.sx, sy = SY ? SY : g.sy;
  uint8_t* sel = reinterpret_cast<uint8_t*>(tile + (size_t)max_out_rows * g.Wo);
  const long long plane = blockIdx.x / nbands;
  const int band = blockIdx.x - (int)(plane * nbands);
  const int h0 = band * band_rows;
  const int h1 = min(h0 + band_rows, g.H);
  const int p_lo = max(ceil_div_pos(h0 + g.py - wy + 1, sy), 0);
  const int p_hi = min((h1 - 1 + g.py) / sy, g.Ho - 1);
  const int n = (p_hi - p_lo + 1) * g.Wo;
  const long long obase = plane * (long long)g.Ho * g.Wo + (long long)p_lo * g.Wo;
  for (int i = threadIdx.x; i < n; i += 256) {
    tile[i] = dy[obase + i];
    sel[i] = argmax[obase + i];
  }
  __syncthreads();
  const int strips_w = (g.W + 3) >> 2;
  float* dxp = dx + plane * (long long)g.H * g.W;
  const bool vec_ok = (g.W & 3) == 0 && (reinterpret_cast<uintptr_t>(dx) & 15) == 0;
  // 32 x 8 threads: strips of four pixels across a row, rows across ty
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int h = h0 + ty; h < h1; h += 8) {
    const int pa = max(ceil_div_pos(h + g.py - wy + 1, sy), 0);
    const int pb = min((h + g.py) / sy, g.Ho - 1);
    for (int sw = tx; sw < strips_w; sw += 32) {
      const int w0 = sw << 2;
      const int qa = max(ceil_div_pos(w0 + g.px - wx + 1, sx), 0);
      const int qb = min((w0 + 3 + g.px) / sx, g.Wo - 1);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int p = pa; p <= pb; ++p) {
        const int ky_mine = h + g.py - p * sy;
        const int rbase = (p - p_lo) * g.Wo;
        for (int q = qa; q <= qb; ++q) {
          const int s = sel[rbase + q];
          const int ky = s / wx, kx = s - ky * wx;
          const int wt = q * sx - g.px + kx - w0;  // position inside the strip
          if (ky == ky_mine && wt >= 0 && wt < 4) {
            const float v = tile[rbase + q];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (wt == j) acc[j] += v;
          }
        }
      }
      float* dst = dxp + (long long)h * g.W + w0;
      if (vec_ok) {
        *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (w0 + j < g.W) dst[j] = acc[j];
      }
    }
  }
}

// Gradient of an average pooling whose single window is the whole unpadded plane (the global
// average pool in front of a classifier): every pixel of a plane receives dy / (H * W).  The
// generic kernel spends its time on index arithmetic here (0.22 ms for the ResNet head).
__global__ void __launch_bounds__(256)
pool_backward_global_avg_kernel(const float* __restrict__ dy, float* __restrict__ dx,
                                long long planes, int hw) {
  const long long total = planes * hw;
  const float div = (float)hw;  // divided, not multiplied by the reciprocal: same bits as the generic kernel
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride)
    dx[t] = dy[t / hw] / div;
}

template <int WX, int WY, int SX, int SY>
void launch_pool_fwd_tile(const float* x, float* y, uint8_t* argmax, const PoolGeo& g, int band,
                          int nbands, size_t smem, cudaStream_t st) {
  pool_forward_max_tile_kernel<WX, WY, SX, SY><<<(unsigned)(g.planes * nbands), 256, smem, st>>>(
      x, y, argmax, g, band, nbands);
}
template <int WX, int WY, int SX, int SY>
void launch_pool_bwd_tile(const float* dy, const uint8_t* argmax, float* dx, const PoolGeo& g,
                          int band, int nbands, int out_rows, size_t smem, cudaStream_t st) {
  pool_backward_max_tile_kernel<WX, WY, SX, SY>
      <<<(unsigned)(g.planes * nbands), 256, smem, st>>>(dy, argmax, dx, g, band, nbands, out_rows);
}
bool is_window(const PoolGeo& g, int wx, int wy, int sx, int sy) {
  return g.wx == wx && g.wy == wy && g.sx == sx && g.sy == sy;
}

// Band height for the tiled kernels: enough outputs per CTA to occupy 256 threads, tile within
// 40 KB.  Returns 0 when a single band does not fit (very wide planes): generic kernels then.
int pool_fwd_band_rows(const PoolGeo& g) {
  int rows = (1024 + g.Wo - 1) / g.Wo;  // ~1024 outputs per CTA (measured best of 256..4096)
  if (rows > g.Ho) rows = g.Ho;
  while (rows > 1 && (size_t)((rows - 1) * g.sy + g.wy) * g.W * 4 > 40 * 1024) --rows;
  if ((size_t)((rows - 1) * g.sy + g.wy) * g.W * 4 > 40 * 1024) return 0;
  return rows;
}
int pool_bwd_band_rows(const PoolGeo& g, int* max_out_rows) {
  int rows = (16384 + g.W - 1) / g.W;  // ~4096 strips of four pixels (measured best of 1K..16K)
  if (rows > g.H) rows = g.H;
  for (;; --rows) {
    const int outs = (rows + g.wy - 2) / g.sy + 2;
    if ((size_t)outs * g.Wo * 5 + 16 <= 40 * 1024 || rows <= 1) {
      *max_out_rows = outs;
      return (size_t)outs * g.Wo * 5 + 16 <= 40 * 1024 ? rows : 0;
    }
  }
}

// Max-pooling gradient with the argmax payload, the hot case of the workloads.  A thread owns
// a strip of four adjacent input pixels of one plane (one 16-byte store) and walks the few
// windows that overlap the strip once, decoding where each window sent its gradient; planes
// come from blockIdx.y so all index arithmetic is 32-bit.
template <typename T>
__global__ void __launch_bounds__(256)
pool_backward_max_strip_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ argmax,
                               T* __restrict__ dx, PoolGeo g) {
  const int strips_w = (g.W + 3) >> 2;
  const int strips = strips_w * g.H;
  const int in_plane = g.H * g.W, out_plane = g.Ho * g.Wo;
  const bool vec_ok = (g.W & 3) == 0 && (reinterpret_cast<uintptr_t>(dx) & 15) == 0 &&
                      sizeof(T) == 4;
  for (long long plane = blockIdx.y; plane < g.planes; plane += gridDim.y) {
    const T* dyp = dy + plane * out_plane;
    const uint8_t* ap = argmax + plane * out_plane;
    T* dxp = dx + plane * in_plane;
    for (int si = blockIdx.x * blockDim.x + threadIdx.x; si < strips;
         si += gridDim.x * blockDim.x) {
      const int h = si / strips_w, w0 = (si - h * strips_w) << 2;
      const int p_lo = max(ceil_div_pos(h + g.py - g.wy + 1, g.sy), 0);
      const int p_hi = min((h + g.py) / g.sy, g.Ho - 1);
      const int q_lo = max(ceil_div_pos(w0 + g.px - g.wx + 1, g.sx), 0);
      const int q_hi = min((w0 + 3 + g.px) / g.sx, g.Wo - 1);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int p = p_lo; p <= p_hi; ++p) {
        const int ky_mine = h + g.py - p * g.sy;
        for (int q = q_lo; q <= q_hi; ++q) {
          const int o = p * g.Wo + q;
          const int sel = ap[o];
          const int ky = sel / g.wx, kx = sel - ky * g.wx;
          const int wt = q * g.sx - g.px + kx - w0;  // position inside the strip
          if (ky == ky_mine && wt >= 0 && wt < 4) {
            const float v = Num<T>::to_f(dyp[o]);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (wt == j) acc[j] += v;
          }
        }
      }
      T* dst = dxp + h * g.W + w0;
      if (vec_ok) {
        *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (w0 + j < g.W) dst[j] = Num<T>::from_f(acc[j]);
      }
    }
  }
}

// ------------------------------------------------------------ channels-last tensors
// x [N][H][W][C]: the channel is the contiguous index, so a thread owns V consecutive
// channels of one output (forward) or input (backward) pixel and every access is one V-wide
// vector, coalesced across the threads of a warp; a window is then wx * wy such vectors.
// Selection rule, NaN behaviour, divisors and the argmax payload (one byte per output element,
// in the tensor's own element order) are those of the kernels above.
template <typename T, int V>
__global__ void __launch_bounds__(256)
pool_forward_cl_kernel(const T* __restrict__ x, T* __restrict__ y, uint8_t* __restrict__ argmax,
                       PoolGeo g, int C, int per_image) {
  // blockIdx.y = image; the index inside an image fits 32 bits (checked by the launcher)
  const unsigned cv = C / V;
  const long long n = blockIdx.y;
  for (unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < (unsigned)per_image;
       t += gridDim.x * blockDim.x) {
    const unsigned pix = t / cv;
    const int c = (int)(t - pix * cv) * V;
    const int p = (int)(pix / (unsigned)g.Wo);
    const int q = (int)(pix - (unsigned)p * (unsigned)g.Wo);
    const int h0 = p * g.sy - g.py, w0 = q * g.sx - g.px;
    const T* xn = x + n * (long long)g.H * g.W * C + c;
    float acc[V];
    int arg[V];
#pragma unroll
    for (int j = 0; j < V; ++j) { acc[j] = g.mode == FLB200_POOL_MAX ? -INFINITY : 0.f; arg[j] = 255; }
    for (int ky = 0; ky < g.wy; ++ky) {
      const int h = h0 + ky;
      if (h < 0 || h >= g.H) continue;
      for (int kx = 0; kx < g.wx; ++kx) {
        const int w = w0 + kx;
        if (w < 0 || w >= g.W) continue;
        const T* src = xn + ((long long)h * g.W + w) * C;
        T vals[V];
        if (V * sizeof(T) == 16) *reinterpret_cast<uint4*>(vals) = *reinterpret_cast<const uint4*>(src);
        else {
#pragma unroll
          for (int j = 0; j < V; ++j) vals[j] = src[j];
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float v = Num<T>::to_f(vals[j]);
          if (g.mode == FLB200_POOL_MAX) {
            if (arg[j] == 255 || v > acc[j] || v != v) { acc[j] = v; arg[j] = ky * g.wx + kx; }
          } else {
            acc[j] += v;
          }
        }
      }
    }
    const float div = g.mode == FLB200_POOL_MAX ? 1.f : window_divisor(g, p, q);
    const long long o = ((n * g.Ho + p) * g.Wo + q) * (long long)C + c;
    T outv[V];
#pragma unroll
    for (int j = 0; j < V; ++j)
      outv[j] = Num<T>::from_f(g.mode == FLB200_POOL_MAX ? acc[j] : acc[j] / div);
    if (V * sizeof(T) == 16) *reinterpret_cast<uint4*>(y + o) = *reinterpret_cast<const uint4*>(outv);
    else {
#pragma unroll
      for (int j = 0; j < V; ++j) y[o + j] = outv[j];
    }
    if (argmax && g.mode == FLB200_POOL_MAX) {
      uint8_t sels[V];
#pragma unroll
      for (int j = 0; j < V; ++j) sels[j] = (uint8_t)arg[j];
      if (V == 4) *reinterpret_cast<uint32_t*>(argmax + o) = *reinterpret_cast<const uint32_t*>(sels);
      else if (V == 8) *reinterpret_cast<uint2*>(argmax + o) = *reinterpret_cast<const uint2*>(sels);
      else {
#pragma unroll
        for (int j = 0; j < V; ++j) argmax[o + j] = sels[j];
      }
    }
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256)
pool_backward_cl_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                        const uint8_t* __restrict__ argmax, T* __restrict__ dx, PoolGeo g, int C,
                        int per_image) {
  const unsigned cv = C / V;
  const long long n = blockIdx.y;
  for (unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < (unsigned)per_image;
       t += gridDim.x * blockDim.x) {
    const unsigned pix = t / cv;
    const int c = (int)(t - pix * cv) * V;
    const int h = (int)(pix / (unsigned)g.W);
    const int w = (int)(pix - (unsigned)h * (unsigned)g.W);
    const int p_lo = max(ceil_div_pos(h + g.py - g.wy + 1, g.sy), 0);
    const int p_hi = min((h + g.py) / g.sy, g.Ho - 1);
    const int q_lo = max(ceil_div_pos(w + g.px - g.wx + 1, g.sx), 0);
    const int q_hi = min((w + g.px) / g.sx, g.Wo - 1);
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    for (int p = p_lo; p <= p_hi; ++p) {
      for (int q = q_lo; q <= q_hi; ++q) {
        const long long o = ((n * g.Ho + p) * g.Wo + q) * (long long)C + c;
        T gv[V];
        if (V * sizeof(T) == 16) *reinterpret_cast<uint4*>(gv) = *reinterpret_cast<const uint4*>(dy + o);
        else {
#pragma unroll
          for (int j = 0; j < V; ++j) gv[j] = dy[o + j];
        }
        if (g.mode == FLB200_POOL_MAX) {
          const int mine = (h + g.py - p * g.sy) * g.wx + (w + g.px - q * g.sx);
          uint8_t sels[V];
          if (argmax) {  // the V window positions in one load (o is a multiple of V)
            if (V == 4) *reinterpret_cast<uint32_t*>(sels) = *reinterpret_cast<const uint32_t*>(argmax + o);
            else if (V == 8) *reinterpret_cast<uint2*>(sels) = *reinterpret_cast<const uint2*>(argmax + o);
            else {
#pragma unroll
              for (int j = 0; j < V; ++j) sels[j] = argmax[o + j];
            }
          }
#pragma unroll
          for (int j = 0; j < V; ++j) {
            int sel;
            if (argmax) {
              sel = sels[j];
            } else {  // recompute the selection of window (p, q) for channel c + j from x
              const int h0 = p * g.sy - g.py, w0 = q * g.sx - g.px;
              float best = -INFINITY;
              sel = 255;
              for (int ky = 0; ky < g.wy; ++ky) {
                const int hh = h0 + ky;
                if (hh < 0 || hh >= g.H) continue;
                for (int kx = 0; kx < g.wx; ++kx) {
                  const int ww = w0 + kx;
                  if (ww < 0 || ww >= g.W) continue;
                  const float v = Num<T>::to_f(x[((n * g.H + hh) * g.W + ww) * (long long)C + c + j]);
                  if (sel == 255 || v > best || v != v) { best = v; sel = ky * g.wx + kx; }
                }
              }
            }
            if (sel == mine) acc[j] += Num<T>::to_f(gv[j]);
          }
        } else {
          const float div = window_divisor(g, p, q);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] += Num<T>::to_f(gv[j]) / div;
        }
      }
    }
    const long long i = ((n * g.H + h) * g.W + w) * (long long)C + c;
    T outv[V];
#pragma unroll
    for (int j = 0; j < V; ++j) outv[j] = Num<T>::from_f(acc[j]);
    if (V * sizeof(T) == 16) *reinterpret_cast<uint4*>(dx + i) = *reinterpret_cast<const uint4*>(outv);
    else {
#pragma unroll
      for (int j = 0; j < V; ++j) dx[i + j] = outv[j];
    }
  }
}

// The hot forward case with everything known at compile time: fp32, max pooling, square
// WIN x WIN window, stride S both ways, four channels per thread.  All WIN * WIN vectors of the
// window are requested before the first comparison (the general kernel's loops have run-time
// bounds, so its loads go out one after the other); the selection then walks them in the same
// order with the same rule, so values and argmax bytes are identical.
template <int WIN, int S>
__global__ void __launch_bounds__(256)
pool_forward_max_cl_fixed_kernel(const float* __restrict__ x, float* __restrict__ y,
                                 uint8_t* __restrict__ argmax, PoolGeo g, int C, int cv_shift,
                                 int per_image) {
  const long long n = blockIdx.y;
  const unsigned cv = (unsigned)C >> 2;
  for (unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < (unsigned)per_image;
       t += gridDim.x * blockDim.x) {
    const unsigned pix = cv_shift >= 0 ? t >> cv_shift : t / cv;
    const int c = (int)(t - pix * cv) * 4;
    const int p = (int)(pix / (unsigned)g.Wo);
    const int q = (int)(pix - (unsigned)p * (unsigned)g.Wo);
    const int h0 = p * S - g.py, w0 = q * S - g.px;
    const float* xn = x + n * (long long)g.H * g.W * C + c;
    float4 v[WIN * WIN];
    bool in[WIN * WIN];
#pragma unroll
    for (int ky = 0; ky < WIN; ++ky)
#pragma unroll
      for (int kx = 0; kx < WIN; ++kx) {
        const int h = h0 + ky, w = w0 + kx;
        const int i = ky * WIN + kx;
        in[i] = h >= 0 && h < g.H && w >= 0 && w < g.W;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in[i]) v[i] = *reinterpret_cast<const float4*>(xn + ((long long)h * g.W + w) * C);
      }
    float acc[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    int arg[4] = {255, 255, 255, 255};
#pragma unroll
    for (int i = 0; i < WIN * WIN; ++i) {
      if (!in[i]) continue;
      const float e[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (arg[j] == 255 || e[j] > acc[j] || e[j] != e[j]) { acc[j] = e[j]; arg[j] = i; }
    }
    const long long o = ((n * g.Ho + p) * g.Wo + q) * (long long)C + c;
    *reinterpret_cast<float4*>(y + o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    if (argmax)
      *reinterpret_cast<uint32_t*>(argmax + o) = (uint32_t)arg[0] | ((uint32_t)arg[1] << 8) |
                                                 ((uint32_t)arg[2] << 16) | ((uint32_t)arg[3] << 24);
  }
}

// The hot case of the above with everything known at compile time: fp32, max pooling with the
// argmax payload, square WIN x WIN window, stride S both ways (3x3 / 2 and 2x2 / 2), four
// channels per thread.  An input pixel lies in at most ceil(WIN / S)^2 windows; their
// candidates are enumerated without divisions or data-dependent loop bounds.
template <int WIN, int S>
__global__ void __launch_bounds__(256)
pool_backward_max_cl_fixed_kernel(const float* __restrict__ dy, const uint8_t* __restrict__ argmax,
                                  float* __restrict__ dx, PoolGeo g, int C, int cv_shift,
                                  int per_image) {
  constexpr int NW = (WIN + S - 1) / S;  // windows per axis that can cover a pixel
  const long long n = blockIdx.y;
  const unsigned cv = (unsigned)C >> 2;
  for (unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < (unsigned)per_image;
       t += gridDim.x * blockDim.x) {
    const unsigned pix = cv_shift >= 0 ? t >> cv_shift : t / cv;
    const int c = (int)(t - pix * cv) * 4;
    const int h = (int)(pix / (unsigned)g.W);
    const int w = (int)(pix - (unsigned)h * (unsigned)g.W);
    const int hp = h + g.py, wp = w + g.px;
    const int p1 = hp / S, q1 = wp / S;  // S is a compile-time constant: shifts
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int a = 0; a < NW; ++a) {
      const int p = p1 - a, ky = hp - p * S;
      if (p < 0 || p >= g.Ho || ky >= WIN) continue;
#pragma unroll
      for (int b = 0; b < NW; ++b) {
        const int q = q1 - b, kx = wp - q * S;
        if (q < 0 || q >= g.Wo || kx >= WIN) continue;
        const long long o = ((n * g.Ho + p) * g.Wo + q) * (long long)C + c;
        const uint32_t sel = *reinterpret_cast<const uint32_t*>(argmax + o);
        const float4 gv = *reinterpret_cast<const float4*>(dy + o);
        const uint32_t mine = (uint32_t)(ky * WIN + kx);
        if ((sel & 0xffu) == mine) acc.x += gv.x;
        if (((sel >> 8) & 0xffu) == mine) acc.y += gv.y;
        if (((sel >> 16) & 0xffu) == mine) acc.z += gv.z;
        if ((sel >> 24) == mine) acc.w += gv.w;
      }
    }
    *reinterpret_cast<float4*>(dx + ((n * g.H + h) * g.W + w) * (long long)C + c) = acc;
  }
}

// The same gradient with a thread per 2 x 2 cell of input pixels (stride 2 both ways): the four
// pixels of a cell lie in the same (at most) 2 x 2 windows, so a thread reads four dy vectors
// and argmax words for four results instead of nine.  Candidates are added in the order of the
// kernel above (nearer window first, rows before columns): identical sums.
template <int WIN>
__global__ void __launch_bounds__(256)
pool_backward_max_cl_cell_kernel(const float* __restrict__ dy, const uint8_t* __restrict__ argmax,
                                 float* __restrict__ dx, PoolGeo g, int C, int cv_shift,
                                 int cells_w, int per_image) {
  const long long n = blockIdx.y;
  const unsigned cv = (unsigned)C >> 2;
  for (unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < (unsigned)per_image;
       t += gridDim.x * blockDim.x) {
    const unsigned cell = cv_shift >= 0 ? t >> cv_shift : t / cv;
    const int c = (int)(t - cell * cv) * 4;
    const int ca = (int)(cell / (unsigned)cells_w);          // cell row: padded rows 2 ca, 2 ca + 1
    const int cb = (int)(cell - (unsigned)ca * (unsigned)cells_w);
    float4 gv[2][2];
    uint32_t sel[2][2];
    bool live[2][2];
#pragma unroll
    for (int pa = 0; pa < 2; ++pa)
#pragma unroll
      for (int qb = 0; qb < 2; ++qb) {
        const int p = ca - pa, q = cb - qb;
        live[pa][qb] = p >= 0 && p < g.Ho && q >= 0 && q < g.Wo;
        gv[pa][qb] = make_float4(0.f, 0.f, 0.f, 0.f);
        sel[pa][qb] = 0xffffffffu;
        if (live[pa][qb]) {
          const long long o = ((n * g.Ho + p) * g.Wo + q) * (long long)C + c;
          sel[pa][qb] = *reinterpret_cast<const uint32_t*>(argmax + o);
          gv[pa][qb] = *reinterpret_cast<const float4*>(dy + o);
        }
      }
#pragma unroll
    for (int dh = 0; dh < 2; ++dh) {
      const int h = 2 * ca + dh - g.py;
      if (h < 0 || h >= g.H) continue;
#pragma unroll
      for (int dw = 0; dw < 2; ++dw) {
        const int w = 2 * cb + dw - g.px;
        if (w < 0 || w >= g.W) continue;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int pa = 0; pa < 2; ++pa) {
          const int ky = dh + 2 * pa;
          if (ky >= WIN) continue;
#pragma unroll
          for (int qb = 0; qb < 2; ++qb) {
            const int kx = dw + 2 * qb;
            if (kx >= WIN || !live[pa][qb]) continue;
            const uint32_t mine = (uint32_t)(ky * WIN + kx), s4 = sel[pa][qb];
            const float4 v = gv[pa][qb];
            if ((s4 & 0xffu) == mine) acc.x += v.x;
            if (((s4 >> 8) & 0xffu) == mine) acc.y += v.y;
            if (((s4 >> 16) & 0xffu) == mine) acc.z += v.z;
            if ((s4 >> 24) == mine) acc.w += v.w;
          }
        }
        *reinterpret_cast<float4*>(dx + ((n * g.H + h) * g.W + w) * (long long)C + c) = acc;
      }
    }
  }
}

template <typename T>
int launch_pool_cl(bool backward, const PoolGeo& g, int C, int N, const void* a, const void* x,
                   const uint8_t* argmax_in, uint8_t* argmax_out, void* out, cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  const long long pixels = backward ? (long long)g.H * g.W : (long long)g.Ho * g.Wo;
  const bool vec = C % V == 0 && aligned16(a) && aligned16(out) && (!x || aligned16(x)) &&
                   (reinterpret_cast<uintptr_t>(argmax_in) & (V - 1)) == 0 &&
                   (reinterpret_cast<uintptr_t>(argmax_out) & (V - 1)) == 0;
  const long long per_image = pixels * (vec ? C / V : C);
  FLB200_REQUIRE(per_image < 0x7fffffffLL && N <= 65535, "pool2d: image too large");
  long long bx = (per_image + 255) / 256;
  if (bx > 4096) bx = 4096;
  const dim3 grid((unsigned)bx, (unsigned)N);
  const int pi = (int)per_image;
  if (!backward) {
    if constexpr (std::is_same<T, float>::value) {
      if (vec && g.mode == FLB200_POOL_MAX && g.wx == g.wy && g.sx == g.sy && g.sx == 2 &&
          (g.wx == 3 || g.wx == 2)) {
        const unsigned cvv = (unsigned)C / 4;
        int shift = -1;
        if ((cvv & (cvv - 1)) == 0) { shift = 0; while ((1u << shift) < cvv) ++shift; }
        if (g.wx == 3)
          pool_forward_max_cl_fixed_kernel<3, 2><<<grid, 256, 0, st>>>(
              static_cast<const float*>(a), static_cast<float*>(out), argmax_out, g, C, shift, pi);
        else
          pool_forward_max_cl_fixed_kernel<2, 2><<<grid, 256, 0, st>>>(
              static_cast<const float*>(a), static_cast<float*>(out), argmax_out, g, C, shift, pi);
        FLB200_AFTER_LAUNCH("pool2d_forward_max_channels_last");
        return FLB200_OK;
      }
    }
    if (vec)
      pool_forward_cl_kernel<T, V><<<grid, 256, 0, st>>>(static_cast<const T*>(a),
                                                         static_cast<T*>(out), argmax_out, g, C, pi);
    else
      pool_forward_cl_kernel<T, 1><<<grid, 256, 0, st>>>(static_cast<const T*>(a),
                                                         static_cast<T*>(out), argmax_out, g, C, pi);
    FLB200_AFTER_LAUNCH("pool2d_forward_channels_last");
  } else {
    if constexpr (std::is_same<T, float>::value) {
      if (vec && g.mode == FLB200_POOL_MAX && argmax_in && g.wx == g.wy && g.sx == g.sy &&
          g.sx == 2 && (g.wx == 3 || g.wx == 2)) {
        const unsigned cvv = (unsigned)C / 4;
        int shift = -1;
        if ((cvv & (cvv - 1)) == 0) { shift = 0; while ((1u << shift) < cvv) ++shift; }
        // cells of 2 x 2 input pixels in padded coordinates
        const long long cells_h = (g.H + g.py + 1) / 2, cells_w = (g.W + g.px + 1) / 2;
        const long long per_cells = cells_h * cells_w * cvv;
        if (per_cells < 0x7fffffffLL) {
          long long cbx = (per_cells + 255) / 256;
          if (cbx > 4096) cbx = 4096;
          const dim3 cgrid((unsigned)cbx, (unsigned)N);
          if (g.wx == 3)
            pool_backward_max_cl_cell_kernel<3><<<cgrid, 256, 0, st>>>(
                static_cast<const float*>(a), argmax_in, static_cast<float*>(out), g, C, shift,
                (int)cells_w, (int)per_cells);
          else
            pool_backward_max_cl_cell_kernel<2><<<cgrid, 256, 0, st>>>(
                static_cast<const float*>(a), argmax_in, static_cast<float*>(out), g, C, shift,
                (int)cells_w, (int)per_cells);
          FLB200_AFTER_LAUNCH("pool2d_backward_max_channels_last");
          return FLB200_OK;
        }
        if (g.wx == 3)
          pool_backward_max_cl_fixed_kernel<3, 2><<<grid, 256, 0, st>>>(
              static_cast<const float*>(a), argmax_in, static_cast<float*>(out), g, C, shift, pi);
        else
          pool_backward_max_cl_fixed_kernel<2, 2><<<grid, 256, 0, st>>>(
              static_cast<const float*>(a), argmax_in, static_cast<float*>(out), g, C, shift, pi);
        FLB200_AFTER_LAUNCH("pool2d_backward_max_channels_last");
        return FLB200_OK;
      }
    }
    if (vec)
      pool_backward_cl_kernel<T, V><<<grid, 256, 0, st>>>(
          static_cast<const T*>(a), static_cast<const T*>(x), argmax_in, static_cast<T*>(out), g, C,
          pi);
    else
      pool_backward_cl_kernel<T, 1><<<grid, 256, 0, st>>>(
          static_cast<const T*>(a), static_cast<const T*>(x), argmax_in, static_cast<T*>(out), g, C,
          pi);
    FLB200_AFTER_LAUNCH("pool2d_backward_channels_last");
  }
  return FLB200_OK;
}

int pool_cl_dispatch(bool backward, const flb200_pool2d_desc* d, const PoolGeo& g, const void* a,
                     const void* x, const uint8_t* argmax_in, uint8_t* argmax_out, void* out,
                     cudaStream_t st) {
  switch (d->dtype) {
    case FLB200_F32:
      return launch_pool_cl<float>(backward, g, d->C, d->N, a, x, argmax_in, argmax_out, out, st);
    case FLB200_F16:
      return launch_pool_cl<__half>(backward, g, d->C, d->N, a, x, argmax_in, argmax_out, out, st);
    case FLB200_BF16:
      return launch_pool_cl<__nv_bfloat16>(backward, g, d->C, d->N, a, x, argmax_in, argmax_out, out,
                                           st);
    default:
      return fail(FLB200_UNSUPPORTED, "pool2d: unknown dtype %d", d->dtype);
  }
}

int make_geo(const char* name, const flb200_pool2d_desc* d, PoolGeo* g) {
  FLB200_REQUIRE(d, "%s: null descriptor", name);
  FLB200_REQUIRE(d->W >= 1 && d->H >= 1 && d->C >= 1 && d->N >= 1, "%s: empty input", name);
  FLB200_REQUIRE(d->wx >= 1 && d->wy >= 1 && d->sx >= 1 && d->sy >= 1 && d->px >= 0 && d->py >= 0,
                 "%s: bad window/stride/padding", name);
  FLB200_REQUIRE(d->mode >= FLB200_POOL_MAX && d->mode <= FLB200_POOL_AVG_EXCLUDE_PAD,
                 "%s: unknown pooling mode %d", name, d->mode);
  // only max pooling keeps a window position in its one-byte argmax payload
  FLB200_REQUIRE(d->mode != FLB200_POOL_MAX || (long long)d->wx * d->wy <= 255,
                 "%s: max-pooling window larger than 255 elements", name);
  FLB200_REQUIRE(d->W + 2 * d->px >= d->wx && d->H + 2 * d->py >= d->wy,
                 "%s: window larger than padded input", name);
  FLB200_REQUIRE(d->layout == FLB200_LAYOUT_NCHW || d->layout == FLB200_LAYOUT_NHWC,
                 "%s: unknown layout %d", name, d->layout);
  g->W = d->W; g->H = d->H;
  g->Wo = 1 + (d->W + 2 * d->px - d->wx) / d->sx;
  g->Ho = 1 + (d->H + 2 * d->py - d->wy) / d->sy;
  g->wx = d->wx; g->wy = d->wy; g->sx = d->sx; g->sy = d->sy; g->px = d->px; g->py = d->py;
  g->mode = d->mode;
  g->planes = (long long)d->C * d->N;
  return FLB200_OK;
}

}  // namespace
}  // namespace flb200

using namespace flb200;

extern "C" {

int flb200_pool2d_output_dims(const flb200_pool2d_desc* d, int32_t* Wo, int32_t* Ho) {
  PoolGeo g;
  if (int st = make_geo("pool2d_output_dims", d, &g)) return st;
  if (Wo) *Wo = g.Wo;
  if (Ho) *Ho = g.Ho;
  return FLB200_OK;
}

int flb200_pool2d_forward(const flb200_pool2d_desc* d, const void* x, void* y, uint8_t* argmax,
                          void* stream) {
  PoolGeo g;
  if (int st = make_geo("pool2d_forward", d, &g)) return st;
  FLB200_REQUIRE(x && y, "pool2d_forward: null tensor");
  const long long total = g.planes * g.Ho * g.Wo;
  const int grid = grid_for(total, 256);
  cudaStream_t st = as_stream(stream);
  if (d->layout == FLB200_LAYOUT_NHWC)
    return pool_cl_dispatch(false, d, g, x, nullptr, nullptr, argmax, y, st);
  if (d->mode == FLB200_POOL_MAX && d->dtype == FLB200_F32) {
    const int band = pool_fwd_band_rows(g);
    const long long nbands = band > 0 ? (g.Ho + band - 1) / band : 0;
    if (band > 0 && g.planes * nbands < 0x7fffffffLL) {
      const size_t smem = (size_t)((band - 1) * g.sy + g.wy) * g.W * sizeof(float);
      const float* xf = static_cast<const float*>(x);
      float* yf = static_cast<float*>(y);
      if (is_window(g, 3, 3, 2, 2))
        launch_pool_fwd_tile<3, 3, 2, 2>(xf, yf, argmax, g, band, (int)nbands, smem, st);
      else if (is_window(g, 2, 2, 2, 2))
        launch_pool_fwd_tile<2, 2, 2, 2>(xf, yf, argmax, g, band, (int)nbands, smem, st);
      else
        launch_pool_fwd_tile<0, 0, 0, 0>(xf, yf, argmax, g, band, (int)nbands, smem, st);
      FLB200_AFTER_LAUNCH("pool2d_forward_max_tile");
      return FLB200_OK;
    }
  }
  switch (d->dtype) {
    case FLB200_F32:
      pool_forward_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x),
                                                       static_cast<float*>(y), argmax, g);
      break;
    case FLB200_F16:
      pool_forward_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x),
                                                        static_cast<__half*>(y), argmax, g);
      break;
    case FLB200_BF16:
      pool_forward_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), argmax, g);
      break;
    default:
      return fail(FLB200_UNSUPPORTED, "pool2d_forward: unknown dtype %d", d->dtype);
  }
  FLB200_AFTER_LAUNCH("pool2d_forward");
  return FLB200_OK;
}

int flb200_pool2d_backward(const flb200_pool2d_desc* d, const void* grad_y, const void* x,
                           const uint8_t* argmax, void* grad_x, void* stream) {
  PoolGeo g;
  if (int st = make_geo("pool2d_backward", d, &g)) return st;
  FLB200_REQUIRE(grad_y && grad_x, "pool2d_backward: null tensor");
  FLB200_REQUIRE(d->mode != FLB200_POOL_MAX || argmax || x,
                 "pool2d_backward: max pooling needs the argmax payload or the input");
  const long long total = g.planes * g.H * g.W;
  const int grid = grid_for(total, 256);
  cudaStream_t st = as_stream(stream);
  if (d->layout == FLB200_LAYOUT_NHWC)
    return pool_cl_dispatch(true, d, g, grad_y, x, argmax, nullptr, grad_x, st);
  if (d->mode == FLB200_POOL_MAX && argmax && d->dtype == FLB200_F32) {
    int out_rows = 0;
    const int band = pool_bwd_band_rows(g, &out_rows);
    const long long nbands = band > 0 ? (g.H + band - 1) / band : 0;
    if (band > 0 && g.planes * nbands < 0x7fffffffLL) {
      const size_t smem = (size_t)out_rows * g.Wo * 5 + 16;
      const float* gyf = static_cast<const float*>(grad_y);
      float* gxf = static_cast<float*>(grad_x);
      if (is_window(g, 3, 3, 2, 2))
        launch_pool_bwd_tile<3, 3, 2, 2>(gyf, argmax, gxf, g, band, (int)nbands, out_rows, smem, st);
      else if (is_window(g, 2, 2, 2, 2))
        launch_pool_bwd_tile<2, 2, 2, 2>(gyf, argmax, gxf, g, band, (int)nbands, out_rows, smem, st);
      else
        launch_pool_bwd_tile<0, 0, 0, 0>(gyf, argmax, gxf, g, band, (int)nbands, out_rows, smem, st);
      FLB200_AFTER_LAUNCH("pool2d_backward_max_tile");
      return FLB200_OK;
    }
    const int strips = ((g.W + 3) / 4) * g.H;
    dim3 sgrid((unsigned)((strips + 255) / 256), (unsigned)(g.planes < 32768 ? g.planes : 32768));
    pool_backward_max_strip_kernel<float><<<sgrid, 256, 0, st>>>(
        static_cast<const float*>(grad_y), argmax, static_cast<float*>(grad_x), g);
    FLB200_AFTER_LAUNCH("pool2d_backward_max");
    return FLB200_OK;
  }
  if (d->mode != FLB200_POOL_MAX && d->dtype == FLB200_F32 && g.Ho == 1 && g.Wo == 1 &&
      g.px == 0 && g.py == 0 && g.wx == g.W && g.wy == g.H && g.H * g.W < (1 << 20)) {
    pool_backward_global_avg_kernel<<<grid, 256, 0, st>>>(
        static_cast<const float*>(grad_y), static_cast<float*>(grad_x), g.planes, g.H * g.W);
    FLB200_AFTER_LAUNCH("pool2d_backward_global_avg");
    return FLB200_OK;
  }
  switch (d->dtype) {
    case FLB200_F32:
      pool_backward_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(grad_y),
                                                        static_cast<const float*>(x), argmax,
                                                        static_cast<float*>(grad_x), g);
      break;
    case FLB200_F16:
      pool_backward_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(grad_y),
                                                         static_cast<const __half*>(x), argmax,
                                                         static_cast<__half*>(grad_x), g);
      break;
    case FLB200_BF16:
      pool_backward_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          static_cast<const __nv_bfloat16*>(grad_y), static_cast<const __nv_bfloat16*>(x), argmax,
          static_cast<__nv_bfloat16*>(grad_x), g);
      break;
    default:
      return fail(FLB200_UNSUPPORTED, "pool2d_backward: unknown dtype %d", d->dtype);
  }
  FLB200_AFTER_LAUNCH("pool2d_backward");
  return FLB200_OK;
}

}  // extern "C"
