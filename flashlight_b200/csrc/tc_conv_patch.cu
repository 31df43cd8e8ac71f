// Host side of the channels-last implicit-GEMM convolution (policies in tc_patch.cuh):
// NCHW -> NHWC copies of the activations, filter repacking, TMA tensor maps, tap tables.
//
// Scratch traffic per pass: one transposed copy of the activation operand (8 bytes per
// element) and a repacked filter; there is no im2col matrix.

#include "tc_conv.cuh"
#include "tc_patch.cuh"

namespace flb200 {
namespace {

inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }
inline int up4(int v) { return (v + 3) / 4 * 4; }

// Where a channels-last copy lives: in the caller's cache when it has a large enough,
// 256-byte aligned buffer for it, else at `fallback` inside the workspace.
struct ClSlot {
  float* buf;
  int32_t* flag;  // the cache's valid flag, or null without a cache buffer
  bool valid;     // the buffer already holds the copy
};
ClSlot cl_slot(flb200_conv2d_cache* c, int which, size_t bytes, float* fallback) {
  ClSlot s{fallback, nullptr, false};
  if (!c) return s;
  void* b = which == 0 ? c->x_cl : c->gy_cl;
  const size_t have = which == 0 ? c->x_cl_bytes : c->gy_cl_bytes;
  if (!b || have < bytes || (reinterpret_cast<uintptr_t>(b) & 255) != 0) return s;
  s.buf = static_cast<float*>(b);
  s.flag = which == 0 ? &c->x_cl_valid : &c->gy_cl_valid;
  s.valid = *s.flag != 0;
  return s;
}

// dst[n][hw][cp] = src[n][c][hw] for c < C, 0 for the padding channels C <= c < cp.
__global__ void __launch_bounds__(256)
nchw_to_nhwc_kernel(const float* __restrict__ src, float* __restrict__ dst, int C, int cp,
                    int HW) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int hw0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const long long n = blockIdx.z;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty + 8 * i, hw = hw0 + tx;
    tile[ty + 8 * i][tx] = (c < C && hw < HW) ? src[(n * C + c) * HW + hw] : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int hw = hw0 + ty + 8 * i, c = c0 + tx;
    if (hw < HW && c < cp) dst[(n * HW + hw) * cp + c] = tile[tx][ty + 8 * i];
  }
}

// The same transposition in 64 x 64 tiles with 16-byte accesses on both sides (four vector loads
// in flight per thread): for HW a multiple of 4 and 16-byte aligned tensors.
__global__ void __launch_bounds__(256)
nchw_to_nhwc_vec_kernel(const float* __restrict__ src, float* __restrict__ dst, int C, int cp,
                        int HW) {
  __shared__ float tile[64][65];
  const int hw0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
  const long long n = blockIdx.z;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 vectors across, 16 rows
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty + 16 * i, hw = hw0 + tx * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < C && hw < HW) v = *reinterpret_cast<const float4*>(src + (n * C + c) * HW + hw);
    tile[ty + 16 * i][tx * 4 + 0] = v.x;
    tile[ty + 16 * i][tx * 4 + 1] = v.y;
    tile[ty + 16 * i][tx * 4 + 2] = v.z;
    tile[ty + 16 * i][tx * 4 + 3] = v.w;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int hw = hw0 + ty + 16 * i, c = c0 + tx * 4;
    if (hw < HW && c < cp) {
      const float4 v = make_float4(tile[tx * 4 + 0][ty + 16 * i], tile[tx * 4 + 1][ty + 16 * i],
                                   tile[tx * 4 + 2][ty + 16 * i], tile[tx * 4 + 3][ty + 16 * i]);
      *reinterpret_cast<float4*>(dst + (n * HW + hw) * cp + c) = v;
    }
  }
}

int to_nhwc(const float* src, float* dst, int N, int C, int cp, int HW, cudaStream_t st) {
  if ((HW & 3) == 0 && (cp & 3) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
    dim3 vgrid((unsigned)((HW + 63) / 64), (unsigned)((cp + 63) / 64), (unsigned)N);
    FLB200_REQUIRE(vgrid.y <= 65535 && vgrid.z <= 65535, "nchw_to_nhwc: extent out of range");
    nchw_to_nhwc_vec_kernel<<<vgrid, 256, 0, st>>>(src, dst, C, cp, HW);
    FLB200_AFTER_LAUNCH("nchw_to_nhwc_vec");
    return FLB200_OK;
  }
  dim3 grid((unsigned)((HW + 31) / 32), (unsigned)((cp + 31) / 32), (unsigned)N);
  FLB200_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "nchw_to_nhwc: extent out of range");
  nchw_to_nhwc_kernel<<<grid, 256, 0, st>>>(src, dst, C, cp, HW);
  FLB200_AFTER_LAUNCH("nchw_to_nhwc");
  return FLB200_OK;
}

// The same transposition of every (sy, sx)-th pixel only: dst[n][p][q][c] = src[n][c][p*sy][q*sx].
__global__ void __launch_bounds__(256)
nchw_to_nhwc_sampled_kernel(const float* __restrict__ src, float* __restrict__ dst, int C, int cp,
                            int HW, int W, int Wo, int HoWo, int sx, int sy) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int hw0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const long long n = blockIdx.z;
  const int o = hw0 + tx;
  const int p = o / Wo, q = o - p * Wo;
  const long long from = (long long)p * sy * W + (long long)q * sx;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty + 8 * i;
    tile[ty + 8 * i][tx] = (c < C && o < HoWo) ? src[(n * C + c) * HW + from] : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int hw = hw0 + ty + 8 * i, c = c0 + tx;
    if (hw < HoWo && c < cp) dst[(n * HoWo + hw) * cp + c] = tile[tx][ty + 8 * i];
  }
}

// A 1 x 1 convolution with a stride and no padding only ever reads every (sy, sx)-th pixel:
// its channels-last copy keeps just those, and the rest of the pass is a stride-1 convolution
// on the Wo x Ho image.  Returns the geometry the forward and backward-filter passes run on.
bool samples_input(const ConvGeo& g) {
  // (a channels-last x is read in place, with the stride in the tensor map)
  return !g.x_cl && g.RS == 1 && g.px == 0 && g.py == 0 && (g.sx > 1 || g.sy > 1);
}
// Backward-filter of a 1 x 1, stride 1, unpadded convolution over channels-last tensors: the
// K index is the pixel, and any 32 consecutive pixels make a K block, so the batch is walked
// as ONE image of N * H * W pixels in a row (no padded patch rows on 14 x 14 or 7 x 7 planes).
ConvGeo cl_wgrad_geo(const ConvGeo& g) {
  ConvGeo e = g;
  if (g.x_cl && g.y_cl && g.RS == 1 && g.sx == 1 && g.sy == 1 && g.px == 0 && g.py == 0 &&
      (long long)g.N * g.HW < 0x7fffffffLL) {
    e.W = e.Wo = g.N * g.HW;
    e.H = e.Ho = 1;
    e.N = 1;
    e.HW = e.HoWo = e.W;
  }
  return e;
}
ConvGeo sampled_geo(const ConvGeo& g) {
  ConvGeo e = g;
  if (samples_input(g)) {
    e.W = g.Wo; e.H = g.Ho; e.HW = g.HoWo;
    e.sx = 1; e.sy = 1;
  }
  return e;
}
// Channels-last copy of x for the forward / backward-filter passes of geometry g.
int x_to_nhwc(const ConvGeo& g, const float* x, float* xt, int cp, cudaStream_t st) {
  if (!samples_input(g)) return to_nhwc(x, xt, g.N, g.C, cp, g.HW, st);
  dim3 grid((unsigned)((g.HoWo + 31) / 32), (unsigned)((cp + 31) / 32), (unsigned)g.N);
  FLB200_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "nchw_to_nhwc: extent out of range");
  nchw_to_nhwc_sampled_kernel<<<grid, 256, 0, st>>>(x, xt, g.C, cp, g.HW, g.W, g.Wo, g.HoWo, g.sx,
                                                   g.sy);
  FLB200_AFTER_LAUNCH("nchw_to_nhwc_sampled");
  return FLB200_OK;
}

// Filter w[co][ci][tap] repacked to out[tap][rows][kp] with (rows, k) = (co, ci) for the
// forward pass and (ci, co) for backward-data; k >= its extent is zero.
__global__ void pack_filter_kernel(const float* __restrict__ w, float* __restrict__ out, int Cout,
                                   int C, int RS, int rows, int kext, int kp, int rows_are_co) {
  const long long total = (long long)RS * rows * kp;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(t % kp);
    const long long r2 = t / kp;
    const int row = (int)(r2 % rows), tap = (int)(r2 / rows);
    float v = 0.f;
    if (k < kext) {
      const int co = rows_are_co ? row : k, ci = rows_are_co ? k : row;
      v = w[((long long)co * C + ci) * RS + tap];
    }
    out[t] = v;
  }
}

// gw[co][ci][tap] = sum over splits of partial[split][tap][co][ci]
__global__ void wgrad_reduce_kernel(const float* __restrict__ partial, float* __restrict__ gw,
                                    int Cout, int C, int RS, int splits) {
  const long long per_split = (long long)RS * Cout * C;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < per_split;
       t += (long long)gridDim.x * blockDim.x) {
    const int ci = (int)(t % C);
    const long long r2 = t / C;
    const int co = (int)(r2 % Cout), tap = (int)(r2 / Cout);
    float s = 0.f;
    for (int sp = 0; sp < splits; ++sp) s += partial[(long long)sp * per_split + t];
    gw[((long long)co * C + ci) * RS + tap] = s;
  }
}

// The same, four input channels per thread (C a multiple of 4, 16-byte aligned partial sums):
// 16-byte loads of every split's slice, same order of additions.
__global__ void wgrad_reduce_vec_kernel(const float4* __restrict__ partial, float* __restrict__ gw,
                                        int Cout, int C4, int RS, int splits) {
  const long long per_split = (long long)RS * Cout * C4;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < per_split;
       t += (long long)gridDim.x * blockDim.x) {
    const int ci = 4 * (int)(t % C4);
    const long long r2 = t / C4;
    const int co = (int)(r2 % Cout), tap = (int)(r2 / Cout);
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp = 0; sp < splits; ++sp) {
      const float4 v = partial[(long long)sp * per_split + t];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    float* dst = gw + ((long long)co * (4 * C4) + ci) * RS + tap;
    if (RS == 1) {
      *reinterpret_cast<float4*>(dst) = s;
    } else {
      dst[0] = s.x; dst[RS] = s.y; dst[2 * RS] = s.z; dst[3 * RS] = s.w;
    }
  }
}

struct Patch { int QW, PH, NB, qw_shift, ph_shift; };
int log2i(int v) { int s = 0; while ((1 << s) < v) ++s; return s; }
// 128-row patch for the forward / backward-data passes.
Patch pick_patch(int Wq, int Hq, int images) {
  Patch p;
  p.QW = 8;
  while (p.QW < Wq && p.QW < 128) p.QW *= 2;
  // rows per patch: the power of two that leaves the fewest padding rows over the batch (14
  // image rows: 7 patches of 2 rows rather than 2 of 8); what is left of the 128 tile rows
  // goes to further images
  const int ph_max = 128 / p.QW;
  long long best = -1;
  p.PH = ph_max;
  for (int ph = ph_max; ph >= 1; ph /= 2) {
    const int nb = ph_max / ph;
    const long long tiles = (long long)((Hq + ph - 1) / ph) * ((images + nb - 1) / nb);
    if (best < 0 || tiles < best) { best = tiles; p.PH = ph; }
  }
  p.NB = ph_max / p.PH;
  p.qw_shift = log2i(p.QW);
  p.ph_shift = log2i(p.PH);
  return p;
}
// 32-pixel patch (the K extent of one stage) for the backward-filter pass.
void pick_k_patch(int Wq, int Hq, int* QW, int* PH) {
  int q = 4;
  while (q < Wq && q < 32) q *= 2;
  int ph = 32 / q;
  (void)Hq;
  *QW = q;
  *PH = ph;
}

// 4-D NHWC map [c, w, h, n] of a tensor with cp channels per pixel.
int nhwc_map(CUtensorMap* m, const float* base, int C, int cp, int W, int H, int N, int box_w,
             int box_h, int box_n, int sx, int sy, int mode) {
  const uint64_t dims[4] = {(uint64_t)C, (uint64_t)W, (uint64_t)H, (uint64_t)N};
  const uint64_t strides[3] = {(uint64_t)cp * 4, (uint64_t)W * cp * 4, (uint64_t)H * W * cp * 4};
  const uint32_t box[4] = {32, (uint32_t)(box_w * sx), (uint32_t)(box_h * sy), (uint32_t)box_n};
  const uint32_t es[4] = {1, (uint32_t)sx, (uint32_t)sy, 1};
  return tc::make_tensor_map(m, base, 4, dims, strides, box, mode, es);
}

// The same tensor with the channel index split into (32 contiguous channels, group of 32):
// [32, w, h, n, ceil(C / 32)].  One box of nbox groups lands in shared memory as nbox
// consecutive [pixels][32 channels] blocks, the layout of an MN-major operand.  Channels past
// C of the last group read the neighbouring pixel (or the bytes after the tensor, which the
// callers keep inside their workspace); such rows / columns of the product are never stored.
int nhwc_map5(CUtensorMap* m, const float* base, int C, int cp, int W, int H, int N, int box_w,
              int box_h, int nbox, int sx, int sy) {
  const uint64_t dims[5] = {32, (uint64_t)W, (uint64_t)H, (uint64_t)N, (uint64_t)((C + 31) / 32)};
  const uint64_t strides[4] = {(uint64_t)cp * 4, (uint64_t)W * cp * 4, (uint64_t)H * W * cp * 4,
                               128};
  const uint32_t box[5] = {32, (uint32_t)(box_w * sx), (uint32_t)(box_h * sy), 1, (uint32_t)nbox};
  const uint32_t es[5] = {1, (uint32_t)sx, (uint32_t)sy, 1, 1};
  return tc::make_tensor_map(m, base, 5, dims, strides, box, tc::kMapMnMajor, es);
}

// Packed filter map [k, rows, taps].
int filter_map(CUtensorMap* m, const float* base, int kext, int kp, int rows, int taps, int bn) {
  const uint64_t dims[3] = {(uint64_t)kext, (uint64_t)rows, (uint64_t)taps};
  const uint64_t strides[2] = {(uint64_t)kp * 4, (uint64_t)rows * kp * 4};
  const uint32_t box[3] = {32, (uint32_t)bn, 1};
  return tc::make_tensor_map(m, base, 3, dims, strides, box, tc::kMapKMajor);
}

// CTA pairs (tc_pair.cuh) for 256-column tiles: each CTA then loads half of the filter tile.
// Measured: 3x3 layers with 256-column tiles run 14 % faster on pairs (with the ring handed
// over two sub-stages at a time); at 128 and 64 columns pairs are slower than single CTAs.
bool patch_uses_pairs(int bn) { return bn >= 256 && !tc::x3_enabled(); }

// Fills the parts of the problem that do not depend on BN and launches with the BN that fits
// the number of output channels.  The filter map must have been made with
// filter_box_rows(bn) rows per box.
struct PatchArgs {
  Patch patch;
  int pix_w, pix_h, images, n_out, cchunks, a_w_mul, a_h_mul;
  int ncls;                                   // parity classes in this launch (1 = forward)
  tc::PatchClass cls[tc::kMaxPatchClasses];   // taps and output offsets of each
  float* out;
  const float* bias;
  int out_H, out_W, out_C, oh_mul, ow_mul, fill_cell, out_cl;
  float* stats;  // EpiStats matrix of the output (forward only) or null
};
int filter_box_rows(int bn) { return patch_uses_pairs(bn) ? bn / 2 : bn; }

template <int BN>
int run_patch(const CUtensorMap& ma, const CUtensorMap& mb, const PatchArgs& a, cudaStream_t st) {
  tc::PatchConvProblem<BN> p;
  p.a_mn_major = 0; p.b_mn_major = 0;
  p.QW = a.patch.QW; p.PH = a.patch.PH; p.NB = a.patch.NB;
  p.qw_shift = a.patch.qw_shift; p.ph_shift = a.patch.ph_shift;
  p.tiles_q = (a.pix_w + p.QW - 1) / p.QW;
  p.tiles_p = (a.pix_h + p.PH - 1) / p.PH;
  p.tiles_b = (a.images + p.NB - 1) / p.NB;
  p.pix_w = a.pix_w; p.pix_h = a.pix_h; p.images = a.images; p.n_out = a.n_out;
  p.cchunks = a.cchunks; p.a_w_mul = a.a_w_mul; p.a_h_mul = a.a_h_mul;
  p.ncls = a.ncls;
  for (int c = 0; c < tc::kMaxPatchClasses; ++c) p.cls[c] = a.cls[c < a.ncls ? c : 0];
  p.out = a.out; p.bias = a.bias;
  p.out_H = a.out_H; p.out_W = a.out_W; p.out_C = a.out_C;
  p.oh_mul = a.oh_mul; p.ow_mul = a.ow_mul;
  p.fill_cell = a.fill_cell;
  p.out_cl = a.out_cl;
  p.stats = a.stats;
  p.tiles_n = (p.n_out + BN - 1) / BN;
  const long long m_tiles = (long long)p.tiles_q * p.tiles_p * p.tiles_b;
  FLB200_REQUIRE(a.ncls >= 1 && a.ncls <= tc::kMaxPatchClasses, "patch conv: bad class count");
  FLB200_REQUIRE(m_tiles * p.tiles_n * a.ncls < 0x7fffffffLL, "patch conv: too many tiles");
  if constexpr (BN >= 256) {
    if (patch_uses_pairs(BN))
    return tc::launch_pair_problem<tc::PatchConvProblem<BN>, BN, 2>(
        "tc_patch_conv_pair", ma, mb, p, ((m_tiles + 1) / 2) * p.tiles_n * a.ncls, st);
  }
  return tc::launch_problem<tc::PatchConvProblem<BN>, BN>("tc_patch_conv", ma, mb, p,
                                                          m_tiles * p.tiles_n * a.ncls, st);
}
int run_patch_any(int bn, const CUtensorMap& ma, const CUtensorMap& mb, const PatchArgs& a,
                  cudaStream_t st) {
  if (bn == 32) return run_patch<32>(ma, mb, a, st);
  if (bn == 64) return run_patch<64>(ma, mb, a, st);
  if (bn == 128) return run_patch<128>(ma, mb, a, st);
  return run_patch<256>(ma, mb, a, st);
}

struct WgradPlan {
  int QW, PH, tiles_q, tiles_p, k_iters, splits, ips, bn;
  int tg, tap_groups, cn_shift, tiles_n;
  size_t partial_bytes;
};
// C = columns per tap, taps = number of taps (the window route passes 32 and kH).
WgradPlan plan_wgrad(const ConvGeo& g, int C, int taps) {
  WgradPlan w;
  pick_k_patch(g.Wo, g.Ho, &w.QW, &w.PH);
  w.tiles_q = (g.Wo + w.QW - 1) / w.QW;
  w.tiles_p = (g.Ho + w.PH - 1) / w.PH;
  w.k_iters = g.N * w.tiles_p * w.tiles_q;
  const int cboxes = (C + 31) / 32;
  if (cboxes >= 8) {
    w.cn_shift = 3; w.tg = 1; w.tap_groups = taps; w.bn = 256;
    w.tiles_n = (C + 255) / 256;
  } else {
    w.cn_shift = log2i(cboxes);
    const int tg_max = 8 >> w.cn_shift;
    w.tap_groups = (taps + tg_max - 1) / tg_max;
    w.tg = (taps + w.tap_groups - 1) / w.tap_groups;
    w.bn = tc::pick_bn(32 * (w.tg << w.cn_shift));
    if (w.bn == 128 && 32 * (w.tg << w.cn_shift) > 128) w.bn = 256;
    w.tiles_n = 1;
  }
  const long long out_tiles =
      (long long)((g.Cout + tc::kBM - 1) / tc::kBM) * w.tiles_n * w.tap_groups;
  tc::plan_splits(out_tiles, w.k_iters, 16, &w.splits, &w.ips);
  const long long splits = w.splits;
  w.partial_bytes = (size_t)splits * taps * g.Cout * C * 4;
  return w;
}
WgradPlan plan_wgrad(const ConvGeo& g) { return plan_wgrad(g, g.C, g.RS); }

inline int wgrad_a_boxes(int Cout) { return Cout >= tc::kBM ? tc::kBM / 32 : (Cout + 31) / 32; }

// Tap geometry of a backward-filter launch: tap t = (t / kW, t % kW) reads x at
// (s * dil_x - pad_x, r * dil_y - pad_y) from the output pixel's origin.
struct WgradTaps { int C, ntaps, kW, dil_x, dil_y, pad_x, pad_y; };

template <int BN>
int run_wgrad(const CUtensorMap& ma, const CUtensorMap& mb, const ConvGeo& g, const WgradTaps& tp,
              const WgradPlan& w, float* partial, cudaStream_t st) {
  tc::PatchWgradProblem<BN> p;
  p.a_mn_major = 1; p.b_mn_major = 1;
  p.QW = w.QW; p.PH = w.PH; p.tiles_q = w.tiles_q; p.tiles_p = w.tiles_p; p.images = g.N;
  p.M = g.Cout; p.N = tp.C;
  p.tiles_m = (g.Cout + tc::kBM - 1) / tc::kBM;
  p.tiles_n = w.tiles_n;
  p.ntaps = tp.ntaps; p.tap_groups = w.tap_groups; p.tg = w.tg; p.cn_shift = w.cn_shift;
  p.a_nbox = wgrad_a_boxes(g.Cout);
  p.splits = w.splits; p.iters_per_split = w.ips; p.k_iters = w.k_iters;
  p.b_w_mul = g.sx; p.b_h_mul = g.sy;
  p.kW = tp.kW; p.dil_x = tp.dil_x; p.dil_y = tp.dil_y; p.pad_x = tp.pad_x; p.pad_y = tp.pad_y;
  p.partial = partial;
  const long long tiles = (long long)p.tiles_m * p.tiles_n * p.tap_groups * p.splits;
  return tc::launch_problem<tc::PatchWgradProblem<BN>, BN>("tc_patch_wgrad", ma, mb, p, tiles,
                                                          st);
}
int run_wgrad_any(const CUtensorMap& ma, const CUtensorMap& mb, const ConvGeo& g,
                  const WgradTaps& tp, const WgradPlan& w, float* partial, cudaStream_t st) {
  if (w.bn == 32) return run_wgrad<32>(ma, mb, g, tp, w, partial, st);
  if (w.bn == 64) return run_wgrad<64>(ma, mb, g, tp, w, partial, st);
  if (w.bn == 128) return run_wgrad<128>(ma, mb, g, tp, w, partial, st);
  return run_wgrad<256>(ma, mb, g, tp, w, partial, st);
}

// ------------------------------------------------ few-channel "row window" route
// With <= 4 input channels a 32-channel K chunk would be almost empty.  Instead the K index
// runs over (s, c): in a zero-padded NHWC copy with 4 channels per pixel the kW taps of one
// filter row are 4*kW <= 32 CONTIGUOUS floats, so one 128-byte row of the A tile is a window
// of 8 pixels starting at the output pixel's first tap.  Windows of neighbouring output
// pixels overlap; the tensor map expresses that with a pixel stride (16 bytes) smaller than
// the window extent.  The filter rows r are the taps of the implicit GEMM (k_iters = kH).
constexpr int kWinPixels = 8;  // 32 floats / 4 channels

// dst[n][hp][wp] = (x[n][0..C)[hp-py][wp-px], 0...) as one float4, zero outside the image.
__global__ void __launch_bounds__(256)
nchw_to_nhwc4_pad_kernel(const float* __restrict__ x, float4* __restrict__ dst, int C, int H,
                         int W, int Hp, int Wp, int py, int px, long long total) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const int wp = (int)(t % Wp);
    const long long r2 = t / Wp;
    const int hp = (int)(r2 % Hp);
    const long long n = r2 / Hp;
    const int h = hp - py, w = wp - px;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (h >= 0 && h < H && w >= 0 && w < W) {
      for (int c = 0; c < C; ++c) v[c] = x[((n * C + c) * H + h) * W + w];
    }
    dst[t] = make_float4(v[0], v[1], v[2], v[3]);
  }
}

// wr[r][co][s*4 + c] = w[co][c][r][s], zero elsewhere (32 floats per row).
__global__ void pack_filter_rows_kernel(const float* __restrict__ w, float* __restrict__ wr,
                                        int Cout, int C, int kH, int kW) {
  const int total = kH * Cout * 32;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gridDim.x * blockDim.x) {
    const int j = t & 31, co = (t >> 5) % Cout, r = (t >> 5) / Cout;
    const int s = j >> 2, c = j & 3;
    wr[t] = (s < kW && c < C) ? w[((co * C + c) * kH + r) * kW + s] : 0.f;
  }
}

// gw[co][c][r][s] = sum over splits of partial[split][co][r*32 + s*4 + c]
__global__ void window_wgrad_reduce_kernel(const float* __restrict__ partial,
                                           float* __restrict__ gw, int Cout, int C, int kH, int kW,
                                           int splits) {
  const int total = Cout * C * kH * kW;
  const long long per_split = (long long)kH * Cout * 32;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gridDim.x * blockDim.x) {
    const int s = t % kW, r = (t / kW) % kH, c = (t / (kW * kH)) % C, co = t / (kW * kH * C);
    const long long src = ((long long)co * kH + r) * 32 + s * 4 + c;
    float acc = 0.f;
    for (int sp = 0; sp < splits; ++sp) acc += partial[(long long)sp * per_split + src];
    gw[t] = acc;
  }
}

struct WindowGeo { int Hp, Wp, starts; };
WindowGeo window_geo(const ConvGeo& g) {
  WindowGeo w;
  w.Hp = g.H + 2 * g.py;
  w.Wp = g.W + 2 * g.px;
  const int need = (g.Wo - 1) * g.sx + kWinPixels;
  if (w.Wp < need) w.Wp = need;
  w.starts = w.Wp - (kWinPixels - 1);
  return w;
}

// [32-float window, window start pixel, padded row, image]: the pixel stride (16 bytes) is
// smaller than the window, i.e. the rows of the view overlap.
int window_map(CUtensorMap* m, const float* base, const WindowGeo& wg, int N, int box_w, int box_h,
               int box_n, int sx, int sy) {
  const uint64_t dims[4] = {32, (uint64_t)wg.starts, (uint64_t)wg.Hp, (uint64_t)N};
  const uint64_t strides[3] = {16, (uint64_t)wg.Wp * 16, (uint64_t)wg.Hp * wg.Wp * 16};
  const uint32_t box[4] = {32, (uint32_t)(box_w * sx), (uint32_t)(box_h * sy), (uint32_t)box_n};
  const uint32_t es[4] = {1, (uint32_t)sx, (uint32_t)sy, 1};
  return tc::make_tensor_map(m, base, 4, dims, strides, box, tc::kMapKMajor, es);
}

// Backward-filter view: a fifth index r (the filter row) steps dy padded rows, so one copy
// of nbox >= kH groups brings the windows of every filter row of a 32-pixel patch as the
// [pixels][32] blocks of an MN-major operand.  Row p*sy + r*dy can pass the image's last
// padded row only for patch rows p >= Ho, where dy is zero and what is read instead (the next
// image, or the bytes after the tensor inside the workspace) is finite.
int window_rows_map(CUtensorMap* m, const float* base, const WindowGeo& wg, int N, int box_w,
                    int box_h, int nbox, int sx, int sy, int kH, int dil_y) {
  const uint64_t dims[5] = {32, (uint64_t)wg.starts, (uint64_t)wg.Hp, (uint64_t)N, (uint64_t)kH};
  const uint64_t strides[4] = {16, (uint64_t)wg.Wp * 16, (uint64_t)wg.Hp * wg.Wp * 16,
                               (uint64_t)dil_y * wg.Wp * 16};
  const uint32_t box[5] = {32, (uint32_t)(box_w * sx), (uint32_t)(box_h * sy), 1, (uint32_t)nbox};
  const uint32_t es[5] = {1, (uint32_t)sx, (uint32_t)sy, 1, 1};
  return tc::make_tensor_map(m, base, 5, dims, strides, box, tc::kMapMnMajor, es);
}

}  // namespace

// ---------------------------------------------------------------- interface
bool patch_conv_supported(const ConvGeo& g) {
  // small channel counts would waste most of each 32-wide K chunk: those stay on the gather route
  if (!(g.groups == 1 && g.RS <= 64 && g.C >= 16 && g.Cout >= 16 && g.sx <= 2 && g.sy <= 2 &&
        g.N <= 65535))
    return false;
  // channels-last tensors are read in place: their pixel stride must be a multiple of 16 bytes
  if (g.x_cl && g.C % 4 != 0) return false;
  if (g.y_cl && g.Cout % 4 != 0) return false;
  return g.x_cl == g.y_cl;
}

// Channels-last tensors are the operands themselves: no copy, no cache, and the scratch holds
// the repacked filter / the split-K partial sums only.
size_t patch_conv_workspace_bytes(const ConvGeo& g0, int which) {
  const ConvGeo g = which == 1 ? g0 : sampled_geo(g0);
  const int cp = up4(g.C), cop = up4(g.Cout);
  const size_t x_copy = g.x_cl ? 0 : up256((size_t)g.N * g.HW * cp * 4);
  const size_t gy_copy = g.y_cl ? 0 : up256((size_t)g.N * g.HoWo * cop * 4);
  if (which == 0) return x_copy + up256((size_t)g.RS * g.Cout * cp * 4);
  if (which == 1) return gy_copy + up256((size_t)g.RS * g.C * cop * 4);
  return x_copy + gy_copy + up256(plan_wgrad(cl_wgrad_geo(g)).partial_bytes);
}

size_t patch_conv_cache_bytes(const ConvGeo& g, int which) {
  if (which == 0) return g.x_cl ? 0 : up256((size_t)g.N * sampled_geo(g).HW * up4(g.C) * 4);
  return g.y_cl ? 0 : up256((size_t)g.N * g.HoWo * up4(g.Cout) * 4);
}

// rows of the statistics matrix: four per pixel patch (one per 32-row quarter of a tile)
long long patch_conv_stats_groups(const ConvGeo& g0) {
  const ConvGeo g = patch_conv_supported(g0) ? sampled_geo(g0) : g0;
  const Patch pt = pick_patch(g.Wo, g.Ho, g.N);
  return 4LL * ((g.Wo + pt.QW - 1) / pt.QW) * ((g.Ho + pt.PH - 1) / pt.PH) *
         ((g.N + pt.NB - 1) / pt.NB);
}

int patch_conv_forward(const ConvGeo& g0, const float* x, const float* w, const float* bias,
                       float* y, void* ws, size_t ws_bytes, cudaStream_t st,
                       flb200_conv2d_cache* cache, const ConvStats* stats) {
  (void)ws_bytes;
  const ConvGeo g = sampled_geo(g0);
  const int cp = up4(g.C);
  char* base = static_cast<char*>(ws);
  const float* xt = x;
  float* wp = reinterpret_cast<float*>(base);
  if (!g.x_cl) {
    const ClSlot xs =
        cl_slot(cache, 0, (size_t)g.N * g.HW * cp * 4, reinterpret_cast<float*>(base));
    wp = reinterpret_cast<float*>(base + up256((size_t)g.N * g.HW * cp * 4));
    if (!xs.valid) {
      if (int rc = x_to_nhwc(g0, x, xs.buf, cp, st)) return rc;
      if (xs.flag) *xs.flag = 1;
    }
    xt = xs.buf;
  }
  pack_filter_kernel<<<grid_for((long long)g.RS * g.Cout * cp, 256), 256, 0, st>>>(
      w, wp, g.Cout, g.C, g.RS, g.Cout, g.C, cp, 1);
  FLB200_AFTER_LAUNCH("pack_filter");
  PatchArgs a{};
  a.patch = pick_patch(g.Wo, g.Ho, g.N);
  a.pix_w = g.Wo; a.pix_h = g.Ho; a.images = g.N; a.n_out = g.Cout;
  a.cchunks = (g.C + tc::kBK - 1) / tc::kBK;
  a.a_w_mul = g.sx; a.a_h_mul = g.sy;
  a.ncls = 1;
  a.cls[0] = tc::PatchClass{tc::TapGrid{g.kH, g.kW, -g.py, g.dy, -g.px, g.dx, 0, 1, 0, 1, g.kW},
                            g.RS, 0, 0};
  a.out = y; a.bias = bias;
  a.out_H = g.Ho; a.out_W = g.Wo; a.out_C = g.Cout;
  a.oh_mul = 1; a.ow_mul = 1;
  a.out_cl = g.y_cl;
  a.stats = stats && g.y_cl ? stats->matrix : nullptr;
  const int bn = tc::pick_bn(g.Cout);
  CUtensorMap ma, mb;
  if (int rc = nhwc_map(&ma, xt, g.C, cp, g.W, g.H, g.N, a.patch.QW, a.patch.PH, a.patch.NB, g.sx,
                        g.sy, tc::kMapKMajor))
    return rc;
  if (int rc = filter_map(&mb, wp, g.C, cp, g.Cout, g.RS, filter_box_rows(bn))) return rc;
  return run_patch_any(bn, ma, mb, a, st);
}

int patch_conv_backward_data(const ConvGeo& g, const float* gy, const float* w, float* gx,
                             void* ws, size_t ws_bytes, cudaStream_t st,
    flb200_conv2d_cache* cache) {
  (void)ws_bytes;
  const int cop = up4(g.Cout);
  char* base = static_cast<char*>(ws);
  const float* gyt = gy;
  float* wd = reinterpret_cast<float*>(base);
  if (!g.y_cl) {
    const ClSlot gs =
        cl_slot(cache, 1, (size_t)g.N * g.HoWo * cop * 4, reinterpret_cast<float*>(base));
    wd = reinterpret_cast<float*>(base + up256((size_t)g.N * g.HoWo * cop * 4));
    if (int rc = to_nhwc(gy, gs.buf, g.N, g.Cout, cop, g.HoWo, st)) return rc;
    if (gs.flag) *gs.flag = 1;  // backward-filter of the same grad_y can take it from here
    gyt = gs.buf;
  }
  pack_filter_kernel<<<grid_for((long long)g.RS * g.C * cop, 256), 256, 0, st>>>(
      w, wd, g.Cout, g.C, g.RS, g.C, g.Cout, cop, 0);
  FLB200_AFTER_LAUNCH("pack_filter");
  const int bn = tc::pick_bn(g.C);
  CUtensorMap mb;
  if (int rc = filter_map(&mb, wd, g.Cout, cop, g.C, g.RS, filter_box_rows(bn))) return rc;
  // One launch per parity class (a, b) of the input pixel: h = p*sy + a, w = q*sx + b.  Only
  // the taps with (a + py - r*dy) divisible by sy reach that class.
  // One launch per parity class (a, b) of the input pixel: h = p*sy + a, w = q*sx + b.  Only
  // the taps with (a + py - r*dy) divisible by sy reach that class; they form an arithmetic
  // progression in r (and likewise in s).  Classes that no tap reaches keep a zero gradient.
  struct Prog { int first, step, count, off0, off_step; };
  auto progression = [](int cls, int pad, int dil, int stride, int kext) {
    Prog pr{0, 1, 0, 0, 0};
    int first = -1, second = -1;
    for (int r = 0; r < kext; ++r)
      if ((cls + pad - r * dil) % stride == 0) {
        if (first < 0) first = r;
        else if (second < 0) second = r;
        ++pr.count;
      }
    if (pr.count == 0) return pr;
    pr.first = first;
    pr.step = second >= 0 ? second - first : 1;
    pr.off0 = (cls + pad - first * dil) / stride;
    pr.off_step = -(pr.step * dil) / stride;
    return pr;
  };
  int empty = 0, live = 0;
  bool origin_live = false;
  for (int ca = 0; ca < g.sy; ++ca)
    for (int cb = 0; cb < g.sx; ++cb) {
      const bool none = progression(ca, g.py, g.dy, g.sy, g.kH).count == 0 ||
                        progression(cb, g.px, g.dx, g.sx, g.kW).count == 0;
      empty += none;
      live += !none;
      if (!none && ca == 0 && cb == 0) origin_live = true;
    }
  // When (0, 0) is the only class that any tap reaches (a 1 x 1 filter without padding) its
  // launch writes the zeros of the other classes itself; otherwise clear gx first.
  const bool fill_cell = live == 1 && origin_live && empty > 0;
  if (empty > 0 && !fill_cell)
    FLB200_CUDA_CHECK(cudaMemsetAsync(gx, 0, (size_t)g.N * g.C * g.HW * 4, st));
  // The classes of one launch must have the same pixel extent (H, W multiples of the stride)
  // and fit the policy's class table; then ONE launch walks all of them, the classes of a
  // pixel patch as consecutive tiles, so that their interleaved stores meet in L2.  Otherwise
  // one launch per class.
  // (Measured on the ResNet-50 layers: 15-31 % faster with 256-column tiles, 6 % slower at 128.)
  const bool merge = !fill_cell && live > 1 && live <= tc::kMaxPatchClasses && g.H % g.sy == 0 &&
                     g.W % g.sx == 0 && bn >= 256;
  PatchArgs a{};
  a.images = g.N; a.n_out = g.C;
  a.cchunks = (g.Cout + tc::kBK - 1) / tc::kBK;
  a.a_w_mul = 1; a.a_h_mul = 1;
  a.out = gx; a.bias = nullptr;
  a.out_H = g.H; a.out_W = g.W; a.out_C = g.C;
  a.oh_mul = g.sy; a.ow_mul = g.sx;
  a.fill_cell = fill_cell ? 1 : 0;
  a.out_cl = g.x_cl;
  auto launch = [&](PatchArgs& args) -> int {
    args.patch = pick_patch(args.pix_w, args.pix_h, g.N);
    CUtensorMap ma;
    if (int rc = nhwc_map(&ma, gyt, g.Cout, cop, g.Wo, g.Ho, g.N, args.patch.QW, args.patch.PH,
                          args.patch.NB, 1, 1, tc::kMapKMajor))
      return rc;
    return run_patch_any(bn, ma, mb, args, st);
  };
  for (int ca = 0; ca < g.sy; ++ca)
    for (int cb = 0; cb < g.sx; ++cb) {
      const Prog ph = progression(ca, g.py, g.dy, g.sy, g.kH);
      const Prog pw = progression(cb, g.px, g.dx, g.sx, g.kW);
      if (ph.count == 0 || pw.count == 0) continue;
      const int pix_h = (g.H - ca + g.sy - 1) / g.sy, pix_w = (g.W - cb + g.sx - 1) / g.sx;
      if (pix_h <= 0 || pix_w <= 0) continue;
      const tc::PatchClass pc{
          tc::TapGrid{ph.count, pw.count, ph.off0, ph.off_step, pw.off0, pw.off_step, ph.first,
                      ph.step, pw.first, pw.step, g.kW},
          ph.count * pw.count, ca, cb};
      a.pix_h = pix_h; a.pix_w = pix_w;
      if (merge) {
        a.cls[a.ncls++] = pc;
      } else {
        a.ncls = 1;
        a.cls[0] = pc;
        if (int rc = launch(a)) return rc;
      }
    }
  if (merge && a.ncls > 0)
    if (int rc = launch(a)) return rc;
  return FLB200_OK;
}

int patch_conv_backward_filter(const ConvGeo& g0, const float* gy, const float* x, float* gw,
                               void* ws, size_t ws_bytes, cudaStream_t st,
                               flb200_conv2d_cache* cache) {
  const ConvGeo g = cl_wgrad_geo(sampled_geo(g0));
  (void)ws_bytes;
  const int cp = up4(g.C), cop = up4(g.Cout);
  const WgradPlan wp = plan_wgrad(g);
  char* base = static_cast<char*>(ws);
  size_t off = 0;
  const float* xt = x;
  if (!g.x_cl) {
    const ClSlot xs =
        cl_slot(cache, 0, (size_t)g.N * g.HW * cp * 4, reinterpret_cast<float*>(base));
    off += up256((size_t)g.N * g.HW * cp * 4);
    if (!xs.valid) {
      if (int rc = x_to_nhwc(g0, x, xs.buf, cp, st)) return rc;
      if (xs.flag) *xs.flag = 1;
    }
    xt = xs.buf;
  }
  const float* gyt = gy;
  if (!g.y_cl) {
    const ClSlot gs =
        cl_slot(cache, 1, (size_t)g.N * g.HoWo * cop * 4, reinterpret_cast<float*>(base + off));
    off += up256((size_t)g.N * g.HoWo * cop * 4);
    if (gs.valid) {
      *gs.flag = 0;  // consumed: the next backward pass brings another grad_y
    } else {
      if (int rc = to_nhwc(gy, gs.buf, g.N, g.Cout, cop, g.HoWo, st)) return rc;
    }
    gyt = gs.buf;
  }
  float* partial = reinterpret_cast<float*>(base + off);
  CUtensorMap ma, mb;
  if (int rc = nhwc_map5(&ma, gyt, g.Cout, cop, g.Wo, g.Ho, g.N, wp.QW, wp.PH,
                         wgrad_a_boxes(g.Cout), 1, 1))
    return rc;
  if (int rc = nhwc_map5(&mb, xt, g.C, cp, g.W, g.H, g.N, wp.QW, wp.PH, 1 << wp.cn_shift, g.sx,
                         g.sy))
    return rc;
  const WgradTaps tp{g.C, g.RS, g.kW, g.dx, g.dy, g.px, g.py};
  if (int rc = run_wgrad_any(ma, mb, g, tp, wp, partial, st)) return rc;
  if (g.C % 4 == 0 && (reinterpret_cast<uintptr_t>(partial) & 15) == 0 &&
      (g.RS != 1 || (reinterpret_cast<uintptr_t>(gw) & 15) == 0))
    wgrad_reduce_vec_kernel<<<grid_for((long long)g.RS * g.Cout * (g.C / 4), 256), 256, 0, st>>>(
        reinterpret_cast<const float4*>(partial), gw, g.Cout, g.C / 4, g.RS, wp.splits);
  else
    wgrad_reduce_kernel<<<grid_for((long long)g.RS * g.Cout * g.C, 256), 256, 0, st>>>(
        partial, gw, g.Cout, g.C, g.RS, wp.splits);
  FLB200_AFTER_LAUNCH("wgrad_reduce");
  return FLB200_OK;
}

// ------------------------------------------------------- row-window interface
bool window_conv_supported(const ConvGeo& g) {
  if (!(g.groups == 1 && g.C <= 4 && g.kW <= kWinPixels && g.dx == 1 && g.Cout >= 16 &&
        g.kH <= 8 && g.sx <= 2 && g.sy <= 2 && g.N <= 65535))
    return false;
  // x is gathered from fl's order into the padded 4-channel copy; y / grad_y may be
  // channels-last (then read and written in place)
  if (g.x_cl || (g.y_cl && g.Cout % 4 != 0)) return false;
  // Rows of the window view overlap (pixel stride < window extent).  Encoding a map reads no
  // memory, so ask the driver up front, with a placeholder base, whether it takes this view;
  // if not, the caller uses the gather route.
  const WindowGeo wg = window_geo(g);
  const Patch pt = pick_patch(g.Wo, g.Ho, g.N);
  int qw, ph;
  pick_k_patch(g.Wo, g.Ho, &qw, &ph);
  CUtensorMap m;
  const float* placeholder = reinterpret_cast<const float*>(uintptr_t(1) << 30);
  return window_map(&m, placeholder, wg, g.N, pt.QW, pt.PH, pt.NB, g.sx, g.sy) == 0 &&
         window_rows_map(&m, placeholder, wg, g.N, qw, ph, 8, g.sx, g.sy, g.kH, g.dy) == 0;
}

size_t window_conv_workspace_bytes(const ConvGeo& g, int which) {
  const WindowGeo wg = window_geo(g);
  const size_t xtp = up256((size_t)g.N * wg.Hp * wg.Wp * 16);
  if (which == 0) return xtp + up256((size_t)g.kH * g.Cout * 32 * 4);
  const int cop = up4(g.Cout);
  // the backward-filter GEMM has 32 columns per tap and kH taps
  return xtp + (g.y_cl ? 0 : up256((size_t)g.N * g.HoWo * cop * 4)) +
         up256(plan_wgrad(g, 32 * g.kH, 1).partial_bytes);
}

size_t window_conv_cache_bytes(const ConvGeo& g, int which) {
  if (which != 0) return 0;  // this route has no backward-data pass to share grad_y with
  const WindowGeo wg = window_geo(g);
  return up256((size_t)g.N * wg.Hp * wg.Wp * 16);
}

int window_conv_forward(const ConvGeo& g, const float* x, const float* w, const float* bias,
                        float* y, void* ws, size_t ws_bytes, cudaStream_t st,
                        flb200_conv2d_cache* cache, const ConvStats* stats) {
  (void)ws_bytes;
  const WindowGeo wg = window_geo(g);
  char* base = static_cast<char*>(ws);
  const ClSlot xs =
      cl_slot(cache, 0, (size_t)g.N * wg.Hp * wg.Wp * 16, reinterpret_cast<float*>(base));
  float* xtp = xs.buf;
  float* wr = reinterpret_cast<float*>(base + up256((size_t)g.N * wg.Hp * wg.Wp * 16));
  PatchArgs a{};
  a.patch = pick_patch(g.Wo, g.Ho, g.N);
  CUtensorMap ma, mb;
  // the overlapping view is the one thing here the driver may refuse: check before launching
  if (int rc = window_map(&ma, xtp, wg, g.N, a.patch.QW, a.patch.PH, a.patch.NB, g.sx, g.sy))
    return rc;
  const int bn = tc::pick_bn(g.Cout);
  if (int rc = filter_map(&mb, wr, 32, 32, g.Cout, g.kH, filter_box_rows(bn))) return rc;
  if (!xs.valid) {
    const long long total = (long long)g.N * wg.Hp * wg.Wp;
    nchw_to_nhwc4_pad_kernel<<<grid_for(total, 256), 256, 0, st>>>(
        x, reinterpret_cast<float4*>(xtp), g.C, g.H, g.W, wg.Hp, wg.Wp, g.py, g.px, total);
    FLB200_AFTER_LAUNCH("nchw_to_nhwc4_pad");
    if (xs.flag) *xs.flag = 1;
  }
  pack_filter_rows_kernel<<<grid_for(g.kH * g.Cout * 32, 256), 256, 0, st>>>(w, wr, g.Cout, g.C,
                                                                            g.kH, g.kW);
  FLB200_AFTER_LAUNCH("pack_filter_rows");
  a.pix_w = g.Wo; a.pix_h = g.Ho; a.images = g.N; a.n_out = g.Cout;
  a.cchunks = 1;
  a.a_w_mul = g.sx; a.a_h_mul = g.sy;
  a.ncls = 1;  // tap r: row offset r*dy, filter row r
  a.cls[0] = tc::PatchClass{tc::TapGrid{g.kH, 1, 0, g.dy, 0, 0, 0, 1, 0, 0, 1}, g.kH, 0, 0};
  a.out = y; a.bias = bias;
  a.out_H = g.Ho; a.out_W = g.Wo; a.out_C = g.Cout;
  a.oh_mul = 1; a.ow_mul = 1;
  a.out_cl = g.y_cl;
  a.stats = stats && g.y_cl ? stats->matrix : nullptr;
  return run_patch_any(bn, ma, mb, a, st);
}

int window_conv_backward_filter(const ConvGeo& g, const float* gy, const float* x, float* gw,
                                void* ws, size_t ws_bytes, cudaStream_t st,
    flb200_conv2d_cache* cache) {
  (void)ws_bytes;
  const WindowGeo wg = window_geo(g);
  const int cop = up4(g.Cout);
  const WgradPlan wp = plan_wgrad(g, 32 * g.kH, 1);
  char* base = static_cast<char*>(ws);
  const ClSlot xs =
      cl_slot(cache, 0, (size_t)g.N * wg.Hp * wg.Wp * 16, reinterpret_cast<float*>(base));
  float* xtp = xs.buf;
  size_t off = up256((size_t)g.N * wg.Hp * wg.Wp * 16);
  const float* gyt = gy;
  float* gy_copy = nullptr;
  if (!g.y_cl) {
    gy_copy = reinterpret_cast<float*>(base + off);
    gyt = gy_copy;
    off += up256((size_t)g.N * g.HoWo * cop * 4);
  }
  float* partial = reinterpret_cast<float*>(base + off);
  CUtensorMap ma, mb;
  if (int rc = window_rows_map(&mb, xtp, wg, g.N, wp.QW, wp.PH, 1 << wp.cn_shift, g.sx, g.sy, g.kH,
                               g.dy)) return rc;
  if (int rc = nhwc_map5(&ma, gyt, g.Cout, cop, g.Wo, g.Ho, g.N, wp.QW, wp.PH,
                         wgrad_a_boxes(g.Cout), 1, 1))
    return rc;
  if (!xs.valid) {
    const long long total = (long long)g.N * wg.Hp * wg.Wp;
    nchw_to_nhwc4_pad_kernel<<<grid_for(total, 256), 256, 0, st>>>(
        x, reinterpret_cast<float4*>(xtp), g.C, g.H, g.W, wg.Hp, wg.Wp, g.py, g.px, total);
    FLB200_AFTER_LAUNCH("nchw_to_nhwc4_pad");
    if (xs.flag) *xs.flag = 1;
  }
  if (gy_copy)
    if (int rc = to_nhwc(gy, gy_copy, g.N, g.Cout, cop, g.HoWo, st)) return rc;
  // One GEMM: M = Cout, N = kH blocks of 32 window floats, K = pixels.  The filter rows are
  // the channel groups of the view, so the launch has a single tap at offset zero.
  const WgradTaps tp{32 * g.kH, 1, 1, 1, 1, 0, 0};
  if (int rc = run_wgrad_any(ma, mb, g, tp, wp, partial, st)) return rc;
  window_wgrad_reduce_kernel<<<grid_for((long long)g.Cout * g.C * g.RS, 256), 256, 0, st>>>(
      partial, gw, g.Cout, g.C, g.kH, g.kW, wp.splits);
  FLB200_AFTER_LAUNCH("window_wgrad_reduce");
  return FLB200_OK;
}

}  // namespace flb200
