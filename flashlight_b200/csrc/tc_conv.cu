// TF32 tensor-core convolution passes built on the tcgen05 contraction (tc_gemm.cuh), all over
// fl's native NCHW buffers (no layout change at the boundary).  Four routes, tried in order:
//
//  * direct 1x1 (stride 1, no padding, H*W a multiple of 4): the image planes ARE the
//    GEMM operands.  TMA reads x[n] / dy[n] as [channels][pixels] matrices (pixel index
//    contiguous = MN-major for forward and backward-data, K-major for backward-filter)
//    straight from the tensors; nothing is copied.
//      forward        y[n](hw, co)  = sum_ci x[n](ci, hw) * w(co, ci)
//      backward data  dx[n](hw, ci) = sum_co dy[n](co, hw) * w(co, ci)
//      backward filt  dw(co, ci)    = sum_{n, hw} dy[n](co, hw) * x[n](ci, hw)   (split-K)
//
//  * channels-last patch route (tc_conv_patch.cu): >= 16 channels in and out, <= 64 taps,
//    stride <= 2.  One NHWC copy of the activation operand, then an implicit GEMM whose tap
//    shifts are TMA coordinates.
//
//  * row-window route (tc_conv_patch.cu): <= 4 input channels (forward, backward-filter).
//
//  * gather route (this file; any filter / stride / padding / dilation, groups == 1): a
//    gather kernel lays the im2col matrix col[k][n][hw_pad] out in scratch (pixel axis
//    padded per image to a multiple of 4, padding = 0) and the passes become plain GEMMs on
//    it.  Backward data gathers dy the same way with the transposed taps; backward filter
//    also copies dy to [co][n][hw_pad].
//
// Algorithmic flops 2*M*N*K of the implicit GEMM; copies and gathers are overhead.
#include "tc_conv.cuh"

#include "tc_gemm.cuh"

namespace flb200 {
namespace {

inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }
inline long long up4(long long v) { return (v + 3) / 4 * 4; }

// ------------------------------------------------------------ gather kernels
// col[k][img][hwp] for k = (ci, r, s): x[img][ci][p*sy-py+r*dy][q*sx-px+s*dx], 0 outside the
// image and on the padding pixels hw >= HoWo.
__global__ void __launch_bounds__(256)
im2col_kernel(const float* __restrict__ x, float* __restrict__ col, ConvGeo g, int hwp,
              long long ld) {
  const int k = blockIdx.y;
  const int ci = k / g.RS, rs = k - ci * g.RS;
  const int r = rs / g.kW, s = rs - r * g.kW;
  const int dh = r * g.dy - g.py, dw = s * g.dx - g.px;
  float* dst = col + (long long)k * ld;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < ld;
       t += (long long)gridDim.x * blockDim.x) {
    const int img = (int)(t / hwp), hw = (int)(t - (long long)img * hwp);
    float v = 0.f;
    if (hw < g.HoWo) {
      const int p = hw / g.Wo, q = hw - p * g.Wo;
      const int h = p * g.sy + dh, w = q * g.sx + dw;
      if (h >= 0 && h < g.H && w >= 0 && w < g.W)
        v = x[((long long)img * g.C + ci) * g.HW + h * g.W + w];
    }
    dst[t] = v;
  }
}

// col2[k][img][hwp_in] for k = (co, r, s): dy[img][co][p][q] with p*sy = h+py-r*dy and
// q*sx = w+px-s*dx when those divide exactly and fall inside the output, else 0.
__global__ void __launch_bounds__(256)
dgrad_gather_kernel(const float* __restrict__ gy, float* __restrict__ col, ConvGeo g, int hwp,
                    long long ld) {
  const int k = blockIdx.y;
  const int co = k / g.RS, rs = k - co * g.RS;
  const int r = rs / g.kW, s = rs - r * g.kW;
  float* dst = col + (long long)k * ld;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < ld;
       t += (long long)gridDim.x * blockDim.x) {
    const int img = (int)(t / hwp), hw = (int)(t - (long long)img * hwp);
    float v = 0.f;
    if (hw < g.HW) {
      const int h = hw / g.W, w = hw - h * g.W;
      const int th = h + g.py - r * g.dy, tw = w + g.px - s * g.dx;
      if (th >= 0 && tw >= 0) {
        const int p = th / g.sy, q = tw / g.sx;
        if (p * g.sy == th && q * g.sx == tw && p < g.Ho && q < g.Wo)
          v = gy[((long long)img * g.Cout + co) * g.HoWo + p * g.Wo + q];
      }
    }
    dst[t] = v;
  }
}

// dst[c][img][hwp] = src[img][c][hw] (0 on padding pixels): dy as a [channels][pixels] matrix.
__global__ void __launch_bounds__(256)
planes_to_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int channels,
                      int hw_count, int hwp, long long ld) {
  const int c = blockIdx.y;
  float* out = dst + (long long)c * ld;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < ld;
       t += (long long)gridDim.x * blockDim.x) {
    const int img = (int)(t / hwp), hw = (int)(t - (long long)img * hwp);
    out[t] = hw < hw_count ? src[((long long)img * channels + c) * hw_count + hw] : 0.f;
  }
}

// wp[co][kp] = w[co][k] for k < kc: same values, row stride padded to a multiple of 4.
__global__ void pad_rows_kernel(const float* __restrict__ w, float* __restrict__ wp, int rows,
                                int kc, int kp) {
  const long long total = (long long)rows * kp;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(t / kp), k = (int)(t - (long long)row * kp);
    wp[t] = k < kc ? w[(long long)row * kc + k] : 0.f;
  }
}

// wt[ci][(co, rs)] = w[co][ci][rs], row stride k2p.
__global__ void transpose_filter_kernel(const float* __restrict__ w, float* __restrict__ wt,
                                        ConvGeo g, int k2p) {
  const long long total = (long long)g.C * k2p;
  const int k2 = g.Cout * g.RS;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const int ci = (int)(t / k2p), k = (int)(t - (long long)ci * k2p);
    float v = 0.f;
    if (k < k2) {
      const int co = k / g.RS, rs = k - co * g.RS;
      v = w[((long long)co * g.C + ci) * g.RS + rs];
    }
    wt[t] = v;
  }
}

// ------------------------------------------------------------- map helpers
int map2d(CUtensorMap* m, const float* base, long long inner, long long outer, long long ld,
          int box_outer, bool mn_major) {
  const uint64_t dims[2] = {(uint64_t)inner, (uint64_t)outer};
  const uint64_t strides[1] = {(uint64_t)ld * 4};
  const uint32_t box[2] = {32, (uint32_t)box_outer};
  return tc::make_tensor_map(m, base, 2, dims, strides, box, mn_major);
}
int map3d(CUtensorMap* m, const float* base, long long inner, long long mid, long long outer,
          long long stride1, long long stride2, int box_mid, bool mn_major) {
  const uint64_t dims[3] = {(uint64_t)inner, (uint64_t)mid, (uint64_t)outer};
  const uint64_t strides[2] = {(uint64_t)stride1 * 4, (uint64_t)stride2 * 4};
  const uint32_t box[3] = {32, (uint32_t)box_mid, 1};
  return tc::make_tensor_map(m, base, 3, dims, strides, box, mn_major);
}
tc::OperandPlan plan_k_major(int rank) {  // dims [K, rows, ...]
  tc::OperandPlan p{};
  p.rank = rank; p.mn_major = 0; p.mn_dim = 1; p.k_dim = 0; p.k2_dim = -1; p.z_dim = -1;
  return p;
}
tc::OperandPlan plan_mn_major(int rank) {  // dims [rows, K, ...]
  tc::OperandPlan p{};
  p.rank = rank; p.mn_major = 1; p.mn_dim = 0; p.k_dim = 1; p.k2_dim = -1; p.z_dim = -1;
  return p;
}

bool direct_1x1(const ConvGeo& g) {
  return !g.x_cl && !g.y_cl && g.kW == 1 && g.kH == 1 && g.sx == 1 && g.sy == 1 && g.px == 0 &&
         g.py == 0 && g.groups == 1 && g.HW % 4 == 0 && g.C % 4 == 0;
}
// The same layer over channels-last tensors: x is the [pixels][C] matrix and y the
// [pixels][Cout] matrix of a plain GEMM, whatever the plane size.
//   forward        y(p, co)  = sum_ci x(p, ci) * w(co, ci)       both operands K-major
//   backward data  dx(p, ci) = sum_co dy(p, co) * wT(ci, co)     wT: filter transposed in scratch
//   backward filt  the channels-last patch route over the batch as one row of pixels
bool cl_1x1(const ConvGeo& g) {
  return g.x_cl && g.y_cl && g.kW == 1 && g.kH == 1 && g.sx == 1 && g.sy == 1 && g.px == 0 &&
         g.py == 0 && g.groups == 1 && g.C % 4 == 0 && g.Cout % 4 == 0 &&
         (long long)g.N * g.HW < 0x7fffffffLL;
}

// wt[ci][co] = w[co][ci] (1 x 1 filters), row stride Cout.
__global__ void transpose_1x1_filter_kernel(const float* __restrict__ w, float* __restrict__ wt,
                                            int Cout, int C) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int ci0 = blockIdx.x * 32, co0 = blockIdx.y * 32;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int co = co0 + ty + 8 * i, ci = ci0 + tx;
    tile[ty + 8 * i][tx] = (co < Cout && ci < C) ? w[(long long)co * C + ci] : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int ci = ci0 + ty + 8 * i, co = co0 + tx;
    if (ci < C && co < Cout) wt[(long long)ci * Cout + co] = tile[tx][ty + 8 * i];
  }
}

struct GeneralSizes {
  int hwp_out, hwp_in;
  long long ld_out, ld_in;  // padded pixel counts N*hwp
  int kc, kp, k2, k2p;
};
GeneralSizes general_sizes(const ConvGeo& g) {
  GeneralSizes s;
  s.hwp_out = (int)up4(g.HoWo);
  s.hwp_in = (int)up4(g.HW);
  s.ld_out = (long long)g.N * s.hwp_out;
  s.ld_in = (long long)g.N * s.hwp_in;
  s.kc = g.C * g.RS;
  s.kp = (int)up4(s.kc);
  s.k2 = g.Cout * g.RS;
  s.k2p = (int)up4(s.k2);
  return s;
}

dim3 gather_grid(long long ld, int rows) {
  long long bx = (ld + 255) / 256;
  if (bx > 4096) bx = 4096;
  return dim3((unsigned)bx, (unsigned)rows);
}

}  // namespace

// -------------------------------------------------------------- interface
size_t tc_conv_workspace_bytes(const ConvGeo& g, int which) {
  if (g.groups != 1) return 0;
  if (cl_1x1(g)) {
    if (which == 0) return 0;
    if (which == 1) return up256((size_t)g.C * g.Cout * 4);
    return patch_conv_supported(g) ? patch_conv_workspace_bytes(g, 2) : 0;
  }
  if (direct_1x1(g)) {
    if (which != 2) return 0;
    const long long k_iters = (long long)g.N * ((g.HW + tc::kBK - 1) / tc::kBK);
    return tc::plan_launch(g.Cout, g.C, k_iters, 1).workspace_bytes;
  }
  if (patch_conv_supported(g)) return patch_conv_workspace_bytes(g, which);
  if (which != 1 && window_conv_supported(g)) return window_conv_workspace_bytes(g, which);
  const GeneralSizes s = general_sizes(g);
  if (which == 0) {
    return up256((size_t)s.kc * s.ld_out * 4) + up256((size_t)g.Cout * s.kp * 4) +
           tc::plan_launch(s.ld_out, g.Cout, (s.kc + tc::kBK - 1) / tc::kBK, 1).workspace_bytes;
  }
  if (which == 1) {
    return up256((size_t)s.k2 * s.ld_in * 4) + up256((size_t)g.C * s.k2p * 4) +
           tc::plan_launch(s.ld_in, g.C, (s.k2 + tc::kBK - 1) / tc::kBK, 1).workspace_bytes;
  }
  return up256((size_t)s.kc * s.ld_out * 4) + up256((size_t)g.Cout * s.ld_out * 4) +
         tc::plan_launch(g.Cout, s.kc, (s.ld_out + tc::kBK - 1) / tc::kBK, 1).workspace_bytes;
}

size_t tc_conv_cache_bytes(const ConvGeo& g, int which) {
  if (g.groups != 1 || !flb200_has_tensor_core_path() || direct_1x1(g)) return 0;
  if (patch_conv_supported(g)) return patch_conv_cache_bytes(g, which);
  if (window_conv_supported(g)) return window_conv_cache_bytes(g, which);
  return 0;
}

bool tc_conv_supported(const ConvGeo& g, int which, size_t workspace_bytes) {
  if (!flb200_has_tensor_core_path()) return false;
  if (g.groups != 1) return false;
  if (cl_1x1(g) && which != 2) return workspace_bytes >= tc_conv_workspace_bytes(g, which);
  // the other channels-last shapes run on the patch / row-window routes or not at all
  if ((g.x_cl || g.y_cl) && !patch_conv_supported(g) && !(which != 1 && window_conv_supported(g)))
    return false;
  if (direct_1x1(g)) return true;  // scratch only speeds up backward-filter (split-K)
  if (patch_conv_supported(g)) return workspace_bytes >= patch_conv_workspace_bytes(g, which);
  if (which != 1 && window_conv_supported(g))
    return workspace_bytes >= window_conv_workspace_bytes(g, which);
  const GeneralSizes s = general_sizes(g);
  if (s.kc > 65535 || s.k2 > 65535) return false;               // gather grids index k in y
  if (s.ld_out >= 0x7fffffffLL || s.ld_in >= 0x7fffffffLL) return false;
  return workspace_bytes >= tc_conv_workspace_bytes(g, which);
}

long long tc_conv_stats_groups(const ConvGeo& g) {
  if (!g.y_cl || g.Cout % 32 != 0) return 0;
  if (cl_1x1(g)) return 4 * (((long long)g.N * g.HW + tc::kBM - 1) / tc::kBM);
  if (direct_1x1(g)) return 0;
  if (patch_conv_supported(g) || window_conv_supported(g)) return patch_conv_stats_groups(g);
  return 0;
}

int tc_conv_forward(const ConvGeo& g, const float* x, const float* w, const float* bias, float* y,
                    void* ws, size_t ws_bytes, cudaStream_t st, flb200_conv2d_cache* cache,
                    const ConvStats* stats) {
  CUtensorMap ma, mb;
  tc::EpiloguePlan ep{};
  ep.out = y;
  ep.alpha = 1.f;
  ep.bias_n = bias;
  const int bn = tc::pick_bn(g.Cout);
  if (cl_1x1(g)) {
    const long long M = (long long)g.N * g.HW, k_iters = (g.C + tc::kBK - 1) / tc::kBK;
    if (int rc = map2d(&ma, x, g.C, M, g.C, tc::kBM, false)) return rc;
    if (int rc = map2d(&mb, w, g.C, g.Cout, g.C, tc::b_box_rows(M, g.Cout, k_iters, false, false),
                       false))
      return rc;
    ep.m_stride = g.Cout;
    ep.n_stride = 1;
    ep.stats = stats ? stats->matrix : nullptr;
    return tc::run(ma, mb, plan_k_major(2), plan_k_major(2), ep, M, g.Cout, k_iters, 1, nullptr, 0,
                   st);
  }
  if (stats && tc_conv_stats_groups(g) == 0)
    return fail(FLB200_UNSUPPORTED, "conv2d_forward: this route takes no output statistics");
  if (direct_1x1(g)) {
    if (int rc = map3d(&ma, x, g.HW, g.C, g.N, g.HW, (long long)g.C * g.HW, 32, true)) return rc;
    // a K-major B tile is one box of all the tile's rows, or of half of them on CTA pairs
    const long long k_iters = (g.C + tc::kBK - 1) / tc::kBK;
    if (int rc = map2d(&mb, w, g.C, g.Cout, g.C, tc::b_box_rows(g.HW, g.Cout, k_iters, true, false), false)) return rc;
    tc::OperandPlan pa = plan_mn_major(3), pb = plan_k_major(2);
    pa.z_dim = 2;
    ep.m_stride = 1;
    ep.n_stride = g.HW;
    ep.z_stride = (long long)g.Cout * g.HW;
    return tc::run(ma, mb, pa, pb, ep, g.HW, g.Cout, (g.C + tc::kBK - 1) / tc::kBK, g.N, nullptr, 0,
                   st);
  }
  if (patch_conv_supported(g))
    return patch_conv_forward(g, x, w, bias, y, ws, ws_bytes, st, cache, stats);
  if (window_conv_supported(g))
    return window_conv_forward(g, x, w, bias, y, ws, ws_bytes, st, cache, stats);
  const GeneralSizes s = general_sizes(g);
  char* base = static_cast<char*>(ws);
  float* col = reinterpret_cast<float*>(base);
  size_t off = up256((size_t)s.kc * s.ld_out * 4);
  float* wp = reinterpret_cast<float*>(base + off);
  off += up256((size_t)g.Cout * s.kp * 4);
  im2col_kernel<<<gather_grid(s.ld_out, s.kc), 256, 0, st>>>(x, col, g, s.hwp_out, s.ld_out);
  FLB200_AFTER_LAUNCH("im2col");
  const float* wsrc = w;
  if (s.kp != s.kc) {
    pad_rows_kernel<<<grid_for((long long)g.Cout * s.kp, 256), 256, 0, st>>>(w, wp, g.Cout, s.kc,
                                                                            s.kp);
    FLB200_AFTER_LAUNCH("pad_filter_rows");
    wsrc = wp;
  }
  if (int rc = map2d(&ma, col, s.ld_out, s.kc, s.ld_out, 32, true)) return rc;
  if (int rc = map2d(&mb, wsrc, s.kc, g.Cout, s.kp, tc::b_box_rows(s.ld_out, g.Cout, (s.kc + tc::kBK - 1) / tc::kBK, true, false), false)) return rc;
  ep.m_div = s.hwp_out;
  ep.m_valid = g.HoWo;
  ep.m_outer = (long long)g.Cout * g.HoWo;
  ep.m_stride = 1;
  ep.n_stride = g.HoWo;
  return tc::run(ma, mb, plan_mn_major(2), plan_k_major(2), ep, s.ld_out, g.Cout,
                 (s.kc + tc::kBK - 1) / tc::kBK, 1, base + off, ws_bytes - off, st);
}

int tc_conv_backward_data(const ConvGeo& g, const float* gy, const float* w, float* gx, void* ws,
                          size_t ws_bytes, cudaStream_t st,
    flb200_conv2d_cache* cache) {
  CUtensorMap ma, mb;
  tc::EpiloguePlan ep{};
  ep.out = gx;
  ep.alpha = 1.f;
  const int bn = tc::pick_bn(g.C);
  if (cl_1x1(g)) {
    const long long M = (long long)g.N * g.HW, k_iters = (g.Cout + tc::kBK - 1) / tc::kBK;
    float* wt = static_cast<float*>(ws);
    dim3 tgrid((unsigned)((g.C + 31) / 32), (unsigned)((g.Cout + 31) / 32));
    transpose_1x1_filter_kernel<<<tgrid, 256, 0, st>>>(w, wt, g.Cout, g.C);
    FLB200_AFTER_LAUNCH("transpose_1x1_filter");
    if (int rc = map2d(&ma, gy, g.Cout, M, g.Cout, tc::kBM, false)) return rc;
    if (int rc = map2d(&mb, wt, g.Cout, g.C, g.Cout, tc::b_box_rows(M, g.C, k_iters, false, false),
                       false))
      return rc;
    ep.m_stride = g.C;
    ep.n_stride = 1;
    return tc::run(ma, mb, plan_k_major(2), plan_k_major(2), ep, M, g.C, k_iters, 1, nullptr, 0, st);
  }
  if (direct_1x1(g)) {
    if (int rc = map3d(&ma, gy, g.HW, g.Cout, g.N, g.HW, (long long)g.Cout * g.HW, 32, true))
      return rc;
    // B(k = co, n = ci) = w[co][ci]: the n index is contiguous.  With a multiple of 32 input
    // channels the map splits ci into (32, group) and the whole B tile is one copy.
    tc::OperandPlan pa = plan_mn_major(3), pb = plan_mn_major(2);
    if (g.C % 32 == 0) {
      const uint64_t dims[3] = {32, (uint64_t)g.Cout, (uint64_t)(g.C / 32)};
      const uint64_t strides[2] = {(uint64_t)g.C * 4, 128};
      const uint32_t box[3] = {32, 32, (uint32_t)(bn / 32)};
      if (int rc = tc::make_tensor_map(&mb, w, 3, dims, strides, box, tc::kMapMnMajor)) return rc;
      pb.rank = 3; pb.mn_dim = 2; pb.k_dim = 1; pb.mn_grouped = 1;
    } else if (int rc = map2d(&mb, w, g.C, g.Cout, g.C, 32, true)) {
      return rc;
    }
    pa.z_dim = 2;
    ep.m_stride = 1;
    ep.n_stride = g.HW;
    ep.z_stride = (long long)g.C * g.HW;
    return tc::run(ma, mb, pa, pb, ep, g.HW, g.C, (g.Cout + tc::kBK - 1) / tc::kBK, g.N, nullptr, 0,
                   st);
  }
  if (patch_conv_supported(g)) return patch_conv_backward_data(g, gy, w, gx, ws, ws_bytes, st, cache);
  const GeneralSizes s = general_sizes(g);
  char* base = static_cast<char*>(ws);
  float* col = reinterpret_cast<float*>(base);
  size_t off = up256((size_t)s.k2 * s.ld_in * 4);
  float* wt = reinterpret_cast<float*>(base + off);
  off += up256((size_t)g.C * s.k2p * 4);
  dgrad_gather_kernel<<<gather_grid(s.ld_in, s.k2), 256, 0, st>>>(gy, col, g, s.hwp_in, s.ld_in);
  FLB200_AFTER_LAUNCH("dgrad_gather");
  transpose_filter_kernel<<<grid_for((long long)g.C * s.k2p, 256), 256, 0, st>>>(w, wt, g, s.k2p);
  FLB200_AFTER_LAUNCH("transpose_filter");
  if (int rc = map2d(&ma, col, s.ld_in, s.k2, s.ld_in, 32, true)) return rc;
  if (int rc = map2d(&mb, wt, s.k2, g.C, s.k2p, tc::b_box_rows(s.ld_in, g.C, (s.k2 + tc::kBK - 1) / tc::kBK, true, false), false)) return rc;
  ep.m_div = s.hwp_in;
  ep.m_valid = g.HW;
  ep.m_outer = (long long)g.C * g.HW;
  ep.m_stride = 1;
  ep.n_stride = g.HW;
  return tc::run(ma, mb, plan_mn_major(2), plan_k_major(2), ep, s.ld_in, g.C,
                 (s.k2 + tc::kBK - 1) / tc::kBK, 1, base + off, ws_bytes - off, st);
}

int tc_conv_backward_filter(const ConvGeo& g, const float* gy, const float* x, float* gw, void* ws,
                            size_t ws_bytes, cudaStream_t st,
    flb200_conv2d_cache* cache) {
  CUtensorMap ma, mb;
  tc::EpiloguePlan ep{};
  ep.out = gw;
  ep.alpha = 1.f;
  ep.n_stride = 1;
  if (direct_1x1(g)) {
    const int bn = tc::pick_bn(g.C);
    const int k_inner = (g.HW + tc::kBK - 1) / tc::kBK;
    if (int rc = map3d(&ma, gy, g.HW, g.Cout, g.N, g.HW, (long long)g.Cout * g.HW, tc::kBM, false))
      return rc;
    if (int rc = map3d(&mb, x, g.HW, g.C, g.N, g.HW, (long long)g.C * g.HW, tc::b_box_rows(g.Cout, g.C, (long long)g.N * k_inner, false, false), false)) return rc;
    tc::OperandPlan pa = plan_k_major(3), pb = plan_k_major(3);
    pa.k2_dim = pb.k2_dim = 2;
    pa.k2_scale = pb.k2_scale = 1;
    pa.k_inner = pb.k_inner = k_inner;
    ep.m_stride = g.C;
    return tc::run(ma, mb, pa, pb, ep, g.Cout, g.C, (long long)g.N * k_inner, 1, ws, ws_bytes, st);
  }
  if (patch_conv_supported(g)) return patch_conv_backward_filter(g, gy, x, gw, ws, ws_bytes, st, cache);
  if (window_conv_supported(g))
    return window_conv_backward_filter(g, gy, x, gw, ws, ws_bytes, st, cache);
  const GeneralSizes s = general_sizes(g);
  const int bn = tc::pick_bn(s.kc);
  char* base = static_cast<char*>(ws);
  float* col = reinterpret_cast<float*>(base);
  size_t off = up256((size_t)s.kc * s.ld_out * 4);
  float* dyt = reinterpret_cast<float*>(base + off);
  off += up256((size_t)g.Cout * s.ld_out * 4);
  im2col_kernel<<<gather_grid(s.ld_out, s.kc), 256, 0, st>>>(x, col, g, s.hwp_out, s.ld_out);
  FLB200_AFTER_LAUNCH("im2col");
  planes_to_rows_kernel<<<gather_grid(s.ld_out, g.Cout), 256, 0, st>>>(gy, dyt, g.Cout, g.HoWo,
                                                                      s.hwp_out, s.ld_out);
  FLB200_AFTER_LAUNCH("planes_to_rows");
  if (int rc = map2d(&ma, dyt, s.ld_out, g.Cout, s.ld_out, tc::kBM, false)) return rc;
  if (int rc = map2d(&mb, col, s.ld_out, s.kc, s.ld_out, tc::b_box_rows(g.Cout, s.kc, (s.ld_out + tc::kBK - 1) / tc::kBK, false, false), false)) return rc;
  ep.m_stride = s.kc;
  return tc::run(ma, mb, plan_k_major(2), plan_k_major(2), ep, g.Cout, s.kc,
                 (s.ld_out + tc::kBK - 1) / tc::kBK, 1, base + off, ws_bytes - off, st);
}

}  // namespace flb200
