// conv2d forward, backward-data and backward-filter(+bias) as implicit GEMMs
// over fl's native layout: x [N][C][H][W], w [Cout][C/groups][kH][kW],
// y [N][Cout][Ho][Wo] (row-major views of fl's column-major tensors; the byte
// buffers are identical, cf. flashlight/fl/autograd/tensor/backend/onednn/Conv2D.cpp:171-178).
// Stands behind fl::AutogradExtension::conv2d / ::conv2dBackwardData /
// ::conv2dBackwardFilterBias (flashlight/fl/autograd/tensor/AutogradExtension.h:58-69,
// 110-138).  Cross-correlation, stride (sx,sy), symmetric zero padding (px,py),
// dilation (dx,dy), groups.
//
// GEMM views (per group):
//   forward   M = Cout/g, N = batch*Ho*Wo, K = (C/g)*kH*kW
//   bwd data  M = C/g,    N = batch*H*W,   K = (Cout/g)*kH*kW
//   bwd filt  M = Cout/g, N = (C/g)*kH*kW, K = batch*Ho*Wo   (split-K)
// STRICT mode: the fp32-FMA kernel of simt_gemm.cuh with im2col loaders below.
// TF32 mode: shapes covered by the tensor-core kernels go to tc_conv, the rest
// fall through to the fp32 kernel.
#include "simt_gemm.cuh"
#include "tc_conv.cuh"
#include "tc_gemm.cuh"

namespace flb200 {

int make_conv_geo(const char* name, const flb200_conv2d_desc* d, ConvGeo* g) {
  FLB200_REQUIRE(d, "%s: null descriptor", name);
  FLB200_REQUIRE(d->W >= 1 && d->H >= 1 && d->C >= 1 && d->N >= 1, "%s: empty input", name);
  FLB200_REQUIRE(d->kW >= 1 && d->kH >= 1 && d->Cout >= 1, "%s: empty filter", name);
  FLB200_REQUIRE(d->sx >= 1 && d->sy >= 1 && d->dx >= 1 && d->dy >= 1 && d->px >= 0 && d->py >= 0,
                 "%s: bad stride/dilation/padding", name);
  FLB200_REQUIRE(d->groups >= 1 && d->C % d->groups == 0 && d->Cout % d->groups == 0,
                 "%s: channels (%d in, %d out) not divisible by groups (%d)", name, d->C, d->Cout,
                 d->groups);
  FLB200_REQUIRE(d->dtype == FLB200_F32 || d->dtype == FLB200_F16 || d->dtype == FLB200_BF16,
                 "%s: unknown dtype %d", name, d->dtype);
  FLB200_REQUIRE(d->math_mode >= FLB200_MATH_STRICT_F32 && d->math_mode <= FLB200_MATH_F32X3,
                 "%s: unknown math mode %d", name, d->math_mode);
  const int ekw = 1 + (d->kW - 1) * d->dx, ekh = 1 + (d->kH - 1) * d->dy;
  FLB200_REQUIRE(d->W + 2 * d->px >= ekw && d->H + 2 * d->py >= ekh,
                 "%s: filter larger than padded input", name);
  g->W = d->W; g->H = d->H; g->C = d->C; g->N = d->N;
  g->kW = d->kW; g->kH = d->kH; g->Cout = d->Cout;
  g->sx = d->sx; g->sy = d->sy; g->px = d->px; g->py = d->py; g->dx = d->dx; g->dy = d->dy;
  g->groups = d->groups;
  g->Wo = 1 + (d->W + 2 * d->px - ekw) / d->sx;
  g->Ho = 1 + (d->H + 2 * d->py - ekh) / d->sy;
  g->Cg = d->C / d->groups;
  g->Coutg = d->Cout / d->groups;
  g->HW = d->H * d->W;
  g->HoWo = g->Ho * g->Wo;
  g->RS = d->kH * d->kW;
  FLB200_REQUIRE(d->layout == FLB200_LAYOUT_NCHW || d->layout == FLB200_LAYOUT_NHWC ||
                     d->layout == FLB200_LAYOUT_NCHW_IN_NHWC_OUT,
                 "%s: unknown layout %d", name, d->layout);
  g->x_cl = d->layout == FLB200_LAYOUT_NHWC;
  g->y_cl = d->layout != FLB200_LAYOUT_NCHW;
  g->x_cs = g->x_cl ? 1 : g->HW;
  g->x_ps = g->x_cl ? d->C : 1;
  g->y_cs = g->y_cl ? 1 : g->HoWo;
  g->y_ps = g->y_cl ? d->Cout : 1;
  return FLB200_OK;
}

namespace {

// ------------------------------------------------------------- forward
// B(k=(ci,r,s), n=(img,p,q)) = x[img][g*Cg+ci][p*sy-py+r*dy][q*sx-px+s*dx]
struct FpropB {
  static constexpr bool kAlongK = false;
  const float* x;
  ConvGeo g;
  long long n_total;
  struct Row { long long base; int h0, w0; };
  struct Kk { int off, dh, dw; };
  __device__ Row row(int n, int z) const {
    if (n >= n_total) return Row{-1, 0, 0};
    const int img = n / g.HoWo, pq = n - img * g.HoWo;
    const int p = pq / g.Wo, q = pq - p * g.Wo;
    return Row{(long long)img * g.C * g.HW + (long long)z * g.Cg * g.x_cs, p * g.sy - g.py,
               q * g.sx - g.px};
  }
  __device__ Kk kk(long long k, int) const {
    const int ki = (int)k;
    const int ci = ki / g.RS, rs = ki - ci * g.RS;
    const int r = rs / g.kW, s = rs - r * g.kW;
    return Kk{ci * g.x_cs, r * g.dy, s * g.dx};
  }
  __device__ float load(const Row& r, const Kk& k) const {
    const int h = r.h0 + k.dh, w = r.w0 + k.dw;
    if (r.base < 0 || h < 0 || h >= g.H || w < 0 || w >= g.W) return 0.f;
    return x[r.base + k.off + (long long)(h * g.W + w) * g.x_ps];
  }
};

struct FpropEpilogue {
  float* y;
  const float* bias;
  ConvGeo g;
  struct Row { long long off; float b; };
  struct Col { long long off; };
  __device__ Row row(int m, int z) const {
    const int co = z * g.Coutg + m;
    return Row{(long long)co * g.y_cs, bias ? bias[co] : 0.f};
  }
  __device__ Col col(int n, int) const {
    const int img = n / g.HoWo, pq = n - img * g.HoWo;
    return Col{(long long)img * g.Cout * g.HoWo + (long long)pq * g.y_ps};
  }
  __device__ void store(const Row& r, const Col& c, float acc) const {
    y[r.off + c.off] = acc + r.b;
  }
};

// ------------------------------------------------------- backward data
// A(m=ci, k=(co,r,s)) = w[g*Coutg+co][ci][r][s]
struct DgradA {
  static constexpr bool kAlongK = true;
  const float* w;
  ConvGeo g;
  struct Row { long long off; };
  struct Kk { long long off; };
  __device__ Row row(int m, int z) const {
    if (m >= g.Cg) return Row{-1};
    return Row{(long long)m * g.RS + (long long)z * g.Coutg * g.Cg * g.RS};
  }
  __device__ Kk kk(long long k, int) const {
    const int ki = (int)k;
    const int co = ki / g.RS, rs = ki - co * g.RS;
    return Kk{(long long)co * g.Cg * g.RS + rs};
  }
  __device__ float load(const Row& r, const Kk& k) const {
    return r.off >= 0 ? w[r.off + k.off] : 0.f;
  }
};

// B(k=(co,r,s), n=(img,h,w)) = gy[img][g*Coutg+co][p][q] with p*sy = h+py-r*dy, q*sx = w+px-s*dx
struct DgradB {
  static constexpr bool kAlongK = false;
  const float* gy;
  ConvGeo g;
  long long n_total;
  struct Row { long long base; int hh, ww; };
  struct Kk { int off, dh, dw; };
  __device__ Row row(int n, int z) const {
    if (n >= n_total) return Row{-1, 0, 0};
    const int img = n / g.HW, hw = n - img * g.HW;
    const int h = hw / g.W, w = hw - h * g.W;
    return Row{(long long)img * g.Cout * g.HoWo + (long long)z * g.Coutg * g.y_cs, h + g.py,
               w + g.px};
  }
  __device__ Kk kk(long long k, int) const {
    const int ki = (int)k;
    const int co = ki / g.RS, rs = ki - co * g.RS;
    const int r = rs / g.kW, s = rs - r * g.kW;
    return Kk{co * g.y_cs, r * g.dy, s * g.dx};
  }
  __device__ float load(const Row& r, const Kk& k) const {
    const int th = r.hh - k.dh, tw = r.ww - k.dw;
    if (r.base < 0 || th < 0 || tw < 0) return 0.f;
    int p = th, q = tw;
    if (g.sy != 1) { p = th / g.sy; if (p * g.sy != th) return 0.f; }
    if (g.sx != 1) { q = tw / g.sx; if (q * g.sx != tw) return 0.f; }
    if (p >= g.Ho || q >= g.Wo) return 0.f;
    return gy[r.base + k.off + (long long)(p * g.Wo + q) * g.y_ps];
  }
};

struct DgradEpilogue {
  float* gx;
  ConvGeo g;
  struct Row { long long off; };
  struct Col { long long off; };
  __device__ Row row(int m, int z) const { return Row{((long long)z * g.Cg + m) * g.x_cs}; }
  __device__ Col col(int n, int) const {
    const int img = n / g.HW, hw = n - img * g.HW;
    return Col{(long long)img * g.C * g.HW + (long long)hw * g.x_ps};
  }
  __device__ void store(const Row& r, const Col& c, float acc) const { gx[r.off + c.off] = acc; }
};

// ----------------------------------------------------- backward filter
// A(m=co, k=(img,p,q)) = gy[img][g*Coutg+co][p][q]
struct WgradA {
  static constexpr bool kAlongK = true;
  const float* gy;
  ConvGeo g;
  struct Row { long long off; };
  struct Kk { long long off; };
  __device__ Row row(int m, int z) const {
    if (m >= g.Coutg) return Row{-1};
    return Row{((long long)z * g.Coutg + m) * g.y_cs};
  }
  __device__ Kk kk(long long k, int) const {
    const long long img = k / g.HoWo;
    const int pq = (int)(k - img * g.HoWo);
    return Kk{img * g.Cout * g.HoWo + (long long)pq * g.y_ps};
  }
  __device__ float load(const Row& r, const Kk& k) const {
    return r.off >= 0 ? gy[r.off + k.off] : 0.f;
  }
};

// B(k=(img,p,q), n=(ci,r,s)) = x[img][g*Cg+ci][p*sy-py+r*dy][q*sx-px+s*dx]
struct WgradB {
  static constexpr bool kAlongK = true;
  const float* x;
  ConvGeo g;
  int n_total;
  struct Row { long long off; int dh, dw; };
  struct Kk { long long base; int h0, w0; };
  __device__ Row row(int n, int z) const {
    if (n >= n_total) return Row{-1, 0, 0};
    const int ci = n / g.RS, rs = n - ci * g.RS;
    const int r = rs / g.kW, s = rs - r * g.kW;
    return Row{((long long)z * g.Cg + ci) * g.x_cs, r * g.dy - g.py, s * g.dx - g.px};
  }
  __device__ Kk kk(long long k, int) const {
    const long long img = k / g.HoWo;
    const int pq = (int)(k - img * g.HoWo);
    const int p = pq / g.Wo, q = pq - p * g.Wo;
    return Kk{img * g.C * g.HW, p * g.sy, q * g.sx};
  }
  __device__ float load(const Row& r, const Kk& k) const {
    const int h = k.h0 + r.dh, w = k.w0 + r.dw;
    if (r.off < 0 || h < 0 || h >= g.H || w < 0 || w >= g.W) return 0.f;
    return x[k.base + r.off + (long long)(h * g.W + w) * g.x_ps];
  }
};

struct WgradEpilogue {
  float* gw;
  ConvGeo g;
  struct Row { long long off; };
  struct Col { long long off; };
  __device__ Row row(int m, int z) const {
    return Row{((long long)z * g.Coutg + m) * ((long long)g.Cg * g.RS)};
  }
  __device__ Col col(int n, int) const { return Col{(long long)n}; }
  __device__ void store(const Row& r, const Col& c, float acc) const { gw[r.off + c.off] = acc; }
};

inline size_t max_sz(size_t a, size_t b) { return a > b ? a : b; }

// The tensor-core routes hand the tensors to TMA (16-byte aligned base addresses) and carve
// 256-byte-aligned sub-buffers out of the workspace that the kernels access with 16-byte
// vectors: an offset view or an odd workspace must not reach them (a misaligned vector access
// is a sticky device fault).  Such calls run on the fp32 kernels, which take any alignment.
inline bool tc_operands_aligned(const void* a, const void* b, const void* c, const void* d,
                                const void* ws) {
  return aligned16(a) && aligned16(b) && aligned16(c) && aligned16(d) && aligned16(ws);
}


// ---- 16-bit tensors ---------------------------------------------------------------------------
// f16 / bf16 convolutions (the reference accepts f16, backend/cudnn/Conv2D.cpp:231,266,321) run
// as: widen the operands into fp32 copies at the front of the workspace, run the fp32 operator
// in the call's math mode (TF32 tensor cores keep 10 mantissa bits, as many as f16 has and more
// than bf16), round the result once to the 16-bit type.  Accumulation is fp32 throughout.
template <typename T>
__global__ void widen_kernel(const T* __restrict__ in, float* __restrict__ out, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
    if (i + 8 <= n && (reinterpret_cast<uintptr_t>(in + i) & 15) == 0) {
      const Vec16<T> v = *reinterpret_cast<const Vec16<T>*>(in + i);
#pragma unroll
      for (int j = 0; j < 8; j += 4)
        *reinterpret_cast<float4*>(out + i + j) =
            make_float4(Num<T>::to_f(v.v[j]), Num<T>::to_f(v.v[j + 1]), Num<T>::to_f(v.v[j + 2]),
                        Num<T>::to_f(v.v[j + 3]));
    } else {
      for (long long j = i; j < n && j < i + 8; ++j) out[j] = Num<T>::to_f(in[j]);
    }
  }
}
template <typename T>
__global__ void narrow_kernel(const float* __restrict__ in, T* __restrict__ out, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
    if (i + 8 <= n && (reinterpret_cast<uintptr_t>(out + i) & 15) == 0) {
      Vec16<T> v;
#pragma unroll
      for (int j = 0; j < 8; ++j) v.v[j] = Num<T>::from_f(in[i + j]);
      *reinterpret_cast<Vec16<T>*>(out + i) = v;
    } else {
      for (long long j = i; j < n && j < i + 8; ++j) out[j] = Num<T>::from_f(in[j]);
    }
  }
}
int widen(const void* in, float* out, long long n, int dtype, cudaStream_t st) {
  if (n == 0 || !in) return FLB200_OK;
  const unsigned grid = (unsigned)std::min<long long>((n / 8 + 255) / 256 + 1, 148 * 8);
  if (dtype == FLB200_F16)
    widen_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(in), out, n);
  else
    widen_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in), out, n);
  FLB200_AFTER_LAUNCH("conv_widen");
  return FLB200_OK;
}
int narrow(const float* in, void* out, long long n, int dtype, cudaStream_t st) {
  if (n == 0 || !out) return FLB200_OK;
  const unsigned grid = (unsigned)std::min<long long>((n / 8 + 255) / 256 + 1, 148 * 8);
  if (dtype == FLB200_F16)
    narrow_kernel<__half><<<grid, 256, 0, st>>>(in, static_cast<__half*>(out), n);
  else
    narrow_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(in, static_cast<__nv_bfloat16*>(out), n);
  FLB200_AFTER_LAUNCH("conv_narrow");
  return FLB200_OK;
}
// byte offsets of the fp32 copies pass `which` needs, in the order of its tensors:
// 0: x, w, bias, y | 1: grad_y, w, grad_x | 2: grad_y, x, grad_w, grad_bias
struct WideCopies {
  long long n[4];
  size_t off[4], total;
};
inline size_t up256c(size_t v) { return (v + 255) / 256 * 256; }
WideCopies wide_copies(const ConvGeo& g, int which) {
  const long long x = (long long)g.N * g.C * g.HW, w = (long long)g.Cout * g.Cg * g.RS,
                  y = (long long)g.N * g.Cout * g.HoWo, b = g.Cout;
  const long long n[3][4] = {{x, w, b, y}, {y, w, x, 0}, {y, x, w, b}};
  WideCopies c{};
  size_t off = 0;
  for (int i = 0; i < 4; ++i) {
    c.n[i] = n[which][i];
    c.off[i] = off;
    off += up256c((size_t)c.n[i] * 4);
  }
  c.total = off;
  return c;
}

}  // namespace
}  // namespace flb200

using namespace flb200;

extern "C" {

int flb200_conv2d_output_dims(const flb200_conv2d_desc* d, int32_t* Wo, int32_t* Ho) {
  ConvGeo g;
  if (int st = make_conv_geo("conv2d_output_dims", d, &g)) return st;
  if (Wo) *Wo = g.Wo;
  if (Ho) *Ho = g.Ho;
  return FLB200_OK;
}

size_t flb200_conv2d_workspace_bytes(const flb200_conv2d_desc* d, int which) {
  ConvGeo g;
  if (make_conv_geo("conv2d_workspace_bytes", d, &g)) return 0;
  size_t need = 0;
  if (which == 0) {
    need = plan_simt(g.Coutg, (long long)g.N * g.HoWo, (long long)g.Cg * g.RS, g.groups)
               .workspace_bytes;
  } else if (which == 1) {
    need = plan_simt(g.Cg, (long long)g.N * g.HW, (long long)g.Coutg * g.RS, g.groups)
               .workspace_bytes;
  } else {
    need = plan_simt(g.Coutg, (long long)g.Cg * g.RS, (long long)g.N * g.HoWo, g.groups)
               .workspace_bytes;
    need = max_sz(need, g.y_cl ? flb200_channel_sum_workspace_bytes((int64_t)g.N * g.HoWo, g.Cout, 1)
                               : flb200_channel_sum_workspace_bytes(g.N, g.Cout, g.HoWo));
  }
  if (d->math_mode != FLB200_MATH_STRICT_F32) need = max_sz(need, tc_conv_workspace_bytes(g, which));
  if (d->dtype != FLB200_F32 && which >= 0 && which <= 2)
    need = up256c(need) + wide_copies(g, which).total;  // fp32 copies of the 16-bit tensors
  return need;
}

int flb200_conv2d_forward(const flb200_conv2d_desc* d, const void* x, const void* w,
                          const void* bias, void* y, void* workspace, size_t workspace_bytes,
                          void* stream) {
  return flb200_conv2d_forward_cached(d, x, w, bias, y, workspace, workspace_bytes, nullptr,
                                      stream);
}

size_t flb200_conv2d_cache_bytes(const flb200_conv2d_desc* d, int which) {
  ConvGeo g;
  if (make_conv_geo("conv2d_cache_bytes", d, &g)) return 0;
  if (d->math_mode == FLB200_MATH_STRICT_F32 || which < 0 || which > 1) return 0;
  return tc_conv_cache_bytes(g, which);
}

int flb200_conv2d_forward_cached(const flb200_conv2d_desc* d, const void* x, const void* w,
                                 const void* bias, void* y, void* workspace,
                                 size_t workspace_bytes, flb200_conv2d_cache* cache,
                                 void* stream) {
  ConvGeo g;
  if (int st = make_conv_geo("conv2d_forward", d, &g)) return st;
  FLB200_REQUIRE(x && w && y, "conv2d_forward: null tensor");
  cudaStream_t st = as_stream(stream);
  if (d->dtype != FLB200_F32) {
    const WideCopies c = wide_copies(g, 0);
    if (!workspace || workspace_bytes < c.total)
      return fail(FLB200_WORKSPACE_TOO_SMALL, "conv2d_forward: workspace %zu < %zu",
                  workspace_bytes, c.total);
    char* ws = static_cast<char*>(workspace);
    float* x32 = reinterpret_cast<float*>(ws + c.off[0]);
    float* w32 = reinterpret_cast<float*>(ws + c.off[1]);
    float* b32 = bias ? reinterpret_cast<float*>(ws + c.off[2]) : nullptr;
    float* y32 = reinterpret_cast<float*>(ws + c.off[3]);
    if (int rc = widen(x, x32, c.n[0], d->dtype, st)) return rc;
    if (int rc = widen(w, w32, c.n[1], d->dtype, st)) return rc;
    if (int rc = widen(bias, b32, c.n[2], d->dtype, st)) return rc;
    flb200_conv2d_desc d32 = *d;
    d32.dtype = FLB200_F32;
    if (int rc = flb200_conv2d_forward_cached(&d32, x32, w32, b32, y32, ws + c.total,
                                              workspace_bytes - c.total, nullptr, stream))
      return rc;
    return narrow(y32, y, c.n[3], d->dtype, st);
  }
  const float* xf = static_cast<const float*>(x);
  const float* wf = static_cast<const float*>(w);
  const float* bf = static_cast<const float*>(bias);
  float* yf = static_cast<float*>(y);
  tc::X3Scope x3(d->math_mode == FLB200_MATH_F32X3);
  if (d->math_mode != FLB200_MATH_STRICT_F32 && tc_operands_aligned(x, w, y, bias, workspace) &&
      tc_conv_supported(g, 0, workspace_bytes))
    return tc_conv_forward(g, xf, wf, bf, yf, workspace, workspace_bytes, st, cache);
  const long long n_total = (long long)g.N * g.HoWo;
  FLB200_REQUIRE(n_total < 0x7fffffffLL, "conv2d_forward: too many output pixels");
  const long long K = (long long)g.Cg * g.RS;
  StridedLoader<true> al{wf, K, 1, (long long)g.Coutg * K, g.Coutg};
  FpropB bl{xf, g, n_total};
  FpropEpilogue ep{yf, bf, g};
  return launch_simt_gemm("conv2d_forward", al, bl, ep, g.Coutg, n_total, K, g.groups, workspace,
                          workspace_bytes, st);
}

size_t flb200_conv2d_stats_bytes(const flb200_conv2d_desc* d, int64_t* groups) {
  ConvGeo g;
  if (groups) *groups = 0;
  if (make_conv_geo("conv2d_stats_bytes", d, &g)) return 0;
  if (d->math_mode == FLB200_MATH_STRICT_F32 || d->dtype != FLB200_F32) return 0;
  const long long n = tc_conv_stats_groups(g);
  if (n == 0 || !tc_conv_supported(g, 0, tc_conv_workspace_bytes(g, 0))) return 0;
  if (groups) *groups = n;
  // CTA pairs may write one phantom tile (four all-zero rows) past the last real one
  return (size_t)(n + 4) * 2 * g.Cout * sizeof(float);
}

int flb200_conv2d_forward_stats(const flb200_conv2d_desc* d, const void* x, const void* w,
                                const void* bias, void* y, float* stats, size_t stats_bytes,
                                void* workspace, size_t workspace_bytes,
                                flb200_conv2d_cache* cache, void* stream) {
  ConvGeo g;
  if (int st = make_conv_geo("conv2d_forward_stats", d, &g)) return st;
  FLB200_REQUIRE(x && w && y && stats, "conv2d_forward_stats: null tensor");
  const size_t need = flb200_conv2d_stats_bytes(d, nullptr);
  if (need == 0 || !tc_operands_aligned(x, w, y, bias, workspace) || !aligned16(stats) ||
      !tc_conv_supported(g, 0, workspace_bytes))
    return fail(FLB200_UNSUPPORTED,
                "conv2d_forward_stats: needs a tensor-core route with a channels-last fp32 output "
                "of a multiple of 32 channels, 16-byte aligned tensors and the forward workspace");
  if (stats_bytes < need)
    return fail(FLB200_WORKSPACE_TOO_SMALL, "conv2d_forward_stats: statistics buffer %zu < %zu",
                stats_bytes, need);
  ConvStats cs{stats};
  tc::X3Scope x3(d->math_mode == FLB200_MATH_F32X3);
  return tc_conv_forward(g, static_cast<const float*>(x), static_cast<const float*>(w),
                         static_cast<const float*>(bias), static_cast<float*>(y), workspace,
                         workspace_bytes, as_stream(stream), cache, &cs);
}

int flb200_conv2d_backward_data(const flb200_conv2d_desc* d, const void* grad_y, const void* w,
                                void* grad_x, void* workspace, size_t workspace_bytes,
                                void* stream) {
  return flb200_conv2d_backward_data_cached(d, grad_y, w, grad_x, workspace, workspace_bytes,
                                            nullptr, stream);
}

int flb200_conv2d_backward_data_cached(const flb200_conv2d_desc* d, const void* grad_y,
                                       const void* w, void* grad_x, void* workspace,
                                       size_t workspace_bytes, flb200_conv2d_cache* cache,
                                       void* stream) {
  ConvGeo g;
  if (int st = make_conv_geo("conv2d_backward_data", d, &g)) return st;
  FLB200_REQUIRE(grad_y && w && grad_x, "conv2d_backward_data: null tensor");
  cudaStream_t st = as_stream(stream);
  if (d->dtype != FLB200_F32) {
    const WideCopies c = wide_copies(g, 1);
    if (!workspace || workspace_bytes < c.total)
      return fail(FLB200_WORKSPACE_TOO_SMALL, "conv2d_backward_data: workspace %zu < %zu",
                  workspace_bytes, c.total);
    char* ws = static_cast<char*>(workspace);
    float* gy32 = reinterpret_cast<float*>(ws + c.off[0]);
    float* w32 = reinterpret_cast<float*>(ws + c.off[1]);
    float* gx32 = reinterpret_cast<float*>(ws + c.off[2]);
    if (int rc = widen(grad_y, gy32, c.n[0], d->dtype, st)) return rc;
    if (int rc = widen(w, w32, c.n[1], d->dtype, st)) return rc;
    flb200_conv2d_desc d32 = *d;
    d32.dtype = FLB200_F32;
    if (int rc = flb200_conv2d_backward_data_cached(&d32, gy32, w32, gx32, ws + c.total,
                                                    workspace_bytes - c.total, nullptr, stream))
      return rc;
    return narrow(gx32, grad_x, c.n[2], d->dtype, st);
  }
  const float* gyf = static_cast<const float*>(grad_y);
  const float* wf = static_cast<const float*>(w);
  float* gxf = static_cast<float*>(grad_x);
  tc::X3Scope x3(d->math_mode == FLB200_MATH_F32X3);
  if (d->math_mode != FLB200_MATH_STRICT_F32 &&
      tc_operands_aligned(grad_y, w, grad_x, nullptr, workspace) &&
      tc_conv_supported(g, 1, workspace_bytes))
    return tc_conv_backward_data(g, gyf, wf, gxf, workspace, workspace_bytes, st, cache);
  const long long n_total = (long long)g.N * g.HW;
  FLB200_REQUIRE(n_total < 0x7fffffffLL, "conv2d_backward_data: too many input pixels");
  DgradA al{wf, g};
  DgradB bl{gyf, g, n_total};
  DgradEpilogue ep{gxf, g};
  return launch_simt_gemm("conv2d_backward_data", al, bl, ep, g.Cg, n_total,
                          (long long)g.Coutg * g.RS, g.groups, workspace, workspace_bytes, st);
}

int flb200_conv2d_backward_filter_bias(const flb200_conv2d_desc* d, const void* grad_y,
                                       const void* x, void* grad_w, void* grad_bias,
                                       void* workspace, size_t workspace_bytes, void* stream) {
  return flb200_conv2d_backward_filter_bias_cached(d, grad_y, x, grad_w, grad_bias, workspace,
                                                   workspace_bytes, nullptr, stream);
}

int flb200_conv2d_backward_filter_bias_cached(const flb200_conv2d_desc* d, const void* grad_y,
                                              const void* x, void* grad_w, void* grad_bias,
                                              void* workspace, size_t workspace_bytes,
                                              flb200_conv2d_cache* cache, void* stream) {
  ConvGeo g;
  if (int st = make_conv_geo("conv2d_backward_filter_bias", d, &g)) return st;
  FLB200_REQUIRE(grad_y && x && grad_w, "conv2d_backward_filter_bias: null tensor");
  cudaStream_t st = as_stream(stream);
  if (d->dtype != FLB200_F32) {
    const WideCopies c = wide_copies(g, 2);
    if (!workspace || workspace_bytes < c.total)
      return fail(FLB200_WORKSPACE_TOO_SMALL, "conv2d_backward_filter_bias: workspace %zu < %zu",
                  workspace_bytes, c.total);
    char* ws = static_cast<char*>(workspace);
    float* gy32 = reinterpret_cast<float*>(ws + c.off[0]);
    float* x32 = reinterpret_cast<float*>(ws + c.off[1]);
    float* gw32 = reinterpret_cast<float*>(ws + c.off[2]);
    float* gb32 = grad_bias ? reinterpret_cast<float*>(ws + c.off[3]) : nullptr;
    if (int rc = widen(grad_y, gy32, c.n[0], d->dtype, st)) return rc;
    if (int rc = widen(x, x32, c.n[1], d->dtype, st)) return rc;
    flb200_conv2d_desc d32 = *d;
    d32.dtype = FLB200_F32;
    if (int rc = flb200_conv2d_backward_filter_bias_cached(&d32, gy32, x32, gw32, gb32,
                                                           ws + c.total, workspace_bytes - c.total,
                                                           nullptr, stream))
      return rc;
    if (int rc = narrow(gw32, grad_w, c.n[2], d->dtype, st)) return rc;
    return narrow(gb32, grad_bias, c.n[3], d->dtype, st);
  }
  const float* gyf = static_cast<const float*>(grad_y);
  const float* xf = static_cast<const float*>(x);
  float* gwf = static_cast<float*>(grad_w);
  int rc;
  tc::X3Scope x3(d->math_mode == FLB200_MATH_F32X3);
  if (d->math_mode != FLB200_MATH_STRICT_F32 &&
      tc_operands_aligned(grad_y, x, grad_w, nullptr, workspace) &&
      tc_conv_supported(g, 2, workspace_bytes)) {
    rc = tc_conv_backward_filter(g, gyf, xf, gwf, workspace, workspace_bytes, st, cache);
  } else {
    const int n_total = g.Cg * g.RS;
    WgradA al{gyf, g};
    WgradB bl{xf, g, n_total};
    WgradEpilogue ep{gwf, g};
    rc = launch_simt_gemm("conv2d_backward_filter", al, bl, ep, g.Coutg, n_total,
                          (long long)g.N * g.HoWo, g.groups, workspace, workspace_bytes, st);
  }
  if (rc) return rc;
  if (grad_bias) {
    // db[co] = sum over batch and output pixels of dy — one pass over dy
    // (flashlight/fl/autograd/tensor/backend/cudnn/Conv2D.cpp:737).
    if (g.y_cl)  // [pixels][Cout]: column sums
      return flb200_channel_sum(grad_y, static_cast<float*>(grad_bias), (int64_t)g.N * g.HoWo,
                                g.Cout, 1, FLB200_F32, workspace, workspace_bytes, stream);
    return flb200_channel_sum(grad_y, static_cast<float*>(grad_bias), g.N, g.Cout, g.HoWo,
                              FLB200_F32, workspace, workspace_bytes, stream);
  }
  return FLB200_OK;
}


int flb200_astype(const void* in, int in_dtype, void* out, int out_dtype, int64_t n,
                  void* stream) {
  FLB200_REQUIRE(n >= 0, "astype: negative length");
  if (n == 0) return FLB200_OK;
  FLB200_REQUIRE(in && out, "astype: null tensor");
  cudaStream_t st = as_stream(stream);
  const bool in16 = in_dtype == FLB200_F16 || in_dtype == FLB200_BF16;
  const bool out16 = out_dtype == FLB200_F16 || out_dtype == FLB200_BF16;
  if (in_dtype == out_dtype) {
    const size_t es = in_dtype == FLB200_F32 ? 4 : 2;
    FLB200_REQUIRE(in_dtype == FLB200_F32 || in16, "astype: unknown dtype %d", in_dtype);
    FLB200_CUDA_CHECK(cudaMemcpyAsync(out, in, (size_t)n * es, cudaMemcpyDeviceToDevice, st));
    return FLB200_OK;
  }
  if (in_dtype == FLB200_F32 && out16) return narrow(static_cast<const float*>(in), out, n, out_dtype, st);
  if (in16 && out_dtype == FLB200_F32) return widen(in, static_cast<float*>(out), n, in_dtype, st);
  return fail(FLB200_UNSUPPORTED, "astype: %d -> %d is not built (f32 <-> f16 / bf16 only)",
              in_dtype, out_dtype);
}

}  // extern "C"
