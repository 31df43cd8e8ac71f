// rnn forward / backward: RELU, TANH, LSTM, GRU; multi-layer; bidirectional.
// Stands behind fl::AutogradExtension::rnn / ::rnnBackward
// (flashlight/fl/autograd/tensor/AutogradExtension.h:96-106, 167-179).
//
// Layouts (row-major views of fl's column-major tensors):
//   x [T][B][I], y [T][B][H*dirs] (forward direction in [0,H), reverse in [H,2H)),
//   hx/cx/hy/cy [L*dirs][B][H], pseudo-layer index p = layer*dirs + direction.
// Flat weights, the cuDNN order the reference relies on
// (flashlight/fl/nn/Utils.cpp:45-84; backend/onednn/RNN.cpp:66-158):
//   for p: W_ih [G*H][In_p], W_hh [G*H][H];   then for p: b_ih [G*H], b_hh [G*H].
// Gate order: LSTM i,f,g,o; GRU r,z,n with n = tanh(Wx + b + r*(Uh + b_hn)).
//
// Structure: per pseudo-layer one large GEMM for all input projections, then a
// time loop of (recurrent GEMM, pointwise cell).  Backward: time loop of
// (pointwise cell gradient, recurrent GEMM for dh), then batched GEMMs over all
// time steps for dW_ih, dW_hh and the gradient of the layer input.
// The reserve space (forward -> backward payload) holds the activated gates,
// cell states, GRU candidates' recurrent part and the outputs of inner layers.
#include <cstdlib>

#include "common.cuh"
#include "rnn_step.cuh"

namespace flb200 {
namespace {

struct RnnDims {
  int I, H, L, B, T, mode, dirs, G;
  long long GH, TB;
};

int make_dims(const char* name, const flb200_rnn_desc* d, RnnDims* r) {
  FLB200_REQUIRE(d, "%s: null descriptor", name);
  FLB200_REQUIRE(d->input_size >= 1 && d->hidden_size >= 1 && d->num_layers >= 1 &&
                     d->batch >= 1 && d->seq_len >= 1,
                 "%s: empty extent", name);
  FLB200_REQUIRE(d->mode >= FLB200_RNN_RELU && d->mode <= FLB200_RNN_GRU, "%s: unknown mode %d",
                 name, d->mode);
  FLB200_REQUIRE(d->dtype == FLB200_F32, "%s: only f32 is built (dtype %d)", name, d->dtype);
  r->I = d->input_size; r->H = d->hidden_size; r->L = d->num_layers; r->B = d->batch;
  r->T = d->seq_len; r->mode = d->mode; r->dirs = d->bidirectional ? 2 : 1;
  r->G = d->mode == FLB200_RNN_LSTM ? 4 : (d->mode == FLB200_RNN_GRU ? 3 : 1);
  r->GH = (long long)r->G * r->H;
  r->TB = (long long)r->T * r->B;
  return FLB200_OK;
}

inline long long in_size(const RnnDims& r, int layer) { return layer == 0 ? r.I : r.H * r.dirs; }

// Offsets (in floats) of W_ih, W_hh, b_ih, b_hh of pseudo-layer p in the flat vector.
struct ParamOffsets { long long w_ih, w_hh, b_ih, b_hh; };
ParamOffsets param_offsets(const RnnDims& r, int p) {
  long long off = 0;
  ParamOffsets po{};
  const int P = r.L * r.dirs;
  for (int q = 0; q < P; ++q) {
    const long long in = in_size(r, q / r.dirs);
    if (q == p) { po.w_ih = off; po.w_hh = off + r.GH * in; }
    off += r.GH * in + r.GH * r.H;
  }
  po.b_ih = off + (long long)p * 2 * r.GH;
  po.b_hh = po.b_ih + r.GH;
  return po;
}
long long num_params(const RnnDims& r) {
  long long n = 0;
  for (int l = 0; l < r.L; ++l) n += r.dirs * (r.GH * in_size(r, l) + r.GH * r.H + 2 * r.GH);
  return n;
}

inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }

// Reserve space: per pseudo-layer gates [T][B][GH], cells [T][B][H] (LSTM),
// q [T][B][H] (GRU); per inner layer its output [T][B][H*dirs].
struct ReserveLayout {
  size_t gates_stride, cell_off, q_off, per_p, inner_y_off, inner_y_stride, dropped_off, total;
};
// dropout: the inner layers' outputs are kept twice, as computed (the layer's own backward pass
// needs its hidden states) and with the dropout mask applied (the input of the layer above).
ReserveLayout reserve_layout(const RnnDims& r, bool dropout = false) {
  ReserveLayout L{};
  size_t off = up256((size_t)r.TB * r.GH * 4);
  L.cell_off = off;
  if (r.mode == FLB200_RNN_LSTM) off += up256((size_t)r.TB * r.H * 4);
  L.q_off = off;
  if (r.mode == FLB200_RNN_GRU) off += up256((size_t)r.TB * r.H * 4);
  L.per_p = off;
  L.inner_y_off = L.per_p * (size_t)(r.L * r.dirs);
  L.inner_y_stride = up256((size_t)r.TB * r.H * r.dirs * 4);
  L.dropped_off = L.inner_y_off + L.inner_y_stride * (size_t)(r.L - 1);
  L.total = L.dropped_off + (dropout ? L.inner_y_stride * (size_t)(r.L - 1) : 0);
  return L;
}

int mm(int math_mode, long long m, long long n, long long k, const float* a, long long a_row,
       long long a_col, const float* b, long long b_row, long long b_col, float* c, long long c_row,
       float beta, void* ws, size_t ws_bytes, void* stream) {
  flb200_matmul_desc d = {};
  d.m = m; d.n = n; d.k = k; d.batch = 1;
  d.a_row = a_row; d.a_col = a_col;
  d.b_row = b_row; d.b_col = b_col;
  d.c_row = c_row; d.c_col = 1;
  d.alpha = 1.f; d.beta = beta;
  d.dtype = FLB200_F32; d.math_mode = math_mode;
  return flb200_matmul(&d, a, b, c, ws, ws_bytes, stream);
}

size_t mm_ws(long long m, long long n, long long k) {
  flb200_matmul_desc d = {};
  d.m = m; d.n = n; d.k = k; d.batch = 1;
  d.math_mode = FLB200_MATH_TF32;
  return flb200_matmul_workspace_bytes(&d);
}

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }

// bias_comb[j] = b_ih[j] + b_hh[j], except the GRU candidate gate keeps b_ih only.
__global__ void combine_bias_kernel(const float* __restrict__ b_ih, const float* __restrict__ b_hh,
                                    float* __restrict__ out, int H, int G, int mode) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= G * H) return;
  const bool cand = mode == FLB200_RNN_GRU && j >= 2 * H;
  out[j] = b_ih[j] + (cand ? 0.f : b_hh[j]);
}

// One time step, forward.  gates: [B][GH] pre-activation in, activated out.
// h_prev/c_prev rows have strides hp_stride / cp_stride; h_out row stride ho_stride.
__global__ void __launch_bounds__(256)
cell_forward_kernel(float* __restrict__ gates, const float* __restrict__ gh,
                    const float* __restrict__ b_hh, const float* __restrict__ h_prev,
                    long long hp_stride, const float* __restrict__ c_prev, long long cp_stride,
                    float* __restrict__ c_out, float* __restrict__ q_out, float* __restrict__ h_out,
                    long long ho_stride, int B, int H, int mode) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx - b * H;
  if (mode == FLB200_RNN_LSTM) {
    float* g = gates + (long long)b * 4 * H;
    const float i = sigmoidf_(g[j]), f = sigmoidf_(g[H + j]);
    const float gg = tanhf(g[2 * H + j]), o = sigmoidf_(g[3 * H + j]);
    const float c = f * c_prev[(long long)b * cp_stride + j] + i * gg;
    g[j] = i; g[H + j] = f; g[2 * H + j] = gg; g[3 * H + j] = o;
    c_out[(long long)b * H + j] = c;
    h_out[(long long)b * ho_stride + j] = o * tanhf(c);
  } else if (mode == FLB200_RNN_GRU) {
    float* g = gates + (long long)b * 3 * H;
    const float* r_h = gh + (long long)b * 3 * H;
    const float r = sigmoidf_(g[j] + r_h[j]);
    const float z = sigmoidf_(g[H + j] + r_h[H + j]);
    const float q = r_h[2 * H + j] + b_hh[2 * H + j];
    const float n = tanhf(g[2 * H + j] + r * q);
    const float hp = h_prev[(long long)b * hp_stride + j];
    g[j] = r; g[H + j] = z; g[2 * H + j] = n;
    q_out[(long long)b * H + j] = q;
    h_out[(long long)b * ho_stride + j] = (1.f - z) * n + z * hp;
  } else {
    float* g = gates + (long long)b * H;
    const float a = g[j];
    const float h = mode == FLB200_RNN_RELU ? fmaxf(a, 0.f) : tanhf(a);
    g[j] = h;
    h_out[(long long)b * ho_stride + j] = h;
  }
}

// One time step, backward.  dh / dc are [B][H] running gradients (updated in
// place: dc becomes dc_prev; for GRU dh becomes the direct part dh*z that the
// recurrent GEMM then accumulates onto).  dgx / dgh: [B][GH] gate gradients on
// the input side and on the recurrent side (same buffer unless GRU).
__global__ void __launch_bounds__(256)
cell_backward_kernel(const float* __restrict__ gates, const float* __restrict__ cells,
                     const float* __restrict__ c_prev, long long cp_stride,
                     const float* __restrict__ q, const float* __restrict__ h_prev,
                     long long hp_stride, const float* __restrict__ dy, long long dy_stride,
                     float* __restrict__ dh, float* __restrict__ dc, float* __restrict__ dgx,
                     float* __restrict__ dgh, int B, int H, int mode) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx - b * H;
  const long long bh = (long long)b * H + j;
  float d = dh[bh];
  if (dy) d += dy[(long long)b * dy_stride + j];
  if (mode == FLB200_RNN_LSTM) {
    const float* g = gates + (long long)b * 4 * H;
    const float i = g[j], f = g[H + j], gg = g[2 * H + j], o = g[3 * H + j];
    const float tc = tanhf(cells[bh]);
    const float dct = dc[bh] + d * o * (1.f - tc * tc);
    float* out = dgx + (long long)b * 4 * H;
    out[j] = dct * gg * i * (1.f - i);
    out[H + j] = dct * c_prev[(long long)b * cp_stride + j] * f * (1.f - f);
    out[2 * H + j] = dct * i * (1.f - gg * gg);
    out[3 * H + j] = d * tc * o * (1.f - o);
    dc[bh] = dct * f;
    dh[bh] = 0.f;  // the recurrent GEMM overwrites it (beta = 0); kept defined for clarity
  } else if (mode == FLB200_RNN_GRU) {
    const float* g = gates + (long long)b * 3 * H;
    const float r = g[j], z = g[H + j], n = g[2 * H + j];
    const float hp = h_prev[(long long)b * hp_stride + j];
    const float dn = d * (1.f - z) * (1.f - n * n);
    const float dz = d * (hp - n) * z * (1.f - z);
    const float dr = dn * q[bh] * r * (1.f - r);
    float* ox = dgx + (long long)b * 3 * H;
    float* oh = dgh + (long long)b * 3 * H;
    ox[j] = dr; ox[H + j] = dz; ox[2 * H + j] = dn;
    oh[j] = dr; oh[H + j] = dz; oh[2 * H + j] = dn * r;
    dh[bh] = d * z;
  } else {
    const float h = gates[(long long)b * H + j];
    const float da = mode == FLB200_RNN_RELU ? (h > 0.f ? d : 0.f) : d * (1.f - h * h);
    dgx[(long long)b * H + j] = da;
    dh[bh] = 0.f;
  }
}

// dst[b][j] = src ? src[b*src_stride + j] : 0
__global__ void copy_rows_kernel(const float* __restrict__ src, long long src_stride,
                                 float* __restrict__ dst, long long dst_stride, int B, int H) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx - b * H;
  dst[(long long)b * dst_stride + j] = src ? src[(long long)b * src_stride + j] : 0.f;
}

struct FwdWs { size_t zero, gh, bias, sync, mm, total; };
FwdWs fwd_ws(const RnnDims& r) {
  FwdWs w{};
  size_t off = 0;
  w.zero = off; off += up256((size_t)r.B * r.H * 4);
  w.gh = off; off += up256((size_t)r.B * r.GH * 4);
  w.bias = off; off += up256((size_t)r.GH * 4);
  w.sync = off; off += 256;  // grid-barrier counter of the persistent recurrence kernel
  w.mm = off;
  size_t m = 0;
  for (int l = 0; l < r.L; ++l) {
    const size_t v = mm_ws(r.TB, r.GH, in_size(r, l));
    if (v > m) m = v;
  }
  const size_t v2 = mm_ws(r.B, r.GH, r.H);
  if (v2 > m) m = v2;
  off += up256(m);
  w.total = off;
  return w;
}

struct BwdWs { size_t dgx, dgh, dya, dyb, dh, dc, zero, sync, xbuf, red, mm, mm_bytes, red_bytes, total; };
BwdWs bwd_ws(const RnnDims& r) {
  BwdWs w{};
  size_t off = 0;
  w.dgx = off; off += up256((size_t)r.TB * r.GH * 4);
  w.dgh = off; if (r.mode == FLB200_RNN_GRU) off += up256((size_t)r.TB * r.GH * 4);
  w.dya = off; off += up256((size_t)r.TB * r.H * r.dirs * 4);
  w.dyb = off; off += up256((size_t)r.TB * r.H * r.dirs * 4);
  w.dh = off; off += up256((size_t)r.B * r.H * 4);
  w.dc = off; off += up256((size_t)r.B * r.H * 4);
  w.zero = off; off += up256((size_t)r.B * r.H * 4);
  w.sync = off; off += 256;  // grid-barrier counter of the persistent recurrence kernel
  w.xbuf = off;              // its per-step exchange of partial sums
  if (r.H == 256 || r.H == 512 || r.H == 1024)
    off += up256(lstm_sequence_backward_scratch_bytes(r.H));
  w.red = off;
  w.red_bytes = flb200_channel_sum_workspace_bytes(r.TB, r.GH, 1);
  off += up256(w.red_bytes);
  w.mm = off;
  size_t m = mm_ws(r.B, r.H, r.GH);
  for (int l = 0; l < r.L; ++l) {
    const long long in = in_size(r, l);
    size_t v = mm_ws(r.GH, in, r.TB);
    if (v > m) m = v;
    v = mm_ws(r.TB, in, r.GH);
    if (v > m) m = v;
  }
  const size_t v3 = mm_ws(r.GH, r.H, r.TB);
  if (v3 > m) m = v3;
  w.mm_bytes = m;
  off += up256(m);
  w.total = off;
  return w;
}

}  // namespace
}  // namespace flb200

using namespace flb200;

extern "C" {

int64_t flb200_rnn_num_params(const flb200_rnn_desc* d) {
  RnnDims r;
  if (make_dims("rnn_num_params", d, &r)) return -1;
  return num_params(r);
}

size_t flb200_rnn_reserve_bytes(const flb200_rnn_desc* d) {
  RnnDims r;
  if (make_dims("rnn_reserve_bytes", d, &r)) return 0;
  return reserve_layout(r).total;
}

// backward: 0 forward with a reserve space, 1 backward, 2 forward without a
// reserve space (inference; the workspace then also holds what the reserve would).
size_t flb200_rnn_workspace_bytes(const flb200_rnn_desc* d, int backward) {
  RnnDims r;
  if (make_dims("rnn_workspace_bytes", d, &r)) return 0;
  if (backward == 1) return bwd_ws(r).total;
  size_t n = fwd_ws(r).total;
  if (backward == 2) n += reserve_layout(r).total;
  return n;
}

// mask != NULL: inter-layer dropout (backend/cudnn/RNN.cpp:83-85), mask [L-1][T][B][H*dirs] of
// 0 / 1, applied with scale 1 / (1 - p) to the input of layers 1 .. L-1.
static int rnn_forward_impl(const flb200_rnn_desc* d, const void* x, const void* hx,
                            const void* cx, const void* w, const void* mask, float drop_p,
                            void* y, void* hy, void* cy, void* reserve, size_t reserve_bytes,
                            void* workspace, size_t workspace_bytes, void* stream) {
  RnnDims r;
  if (int st = make_dims("rnn_forward", d, &r)) return st;
  FLB200_REQUIRE(x && w && y, "rnn_forward: null tensor");
  FLB200_REQUIRE(!mask || (drop_p >= 0.f && drop_p < 1.f), "rnn_forward: dropout outside [0, 1)");
  const bool dropout = mask != nullptr && r.L > 1;
  const float drop_scale = dropout ? 1.f / (1.f - drop_p) : 1.f;
  const ReserveLayout RL = reserve_layout(r, dropout);
  const FwdWs W = fwd_ws(r);
  char* ws = static_cast<char*>(workspace);
  char* rs = static_cast<char*>(reserve);
  size_t need = W.total;
  if (!rs) need += RL.total;
  if (!ws || workspace_bytes < need)
    return fail(FLB200_WORKSPACE_TOO_SMALL, "rnn_forward: workspace %zu < %zu", workspace_bytes,
                need);
  if (rs) {
    if (reserve_bytes < RL.total)
      return fail(FLB200_WORKSPACE_TOO_SMALL, "rnn_forward: reserve %zu < %zu", reserve_bytes,
                  RL.total);
  } else {
    rs = ws + W.total;
  }
  cudaStream_t st = as_stream(stream);
  const float* wf = static_cast<const float*>(w);
  const float* hxf = static_cast<const float*>(hx);
  const float* cxf = static_cast<const float*>(cx);
  float* zero = reinterpret_cast<float*>(ws + W.zero);
  float* gh = reinterpret_cast<float*>(ws + W.gh);
  float* bias = reinterpret_cast<float*>(ws + W.bias);
  void* mmws = ws + W.mm;
  const size_t mmws_bytes = workspace_bytes - W.mm > 0 ? (W.total - W.mm) : 0;
  FLB200_CUDA_CHECK(cudaMemsetAsync(zero, 0, (size_t)r.B * r.H * 4, st));
  const int H = r.H, B = r.B, T = r.T;
  const long long GH = r.GH, BH = (long long)B * H;
  const int cell_grid = (B * H + 255) / 256;

  for (int l = 0; l < r.L; ++l) {
    const long long In = in_size(r, l);
    const float* in = l == 0 ? static_cast<const float*>(x)
                             : reinterpret_cast<const float*>(
                                   rs + (dropout ? RL.dropped_off : RL.inner_y_off) +
                                   RL.inner_y_stride * (size_t)(l - 1));
    float* out = l == r.L - 1 ? static_cast<float*>(y)
                              : reinterpret_cast<float*>(rs + RL.inner_y_off +
                                                         RL.inner_y_stride * (size_t)l);
    const long long out_stride = (long long)H * r.dirs;
    for (int dir = 0; dir < r.dirs; ++dir) {
      const int p = l * r.dirs + dir;
      const ParamOffsets po = param_offsets(r, p);
      float* gates = reinterpret_cast<float*>(rs + RL.per_p * (size_t)p);
      float* cells = reinterpret_cast<float*>(rs + RL.per_p * (size_t)p + RL.cell_off);
      float* qbuf = reinterpret_cast<float*>(rs + RL.per_p * (size_t)p + RL.q_off);
      combine_bias_kernel<<<(unsigned)((GH + 255) / 256), 256, 0, st>>>(wf + po.b_ih, wf + po.b_hh,
                                                                        bias, H, r.G, r.mode);
      FLB200_AFTER_LAUNCH("rnn_combine_bias");
      // all input projections of this pseudo-layer: gates[TB][GH] = in * W_ih^T + bias
      if (int rc = mm(d->math_mode, r.TB, GH, In, in, In, 1, wf + po.w_ih, 1, In, gates, GH, 0.f,
                      mmws, mmws_bytes, stream))
        return rc;
      if (int rc = flb200_channel_bias_add(gates, bias, gates, r.TB, GH, 1, FLB200_F32, stream))
        return rc;
      const float* h_prev = hxf ? hxf + (long long)p * BH : zero;
      long long hp_stride = H;
      const float* c_prev = cxf ? cxf + (long long)p * BH : zero;
      // LSTM in TF32 mode: one fused kernel per step (contraction + reduction + cell)
      const bool fused = r.mode == FLB200_RNN_LSTM && lstm_step_supported(d->math_mode, B, H);
      CUtensorMap map_whh;
      if (fused)
        if (int rc = lstm_step_weight_map(&map_whh, wf + po.w_hh, H)) return rc;
      // ... or, where the device can hold the whole launch at once, ONE persistent kernel for
      // all T steps with W_hh resident in shared memory (FLB200_RNN_PERSISTENT=0: per step)
      static const bool persistent_off = [] {
        const char* v = getenv("FLB200_RNN_PERSISTENT");
        return v && v[0] == '0';
      }();
      int first_step = 0;
      if (r.mode != FLB200_RNN_LSTM && !persistent_off &&
          lstm_sequence_supported(d->math_mode, B, H, r.G)) {
        // GRU and the plain cells: the same persistent kernel with three gates / one; the
        // GRU's reserve tensor q takes the place of the cell states
        const bool gru = r.mode == FLB200_RNN_GRU;
        if (int rc = lstm_step_weight_map(&map_whh, wf + po.w_hh, H, r.G)) return rc;
        if (int rc = lstm_sequence_forward(
                map_whh, gates, gru ? qbuf : nullptr, out + (long long)dir * H, out_stride, h_prev,
                nullptr, reinterpret_cast<unsigned*>(ws + W.sync), T, B, H, dir, 0, -1, st, r.G,
                gru ? wf + po.b_hh + 2 * H : nullptr, r.mode == FLB200_RNN_RELU ? 0 : 1))
          return rc;
        const int t_last = dir == 0 ? T - 1 : 0;
        h_prev = out + (long long)t_last * B * out_stride + (long long)dir * H;
        hp_stride = out_stride;
        first_step = T;
      }
      if (fused && !persistent_off && lstm_sequence_supported(d->math_mode, B, H)) {
        if (int rc = lstm_sequence_forward(
                map_whh, gates, cells, out + (long long)dir * H, out_stride, h_prev, c_prev,
                reinterpret_cast<unsigned*>(ws + W.sync), T, B, H, dir, 0, -1, st))
          return rc;
        const int t_last = dir == 0 ? T - 1 : 0;
        h_prev = out + (long long)t_last * B * out_stride + (long long)dir * H;
        hp_stride = out_stride;
        c_prev = cells + (long long)t_last * BH;
        first_step = T;
      }
      for (int step = first_step; step < T; ++step) {
        const int t = dir == 0 ? step : T - 1 - step;
        float* g_t = gates + (long long)t * B * GH;
        float* h_t = out + (long long)t * B * out_stride + (long long)dir * H;
        if (fused) {
          if (int rc = lstm_step_forward(map_whh, h_prev, hp_stride, g_t, c_prev, H,
                                         cells + (long long)t * BH, h_t, out_stride, B, H, st))
            return rc;
          h_prev = h_t;
          hp_stride = out_stride;
          c_prev = cells + (long long)t * BH;
          continue;
        }
        if (r.mode == FLB200_RNN_GRU) {
          if (int rc = mm(d->math_mode, B, GH, H, h_prev, hp_stride, 1, wf + po.w_hh, 1, H, gh, GH,
                          0.f, mmws, mmws_bytes, stream))
            return rc;
        } else {
          if (int rc = mm(d->math_mode, B, GH, H, h_prev, hp_stride, 1, wf + po.w_hh, 1, H, g_t,
                          GH, 1.f, mmws, mmws_bytes, stream))
            return rc;
        }
        cell_forward_kernel<<<cell_grid, 256, 0, st>>>(
            g_t, gh, wf + po.b_hh, h_prev, hp_stride, c_prev, H, cells + (long long)t * BH,
            qbuf + (long long)t * BH, h_t, out_stride, B, H, r.mode);
        FLB200_AFTER_LAUNCH("rnn_cell_forward");
        h_prev = h_t;
        hp_stride = out_stride;
        c_prev = cells + (long long)t * BH;
      }
      if (hy) {
        copy_rows_kernel<<<cell_grid, 256, 0, st>>>(h_prev, hp_stride,
                                                    static_cast<float*>(hy) + (long long)p * BH, H,
                                                    B, H);
        FLB200_AFTER_LAUNCH("rnn_copy_hy");
      }
      if (cy && r.mode == FLB200_RNN_LSTM) {
        copy_rows_kernel<<<cell_grid, 256, 0, st>>>(c_prev, H,
                                                    static_cast<float*>(cy) + (long long)p * BH, H,
                                                    B, H);
        FLB200_AFTER_LAUNCH("rnn_copy_cy");
      }
    }
    if (dropout && l < r.L - 1) {
      const long long n = r.TB * out_stride;
      if (int rc = flb200_dropout_apply(
              out, static_cast<const float*>(mask) + (long long)l * n,
              rs + RL.dropped_off + RL.inner_y_stride * (size_t)l, drop_scale, n, FLB200_F32,
              stream))
        return rc;
    }
  }
  return FLB200_OK;
}

static int rnn_backward_impl(const flb200_rnn_desc* d, const void* x, const void* hx,
                             const void* cx, const void* w, const void* mask, float drop_p,
                             const void* y, const void* grad_y, const void* grad_hy,
                             const void* grad_cy, void* grad_x, void* grad_hx, void* grad_cx,
                             void* grad_w, const void* reserve, size_t reserve_bytes,
                             void* workspace, size_t workspace_bytes, void* stream) {
  RnnDims r;
  if (int st = make_dims("rnn_backward", d, &r)) return st;
  FLB200_REQUIRE(x && w && y && grad_x && grad_w, "rnn_backward: null tensor");
  FLB200_REQUIRE(reserve, "rnn_backward: the reserve space written by rnn_forward is required");
  FLB200_REQUIRE(!mask || (drop_p >= 0.f && drop_p < 1.f), "rnn_backward: dropout outside [0, 1)");
  const bool dropout = mask != nullptr && r.L > 1;
  const float drop_scale = dropout ? 1.f / (1.f - drop_p) : 1.f;
  const ReserveLayout RL = reserve_layout(r, dropout);
  if (reserve_bytes < RL.total)
    return fail(FLB200_WORKSPACE_TOO_SMALL, "rnn_backward: reserve %zu < %zu", reserve_bytes,
                RL.total);
  const BwdWs W = bwd_ws(r);
  if (!workspace || workspace_bytes < W.total)
    return fail(FLB200_WORKSPACE_TOO_SMALL, "rnn_backward: workspace %zu < %zu", workspace_bytes,
                W.total);
  cudaStream_t st = as_stream(stream);
  char* ws = static_cast<char*>(workspace);
  const char* rs = static_cast<const char*>(reserve);
  const float* wf = static_cast<const float*>(w);
  float* gwf = static_cast<float*>(grad_w);
  const float* hxf = static_cast<const float*>(hx);
  const float* cxf = static_cast<const float*>(cx);
  float* dgx = reinterpret_cast<float*>(ws + W.dgx);
  float* dgh = r.mode == FLB200_RNN_GRU ? reinterpret_cast<float*>(ws + W.dgh) : dgx;
  float* dy_bufs[2] = {reinterpret_cast<float*>(ws + W.dya), reinterpret_cast<float*>(ws + W.dyb)};
  float* dh = reinterpret_cast<float*>(ws + W.dh);
  float* dc = reinterpret_cast<float*>(ws + W.dc);
  float* zero = reinterpret_cast<float*>(ws + W.zero);
  void* red = ws + W.red;
  void* mmws = ws + W.mm;
  const size_t mmws_bytes = W.mm_bytes;
  FLB200_CUDA_CHECK(cudaMemsetAsync(zero, 0, (size_t)r.B * r.H * 4, st));
  const int H = r.H, B = r.B, T = r.T;
  const long long GH = r.GH, BH = (long long)B * H;
  const int cell_grid = (B * H + 255) / 256;
  const long long ys = (long long)H * r.dirs;

  for (int l = r.L - 1; l >= 0; --l) {
    const long long In = in_size(r, l);
    // the layer's input as the forward pass fed it: with dropout, the masked copy
    const float* in = l == 0 ? static_cast<const float*>(x)
                             : reinterpret_cast<const float*>(
                                   rs + (dropout ? RL.dropped_off : RL.inner_y_off) +
                                   RL.inner_y_stride * (size_t)(l - 1));
    const float* out = l == r.L - 1 ? static_cast<const float*>(y)
                                    : reinterpret_cast<const float*>(rs + RL.inner_y_off +
                                                                     RL.inner_y_stride * (size_t)l);
    // gradient w.r.t. this layer's output: the caller's grad_y for the top
    // layer, else what the layer above left in the ping-pong buffer.
    const float* dy_l = l == r.L - 1 ? static_cast<const float*>(grad_y) : dy_bufs[(l + 1) & 1];
    float* din = l == 0 ? static_cast<float*>(grad_x) : dy_bufs[l & 1];
    for (int dir = 0; dir < r.dirs; ++dir) {
      const int p = l * r.dirs + dir;
      const ParamOffsets po = param_offsets(r, p);
      const float* gates = reinterpret_cast<const float*>(rs + RL.per_p * (size_t)p);
      const float* cells = reinterpret_cast<const float*>(rs + RL.per_p * (size_t)p + RL.cell_off);
      const float* qbuf = reinterpret_cast<const float*>(rs + RL.per_p * (size_t)p + RL.q_off);
      // LSTM in TF32 mode on a device that holds the whole launch at once: the recurrence of
      // all T steps in ONE persistent kernel (FLB200_RNN_PERSISTENT=0: kernels per step)
      static const bool persistent_off = [] {
        const char* v = getenv("FLB200_RNN_PERSISTENT");
        return v && v[0] == '0';
      }();
      const bool lstm = r.mode == FLB200_RNN_LSTM, gru = r.mode == FLB200_RNN_GRU;
      const bool persistent = !persistent_off &&
                              lstm_sequence_backward_supported(d->math_mode, B, H, r.G);
      if (persistent) {
        // (GRU: q in the place of the cell states, h0 in the place of c0, no cell-state
        // gradients, the recurrent side's gate gradients in dgh; plain cells: gates only)
        CUtensorMap map_wt;
        if (int rc = lstm_sequence_weight_map_transposed(&map_wt, wf + po.w_hh, H, r.G)) return rc;
        const float* first_state = lstm ? (cxf ? cxf + (long long)p * BH : zero)
                                        : (hxf ? hxf + (long long)p * BH : zero);
        if (int rc = lstm_sequence_backward(
                map_wt, gates, lstm ? cells : qbuf, first_state,
                dy_l ? dy_l + (long long)dir * H : nullptr, ys,
                grad_hy ? static_cast<const float*>(grad_hy) + (long long)p * BH : nullptr,
                lstm && grad_cy ? static_cast<const float*>(grad_cy) + (long long)p * BH : nullptr,
                dgx, dh, dc, reinterpret_cast<float*>(ws + W.xbuf),
                reinterpret_cast<unsigned*>(ws + W.sync), T, B, H, dir, st, r.G, dgh,
                out + (long long)dir * H, ys, r.mode == FLB200_RNN_RELU ? 0 : 1))
          return rc;
      }
      if (!persistent) {
      copy_rows_kernel<<<cell_grid, 256, 0, st>>>(
          grad_hy ? static_cast<const float*>(grad_hy) + (long long)p * BH : nullptr, H, dh, H, B,
          H);
      FLB200_AFTER_LAUNCH("rnn_init_dh");
      copy_rows_kernel<<<cell_grid, 256, 0, st>>>(
          grad_cy && r.mode == FLB200_RNN_LSTM
              ? static_cast<const float*>(grad_cy) + (long long)p * BH
              : nullptr,
          H, dc, H, B, H);
      FLB200_AFTER_LAUNCH("rnn_init_dc");
      // walk time against the direction of the forward recurrence
      for (int step = T - 1; step >= 0; --step) {
        const int t = dir == 0 ? step : T - 1 - step;
        const int t_prev = dir == 0 ? t - 1 : t + 1;  // index of h_{prev} in `out`
        const bool first = step == 0;
        const float* h_prev = first ? (hxf ? hxf + (long long)p * BH : zero)
                                    : out + (long long)t_prev * B * ys + (long long)dir * H;
        const long long hp_stride = first ? H : ys;
        const float* c_prev = first ? (cxf ? cxf + (long long)p * BH : zero)
                                    : cells + (long long)t_prev * BH;
        cell_backward_kernel<<<cell_grid, 256, 0, st>>>(
            gates + (long long)t * B * GH, cells + (long long)t * BH, c_prev, H,
            qbuf + (long long)t * BH, h_prev, hp_stride,
            dy_l ? dy_l + (long long)t * B * ys + (long long)dir * H : nullptr, ys, dh, dc,
            dgx + (long long)t * B * GH, dgh + (long long)t * B * GH, B, H, r.mode);
        FLB200_AFTER_LAUNCH("rnn_cell_backward");
        // dh_prev (+)= dgates_h[t] * W_hh
        if (int rc = mm(d->math_mode, B, H, GH, dgh + (long long)t * B * GH, GH, 1, wf + po.w_hh, H,
                        1, dh, H, r.mode == FLB200_RNN_GRU ? 1.f : 0.f, mmws, mmws_bytes, stream))
          return rc;
      }
      }  // !persistent
      if (grad_hx) {
        copy_rows_kernel<<<cell_grid, 256, 0, st>>>(
            dh, H, static_cast<float*>(grad_hx) + (long long)p * BH, H, B, H);
        FLB200_AFTER_LAUNCH("rnn_copy_dhx");
      }
      if (grad_cx && r.mode == FLB200_RNN_LSTM) {
        copy_rows_kernel<<<cell_grid, 256, 0, st>>>(
            dc, H, static_cast<float*>(grad_cx) + (long long)p * BH, H, B, H);
        FLB200_AFTER_LAUNCH("rnn_copy_dcx");
      }
      // dW_ih[GH][In] = dgx^T * in   (K = T*B)
      if (int rc = mm(d->math_mode, GH, In, r.TB, dgx, 1, GH, in, In, 1, gwf + po.w_ih, In, 0.f,
                      mmws, mmws_bytes, stream))
        return rc;
      // dW_hh[GH][H] = sum_t dgh[t]^T * h_prev[t]: all steps that have a
      // predecessor inside `out` in one GEMM, then the boundary step with hx.
      if (T > 1) {
        // forward direction: steps t = 1..T-1 pair with out[t-1]; reverse: t = 0..T-2 with out[t+1]
        const float* dg0 = dir == 0 ? dgh + (long long)B * GH : dgh;
        const float* hp0 = dir == 0 ? out + (long long)dir * H : out + (long long)B * ys + (long long)dir * H;
        if (int rc = mm(d->math_mode, GH, H, (long long)(T - 1) * B, dg0, 1, GH, hp0, ys, 1,
                        gwf + po.w_hh, H, 0.f, mmws, mmws_bytes, stream))
          return rc;
      }
      {
        const int tb = dir == 0 ? 0 : T - 1;  // boundary step
        const float* hb = hxf ? hxf + (long long)p * BH : zero;
        if (int rc = mm(d->math_mode, GH, H, B, dgh + (long long)tb * B * GH, 1, GH, hb, H, 1,
                        gwf + po.w_hh, H, T > 1 ? 1.f : 0.f, mmws, mmws_bytes, stream))
          return rc;
      }
      // bias gradients: column sums of the gate gradients over all (t, b)
      if (int rc = flb200_channel_sum(dgx, gwf + po.b_ih, r.TB, GH, 1, FLB200_F32, red,
                                      W.red_bytes, stream))
        return rc;
      if (int rc = flb200_channel_sum(dgh, gwf + po.b_hh, r.TB, GH, 1, FLB200_F32, red,
                                      W.red_bytes, stream))
        return rc;
      // gradient of the layer input: din[TB][In] (+)= dgx * W_ih
      if (int rc = mm(d->math_mode, r.TB, In, GH, dgx, GH, 1, wf + po.w_ih, In, 1, din, In,
                      dir == 0 ? 0.f : 1.f, mmws, mmws_bytes, stream))
        return rc;
    }
    if (dropout && l > 0) {
      // din is the gradient of the MASKED output of the layer below
      const long long n = r.TB * In;
      if (int rc = flb200_dropout_apply(din, static_cast<const float*>(mask) + (long long)(l - 1) * n,
                                        din, drop_scale, n, FLB200_F32, stream))
        return rc;
    }
  }
  return FLB200_OK;
}

int flb200_rnn_forward(const flb200_rnn_desc* d, const void* x, const void* hx, const void* cx,
                       const void* w, void* y, void* hy, void* cy, void* reserve,
                       size_t reserve_bytes, void* workspace, size_t workspace_bytes,
                       void* stream) {
  return rnn_forward_impl(d, x, hx, cx, w, nullptr, 0.f, y, hy, cy, reserve, reserve_bytes,
                          workspace, workspace_bytes, stream);
}

int flb200_rnn_backward(const flb200_rnn_desc* d, const void* x, const void* hx, const void* cx,
                        const void* w, const void* y, const void* grad_y, const void* grad_hy,
                        const void* grad_cy, void* grad_x, void* grad_hx, void* grad_cx,
                        void* grad_w, const void* reserve, size_t reserve_bytes, void* workspace,
                        size_t workspace_bytes, void* stream) {
  return rnn_backward_impl(d, x, hx, cx, w, nullptr, 0.f, y, grad_y, grad_hy, grad_cy, grad_x,
                           grad_hx, grad_cx, grad_w, reserve, reserve_bytes, workspace,
                           workspace_bytes, stream);
}

int64_t flb200_rnn_dropout_mask_elements(const flb200_rnn_desc* d) {
  RnnDims r;
  if (make_dims("rnn_dropout_mask_elements", d, &r)) return -1;
  return (long long)(r.L - 1) * r.TB * r.H * r.dirs;
}

size_t flb200_rnn_reserve_bytes_dropout(const flb200_rnn_desc* d) {
  RnnDims r;
  if (make_dims("rnn_reserve_bytes_dropout", d, &r)) return 0;
  return reserve_layout(r, r.L > 1).total;
}

int flb200_rnn_forward_dropout(const flb200_rnn_desc* d, const void* x, const void* hx,
                               const void* cx, const void* w, const void* mask, float p, void* y,
                               void* hy, void* cy, void* reserve, size_t reserve_bytes,
                               void* workspace, size_t workspace_bytes, void* stream) {
  FLB200_REQUIRE(mask || flb200_rnn_dropout_mask_elements(d) == 0,
                 "rnn_forward_dropout: null mask");
  return rnn_forward_impl(d, x, hx, cx, w, mask, p, y, hy, cy, reserve, reserve_bytes, workspace,
                          workspace_bytes, stream);
}

int flb200_rnn_backward_dropout(const flb200_rnn_desc* d, const void* x, const void* hx,
                                const void* cx, const void* w, const void* mask, float p,
                                const void* y, const void* grad_y, const void* grad_hy,
                                const void* grad_cy, void* grad_x, void* grad_hx, void* grad_cx,
                                void* grad_w, const void* reserve, size_t reserve_bytes,
                                void* workspace, size_t workspace_bytes, void* stream) {
  FLB200_REQUIRE(mask || flb200_rnn_dropout_mask_elements(d) == 0,
                 "rnn_backward_dropout: null mask");
  return rnn_backward_impl(d, x, hx, cx, w, mask, p, y, grad_y, grad_hy, grad_cy, grad_x, grad_hx,
                           grad_cx, grad_w, reserve, reserve_bytes, workspace, workspace_bytes,
                           stream);
}

// ---- self-test of the bounded waits -------------------------------------------------------
size_t flb200_selftest_bounded_wait_workspace_bytes(void) {
  // W_hh [4H][H], gates [T][B][4H], cells and output [T][B][H], h0 / c0 [B][H], the counter
  const size_t H = 256, B = 4, T = 3;
  return (4 * H * H + T * B * 4 * H + 2 * T * B * H + 2 * B * H) * 4 + 256;
}

int flb200_selftest_bounded_wait(double budget_ms, void* workspace, size_t workspace_bytes,
                                 void* stream) {
  const int H = 256, B = 4, T = 3;
  FLB200_REQUIRE(workspace && workspace_bytes >= flb200_selftest_bounded_wait_workspace_bytes(),
                 "selftest_bounded_wait: workspace too small");
  FLB200_REQUIRE(budget_ms > 0.0 && budget_ms <= 1000.0, "selftest_bounded_wait: budget in (0, 1000] ms");
  if (!lstm_sequence_supported(FLB200_MATH_TF32, B, H))
    return fail(FLB200_UNSUPPORTED, "selftest_bounded_wait: the persistent kernel cannot run here");
  cudaStream_t st = as_stream(stream);
  FLB200_CUDA_CHECK(cudaMemsetAsync(workspace, 0, flb200_selftest_bounded_wait_workspace_bytes(), st));
  float* w = static_cast<float*>(workspace);
  float* gates = w + 4 * H * H;
  float* cells = gates + T * B * 4 * H;
  float* out = cells + T * B * H;
  float* h0 = out + T * B * H;
  float* c0 = h0 + B * H;
  unsigned* sync = reinterpret_cast<unsigned*>(c0 + B * H);
  CUtensorMap map;
  if (int rc = lstm_step_weight_map(&map, w, H)) return rc;
  // CTA 0 never arrives at the grid barrier: every CTA's wait for step 1 runs out after
  // budget_ms (at ~2 GHz), raises the status flag and the kernel still ends by itself
  return lstm_sequence_forward(map, gates, cells, out, H, h0, c0, sync, T, B, H, 0,
                               (long long)(budget_ms * 2.0e6), 0, st);
}

}  // extern "C"
