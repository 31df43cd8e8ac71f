// matmul on strided row-major views and the three GEMMs of fl::linear's
// gradFunc (flashlight/fl/autograd/Functions.cpp:827-946, 1255-1309;
// TensorBackend::matmul, flashlight/fl/tensor/TensorBackend.h:213-217).
// STRICT mode runs the fp32-FMA kernel of simt_gemm.cuh; TF32 mode hands the
// shapes the tensor-core kernel covers to tc_gemm (tcgen05, fp32 accumulate in
// tensor memory) and everything else to the fp32 kernel.
#include "simt_gemm.cuh"
#include "tc_gemm.cuh"

namespace flb200 {
namespace {

int matmul_simt(const flb200_matmul_desc* d, const void* a, const void* b, void* c, void* ws,
                size_t ws_bytes, cudaStream_t st) {
  StridedEpilogue ep{static_cast<float*>(c), d->c_row, d->c_col, d->c_batch, d->alpha, d->beta};
  const bool a_k = d->a_col == 1 || d->a_row != 1;  // read A along k unless m is the unit stride
  const bool b_k = d->b_row == 1 && d->b_col != 1;  // read B along k only when k is the unit stride
  const float* ap = static_cast<const float*>(a);
  const float* bp = static_cast<const float*>(b);
  // Operand B is indexed (row = n, k): row stride is b_col, k stride is b_row.
#define FLB200_MM(AK, BK_)                                                                     \
  return launch_simt_gemm("matmul", StridedLoader<AK>{ap, d->a_row, d->a_col, d->a_batch, (int)d->m}, \
                          StridedLoader<BK_>{bp, d->b_col, d->b_row, d->b_batch, (int)d->n}, ep, \
                          d->m, d->n, d->k, d->batch, ws, ws_bytes, st)
  if (a_k && b_k) FLB200_MM(true, true);
  if (a_k && !b_k) FLB200_MM(true, false);
  if (!a_k && b_k) FLB200_MM(false, true);
  FLB200_MM(false, false);
#undef FLB200_MM
}

int check_desc(const flb200_matmul_desc* d, const void* a, const void* b, const void* c) {
  FLB200_REQUIRE(d, "matmul: null descriptor");
  FLB200_REQUIRE(d->m >= 0 && d->n >= 0 && d->k >= 0 && d->batch >= 1, "matmul: negative extent");
  FLB200_REQUIRE(d->dtype == FLB200_F32 || d->dtype == FLB200_BF16,
                 "matmul: f32 and bf16 are built (dtype %d)", d->dtype);
  FLB200_REQUIRE(d->math_mode >= FLB200_MATH_STRICT_F32 && d->math_mode <= FLB200_MATH_F32X3,
                 "matmul: unknown math mode %d", d->math_mode);
  FLB200_REQUIRE((a && b && c) || d->m == 0 || d->n == 0, "matmul: null matrix");
  return FLB200_OK;
}

int run_matmul(const flb200_matmul_desc* d, const void* a, const void* b, void* c, void* ws,
               size_t ws_bytes, void* stream) {
  if (int st = check_desc(d, a, b, c)) return st;
  if (d->m == 0 || d->n == 0) return FLB200_OK;
  cudaStream_t st = as_stream(stream);
  if (d->dtype == FLB200_BF16) {
    // bf16 operands, fp32 accumulation, bf16 result: tensor cores only (no fp32-FMA kernel
    // reads bf16), whatever the math mode says
    if (!tc_gemm_supported(d, a, b, c))
      return fail(FLB200_UNSUPPORTED,
                  "matmul: bf16 needs the tensor-core path (sm_100, 16-byte aligned operands "
                  "with one unit stride each)");
    return tc_gemm_run(d, a, b, c, ws, ws_bytes, st);
  }
  tc::X3Scope x3(d->math_mode == FLB200_MATH_F32X3);
  if (d->math_mode != FLB200_MATH_STRICT_F32 && tc_gemm_supported(d, a, b, c))
    return tc_gemm_run(d, a, b, c, ws, ws_bytes, st);
  return matmul_simt(d, a, b, c, ws, ws_bytes, st);
}

}  // namespace
}  // namespace flb200

using namespace flb200;

extern "C" {

size_t flb200_matmul_workspace_bytes(const flb200_matmul_desc* d) {
  if (!d || d->m <= 0 || d->n <= 0 || d->batch <= 0) return 0;
  size_t need = plan_simt(d->m, d->n, d->k, d->batch).workspace_bytes;
  const size_t tc = tc_gemm_workspace_bytes(d);
  return need > tc ? need : tc;
}

int flb200_matmul(const flb200_matmul_desc* d, const void* a, const void* b, void* c,
                  void* workspace, size_t workspace_bytes, void* stream) {
  return run_matmul(d, a, b, c, workspace, workspace_bytes, stream);
}

// which: 0 forward, 1 backward-input, 2 backward-weight.  A NULL / short
// workspace is accepted by the three calls: the contraction then runs unsplit.
size_t flb200_linear_workspace_bytes(int64_t O, int64_t I, int64_t cols, int which) {
  flb200_matmul_desc d = {};
  d.batch = 1;
  if (which == 0) { d.m = cols; d.n = O; d.k = I; }
  else if (which == 1) { d.m = cols; d.n = I; d.k = O; }
  else { d.m = I; d.n = O; d.k = cols; }
  return flb200_matmul_workspace_bytes(&d);
}

// fl layout (column-major): weight (o,i) at o + i*O; x (i,col) at i + col*I;
// y (o,col) at o + col*O.  Row-major GEMM views used below:
//   forward          Y[col][o]  = sum_i X[col][i] * Wt[i][o]      (+ bias[o])
//   backward input   dX[col][i] = sum_o dY[col][o] * W(o,i)
//   backward weight  dWt[i][o]  = sum_col X[col][i] * dY[col][o]
int flb200_linear_forward(int64_t O, int64_t I, int64_t cols, const void* weight, const void* x,
                          const void* bias, void* y, int math_mode, void* workspace,
                          size_t workspace_bytes, void* stream) {
  flb200_matmul_desc d = {};
  d.m = cols; d.n = O; d.k = I; d.batch = 1;
  d.a_row = I; d.a_col = 1;
  d.b_row = O; d.b_col = 1;
  d.c_row = O; d.c_col = 1;
  d.alpha = 1.f; d.beta = 0.f;
  d.dtype = FLB200_F32; d.math_mode = math_mode;
  if (int st = run_matmul(&d, x, weight, y, workspace, workspace_bytes, stream)) return st;
  if (bias) return flb200_channel_bias_add(y, static_cast<const float*>(bias), y, cols, O, 1,
                                           FLB200_F32, stream);
  return FLB200_OK;
}

int flb200_linear_bias_act_forward(int64_t O, int64_t I, int64_t cols, const void* weight,
                                   const void* x, const float* bias, void* y, void* pre, int act,
                                   int dtype, int math_mode, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  FLB200_REQUIRE(act == FLB200_ACT_NONE || act == FLB200_ACT_GELU,
                 "linear_bias_act_forward: unknown activation %d", act);
  FLB200_REQUIRE(act != FLB200_ACT_NONE || pre == nullptr,
                 "linear_bias_act_forward: a pre-activation copy needs an activation");
  flb200_matmul_desc d = {};
  d.m = cols; d.n = O; d.k = I; d.batch = 1;
  d.a_row = I; d.a_col = 1;
  d.b_row = O; d.b_col = 1;
  d.c_row = O; d.c_col = 1;
  d.alpha = 1.f; d.beta = 0.f;
  d.dtype = dtype; d.math_mode = math_mode;
  if (int st = check_desc(&d, x, weight, y)) return st;
  if (cols == 0 || O == 0) return FLB200_OK;
  if ((dtype != FLB200_BF16 && math_mode == FLB200_MATH_STRICT_F32) ||
      !tc_gemm_supported(&d, x, weight, y) || (bias && !aligned16(bias)))
    return fail(FLB200_UNSUPPORTED,
                "linear_bias_act_forward: needs the tensor-core path (run linear, bias and "
                "activation one by one)");
  tc::X3Scope x3(dtype == FLB200_F32 && math_mode == FLB200_MATH_F32X3);
  return tc_gemm_run(&d, x, weight, y, workspace, workspace_bytes, as_stream(stream), bias, act,
                     pre);
}

int flb200_linear_backward_input(int64_t O, int64_t I, int64_t cols, const void* weight,
                                 const void* grad_y, void* grad_x, int math_mode, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  flb200_matmul_desc d = {};
  d.m = cols; d.n = I; d.k = O; d.batch = 1;
  d.a_row = O; d.a_col = 1;          // dY[col][o]
  d.b_row = 1; d.b_col = O;          // B(k=o, n=i) = W(o,i) at o + i*O
  d.c_row = I; d.c_col = 1;
  d.alpha = 1.f; d.beta = 0.f;
  d.dtype = FLB200_F32; d.math_mode = math_mode;
  return run_matmul(&d, grad_y, weight, grad_x, workspace, workspace_bytes, stream);
}

int flb200_linear_backward_weight(int64_t O, int64_t I, int64_t cols, const void* grad_y,
                                  const void* x, void* grad_w, int math_mode, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  flb200_matmul_desc d = {};
  d.m = I; d.n = O; d.k = cols; d.batch = 1;
  d.a_row = 1; d.a_col = I;          // A(m=i, k=col) = X[col][i]
  d.b_row = O; d.b_col = 1;          // B(k=col, n=o) = dY[col][o]
  d.c_row = O; d.c_col = 1;          // dWt[i][o]
  d.alpha = 1.f; d.beta = 0.f;
  d.dtype = FLB200_F32; d.math_mode = math_mode;
  return run_matmul(&d, x, grad_y, grad_w, workspace, workspace_bytes, stream);
}

}  // extern "C"
