/*
 * flb200 — C ABI of the B200 (sm_100a) autograd-backward kernel library.
 *
 * Every entry point takes raw DEVICE pointers, extents in Flashlight order
 * (column-major: dim 0 is the fastest; an fl tensor [W,H,C,N] is the same bytes
 * as a row-major NCHW array) and a CUDA stream (passed as void* so that this
 * header needs no CUDA include).  Every entry point returns an int status
 * (FLB200_OK == 0) and never throws, exits or allocates device memory: scratch
 * is passed in by the caller, sized by the matching *_workspace_bytes query.
 * The last error text of the calling thread is kept in flb200_last_error().
 *
 * Each declaration names the Flashlight interface it stands behind
 * (path within the flashlight project : line).
 */
#ifndef FLB200_H_
#define FLB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- status */
enum {
  FLB200_OK = 0,
  FLB200_INVALID_ARG = 1,     /* maps to std::invalid_argument on the C++ side */
  FLB200_UNSUPPORTED = 2,     /* dtype / mode not built */
  FLB200_LAUNCH_FAILURE = 3,  /* a CUDA call returned an error */
  FLB200_TIMEOUT = 4,         /* a bounded device-side wait ran out */
  FLB200_WORKSPACE_TOO_SMALL = 5
};

/* fl::dtype subset (flashlight/fl/tensor/Types.h:17-30) + bf16 */
enum { FLB200_F32 = 0, FLB200_F16 = 1, FLB200_BF16 = 2 };

/* fl::PoolingMode (flashlight/fl/autograd/tensor/AutogradOps.h) */
enum { FLB200_POOL_MAX = 0, FLB200_POOL_AVG_INCLUDE_PAD = 1, FLB200_POOL_AVG_EXCLUDE_PAD = 2 };

/* fl::RnnMode (flashlight/fl/autograd/tensor/AutogradOps.h) */
enum { FLB200_RNN_RELU = 0, FLB200_RNN_TANH = 1, FLB200_RNN_LSTM = 2, FLB200_RNN_GRU = 3 };

/* Arithmetic mode of the dense contractions; the counterpart of
 * fl::KernelMode {F32, F32_ALLOW_CONVERSION, F16} (flashlight/fl/common/Defines.h:100).
 * STRICT = fp32 FMA everywhere (meets 1e-4 parity); TF32 = tcgen05 kind::tf32
 * with fp32 accumulation in tensor memory where a tensor-core kernel exists for
 * the shape, fp32 FMA otherwise. */
/* STRICT_F32: fp32 FMA kernels.  TF32: tensor cores, operands read with a 10-bit mantissa.
 * F32X3: tensor cores with every operand split into a TF32-exact high part and the remainder
 * and three passes per product (a_lo*b_hi + a_hi*b_lo + a_hi*b_hi): products carry about 21
 * mantissa bits, fp32 accumulation in tensor memory: errors of a few 1e-6 of the result's scale
 * (TF32: ~1e-3), at about two thirds of the TF32 speed on a ResNet-50 step. */
enum { FLB200_MATH_STRICT_F32 = 0, FLB200_MATH_TF32 = 1, FLB200_MATH_F32X3 = 2 };

/* Memory layout of image tensors.  NCHW is fl's own: an fl tensor [W,H,C,N] (column-major) read
 * row-major.  NHWC ("channels-last") is the same logical tensor stored as fl [C,W,H,N]: the
 * layout the tensor-core convolutions read natively (a filter tap then shifts whole pixels and
 * the contiguous index is the channel), so a network that keeps its activations channels-last
 * between operators pays for no layout copy at all.  Filters, biases and statistics keep the
 * reference layout in every mode.  NCHW_IN_NHWC_OUT is for a network's first convolution: x
 * (and nothing else) arrives in fl's order, y / grad_y are channels-last. */
enum { FLB200_LAYOUT_NCHW = 0, FLB200_LAYOUT_NCHW_IN_NHWC_OUT = 2, FLB200_LAYOUT_NHWC = 3 };

/* fl::ReduceMode (flashlight/fl/autograd/Functions.h) */
enum { FLB200_REDUCE_NONE = 0, FLB200_REDUCE_MEAN = 1, FLB200_REDUCE_SUM = 2 };

int flb200_abi_version(void);
const char* flb200_status_string(int status);
const char* flb200_last_error(void);
/* Number of kernels this library has launched from the calling process so far. */
long long flb200_kernel_launches(void);
/* 1 when the tcgen05 kernels can run: the current device is sm_100 and the driver exports
 * cuTensorMapEncodeTiled. */
int flb200_has_tensor_core_path(void);
/* Number of tcgen05 contraction kernels launched so far (subset of flb200_kernel_launches). */
long long flb200_tc_kernel_launches(void);
/* Every wait inside a tensor-core kernel is bounded; one that runs out raises a device flag
 * and the kernel drains and returns.  This call synchronises the stream, reads and clears
 * the flag and returns FLB200_TIMEOUT if it was set. */
int flb200_tc_poll_status(void* stream);

/* ------------------------------------------------- conv2d (a3, a4, a8) */
/* Geometry of one fl::conv2d call.  x [W,H,C,N], w [kW,kH,C/groups,Cout],
 * bias [1,1,Cout,1] or absent, y [Wo,Ho,Cout,N] with
 * Wo = 1 + (W + 2 px - (1 + (kW-1) dx)) / sx  (same for H)
 * — flashlight/fl/autograd/tensor/backend/onednn/Conv2D.cpp:179-188. */
typedef struct flb200_conv2d_desc {
  int32_t W, H, C, N;
  int32_t kW, kH, Cout;
  int32_t sx, sy, px, py, dx, dy, groups;
  int32_t dtype;      /* FLB200_F32; FLB200_F16 / FLB200_BF16: every tensor of the call in that
                       * type, fp32 accumulation (operands are widened into the workspace) */
  int32_t math_mode;  /* FLB200_MATH_* */
  int32_t layout;     /* FLB200_LAYOUT_* of x / grad_x and y / grad_y (0 = fl's own) */
} flb200_conv2d_desc;

int flb200_conv2d_output_dims(const flb200_conv2d_desc* d, int32_t* Wo, int32_t* Ho);

/* which: 0 forward, 1 backward-data, 2 backward-filter(+bias).
 * Alignment: any 4-byte aligned tensor and workspace is accepted.  The tensor-core modes
 * (TF32, F32X3) only engage when x / w / y (grad_y, grad_x, grad_w) and the workspace start on
 * 16-byte boundaries (TMA and 16-byte vector accesses); a call with an offset view or an odd
 * workspace runs on the fp32 kernels instead, with fp32 results. */
size_t flb200_conv2d_workspace_bytes(const flb200_conv2d_desc* d, int which);

/* fl::AutogradExtension::conv2d — flashlight/fl/autograd/tensor/AutogradExtension.h:58-69.
 * bias may be NULL. */
int flb200_conv2d_forward(const flb200_conv2d_desc* d, const void* x, const void* w,
                          const void* bias, void* y, void* workspace,
                          size_t workspace_bytes, void* stream);

/* fl::AutogradExtension::conv2dBackwardData — AutogradExtension.h:110-122.
 * grad_x [W,H,C,N] is fully overwritten. */
int flb200_conv2d_backward_data(const flb200_conv2d_desc* d, const void* grad_y,
                                const void* w, void* grad_x, void* workspace,
                                size_t workspace_bytes, void* stream);

/* fl::AutogradExtension::conv2dBackwardFilterBias — AutogradExtension.h:124-138.
 * grad_w [kW,kH,C/groups,Cout] is fully overwritten; grad_bias [Cout] may be
 * NULL (the reference skips it when bias is empty:
 * flashlight/fl/autograd/tensor/backend/cudnn/Conv2D.cpp:753). */
int flb200_conv2d_backward_filter_bias(const flb200_conv2d_desc* d, const void* grad_y,
                                       const void* x, void* grad_w, void* grad_bias,
                                       void* workspace, size_t workspace_bytes,
                                       void* stream);

/* Keeping layout copies between the calls of one convolution.  The tensor-core routes read
 * x and grad_y from channels-last copies; a caller that passes the same cache to the forward
 * call and to both backward calls of one fl::conv2d lets backward-filter reuse the copy of x
 * made by forward and the copy of grad_y made by backward-data instead of making them again.
 * The reference hands every backend the same kind of per-call-site state:
 * std::shared_ptr<detail::AutogradPayload> in flashlight/fl/autograd/tensor/
 * AutogradExtension.h:58-69, 110-138 (created once per call site in
 * flashlight/fl/autograd/Functions.cpp:1341).  The caller owns both buffers (sizes from
 * flb200_conv2d_cache_bytes; a NULL or short buffer is simply not used) and the flags:
 *   x_cl_valid   set by forward (and by backward-filter when it had to make the copy);
 *                clear it when x changes.
 *   gy_cl_valid  set by backward-data, consumed and cleared by backward-filter, which
 *                therefore must be called with the same grad_y as that backward-data call.
 * Routes that make no such copy leave the cache untouched. */
typedef struct flb200_conv2d_cache {
  void* x_cl;
  size_t x_cl_bytes;
  int32_t x_cl_valid;
  void* gy_cl;
  size_t gy_cl_bytes;
  int32_t gy_cl_valid;
} flb200_conv2d_cache;

/* which: 0 the copy of x, 1 the copy of grad_y; 0 bytes when the route keeps none. */
size_t flb200_conv2d_cache_bytes(const flb200_conv2d_desc* d, int which);

/* The three calls above with a cache (may be NULL: then they are the calls above). */
int flb200_conv2d_forward_cached(const flb200_conv2d_desc* d, const void* x, const void* w,
                                 const void* bias, void* y, void* workspace,
                                 size_t workspace_bytes, flb200_conv2d_cache* cache,
                                 void* stream);
int flb200_conv2d_backward_data_cached(const flb200_conv2d_desc* d, const void* grad_y,
                                       const void* w, void* grad_x, void* workspace,
                                       size_t workspace_bytes, flb200_conv2d_cache* cache,
                                       void* stream);
int flb200_conv2d_backward_filter_bias_cached(const flb200_conv2d_desc* d, const void* grad_y,
                                              const void* x, void* grad_w, void* grad_bias,
                                              void* workspace, size_t workspace_bytes,
                                              flb200_conv2d_cache* cache, void* stream);

/* ------------------------------------------------------- pool2d (a5, a8) */
/* Forward convolution that also takes the batch-norm statistics of its output while the
 * accumulators are stored — the conv + batch-norm pairing of
 * flashlight/pkg/vision/models/Resnet.cpp:67-121: `stats` receives a matrix of `groups` rows of
 * 2 * Cout floats (flb200_conv2d_stats_bytes gives its size and the row count) whose column sums
 * are, per output channel, the sum of y ([0, Cout)) and the sum of y^2 ([Cout, 2 Cout)) — one row
 * per 32 output pixels, written without atomics, so results do not depend on timing.
 * flb200_batchnorm_forward_from_stats reduces that small matrix instead of reading y again.
 * Tensor-core modes, fp32, channels-last output, Cout a multiple of 32; elsewhere
 * flb200_conv2d_stats_bytes returns 0.  The workspace is that of flb200_conv2d_forward. */
size_t flb200_conv2d_stats_bytes(const flb200_conv2d_desc* d, int64_t* groups);
int flb200_conv2d_forward_stats(const flb200_conv2d_desc* d, const void* x, const void* w,
                                const void* bias, void* y, float* stats, size_t stats_bytes,
                                void* workspace, size_t workspace_bytes,
                                flb200_conv2d_cache* cache, void* stream);

typedef struct flb200_pool2d_desc {
  int32_t W, H, C, N;
  int32_t wx, wy, sx, sy, px, py;
  int32_t mode;   /* FLB200_POOL_* */
  int32_t dtype;  /* FLB200_F32 / F16 / BF16 */
  int32_t layout; /* FLB200_LAYOUT_NCHW or FLB200_LAYOUT_NHWC (x, y, argmax and gradients alike) */
} flb200_pool2d_desc;

/* Wo = 1 + (W + 2 px - wx) / sx — flashlight/fl/autograd/tensor/backend/onednn/Pool2D.cpp:100-102 */
int flb200_pool2d_output_dims(const flb200_pool2d_desc* d, int32_t* Wo, int32_t* Ho);

/* fl::AutogradExtension::pool2d — AutogradExtension.h:71-80.
 * argmax (optional, MAX mode only): one byte per output element holding the
 * window position ky*wx+kx of the selected input; this is the payload that
 * backward consumes (the oneDNN backend keeps a workspace the same way:
 * backend/onednn/Pool2D.cpp:71-76).  Ties go to the first in-bounds element in
 * scan order (ky outer, kx inner); NaN propagates. */
int flb200_pool2d_forward(const flb200_pool2d_desc* d, const void* x, void* y,
                          uint8_t* argmax, void* stream);

/* fl::AutogradExtension::pool2dBackward — AutogradExtension.h:141-152.
 * argmax may be NULL: the selection is then recomputed from x (the cuDNN
 * backend also works from x and y: backend/cudnn/Pool2D.cpp:73-122). x may be
 * NULL when argmax is given or mode is an average. */
int flb200_pool2d_backward(const flb200_pool2d_desc* d, const void* grad_y,
                           const void* x, const uint8_t* argmax, void* grad_x,
                           void* stream);

/* ---------------------------------------------------- batchnorm (a6, a8) */
/* Geometry after fl's axes rule (backend/cudnn/BatchNorm.cpp:22-75): the input
 * is [outer][channels][inner] row-major; statistics are per channel over
 * outer*inner elements.  Per-activation mode (min axis 0) is inner == 1. */
typedef struct flb200_batchnorm_desc {
  int64_t outer, channels, inner;
  int32_t dtype;  /* of x, y and their gradients: FLB200_F32 / F16 / BF16; weight, bias, the
                   * statistics and their gradients are fp32 whatever it is (the reference's
                   * f16 batch-norm, backend/cudnn/BatchNorm.cpp:92-95) */
} flb200_batchnorm_desc;

/* Turns (shape, axes) into the descriptor; returns FLB200_INVALID_ARG for axes
 * that are out of range or not contiguous, like the reference. */
int flb200_batchnorm_geometry(const int64_t* shape, int ndim, const int32_t* axes,
                              int naxes, flb200_batchnorm_desc* out);

size_t flb200_batchnorm_workspace_bytes(const flb200_batchnorm_desc* d);

/* fl::AutogradExtension::batchnorm — AutogradExtension.h:82-94.
 * train != 0: batch statistics; save_mean[c] = mean, save_invstd[c] =
 * 1/sqrt(biased var + eps) (what cuDNN's saveVar slot holds); running stats
 * (optional) updated as r = (1-momentum) r + momentum * batch (unbiased var).
 * train == 0: normalises with running_mean / running_var.
 * weight / bias may be NULL (ones / zeros). */
int flb200_batchnorm_forward(const flb200_batchnorm_desc* d, const void* x,
                             const float* weight, const float* bias,
                             float* running_mean, float* running_var,
                             float* save_mean, float* save_invstd, int train,
                             double momentum, double epsilon, void* y,
                             void* workspace, size_t workspace_bytes, void* stream);

/* fl::AutogradExtension::batchnormBackward — AutogradExtension.h:155-164.
 * Always writes grad_x, grad_weight, grad_bias. */
int flb200_batchnorm_backward(const flb200_batchnorm_desc* d, const void* grad_y,
                              const void* x, const float* weight,
                              const float* save_mean, const float* save_invstd,
                              void* grad_x, float* grad_weight, float* grad_bias,
                              void* workspace, size_t workspace_bytes, void* stream);

/* relu(batchnorm(x)) as one operator (the conv -> BatchNorm -> ReLU chain of
 * flashlight/pkg/vision/models/Resnet.cpp:67-121): the apply pass clamps at zero, and the
 * backward passes rebuild the relu predicate from x (the normalised value is recomputed with
 * the very expression forward used), so the relu costs no pass of its own in either
 * direction and nothing extra is saved.  Arguments as flb200_batchnorm_forward / _backward;
 * backward also takes the bias (NULL = zeros) and grad_y is the gradient of the relu output. */
int flb200_batchnorm_relu_forward(const flb200_batchnorm_desc* d, const void* x,
                                  const float* weight, const float* bias,
                                  float* running_mean, float* running_var,
                                  float* save_mean, float* save_invstd, int train,
                                  double momentum, double epsilon, void* y,
                                  void* workspace, size_t workspace_bytes, void* stream);
/* y = relu(batchnorm(x) + addend): the last BatchNorm of a residual block fused with the block's
 * join (Resnet.cpp:67-121), plus the bit mask of the predicate for
 * flb200_batchnorm_add_relu_backward: `mask` needs n bytes (channel rows of a multiple of 8
 * elements use one byte per 8 elements, in the layout of flb200_relu_forward_mask; of a multiple
 * of 4, one byte per 4; other rows one byte per element).  f32, 16-byte aligned, spatial layout
 * (inner > 1); otherwise FLB200_UNSUPPORTED (run the two operators separately). */
int flb200_batchnorm_add_relu_forward(const flb200_batchnorm_desc* d, const void* x,
                                      const void* addend, const float* weight,
                                      const float* bias, float* running_mean,
                                      float* running_var, float* save_mean,
                                      float* save_invstd, int train, double momentum,
                                      double epsilon, void* y, uint8_t* mask, void* workspace,
                                      size_t workspace_bytes, void* stream);
/* Training-mode batch-norm forward whose statistics come from the matrix a convolution wrote for
 * x (flb200_conv2d_forward_stats: `groups` rows of 2 * channels floats) instead of a pass over x.
 * addend != NULL: the relu(batchnorm(x) + addend) form (mask required); else relu != 0:
 * relu(batchnorm(x)); else the plain operator.  Everything else as in the functions above;
 * workspace: flb200_batchnorm_from_stats_workspace_bytes. */
size_t flb200_batchnorm_from_stats_workspace_bytes(const flb200_batchnorm_desc* d, int64_t groups);
int flb200_batchnorm_forward_from_stats(const flb200_batchnorm_desc* d, const void* x,
                                        const void* addend, int relu, const float* stats,
                                        int64_t groups, const float* weight, const float* bias,
                                        float* running_mean, float* running_var,
                                        float* save_mean, float* save_invstd, double momentum,
                                        double epsilon, void* y, uint8_t* mask, void* workspace,
                                        size_t workspace_bytes, void* stream);
/* Gradient of flb200_batchnorm_add_relu_forward given the gradients of its output's consumers
 * (grad_y_b may be NULL): grad_sum = mask ? grad_y_a + grad_y_b : 0 is written (the addend's
 * gradient) while the first batch-norm pass reduces it, then grad_x / grad_weight / grad_bias
 * as flb200_batchnorm_backward.  Same shape restrictions as the forward call. */
int flb200_batchnorm_add_relu_backward(const flb200_batchnorm_desc* d, const uint8_t* mask,
                                       const void* grad_y_a, const void* grad_y_b,
                                       const void* x, const float* weight,
                                       const float* save_mean, const float* save_invstd,
                                       void* grad_sum, void* grad_x, float* grad_weight,
                                       float* grad_bias, void* workspace,
                                       size_t workspace_bytes, void* stream);
int flb200_batchnorm_relu_backward(const flb200_batchnorm_desc* d, const void* grad_y,
                                   const void* x, const float* weight, const float* bias,
                                   const float* save_mean, const float* save_invstd,
                                   void* grad_x, float* grad_weight, float* grad_bias,
                                   void* workspace, size_t workspace_bytes, void* stream);

/* --------------------------------------------------------- matmul (a9) */
/* C[m,n] = alpha * sum_k A(m,k) B(k,n) + beta * C[m,n] on ROW-MAJOR views with
 * explicit element strides, so that every fl::matmul / matmulTN / matmulNT
 * (flashlight/fl/autograd/Functions.cpp:827-946; TensorBackend::matmul,
 * flashlight/fl/tensor/TensorBackend.h:213-217) is one call.  batch > 1 walks
 * the batch strides (0 = broadcast). */
typedef struct flb200_matmul_desc {
  int64_t m, n, k, batch;
  int64_t a_row, a_col, a_batch; /* A(i,kk) at a[i*a_row + kk*a_col + b*a_batch] */
  int64_t b_row, b_col, b_batch; /* B(kk,j) at b[kk*b_row + j*b_col + b*b_batch] */
  int64_t c_row, c_col, c_batch;
  float alpha, beta;
  int32_t dtype;      /* FLB200_F32, or FLB200_BF16: bf16 A, B and C, fp32 accumulation on the
                       * tensor cores (needs 16-byte aligned operands with one unit stride each) */
  int32_t math_mode;  /* FLB200_MATH_* */
} flb200_matmul_desc;

size_t flb200_matmul_workspace_bytes(const flb200_matmul_desc* d);
int flb200_matmul(const flb200_matmul_desc* d, const void* a, const void* b, void* c,
                  void* workspace, size_t workspace_bytes, void* stream);

/* fl::linear gradFunc pieces (Functions.cpp:1255-1309) on fl-layout buffers:
 * weight [O,I], x [I,cols], y / grad_y [O,cols] (all column-major).  which:
 * 0 forward, 1 backward-input, 2 backward-weight.  workspace may be NULL (the
 * contraction then runs without split-K). */
size_t flb200_linear_workspace_bytes(int64_t O, int64_t I, int64_t cols, int which);
int flb200_linear_forward(int64_t O, int64_t I, int64_t cols, const void* weight,
                          const void* x, const void* bias, void* y, int math_mode,
                          void* workspace, size_t workspace_bytes, void* stream);
/* Linear + bias + activation in one kernel (Linear + bias + GELU of
 * flashlight/pkg/vision/nn/VisionTransformer.cpp:101-110 and of the Transformer feed-forward
 * block): y = act(x W + bias) with bias (fp32, may be NULL) and the activation applied where the
 * accumulators are stored; `pre` (may be NULL) also receives x W + bias, which the activation's
 * gradient needs.  dtype FLB200_F32 (tensor-core math modes) or FLB200_BF16; O a multiple of 32.
 * FLB200_UNSUPPORTED where the tensor-core path does not cover the call: run flb200_linear_forward
 * / flb200_matmul, the bias and the activation one by one. */
enum { FLB200_ACT_NONE = 0, FLB200_ACT_GELU = 1 };
int flb200_linear_bias_act_forward(int64_t O, int64_t I, int64_t cols, const void* weight,
                                   const void* x, const float* bias, void* y, void* pre, int act,
                                   int dtype, int math_mode, void* workspace,
                                   size_t workspace_bytes, void* stream);
int flb200_linear_backward_input(int64_t O, int64_t I, int64_t cols, const void* weight,
                                 const void* grad_y, void* grad_x, int math_mode,
                                 void* workspace, size_t workspace_bytes, void* stream);
int flb200_linear_backward_weight(int64_t O, int64_t I, int64_t cols, const void* grad_y,
                                  const void* x, void* grad_w, int math_mode,
                                  void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------- bandwidth-bound gradFuncs (a10-a12) */
/* out[c] = sum over outer, inner of in[o][c][i]  — conv bias gradient
 * (backend/cudnn/Conv2D.cpp:737) with (N, Cout, Ho*Wo), and detail::sumAs for a
 * linear bias (Functions.cpp:44-58, 1285-1289) with (cols, O, 1). */
size_t flb200_channel_sum_workspace_bytes(int64_t outer, int64_t channels, int64_t inner);
int flb200_channel_sum(const void* in, float* out, int64_t outer, int64_t channels,
                       int64_t inner, int dtype, void* workspace,
                       size_t workspace_bytes, void* stream);

/* flb200_channel_sum for callers that cannot allocate device memory at the time of the call
 * (code running inside a framework's memory-manager callback or out-of-memory handler, hosts
 * that hand out their whole device budget at start-up).  It has no counterpart in the reference.
 * The partial sums live in a 1 MiB array built into the library (held by every GPU that loads
 * it, until the process exits); shapes that need more are refused with FLB200_INVALID_ARG — use
 * flb200_channel_sum with your own scratch for those.  Calls neither cudaMalloc nor cudaFree.
 * The first call on a device looks up the array's device address (thread-safe); that lookup can
 * make the CUDA runtime load the library's device code, which may allocate.  So make one warm-up
 * call per device at start-up, before any stream capture begins and before the situation in
 * which allocating is forbidden: from the second call on nothing is allocated.  All calls share
 * the one array: two calls that may overlap on the GPU (different streams, no ordering between
 * them) race and give wrong sums. */
int flb200_channel_sum_static_scratch(const void* in, float* out, int64_t outer,
                                      int64_t channels, int64_t inner, int dtype, void* stream);

/* The affine part of fl::LayerNorm (flashlight/fl/nn/modules/LayerNorm.cpp:112-128: the
 * normalised tensor times tileAs(weight) plus tileAs(bias)) on rows of `features` contiguous
 * elements, as one kernel:  y[r][f] = xhat[r][f] * weight[f] + bias[f]  (bias may be NULL).
 * weight / bias are fp32 whatever the activations' dtype (fp32 master parameters are used as
 * they are).  In place allowed. */
int flb200_layernorm_affine_forward(const void* xhat, const float* weight, const float* bias,
                                    void* y, int64_t rows, int64_t features, int dtype,
                                    void* stream);
/* Its gradient chain (the tileAs / sumAs products of Functions.cpp:27-58, 537-566) in two
 * kernels: grad_weight[f] = sum_r grad_y * xhat and grad_bias[f] = sum_r grad_y from one pass
 * over both tensors (fp32, either may be NULL), grad_xhat = grad_y * weight (may be NULL). */
size_t flb200_layernorm_affine_workspace_bytes(int64_t rows, int64_t features);
int flb200_layernorm_affine_backward(const void* grad_y, const void* xhat, const float* weight,
                                     void* grad_xhat, float* grad_weight, float* grad_bias,
                                     int64_t rows, int64_t features, int dtype, void* workspace,
                                     size_t workspace_bytes, void* stream);

/* fl::LayerNorm over rows of `features` elements as one operator each way
 * (flashlight/fl/nn/modules/LayerNorm.cpp:66-128: batchnorm over the normalised axes, then
 * tileAs(weight) * x_hat + tileAs(bias)): forward reads x once and writes y = x_hat * weight +
 * bias and x_hat (kept for the gradient; NULL: not written) plus the rows' mean and inverse
 * standard deviation (fp32, either may be NULL); weight / bias fp32 or NULL; features <= 2048.
 * Backward: grad_x = invstd * (g - mean(g) - x_hat * mean(g * x_hat)) with g = grad_y * weight
 * from one pass over grad_y and x_hat, and grad_weight = sum_rows grad_y * x_hat, grad_bias =
 * sum_rows grad_y from a second one (any of the three outputs may be NULL). */
int flb200_layernorm_forward(const void* x, const float* weight, const float* bias, void* y,
                             void* xhat, float* mean, float* invstd, int64_t rows,
                             int64_t features, double epsilon, int dtype, void* stream);
size_t flb200_layernorm_backward_workspace_bytes(int64_t rows, int64_t features);
int flb200_layernorm_backward(const void* grad_y, const void* xhat, const float* weight,
                              const float* invstd, void* grad_x, float* grad_weight,
                              float* grad_bias, int64_t rows, int64_t features, int dtype,
                              void* workspace, size_t workspace_bytes, void* stream);

/* y[o][c][i] = x[o][c][i] + bias[c] (tile + add, Functions.cpp:1270-1275). In place allowed. */
int flb200_channel_bias_add(const void* x, const float* bias, void* y, int64_t outer,
                            int64_t channels, int64_t inner, int dtype, void* stream);

/* relu with the predicate kept as one bit per element instead of a tensor: the reference's
 * gradFunc multiplies dy by (result > 0) and keeps `result` alive for that
 * (Functions.cpp:329-338, 1787-1789); here forward also writes mask[i / 8] bit (i % 8) = x[i] > 0
 * (ceil(n / 8) bytes, caller-owned) and backward reads dy and the mask only.  f32, 16-byte
 * aligned tensors. */
int flb200_relu_forward_mask(const void* x, void* y, uint8_t* mask, int64_t n, int dtype,
                             void* stream);
int flb200_relu_backward_mask(const uint8_t* mask, const void* grad_y, void* grad_x, int64_t n,
                              int dtype, void* stream);
/* The residual join of a bottleneck block, relu(out + shortcut)
 * (flashlight/pkg/vision/models/Resnet.cpp:67-121: operator+ then ReLU), in one pass:
 * y = max(a + b, 0) and the mask of (a + b) > 0; 12.1 bytes per element instead of 20.
 * Its gradient is the same for both addends: flb200_relu_backward_mask, or, when the output
 * had two consumers, flb200_relu_backward_mask_sum, which adds their two gradients on the fly
 * (what Variable::addGrad, Variable.cpp:196-211, does with a whole-tensor addition):
 * grad_x = mask ? grad_y_a + grad_y_b : 0. */
int flb200_add_relu_forward_mask(const void* a, const void* b, void* y, uint8_t* mask, int64_t n,
                                 int dtype, void* stream);
int flb200_relu_backward_mask_sum(const uint8_t* mask, const void* grad_y_a, const void* grad_y_b,
                                  void* grad_x, int64_t n, int dtype, void* stream);

/* relu = max(x, 0) (Functions.cpp:1787-1789); gradient (x > 0) * dy (Functions.cpp:329-338). */
int flb200_relu_forward(const void* x, void* y, int64_t n, int dtype, void* stream);
int flb200_relu_backward(const void* x, const void* grad_y, void* grad_x, int64_t n,
                         int dtype, void* stream);
/* gelu, tanh form with 0.7978845608 and 0.044715 (Functions.cpp:1791-1796). */
int flb200_gelu_forward(const void* x, void* y, int64_t n, int dtype, void* stream);
int flb200_gelu_backward(const void* x, const void* grad_y, void* grad_x, int64_t n,
                         int dtype, void* stream);
/* tanh: gradient (1 - y^2) * dy from the saved OUTPUT (Functions.cpp:454-463). */
int flb200_tanh_forward(const void* x, void* y, int64_t n, int dtype, void* stream);
int flb200_tanh_backward(const void* y, const void* grad_y, void* grad_x, int64_t n,
                         int dtype, void* stream);
/* dropout: out = in * mask * scale, scale = 1/(1-p); the same call serves the
 * forward (in = x) and the gradient (in = dy) (Functions.cpp:1777-1785). mask
 * holds 0/1 in the tensor's dtype, as the reference materialises it. */
int flb200_dropout_apply(const void* in, const void* mask, void* out, float scale,
                         int64_t n, int dtype, void* stream);
/* The Bernoulli mask the reference draws with `rand(shape) > ratio` (Functions.cpp:1779-1781)
 * for dropout: out[i] = 1 with probability keep_prob, else 0, from a counter-based generator
 * (Philox4x32-10): the values depend on (seed, offset, i) only, never on the launch shape;
 * element i uses counter offset + i / 4, so consecutive masks advance `offset` by (n + 3) / 4. */
int flb200_bernoulli_mask(void* out, int64_t n, float keep_prob, uint64_t seed, uint64_t offset,
                          int dtype, void* stream);
/* out = a + b: Variable::addGrad fan-in accumulation (flashlight/fl/autograd/Variable.cpp:205-211). In place allowed. */
int flb200_add(const void* a, const void* b, void* out, int64_t n, int dtype, void* stream);
/* Variable::astype (flashlight/fl/autograd/Variable.cpp:91-100) between f32 and f16 / bf16
 * (round to nearest even), 16 bytes per thread; the same type on both sides is a copy. */
int flb200_astype(const void* in, int in_dtype, void* out, int out_dtype, int64_t n,
                  void* stream);
/* fl::reorder (Functions.cpp:513-535) where the innermost run stays contiguous (the head split
 * and merge of an attention block: [B,T,3,h,hd] <-> [3,B,h,T,hd], [B,h,T,hd] <-> [B,T,h,hd]):
 * out is contiguous with outer extents dims[0..3] (slowest first) and runs of `inner` elements;
 * in_strides[k] = input stride, in elements, of output index k.  inner * element size and every
 * stride must be multiples of 16 bytes, both tensors 16-byte aligned (else INVALID_ARG). */
int flb200_reorder(const void* in, void* out, const int64_t* dims, const int64_t* in_strides,
                   int64_t inner, int dtype, void* stream);

/* fl::SGDOptimizer::step for one parameter in one pass
 * (flashlight/fl/optim/SGDOptimizer.cpp:38-68):
 *   g = grad_scale * grad + weight_decay * p;   v = momentum * v + g   (momentum != 0)
 *   g = nesterov ? g + momentum * v : v;        p = p - lr * g
 * grad_scale folds the 1/world-size of the data-parallel average
 * (flashlight/fl/nn/DistributedUtils.cpp:16-22); zero_grad != 0 clears grad in the same pass
 * (the zeroGrad() of the next step).  velocity may be NULL when momentum == 0.  Unlike the
 * reference, grad is not left holding the update direction.  f32. */
int flb200_sgd_step(void* param, void* grad, void* velocity, int64_t n, float lr, float momentum,
                    float weight_decay, int nesterov, float grad_scale, int zero_grad, int dtype,
                    void* stream);

/* fl::embedding (Functions.cpp:1707-1749): out row r = table row ids[r]; table [vocab][dim]
 * row-major (fl [dim, vocab]), ids int32 or int64, out [rows][dim].  Ids outside [0, vocab)
 * give a zero row / are ignored by the gradient. */
enum { FLB200_IDS_I32 = 0, FLB200_IDS_I64 = 1 };
int flb200_embedding_forward(const void* table, const void* ids, int ids_dtype, void* out,
                             int64_t rows, int64_t dim, int64_t vocab, int dtype, void* stream);
/* Its gradient: grad_table [vocab][dim] (f32, fully overwritten) = sum of the grad_out rows of
 * every position holding that id, added in increasing position order (no atomics; the
 * reference's kernel uses atomicAdd: flashlight/fl/tensor/backend/af/AdvancedIndex.cu:28-79). */
int flb200_embedding_backward(const void* grad_out, const void* ids, int ids_dtype,
                              float* grad_table, int64_t rows, int64_t dim, int64_t vocab,
                              int dtype, void* stream);

/* softmax over fl dim 0 (Functions.cpp:1021-1042) of attention scores, with the score scale and
 * the causal mask of flashlight/fl/contrib/modules/Transformer.cpp:112-119 folded in:
 * x, y [cols, rows]; y = softmax(scale * x + mask), where with causal_period = T > 0 the rows
 * are T x cols matrices stacked along rows and column c of row r is masked (-inf) when
 * c > r mod T; causal_period = 0: no mask.  cols <= 2048.
 * Gradient: grad_x = scale * y * (grad_y - sum_c grad_y * y). */
int flb200_softmax_forward(const void* x, void* y, int64_t cols, int64_t rows, float scale,
                           int64_t causal_period, int dtype, void* stream);
int flb200_softmax_backward(const void* y, const void* grad_y, void* grad_x, int64_t cols,
                            int64_t rows, float scale, int dtype, void* stream);
/* The forward pass that also keeps lse[row] = log sum_c exp(scale * x[row][c]) over the unmasked
 * columns (fp32): all that flb200_attention_backward needs of the scores. */
int flb200_softmax_forward_lse(const void* x, void* y, float* lse, int64_t cols, int64_t rows,
                               float scale, int64_t causal_period, int dtype, void* stream);

/* Gradient of o = softmax(scale * q k^T [+ causal mask]) v, the chain of
 * flashlight/fl/autograd/Functions.cpp:1828-1891 (matmulNT, softmax, matmul) as one flash-style
 * kernel: the T x T scores and probabilities are recomputed block by block in tensor memory from
 * q, k and lse instead of being kept from the forward pass or written by the backward pass.
 * q, k, v, o, grad_o, grad_q, grad_k, grad_v: [batch_heads][seq_len][head_dim] row-major;
 * lse [batch_heads][seq_len] from flb200_softmax_forward_lse; causal: key c of query r is masked
 * when c > r.  Built for FLB200_BF16, head_dim 64, seq_len a multiple of 128
 * (flb200_attention_backward_supported); the workspace holds fp32 sums of grad_q. */
int flb200_attention_backward_supported(int64_t seq_len, int64_t head_dim, int dtype);
size_t flb200_attention_backward_workspace_bytes(int64_t batch_heads, int64_t seq_len,
                                                 int64_t head_dim);
int flb200_attention_backward(const void* q, const void* k, const void* v, const void* o,
                              const void* grad_o, const float* lse, void* grad_q, void* grad_k,
                              void* grad_v, int64_t batch_heads, int64_t seq_len,
                              int64_t head_dim, float scale, int causal, int dtype,
                              void* workspace, size_t workspace_bytes, void* stream);

/* logSoftmax over fl dim 0: x, y [C, X] column-major (Functions.cpp:1044-1070). */
int flb200_log_softmax_forward(const void* x, void* y, int64_t C, int64_t X, int dtype,
                               void* stream);
/* grad_x = grad_y - exp(y) * sum_c grad_y (Functions.cpp:1062-1067). */
int flb200_log_softmax_backward(const void* y, const void* grad_y, void* grad_x, int64_t C,
                                int64_t X, int dtype, void* stream);

/* categoricalCrossEntropy (Functions.cpp:1078-1154): logp [C,X], targets int32 [X].
 * loss: [X] for NONE, [1] otherwise; count_out (optional) receives the number
 * of targets != ignore_index (the MEAN denominator).  A target outside [0,C)
 * that is not ignore_index makes bad_target_flag (device int, optional) nonzero
 * and contributes 0 — the host side turns that into std::invalid_argument. */
size_t flb200_cce_workspace_bytes(int64_t X);
int flb200_cce_forward(const void* logp, const int32_t* targets, float* loss,
                       int32_t* count_out, int32_t* bad_target_flag, int64_t C, int64_t X,
                       int reduction, int ignore_index, int dtype, void* workspace,
                       size_t workspace_bytes, void* stream);
/* grad_logp [C,X] is fully written: -(g) at the target row, 0 elsewhere, where
 * g = grad_loss[x] (NONE), grad_loss[0]/count (MEAN), grad_loss[0] (SUM);
 * count is read from the device int written by the forward call. */
int flb200_cce_backward(const float* grad_loss, const int32_t* targets,
                        const int32_t* count, void* grad_logp, int64_t C, int64_t X,
                        int reduction, int ignore_index, int dtype, void* stream);
/* logSoftmax + categoricalCrossEntropy gradient in one pass:
 * grad_x = (exp(y) - onehot) * g   (the chain of the two gradFuncs above). */
int flb200_log_softmax_cce_backward(const void* y, const float* grad_loss,
                                    const int32_t* targets, const int32_t* count,
                                    void* grad_x, int64_t C, int64_t X, int reduction,
                                    int ignore_index, int dtype, void* stream);

/* ----------------------------------------------------------- rnn (a7, a8) */
/* x [I,B,T], y [H*dirs,B,T], hx/cx/hy/cy [H,B,L*dirs]; w flat in the cuDNN
 * order the reference uses (flashlight/fl/nn/Utils.cpp:45-84;
 * backend/onednn/RNN.cpp:66-158): for every pseudo-layer (layer-major, forward
 * direction then reverse) W_ih [G*H, In] and W_hh [G*H, H] row-major; then for
 * every pseudo-layer b_ih [G*H], b_hh [G*H].  Gate order LSTM i,f,g,o; GRU
 * r,z,n with the reset gate applied after the recurrent product. */
typedef struct flb200_rnn_desc {
  int32_t input_size, hidden_size, num_layers, batch, seq_len;
  int32_t mode;           /* FLB200_RNN_* */
  int32_t bidirectional;  /* 0 / 1 */
  int32_t dtype;          /* FLB200_F32 */
  int32_t math_mode;
} flb200_rnn_desc;

int64_t flb200_rnn_num_params(const flb200_rnn_desc* d);
/* reserve space written by forward and read by backward (the payload). */
size_t flb200_rnn_reserve_bytes(const flb200_rnn_desc* d);
size_t flb200_rnn_workspace_bytes(const flb200_rnn_desc* d, int backward);

/* fl::AutogradExtension::rnn — AutogradExtension.h:96-106. hx, cx may be NULL (zeros);
 * hy, cy may be NULL; reserve may be NULL for inference. */
int flb200_rnn_forward(const flb200_rnn_desc* d, const void* x, const void* hx,
                       const void* cx, const void* w, void* y, void* hy, void* cy,
                       void* reserve, size_t reserve_bytes, void* workspace,
                       size_t workspace_bytes, void* stream);
/* fl::AutogradExtension::rnnBackward — AutogradExtension.h:167-179. grad_y, grad_hy,
 * grad_cy may be NULL (zeros: backend/cudnn/RNN.cpp:269-272); grad_hx / grad_cx may be NULL. */
int flb200_rnn_backward(const flb200_rnn_desc* d, const void* x, const void* hx,
                        const void* cx, const void* w, const void* y,
                        const void* grad_y, const void* grad_hy, const void* grad_cy,
                        void* grad_x, void* grad_hx, void* grad_cx, void* grad_w,
                        const void* reserve, size_t reserve_bytes, void* workspace,
                        size_t workspace_bytes, void* stream);

/* Inter-layer dropout (the `dropout` argument of AutogradExtension::rnn / rnnBackward,
 * AutogradExtension.h:96-106,167-179; applied by cuDNN to the input of every layer but the first,
 * backend/cudnn/RNN.cpp:83-85): the mask is DATA, [num_layers - 1][seq_len][batch][hidden * dirs]
 * floats of 0 / 1 (flb200_bernoulli_mask draws one), scaled by 1 / (1 - p) when applied, and the
 * same mask must be passed to the backward call.  The reserve space is larger
 * (flb200_rnn_reserve_bytes_dropout): inner outputs are kept with and without the mask. */
int64_t flb200_rnn_dropout_mask_elements(const flb200_rnn_desc* d);
size_t flb200_rnn_reserve_bytes_dropout(const flb200_rnn_desc* d);
int flb200_rnn_forward_dropout(const flb200_rnn_desc* d, const void* x, const void* hx,
                               const void* cx, const void* w, const void* mask, float p, void* y,
                               void* hy, void* cy, void* reserve, size_t reserve_bytes,
                               void* workspace, size_t workspace_bytes, void* stream);
int flb200_rnn_backward_dropout(const flb200_rnn_desc* d, const void* x, const void* hx,
                                const void* cx, const void* w, const void* mask, float p,
                                const void* y, const void* grad_y, const void* grad_hy,
                                const void* grad_cy, void* grad_x, void* grad_hx, void* grad_cx,
                                void* grad_w, const void* reserve, size_t reserve_bytes,
                                void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------- diagnostics */
/* Self-test of the bounded device-side waits (no counterpart in the reference): runs the
 * persistent LSTM recurrence kernel on a tiny all-zero problem in which one thread block never
 * arrives at the per-step grid barrier.  Every other block's wait runs out after `budget_ms`,
 * raises the library's device status flag, and the kernel ends by itself with the context
 * intact; a following flb200_tc_poll_status() returns FLB200_TIMEOUT and clears the flag.
 * FLB200_UNSUPPORTED where that kernel cannot run (not sm_100, or the device cannot hold its
 * blocks at once). */
size_t flb200_selftest_bounded_wait_workspace_bytes(void);
int flb200_selftest_bounded_wait(double budget_ms, void* workspace, size_t workspace_bytes,
                                 void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLB200_H_ */
