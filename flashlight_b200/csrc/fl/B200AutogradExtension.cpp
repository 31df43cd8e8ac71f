/*
 * Host code of B200AutogradExtension: fl::Tensor in, C ABI call, fl::Tensor out.
 * The structure of each method follows what the cuDNN backend does around its library calls
 * (flashlight/fl/autograd/tensor/backend/cudnn/Conv2D.cpp:242-357, Pool2D.cpp:17-122,
 * BatchNorm.cpp:79-265, RNN.cpp:60-373) with the library call replaced by flb200_*.
 */
#include "B200AutogradExtension.h"

#include <atomic>
#include <cstdlib>

#include <algorithm>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include "flashlight/fl/common/DevicePtr.h"
#include "flashlight/fl/common/DynamicBenchmark.h"
#include "flashlight/fl/tensor/Compute.h"
#include "flashlight/fl/tensor/TensorBase.h"
#include "flb200.h"

namespace fl {
namespace {

// FLB200_INVALID_ARG is a caller error (std::invalid_argument, like cudnnCheckErr for bad
// parameters: flashlight/fl/autograd/tensor/backend/cudnn/CudnnUtils.cpp:88-99); the rest are
// run-time failures.
void check(int status, const char* where) {
  if (status == FLB200_OK) {
    return;
  }
  const std::string msg = std::string(where) + ": " + flb200_status_string(status) + " - " +
      flb200_last_error();
  if (status == FLB200_INVALID_ARG) {
    throw std::invalid_argument(msg);
  }
  throw std::runtime_error(msg);
}

long long dimOr1(const Tensor& t, int i) {
  return t.ndim() > i ? t.dim(i) : 1;
}

void requireF32(const Tensor& t, const char* what) {
  if (!t.isEmpty() && t.type() != fl::dtype::f32) {
    throw std::invalid_argument(std::string(what) + ": the B200 extension needs f32 tensors");
  }
}

// Activations of the convolution, pooling and batch-norm operators may be f32 or f16 (the
// types the cuDNN extension takes for them, minus f64): the library's type code.
int activationType(const Tensor& t, const char* what) {
  if (t.type() == fl::dtype::f32) {
    return FLB200_F32;
  }
  if (t.type() == fl::dtype::f16) {
    return FLB200_F16;
  }
  throw std::invalid_argument(std::string(what) + ": the B200 extension needs f32 or f16 tensors");
}
void requireSameType(const Tensor& t, const Tensor& like, const char* what) {
  if (!t.isEmpty() && t.type() != like.type()) {
    throw std::invalid_argument(std::string(what) + ": all tensors of the call must share a type");
  }
}

Tensor scratch(size_t bytes) {
  return Tensor({static_cast<long long>(std::max<size_t>(bytes, 1))}, fl::dtype::b8);
}

struct PoolPayload : detail::AutogradPayloadData {
  Tensor argmax; // one byte per output element: selected window position
};

// Channels-last copies of x and grad_y that the tensor-core convolution routes keep between
// the forward, backward-data and backward-filter calls of one fl::conv2d.
struct ConvPayload : detail::AutogradPayloadData {
  Tensor xCl, gyCl;
  flb200_conv2d_cache cache{};
  const void* gyFrom = nullptr; // device address of the grad_y that gyCl was made from
};

struct RnnPayload : detail::AutogradPayloadData {
  Tensor reserve;
  Tensor dropoutMask; // [H * dirs, B, T, L - 1] of 0 / 1 when inter-layer dropout is on
};

// Counter of the dropout-mask stream: every mask continues where the last one ended, so two
// calls never reuse random numbers (the seed is fixed per process unless FLB200_SEED is set).
uint64_t nextMaskOffset(int64_t elements) {
  static std::atomic<uint64_t> offset{0};
  return offset.fetch_add(static_cast<uint64_t>((elements + 3) / 4));
}
uint64_t maskSeed() {
  static const uint64_t seed = [] {
    const char* v = std::getenv("FLB200_SEED");
    return v ? std::strtoull(v, nullptr, 10) : 0x5eed5eedULL;
  }();
  return seed;
}

flb200_conv2d_desc convDesc(
    const Tensor& input,
    const Tensor& weights,
    int sx, int sy, int px, int py, int dx, int dy, int groups, int mathMode) {
  flb200_conv2d_desc d;
  d.W = static_cast<int>(dimOr1(input, 0));
  d.H = static_cast<int>(dimOr1(input, 1));
  d.C = static_cast<int>(dimOr1(input, 2));
  d.N = static_cast<int>(dimOr1(input, 3));
  d.kW = static_cast<int>(dimOr1(weights, 0));
  d.kH = static_cast<int>(dimOr1(weights, 1));
  d.Cout = static_cast<int>(dimOr1(weights, 3));
  d.sx = sx; d.sy = sy; d.px = px; d.py = py; d.dx = dx; d.dy = dy; d.groups = groups;
  d.dtype = activationType(input, "conv2d");
  d.math_mode = mathMode;
  d.layout = FLB200_LAYOUT_NCHW;  // fl tensors are [W,H,C,N]
  if (dimOr1(weights, 2) * groups != d.C) {
    throw std::invalid_argument("conv2d: weight channels x groups do not match the input");
  }
  return d;
}

flb200_pool2d_desc poolDesc(
    const Tensor& input, int wx, int wy, int sx, int sy, int px, int py, PoolingMode mode) {
  flb200_pool2d_desc d;
  d.W = static_cast<int>(dimOr1(input, 0));
  d.H = static_cast<int>(dimOr1(input, 1));
  d.C = static_cast<int>(dimOr1(input, 2));
  d.N = static_cast<int>(dimOr1(input, 3));
  d.wx = wx; d.wy = wy; d.sx = sx; d.sy = sy; d.px = px; d.py = py;
  d.mode = static_cast<int>(mode);
  d.dtype = activationType(input, "pool2d");
  d.layout = FLB200_LAYOUT_NCHW;
  return d;
}

flb200_batchnorm_desc bnDesc(const Tensor& input, const std::vector<int>& axes) {
  std::vector<int64_t> shape(input.ndim());
  for (int i = 0; i < input.ndim(); ++i) {
    shape[i] = input.dim(i);
  }
  std::vector<int32_t> ax(axes.begin(), axes.end());
  flb200_batchnorm_desc d;
  check(
      flb200_batchnorm_geometry(
          shape.data(), input.ndim(), ax.data(), static_cast<int>(ax.size()), &d),
      "batchnorm");
  d.dtype = activationType(input, "batchnorm");  // parameters and statistics stay f32
  return d;
}

flb200_rnn_desc rnnDesc(
    const Tensor& input, int hiddenSize, int numLayers, RnnMode mode, bool bidirectional,
    int mathMode) {
  flb200_rnn_desc d;
  d.input_size = static_cast<int>(dimOr1(input, 0));
  d.batch = static_cast<int>(dimOr1(input, 1));
  d.seq_len = static_cast<int>(dimOr1(input, 2));
  d.hidden_size = hiddenSize;
  d.num_layers = numLayers;
  d.mode = static_cast<int>(mode);
  d.bidirectional = bidirectional ? 1 : 0;
  d.dtype = FLB200_F32;
  d.math_mode = mathMode;
  return d;
}

void* ptrOrNull(const Tensor& t, DevicePtr& holder) {
  if (t.isEmpty()) {
    return nullptr;
  }
  holder = DevicePtr(t);
  return holder.get();
}

// The conv payload of this call site, created on first use; null when the route keeps no
// copies or the caller passed no payload.
std::shared_ptr<ConvPayload> convPayload(
    const flb200_conv2d_desc& d, const std::shared_ptr<detail::AutogradPayload>& payload) {
  if (!payload) {
    return nullptr;
  }
  if (payload->data) {
    // only conv2d call sites hand this payload to the convolution methods
    return std::static_pointer_cast<ConvPayload>(payload->data);
  }
  const size_t xBytes = flb200_conv2d_cache_bytes(&d, 0);
  const size_t gyBytes = flb200_conv2d_cache_bytes(&d, 1);
  if (xBytes == 0 && gyBytes == 0) {
    return nullptr;
  }
  auto data = std::make_shared<ConvPayload>();
  data->cache.x_cl_bytes = xBytes;
  data->cache.gy_cl_bytes = gyBytes;
  payload->data = data;
  return data;
}

// Allocates the buffer of one slot on first use and returns a pointer holder for it.
void bindSlot(Tensor& buf, size_t bytes, DevicePtr& holder, void** slot) {
  if (bytes == 0) {
    *slot = nullptr;
    return;
  }
  if (buf.isEmpty()) {
    buf = scratch(bytes);
  }
  holder = DevicePtr(buf);
  *slot = holder.get();
}

} // namespace

B200AutogradExtension::B200AutogradExtension() : mathMode_(FLB200_MATH_STRICT_F32) {
  const char* env = std::getenv("FLB200_TF32");
  if (env && env[0] != '\0' && env[0] != '0') {
    mathMode_ = FLB200_MATH_TF32;
  }
  if (const char* poll = std::getenv("FLB200_POLL_EVERY_CALL")) {
    pollEveryCall_ = poll[0] != '\0' && poll[0] != '0';
  }
  // FLB200_MATH=strict|tf32|f32x3 names the mode and wins over FLB200_TF32
  if (const char* name = std::getenv("FLB200_MATH")) {
    const std::string mode(name);
    if (mode == "strict") {
      mathMode_ = FLB200_MATH_STRICT_F32;
    } else if (mode == "tf32") {
      mathMode_ = FLB200_MATH_TF32;
    } else if (mode == "f32x3") {
      mathMode_ = FLB200_MATH_F32X3;
    }
  }
}

void B200AutogradExtension::checkDeviceWaits() {
  check(flb200_tc_poll_status(stream().handle()), "B200AutogradExtension");
}

const CUDAStream& B200AutogradExtension::stream() {
  if (!stream_) {
    stream_ = CUDAStream::createManaged();
  }
  return *stream_;
}

bool B200AutogradExtension::isDataTypeSupported(const fl::dtype& dtype) const {
  // f16: convolution, pooling and batch-norm activations (fp32 accumulation; batch-norm
  // parameters stay f32, as in backend/cudnn/BatchNorm.cpp:92-95).  The rnn operator is f32.
  return dtype == fl::dtype::f32 || dtype == fl::dtype::f16;
}

/**************************** conv2d ****************************/
Tensor B200AutogradExtension::conv2d(
    const Tensor& input, const Tensor& weights, const Tensor& bias, const int sx, const int sy,
    const int px, const int py, const int dx, const int dy, const int groups,
    std::shared_ptr<detail::AutogradPayload> payload) {
  requireSameType(weights, input, "conv2d");
  requireSameType(bias, input, "conv2d");
  const auto d = convDesc(input, weights, sx, sy, px, py, dx, dy, groups, mathMode_);
  int32_t wo = 0, ho = 0;
  check(flb200_conv2d_output_dims(&d, &wo, &ho), "conv2d");
  auto output = Tensor({wo, ho, d.Cout, d.N}, input.type());
  const size_t wsBytes = flb200_conv2d_workspace_bytes(&d, 0);
  auto ws = scratch(wsBytes);
  {
    DevicePtr inPtr(input), wtPtr(weights), outPtr(output), wsPtr(ws), bsPtr, xClPtr;
    void* bs = ptrOrNull(bias, bsPtr);
    const auto& st = stream();
    auto conv = convPayload(d, payload);
    if (conv) {
      bindSlot(conv->xCl, conv->cache.x_cl_bytes, xClPtr, &conv->cache.x_cl);
      conv->cache.x_cl_valid = 0;
      conv->cache.gy_cl = nullptr; // no grad_y yet
      relativeSync(st, {conv->xCl});
    }
    relativeSync(st, {input, weights, bias, output, ws});
    check(
        flb200_conv2d_forward_cached(
            &d, inPtr.get(), wtPtr.get(), bs, outPtr.get(), wsPtr.get(), wsBytes,
            conv ? &conv->cache : nullptr, st.handle()),
        "conv2d");
    relativeSync({output}, st);
    if (pollEveryCall_) {
      checkDeviceWaits();
    }
  }
  return output;
}

/**************************** run-time kernel-mode selection ****************************/
std::shared_ptr<fl::DynamicBenchmark> B200AutogradExtension::createBenchmarkOptions() {
  return std::make_shared<fl::DynamicBenchmark>(
      std::make_shared<fl::DynamicBenchmarkOptions<KernelMode>>(
          std::vector<KernelMode>(
              {KernelMode::F32, KernelMode::F32_ALLOW_CONVERSION, KernelMode::F32_SPLIT}),
          fl::kDynamicBenchmarkDefaultCount));
}

int B200AutogradExtension::modeFor(const std::shared_ptr<DynamicBenchmark>& bench) const {
  if (!bench || !DynamicBenchmark::getBenchmarkMode()) {
    return mathMode_;
  }
  switch (bench->getOptions<DynamicBenchmarkOptions<KernelMode>>()->currentOption()) {
    case KernelMode::F32:
      return FLB200_MATH_STRICT_F32;
    case KernelMode::F32_ALLOW_CONVERSION:
      return FLB200_MATH_TF32;
    case KernelMode::F32_SPLIT:
      return FLB200_MATH_F32X3;
  }
  return mathMode_;
}

namespace {
// Times `fn` for the benchmark's current option while tuning is on (DynamicBenchmark::audit
// synchronises the device around it), else just runs it.
template <typename F>
void audited(const std::shared_ptr<DynamicBenchmark>& bench, F&& fn) {
  if (bench && DynamicBenchmark::getBenchmarkMode()) {
    bench->audit(fn);
  } else {
    fn();
  }
}
} // namespace

Tensor B200AutogradExtension::conv2dBackwardData(
    const Tensor& gradOutput, const Tensor& input, const Tensor& weight, const int sx,
    const int sy, const int px, const int py, const int dx, const int dy, const int groups,
    std::shared_ptr<DynamicBenchmark> dataGradBenchmark,
    std::shared_ptr<detail::AutogradPayload> payload) {
  requireSameType(gradOutput, input, "conv2dBackwardData");
  requireSameType(weight, input, "conv2dBackwardData");
  const auto d =
      convDesc(input, weight, sx, sy, px, py, dx, dy, groups, modeFor(dataGradBenchmark));
  auto gradInput = Tensor(input.shape(), input.type());
  const size_t wsBytes = flb200_conv2d_workspace_bytes(&d, 1);
  auto ws = scratch(wsBytes);
  {
    DevicePtr goPtr(gradOutput), wtPtr(weight), giPtr(gradInput), wsPtr(ws), xClPtr, gyClPtr;
    const auto& st = stream();
    auto conv = convPayload(d, payload);
    if (conv) {
      bindSlot(conv->xCl, conv->cache.x_cl_bytes, xClPtr, &conv->cache.x_cl);
      bindSlot(conv->gyCl, conv->cache.gy_cl_bytes, gyClPtr, &conv->cache.gy_cl);
      conv->cache.gy_cl_valid = 0;
      conv->gyFrom = goPtr.get();
      relativeSync(st, {conv->xCl, conv->gyCl});
    }
    relativeSync(st, {gradOutput, weight, gradInput, ws});
    audited(dataGradBenchmark, [&] {
      check(
          flb200_conv2d_backward_data_cached(
              &d, goPtr.get(), wtPtr.get(), giPtr.get(), wsPtr.get(), wsBytes,
              conv ? &conv->cache : nullptr, st.handle()),
          "conv2dBackwardData");
      relativeSync({gradInput}, st);
    });
    if (pollEveryCall_) {
      checkDeviceWaits();
    }
  }
  return gradInput;
}

std::pair<Tensor, Tensor> B200AutogradExtension::conv2dBackwardFilterBias(
    const Tensor& gradOutput, const Tensor& input, const Tensor& weights, const Tensor& bias,
    const int sx, const int sy, const int px, const int py, const int dx, const int dy,
    const int groups, std::shared_ptr<DynamicBenchmark> filterGradBenchmark,
    std::shared_ptr<DynamicBenchmark> /* biasGradBenchmark: the bias gradient is a reduction */,
    std::shared_ptr<detail::AutogradPayload> payload) {
  requireSameType(gradOutput, input, "conv2dBackwardFilterBias");
  requireSameType(weights, input, "conv2dBackwardFilterBias");
  const auto d =
      convDesc(input, weights, sx, sy, px, py, dx, dy, groups, modeFor(filterGradBenchmark));
  auto gradWeights = Tensor(weights.shape(), weights.type());
  // the bias gradient is skipped when there is no bias (cudnn/Conv2D.cpp:753)
  Tensor gradBias;
  if (!bias.isEmpty()) {
    gradBias = Tensor(bias.shape(), bias.type());
  }
  const size_t wsBytes = flb200_conv2d_workspace_bytes(&d, 2);
  auto ws = scratch(wsBytes);
  {
    DevicePtr goPtr(gradOutput), inPtr(input), gwPtr(gradWeights), wsPtr(ws), gbPtr, xClPtr,
        gyClPtr;
    void* gb = ptrOrNull(gradBias, gbPtr);
    const auto& st = stream();
    auto conv = convPayload(d, payload);
    if (conv) {
      bindSlot(conv->xCl, conv->cache.x_cl_bytes, xClPtr, &conv->cache.x_cl);
      if (!conv->gyCl.isEmpty()) {
        bindSlot(conv->gyCl, conv->cache.gy_cl_bytes, gyClPtr, &conv->cache.gy_cl);
      } else {
        conv->cache.gy_cl = nullptr;
      }
      // the copy of grad_y is only good for the tensor backward-data made it from
      if (conv->gyFrom != goPtr.get()) {
        conv->cache.gy_cl_valid = 0;
      }
      relativeSync(st, {conv->xCl, conv->gyCl});
    }
    relativeSync(st, {gradOutput, input, gradWeights, gradBias, ws});
    audited(filterGradBenchmark, [&] {
      check(
          flb200_conv2d_backward_filter_bias_cached(
              &d, goPtr.get(), inPtr.get(), gwPtr.get(), gb, wsPtr.get(), wsBytes,
              conv ? &conv->cache : nullptr, st.handle()),
          "conv2dBackwardFilterBias");
      relativeSync({gradWeights, gradBias}, st);
    });
    if (conv) {
      conv->gyCl = Tensor(); // dead after this pass; x stays for a later backward
      conv->gyFrom = nullptr;
      conv->cache.gy_cl = nullptr;
      conv->cache.gy_cl_valid = 0;
    }
    relativeSync({gradWeights, gradBias}, st);
    if (pollEveryCall_) {
      checkDeviceWaits();
    }
  }
  return {gradWeights, gradBias};
}

/**************************** pool2d ****************************/
Tensor B200AutogradExtension::pool2d(
    const Tensor& input, const int wx, const int wy, const int sx, const int sy, const int px,
    const int py, const PoolingMode mode, std::shared_ptr<detail::AutogradPayload> payload) {
  const auto d = poolDesc(input, wx, wy, sx, sy, px, py, mode);
  int32_t wo = 0, ho = 0;
  check(flb200_pool2d_output_dims(&d, &wo, &ho), "pool2d");
  auto output = Tensor({wo, ho, d.C, d.N}, input.type());
  // The argmax tensor is created inside the payload and used from there (as the cuDNN backend
  // does with its reserve space, cudnn/RNN.cpp:157-175): copying an fl::Tensor may be an eager
  // deep copy or copy-on-write depending on the tensor backend, and a copy taken before the
  // kernel ran would not see what it writes.
  Tensor none;
  std::shared_ptr<PoolPayload> data;
  if (payload && mode == PoolingMode::MAX) {
    data = std::make_shared<PoolPayload>();
    data->argmax = Tensor({wo, ho, d.C, d.N}, fl::dtype::u8);
    payload->data = data;
  }
  const Tensor& argmax = data ? data->argmax : none;
  {
    DevicePtr inPtr(input), outPtr(output), amPtr;
    void* am = ptrOrNull(argmax, amPtr);
    const auto& st = stream();
    relativeSync(st, {input, output, argmax});
    check(
        flb200_pool2d_forward(
            &d, inPtr.get(), outPtr.get(), static_cast<uint8_t*>(am), st.handle()),
        "pool2d");
    relativeSync({output, argmax}, st);
    if (pollEveryCall_) {
      checkDeviceWaits();
    }
  }
  return output;
}

Tensor B200AutogradExtension::pool2dBackward(
    const Tensor& gradOutput, const Tensor& input, const Tensor& /* poolOutput */, const int wx,
    const int wy, const int sx, const int sy, const int px, const int py, const PoolingMode mode,
    std::shared_ptr<detail::AutogradPayload> payload) {
  requireSameType(gradOutput, input, "pool2dBackward");
  const auto d = poolDesc(input, wx, wy, sx, sy, px, py, mode);
  auto gradInput = Tensor(input.shape(), input.type());
  Tensor none;
  const Tensor& argmax = payload && payload->data
      ? std::static_pointer_cast<PoolPayload>(payload->data)->argmax
      : none;
  {
    DevicePtr goPtr(gradOutput), inPtr(input), giPtr(gradInput), amPtr;
    void* am = ptrOrNull(argmax, amPtr);
    const auto& st = stream();
    relativeSync(st, {gradOutput, input, gradInput, argmax});
    check(
        flb200_pool2d_backward(
            &d, goPtr.get(), inPtr.get(), static_cast<const uint8_t*>(am), giPtr.get(),
            st.handle()),
        "pool2dBackward");
    relativeSync({gradInput}, st);
    if (pollEveryCall_) {
      checkDeviceWaits();
    }
  }
  return gradInput;
}

/**************************** batchnorm ****************************/
Tensor B200AutogradExtension::batchnorm(
    Tensor& saveMean, Tensor& saveVar, const Tensor& input, const Tensor& weight,
    const Tensor& bias, Tensor& runningMean, Tensor& runningVar, const std::vector<int>& axes,
    const bool train, const double momentum, const double epsilon,
    std::shared_ptr<detail::AutogradPayload>) {
  requireF32(weight, "batchnorm");
  requireF32(bias, "batchnorm");
  auto d = bnDesc(input, axes);
  const long long features = d.channels;
  if (!weight.isEmpty() && weight.elements() != features) {
    throw std::invalid_argument("[BatchNorm] Invalid shape for weight.");
  }
  if (!bias.isEmpty() && bias.elements() != features) {
    throw std::invalid_argument("[BatchNorm] Invalid shape for bias.");
  }
  auto output = Tensor(input.shape(), input.type());
  if (train) {
    saveMean = Tensor({features}, fl::dtype::f32);
    saveVar = Tensor({features}, fl::dtype::f32);
  }
  const size_t wsBytes = flb200_batchnorm_workspace_bytes(&d);
  auto ws = scratch(wsBytes);
  {
    DevicePtr inPtr(input), outPtr(output), wsPtr(ws), wtPtr, bsPtr, rmPtr, rvPtr, smPtr, svPtr;
    const auto& st = stream();
    relativeSync(st, {input, output, weight, bias, runningMean, runningVar, saveMean, saveVar, ws});
    check(
        flb200_batchnorm_forward(
            &d, inPtr.get(), static_cast<const float*>(ptrOrNull(weight, wtPtr)),
            static_cast<const float*>(ptrOrNull(bias, bsPtr)),
            static_cast<float*>(ptrOrNull(runningMean, rmPtr)),
            static_cast<float*>(ptrOrNull(runningVar, rvPtr)),
            static_cast<float*>(ptrOrNull(saveMean, smPtr)),
            static_cast<float*>(ptrOrNull(saveVar, svPtr)), train ? 1 : 0, momentum, epsilon,
            outPtr.get(), wsPtr.get(), wsBytes, st.handle()),
        "batchnorm");
    relativeSync({output, runningMean, runningVar, saveMean, saveVar}, st);
    if (pollEveryCall_) {
      checkDeviceWaits();
    }
  }
  return output;
}

std::tuple<Tensor, Tensor, Tensor> B200AutogradExtension::batchnormBackward(
    const Tensor& gradOutput, const Tensor& saveMean, const Tensor& saveVar, const Tensor& input,
    const Tensor& weight, const std::vector<int>& axes, const bool train, const float /* eps */,
    std::shared_ptr<detail::AutogradPayload>) {
  if (!train) {
    throw std::logic_error("can't compute batchnorm grad when train was not specified");
  }
  requireSameType(gradOutput, input, "batchnormBackward");
  requireF32(weight, "batchnormBackward");
  auto d = bnDesc(input, axes);
  const long long features = d.channels;
  auto gradIn = Tensor(input.shape(), input.type());
  auto gradWt = Tensor({features}, fl::dtype::f32);
  auto gradBs = Tensor({features}, fl::dtype::f32);
  const size_t wsBytes = flb200_batchnorm_workspace_bytes(&d);
  auto ws = scratch(wsBytes);
  {
    DevicePtr goPtr(gradOutput), inPtr(input), smPtr(saveMean), svPtr(saveVar), giPtr(gradIn),
        gwPtr(gradWt), gbPtr(gradBs), wsPtr(ws), wtPtr;
    const auto& st = stream();
    relativeSync(st, {gradOutput, input, weight, saveMean, saveVar, gradIn, gradWt, gradBs, ws});
    check(
        flb200_batchnorm_backward(
            &d, goPtr.get(), inPtr.get(), static_cast<const float*>(ptrOrNull(weight, wtPtr)),
            static_cast<const float*>(smPtr.get()), static_cast<const float*>(svPtr.get()),
            giPtr.get(), static_cast<float*>(gwPtr.get()), static_cast<float*>(gbPtr.get()),
            wsPtr.get(), wsBytes, st.handle()),
        "batchnormBackward");
    relativeSync({gradIn, gradWt, gradBs}, st);
    if (pollEveryCall_) {
      checkDeviceWaits();
    }
  }
  return std::make_tuple(gradIn, gradWt, gradBs);
}

/**************************** rnn ****************************/
std::tuple<Tensor, Tensor, Tensor> B200AutogradExtension::rnn(
    const Tensor& input, const Tensor& hiddenState, const Tensor& cellState,
    const Tensor& weights, const int hiddenSize, const int numLayers, const RnnMode mode,
    const bool bidirectional, const float dropout,
    std::shared_ptr<detail::AutogradPayload> payload) {
  if (dropout < 0.f || dropout >= 1.f) {
    throw std::invalid_argument("rnn: dropout must be in [0, 1)");
  }
  requireF32(input, "rnn");
  requireF32(weights, "rnn");
  const auto d = rnnDesc(input, hiddenSize, numLayers, mode, bidirectional, mathMode_);
  if (weights.elements() != flb200_rnn_num_params(&d)) {
    throw std::invalid_argument("rnn: invalid weights tensor size");
  }
  const auto x = input.asContiguousTensor();
  const auto hx = hiddenState.isEmpty() ? hiddenState : hiddenState.asContiguousTensor();
  const auto cx = cellState.isEmpty() ? cellState : cellState.asContiguousTensor();
  const auto w = weights.asContiguousTensor();
  const int dirs = bidirectional ? 2 : 1;
  auto y = Tensor({hiddenSize * dirs, d.batch, d.seq_len}, input.type());
  auto hy = Tensor({hiddenSize, d.batch, numLayers * dirs}, input.type());
  Tensor cy;
  if (mode == RnnMode::LSTM) {
    cy = Tensor({hiddenSize, d.batch, numLayers * dirs}, input.type());
  }
  Tensor none;
  // Inter-layer dropout (cudnn/RNN.cpp:83-85): the mask is drawn by the library's counter-based
  // generator and lives in the payload, where rnnBackward finds it.
  const bool useDropout = dropout > 0.f && numLayers > 1;
  const int64_t maskElements = useDropout ? flb200_rnn_dropout_mask_elements(&d) : 0;
  std::shared_ptr<RnnPayload> data;
  size_t reserveBytes = 0;
  if (payload) {  // created inside the payload and used from there (see pool2d)
    reserveBytes = useDropout ? flb200_rnn_reserve_bytes_dropout(&d) : flb200_rnn_reserve_bytes(&d);
    data = std::make_shared<RnnPayload>();
    data->reserve = scratch(reserveBytes);
    if (useDropout) {
      data->dropoutMask = Tensor({hiddenSize * dirs, d.batch, d.seq_len, numLayers - 1}, dtype::f32);
    }
    payload->data = data;
  }
  Tensor localMask;
  if (useDropout && !data) {
    localMask = Tensor({hiddenSize * dirs, d.batch, d.seq_len, numLayers - 1}, dtype::f32);
  }
  const Tensor& reserve = data ? data->reserve : none;
  const Tensor& mask = data ? data->dropoutMask : localMask;
  size_t wsBytes = flb200_rnn_workspace_bytes(&d, payload ? 0 : 2);
  if (!payload && useDropout) {
    wsBytes += flb200_rnn_reserve_bytes_dropout(&d);
  }
  auto ws = scratch(wsBytes);
  {
    DevicePtr xPtr(x), wPtr(w), yPtr(y), hyPtr(hy), wsPtr(ws), hxPtr, cxPtr, cyPtr, rsPtr, mkPtr;
    const auto& st = stream();
    relativeSync(st, {x, hx, cx, w, y, hy, cy, reserve, ws, mask});
    if (useDropout) {
      check(
          flb200_bernoulli_mask(
              ptrOrNull(mask, mkPtr), maskElements, 1.f - dropout, maskSeed(),
              nextMaskOffset(maskElements), FLB200_F32, st.handle()),
          "rnn");
      check(
          flb200_rnn_forward_dropout(
              &d, xPtr.get(), ptrOrNull(hx, hxPtr), ptrOrNull(cx, cxPtr), wPtr.get(), mkPtr.get(),
              dropout, yPtr.get(), hyPtr.get(), ptrOrNull(cy, cyPtr), ptrOrNull(reserve, rsPtr),
              reserveBytes, wsPtr.get(), wsBytes, st.handle()),
          "rnn");
    } else {
      check(
          flb200_rnn_forward(
              &d, xPtr.get(), ptrOrNull(hx, hxPtr), ptrOrNull(cx, cxPtr), wPtr.get(), yPtr.get(),
              hyPtr.get(), ptrOrNull(cy, cyPtr), ptrOrNull(reserve, rsPtr), reserveBytes,
              wsPtr.get(), wsBytes, st.handle()),
          "rnn");
    }
    relativeSync({y, hy, cy, reserve, mask}, st);
    if (pollEveryCall_) {
      checkDeviceWaits();
    }

  }
  return std::make_tuple(y, hy, cy);
}

std::tuple<Tensor, Tensor, Tensor, Tensor> B200AutogradExtension::rnnBackward(
    const Tensor& input, const Tensor& hiddenState, const Tensor& cellState,
    const Tensor& weights, const std::shared_ptr<detail::RNNGradData> gradData,
    const Tensor& output, const int numLayers, const int hiddenSize, const RnnMode mode,
    const bool bidirectional, const float dropProb,
    std::shared_ptr<detail::AutogradPayload> payload) {
  if (!payload || !payload->data) {
    throw std::invalid_argument(
        "B200AutogradExtension::rnnBackward given null detail::AutogradPayload");
  }
  const auto d = rnnDesc(input, hiddenSize, numLayers, mode, bidirectional, mathMode_);
  const Tensor& reserve = std::static_pointer_cast<RnnPayload>(payload->data)->reserve;
  const Tensor& mask = std::static_pointer_cast<RnnPayload>(payload->data)->dropoutMask;
  const auto x = input.asContiguousTensor();
  const auto hx = hiddenState.isEmpty() ? hiddenState : hiddenState.asContiguousTensor();
  const auto cx = cellState.isEmpty() ? cellState : cellState.asContiguousTensor();
  const auto w = weights.asContiguousTensor();
  const auto y = output.asContiguousTensor();
  // absent output gradients count as zeros (cudnn/RNN.cpp:269-272)
  const Tensor dy = gradData ? gradData->dy : Tensor();
  const Tensor dhy = gradData ? gradData->dhy : Tensor();
  const Tensor dcy = gradData ? gradData->dcy : Tensor();
  auto dx = Tensor(input.shape(), input.type());
  const int dirs = bidirectional ? 2 : 1;
  auto dhx = Tensor({hiddenSize, d.batch, numLayers * dirs}, input.type());
  Tensor dcx;
  if (mode == RnnMode::LSTM) {
    dcx = Tensor({hiddenSize, d.batch, numLayers * dirs}, input.type());
  }
  auto dw = Tensor(weights.shape(), weights.type());
  const size_t wsBytes = flb200_rnn_workspace_bytes(&d, 1);
  auto ws = scratch(wsBytes);
  {
    DevicePtr xPtr(x), wPtr(w), yPtr(y), dxPtr(dx), dhxPtr(dhx), dwPtr(dw), rsPtr(reserve),
        wsPtr(ws), hxPtr, cxPtr, dyPtr, dhyPtr, dcyPtr, dcxPtr, mkPtr;
    const auto& st = stream();
    relativeSync(st, {x, hx, cx, w, y, dy, dhy, dcy, dx, dhx, dcx, dw, reserve, ws, mask});
    if (!mask.isEmpty()) {
      check(
          flb200_rnn_backward_dropout(
              &d, xPtr.get(), ptrOrNull(hx, hxPtr), ptrOrNull(cx, cxPtr), wPtr.get(),
              ptrOrNull(mask, mkPtr), dropProb, yPtr.get(), ptrOrNull(dy, dyPtr),
              ptrOrNull(dhy, dhyPtr), ptrOrNull(dcy, dcyPtr), dxPtr.get(), dhxPtr.get(),
              ptrOrNull(dcx, dcxPtr), dwPtr.get(), rsPtr.get(),
              static_cast<size_t>(reserve.elements()), wsPtr.get(), wsBytes, st.handle()),
          "rnnBackward");
    } else {
      check(
          flb200_rnn_backward(
              &d, xPtr.get(), ptrOrNull(hx, hxPtr), ptrOrNull(cx, cxPtr), wPtr.get(), yPtr.get(),
              ptrOrNull(dy, dyPtr), ptrOrNull(dhy, dhyPtr), ptrOrNull(dcy, dcyPtr), dxPtr.get(),
              dhxPtr.get(), ptrOrNull(dcx, dcxPtr), dwPtr.get(), rsPtr.get(),
              static_cast<size_t>(reserve.elements()), wsPtr.get(), wsBytes, st.handle()),
          "rnnBackward");
    }
    relativeSync({dx, dhx, dcx, dw}, st);
    if (pollEveryCall_) {
      checkDeviceWaits();
    }
  }
  return std::make_tuple(dx, dhx, dcx, dw);
}

} // namespace fl
