/*
 * B200AutogradExtension — the sm_100a implementation of fl::AutogradExtension
 * (flashlight/fl/autograd/tensor/AutogradExtension.h:46-180).  Every operator forwards to the C
 * ABI of libflb200.so (include/flb200.h); this class only does what the cuDNN backend's host
 * code does around its library calls: shape / dtype checks, output and scratch allocation as
 * fl::Tensor, raw pointers through fl::DevicePtr, stream ordering with relativeSync, payloads.
 *
 * Register it for the tensor backend in use, and make it the only autograd registration for
 * that backend (the registry is first-wins, flashlight/fl/tensor/TensorExtension.cpp:13-30):
 *
 *   FL_REGISTER_TENSOR_EXTENSION(B200AutogradExtension, TensorBackendType::ArrayFire);
 */
#pragma once

#include <memory>

#include "flashlight/fl/autograd/tensor/AutogradExtension.h"
#include "flashlight/fl/runtime/CUDAStream.h"

namespace fl {

class B200AutogradExtension final : public AutogradExtension {
 public:
  B200AutogradExtension();

  // fp32 is the built dtype of the dense operators (f16 / bf16 exist for the element-wise ones)
  bool isDataTypeSupported(const fl::dtype& dtype) const override;

  // The arithmetic a convolution gradient may run in, in the order DynamicBenchmark tries them
  // (the counterpart of CudnnAutogradExtension::KernelMode,
  // flashlight/fl/autograd/tensor/backend/cudnn/CudnnAutogradExtension.h:24): fp32 FMA, TF32
  // tensor cores ("allow conversion"), and the three-pass TF32 split with fp32-grade results.
  enum class KernelMode { F32 = 0, F32_ALLOW_CONVERSION = 1, F32_SPLIT = 2 };

  // Options for a Conv2D module's run-time autotune (flashlight/fl/common/DynamicBenchmark.h:
  // 196-263): while DynamicBenchmark::getBenchmarkMode() is on, conv2dBackwardData and
  // conv2dBackwardFilterBias time each mode kDynamicBenchmarkDefaultCount times through
  // DynamicBenchmark::audit and then keep the fastest, as the cuDNN extension does
  // (cudnn/Conv2D.cpp:401-405,466-535); with benchmark mode off they run in the extension's
  // configured mode.
  std::shared_ptr<fl::DynamicBenchmark> createBenchmarkOptions() override;

  // Every wait inside the tensor-core kernels is bounded: one that runs out raises a device
  // flag and the kernel returns with partial results instead of hanging the GPU.  This call
  // synchronises the extension's stream, reads and clears the flag and throws
  // std::runtime_error if it was set.  Call it wherever the host synchronises anyway (end of
  // a step, before reading a loss); with FLB200_POLL_EVERY_CALL=1 in the environment every
  // operator does it after its launch (debugging aid: it serialises host and device).
  void checkDeviceWaits();

  /**************************** Forward ****************************/
  Tensor conv2d(
      const Tensor& input, const Tensor& weights, const Tensor& bias, const int sx, const int sy,
      const int px, const int py, const int dx, const int dy, const int groups,
      std::shared_ptr<detail::AutogradPayload> payload) override;

  Tensor pool2d(
      const Tensor& input, const int wx, const int wy, const int sx, const int sy, const int px,
      const int py, const PoolingMode mode,
      std::shared_ptr<detail::AutogradPayload> payload) override;

  Tensor batchnorm(
      Tensor& saveMean, Tensor& saveVar, const Tensor& input, const Tensor& weight,
      const Tensor& bias, Tensor& runningMean, Tensor& runningVar, const std::vector<int>& axes,
      const bool train, const double momentum, const double epsilon,
      std::shared_ptr<detail::AutogradPayload> payload) override;

  std::tuple<Tensor, Tensor, Tensor> rnn(
      const Tensor& input, const Tensor& hiddenState, const Tensor& cellState,
      const Tensor& weights, const int hiddenSize, const int numLayers, const RnnMode mode,
      const bool bidirectional, const float dropout,
      std::shared_ptr<detail::AutogradPayload> payload) override;

  /**************************** Backward ****************************/
  Tensor conv2dBackwardData(
      const Tensor& gradOutput, const Tensor& input, const Tensor& weight, const int sx,
      const int sy, const int px, const int py, const int dx, const int dy, const int groups,
      std::shared_ptr<DynamicBenchmark> dataGradBenchmark,
      std::shared_ptr<detail::AutogradPayload> payload) override;

  std::pair<Tensor, Tensor> conv2dBackwardFilterBias(
      const Tensor& gradOutput, const Tensor& input, const Tensor& weights, const Tensor& bias,
      const int sx, const int sy, const int px, const int py, const int dx, const int dy,
      const int groups, std::shared_ptr<DynamicBenchmark> filterBench,
      std::shared_ptr<DynamicBenchmark> biasBench,
      std::shared_ptr<detail::AutogradPayload> autogradPayload) override;

  Tensor pool2dBackward(
      const Tensor& gradOutput, const Tensor& input, const Tensor& poolOutput, const int wx,
      const int wy, const int sx, const int sy, const int px, const int py, const PoolingMode mode,
      std::shared_ptr<detail::AutogradPayload> payload) override;

  std::tuple<Tensor, Tensor, Tensor> batchnormBackward(
      const Tensor& gradOutput, const Tensor& saveMean, const Tensor& saveVar,
      const Tensor& input, const Tensor& weight, const std::vector<int>& axes, const bool train,
      const float epsilon, std::shared_ptr<detail::AutogradPayload> payload) override;

  std::tuple<Tensor, Tensor, Tensor, Tensor> rnnBackward(
      const Tensor& input, const Tensor& hiddenState, const Tensor& cellState,
      const Tensor& weights, const std::shared_ptr<detail::RNNGradData> gradData,
      const Tensor& output, const int numLayers, const int hiddenSize, const RnnMode mode,
      const bool bidirectional, const float dropProb,
      std::shared_ptr<detail::AutogradPayload> payload) override;

 private:
  // math mode of one audited call: the benchmark's current option while tuning is on
  int modeFor(const std::shared_ptr<DynamicBenchmark>& bench) const;

  // FLB200_MATH_STRICT_F32, _TF32 or _F32X3 (environment FLB200_MATH=strict|tf32|f32x3, or
  // FLB200_TF32=1; read once)
  int mathMode_;
  bool pollEveryCall_ = false;
  // the stream the kernels run on; ordered against the tensors' streams around every call
  std::shared_ptr<CUDAStream> stream_;
  const CUDAStream& stream();
};

} // namespace fl
