/*
 * B200Tensor / B200Backend — the smallest fl::TensorAdapterBase / fl::TensorBackend pair that
 * lets B200AutogradExtension run behind fl::Tensor without ArrayFire: device buffers owned by
 * the tensor, creation from host or device memory, host read-back, device pointers with lock
 * counting (what fl::DevicePtr needs, flashlight/fl/common/DevicePtr.cpp:16-33), and a CUDA
 * stream per backend for fl::relativeSync (flashlight/fl/tensor/Compute.cpp:70-98).
 *
 * Interfaces: flashlight/fl/tensor/TensorAdapter.h:41-263, TensorBackend.h:36-305.  The
 * TensorBackendType enum is closed (flashlight/fl/tensor/TensorBase.h:32), so the pair lives in
 * the `Stub` slot and derives from the reference's stub classes: every tensor operation this
 * harness does not implement throws "unimplemented" exactly like the stub
 * (flashlight/fl/tensor/backend/stub/StubBackend.cpp).  In a full Flashlight build the
 * extension is registered for the ArrayFire backend instead and this pair is not used.
 */
#pragma once

#include <memory>
#include <string>

#include "flashlight/fl/runtime/CUDAStream.h"
#include "flashlight/fl/tensor/backend/stub/StubBackend.h"
#include "flashlight/fl/tensor/backend/stub/StubTensor.h"

namespace fl {

class B200Backend : public StubBackend {
 public:
  static B200Backend& getInstance();
  void eval(const Tensor& tensor) override; // nothing is lazy here
  bool supportsDataType(const fl::dtype& dtype) const override;
  // the stream tensor copies run on; extensions order their own streams against it
  const CUDAStream& stream();

 private:
  B200Backend() = default;
  std::shared_ptr<CUDAStream> stream_;
};

class B200Tensor : public StubTensor {
 public:
  B200Tensor();
  B200Tensor(const Shape& shape, fl::dtype type, const void* ptr, Location memoryLocation);
  B200Tensor(
      const Dim nRows, const Dim nCols, const Tensor& values, const Tensor& rowIdx,
      const Tensor& colIdx, StorageType storageType);
  ~B200Tensor() override = default;

  std::unique_ptr<TensorAdapterBase> clone() const override; // deep copy
  TensorBackendType backendType() const override;
  TensorBackend& backend() const override;
  Tensor copy() override;
  Tensor shallowCopy() override; // shares the buffer
  const Shape& shape() override;
  dtype type() override;
  bool isSparse() override;
  Location location() override;
  void scalar(void* out) override;
  void device(void** out) override;
  void host(void* out) override;
  void unlock() override;
  bool isLocked() override;
  bool isContiguous() override;
  Shape strides() override;
  const Stream& stream() const override;
  Tensor astype(const dtype type) override; // same type, or f32 <-> f16
  Tensor flatten() const override;
  Tensor asContiguousTensor() override;
  void setContext(void* context) override;
  void* getContext() override;
  std::string toString() override;
  std::ostream& operator<<(std::ostream& ostr) override;

 private:
  struct Buffer; // device allocation, freed with the last tensor that shares it
  std::shared_ptr<Buffer> buf_;
  Shape shape_{0};
  fl::dtype type_{fl::dtype::f32};
  void* context_{nullptr};
  size_t bytes() const;
};

} // namespace fl
