/* See B200Tensor.h. */
#include "B200Tensor.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <sstream>
#include <stdexcept>
#include <vector>

#include "flashlight/fl/tensor/TensorBase.h"

namespace fl {
namespace {

void cudaCheck(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    throw std::runtime_error(std::string("B200Tensor: ") + what + ": " + cudaGetErrorString(e));
  }
}

Tensor wrap(std::unique_ptr<TensorAdapterBase> a) {
  return Tensor(std::move(a));
}

} // namespace

/******************************* backend *******************************/
B200Backend& B200Backend::getInstance() {
  static B200Backend instance;
  return instance;
}

void B200Backend::eval(const Tensor& /* tensor */) {}

bool B200Backend::supportsDataType(const fl::dtype& dtype) const {
  return dtype == fl::dtype::f32 || dtype == fl::dtype::f16 || dtype == fl::dtype::b8 ||
      dtype == fl::dtype::u8 || dtype == fl::dtype::s32;
}

const CUDAStream& B200Backend::stream() {
  if (!stream_) {
    stream_ = CUDAStream::createManaged();
  }
  return *stream_;
}

/******************************* tensor *******************************/
// Device memory comes from the CUDA stream-ordered pool on the backend's stream: allocating and
// freeing a tensor neither synchronises the device nor calls into the driver's allocator in the
// steady state (the pool keeps what was freed).  Every B200Tensor computes on that one stream
// and the extension orders its own stream against it with relativeSync before a tensor it used
// can be freed, so stream order is enough to make reuse safe.
struct B200Tensor::Buffer {
  void* ptr = nullptr;
  size_t bytes = 0;
  int locks = 0;
  explicit Buffer(size_t n) : bytes(n) {
    if (n > 0) {
      static const bool configured = [] {
        int dev = 0;
        cudaMemPool_t pool = nullptr;
        unsigned long long keep = ~0ull;  // never trim the pool at synchronisation points
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
          cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
        }
        return true;
      }();
      (void)configured;
      cudaCheck(
          cudaMallocAsync(&ptr, n, B200Backend::getInstance().stream().handle()),
          "cudaMallocAsync");
    }
  }
  ~Buffer() {
    if (ptr) {
      cudaFreeAsync(ptr, B200Backend::getInstance().stream().handle());
    }
  }
  Buffer(const Buffer&) = delete;
  Buffer& operator=(const Buffer&) = delete;
};

B200Tensor::B200Tensor() : buf_(std::make_shared<Buffer>(0)) {}

B200Tensor::B200Tensor(
    const Shape& shape, fl::dtype type, const void* ptr, Location memoryLocation)
    : shape_(shape), type_(type) {
  buf_ = std::make_shared<Buffer>(bytes());
  if (ptr && buf_->bytes > 0) {
    const auto kind =
        memoryLocation == Location::Host ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
    const auto st = B200Backend::getInstance().stream().handle();
    cudaCheck(cudaMemcpyAsync(buf_->ptr, ptr, buf_->bytes, kind, st), "copy into a new tensor");
    if (memoryLocation == Location::Host) {
      cudaCheck(cudaStreamSynchronize(st), "sync"); // the host buffer may go away after the call
    }
  }
}

B200Tensor::B200Tensor(
    const Dim, const Dim, const Tensor&, const Tensor&, const Tensor&, StorageType) {
  throw std::invalid_argument("B200Tensor: sparse tensors are not built");
}

size_t B200Tensor::bytes() const {
  return static_cast<size_t>(shape_.elements()) * fl::getTypeSize(type_);
}

std::unique_ptr<TensorAdapterBase> B200Tensor::clone() const {
  return std::make_unique<B200Tensor>(shape_, type_, buf_->ptr, Location::Device);
}

TensorBackendType B200Tensor::backendType() const {
  return TensorBackendType::Stub;
}

TensorBackend& B200Tensor::backend() const {
  return B200Backend::getInstance();
}

Tensor B200Tensor::copy() {
  return wrap(clone());
}

Tensor B200Tensor::shallowCopy() {
  auto t = std::make_unique<B200Tensor>();
  t->buf_ = buf_;
  t->shape_ = shape_;
  t->type_ = type_;
  t->context_ = context_;
  return wrap(std::move(t));
}

const Shape& B200Tensor::shape() {
  return shape_;
}

dtype B200Tensor::type() {
  return type_;
}

bool B200Tensor::isSparse() {
  return false;
}

Location B200Tensor::location() {
  return Location::Device;
}

void B200Tensor::scalar(void* out) {
  if (buf_->bytes == 0) {
    throw std::invalid_argument("B200Tensor::scalar called on an empty tensor");
  }
  const auto st = B200Backend::getInstance().stream().handle();
  cudaCheck(cudaStreamSynchronize(st), "sync");
  cudaCheck(cudaMemcpy(out, buf_->ptr, fl::getTypeSize(type_), cudaMemcpyDeviceToHost), "scalar");
}

void B200Tensor::device(void** out) {
  ++buf_->locks;
  *out = buf_->ptr;
}

void B200Tensor::host(void* out) {
  if (buf_->bytes == 0) {
    return;
  }
  // every stream that produced this tensor made the tensor's stream wait on it
  // (relativeSync({outputs}, extensionStream)), so syncing the tensor's stream is enough
  const auto st = B200Backend::getInstance().stream().handle();
  cudaCheck(cudaStreamSynchronize(st), "sync");
  cudaCheck(cudaMemcpy(out, buf_->ptr, buf_->bytes, cudaMemcpyDeviceToHost), "host");
}

void B200Tensor::unlock() {
  if (buf_->locks > 0) {
    --buf_->locks;
  }
}

bool B200Tensor::isLocked() {
  return buf_->locks > 0;
}

bool B200Tensor::isContiguous() {
  return true;
}

Shape B200Tensor::strides() {
  std::vector<Dim> s(shape_.ndim());
  Dim acc = 1;
  for (int i = 0; i < shape_.ndim(); ++i) {
    s[i] = acc;
    acc *= shape_.dim(i);
  }
  return Shape(s);
}

const Stream& B200Tensor::stream() const {
  return B200Backend::getInstance().stream();
}

// f32 <-> f16 through the host (round to nearest even): this tensor type exists to drive the
// extension from tests, so the conversion favours being obviously right over being fast.
Tensor B200Tensor::astype(const dtype type) {
  if (type == type_) {
    return copy();
  }
  const bool widen = type_ == fl::dtype::f16 && type == fl::dtype::f32;
  const bool narrow = type_ == fl::dtype::f32 && type == fl::dtype::f16;
  if (!widen && !narrow) {
    throw std::invalid_argument("B200Tensor::astype - only f32 <-> f16 conversions are built");
  }
  const size_t n = static_cast<size_t>(shape_.elements());
  std::vector<float> wide(n);
  std::vector<__half> half(n);
  if (narrow) {
    host(wide.data());
    for (size_t i = 0; i < n; ++i) {
      half[i] = __float2half_rn(wide[i]);
    }
    return toTensor<B200Tensor>(shape_, type, half.data(), Location::Host);
  }
  host(half.data());
  for (size_t i = 0; i < n; ++i) {
    wide[i] = __half2float(half[i]);
  }
  return toTensor<B200Tensor>(shape_, type, wide.data(), Location::Host);
}

Tensor B200Tensor::flatten() const {
  auto t = std::make_unique<B200Tensor>();
  t->buf_ = buf_;
  t->shape_ = Shape({shape_.elements()});
  t->type_ = type_;
  return wrap(std::move(t));
}

Tensor B200Tensor::asContiguousTensor() {
  return shallowCopy();
}

void B200Tensor::setContext(void* context) {
  context_ = context;
}

void* B200Tensor::getContext() {
  return context_;
}

std::string B200Tensor::toString() {
  std::ostringstream os;
  os << "B200Tensor" << shape_ << " on the device";
  return os.str();
}

std::ostream& B200Tensor::operator<<(std::ostream& ostr) {
  return ostr << toString();
}

} // namespace fl
