/* The backend half of fl::distributed over libflb200_dist.so.
 *
 * A Flashlight distributed backend is one translation unit that defines the Tensor-level free
 * functions declared in flashlight/fl/distributed/DistributedApi.h:33-136 — distributedInit,
 * allReduce(Tensor&, bool), allReduceMultiple(std::vector<Tensor*>, bool, bool),
 * syncDistributed, getWorldRank, getWorldSize — while DistributedApi.cpp supplies the Variable
 * overloads, barrier() and isDistributedInit() on top of them.  This file is that unit for B200:
 * it replaces flashlight/fl/distributed/backend/cuda/DistributedBackend.cpp in the build
 * (select it where FL_DISTRIBUTED_BACKEND names the NCCL backend) and forwards to the C ABI of
 * flb200_dist.h.  MPI rendezvous is not offered (DistributedInit::MPI throws like an unknown
 * method does in the reference); FILE_SYSTEM is.
 *
 * DistributedApi.h includes Variable.h and with it the cereal serialisation headers.  Where those
 * are installed the real header is used and detail::DistributedInfo is filled in; where they are
 * not, the same signatures are declared here so that the unit still compiles, links and can be
 * driven through fl::Tensor objects.
 */
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "flashlight/fl/common/Defines.h"
#include "flashlight/fl/common/DevicePtr.h"
#include "flashlight/fl/runtime/CUDAStream.h"
#include "flashlight/fl/runtime/DeviceManager.h"
#include "flashlight/fl/tensor/TensorBase.h"
#include "flb200_dist.h"

#if __has_include(<cereal/access.hpp>)
#include "flashlight/fl/distributed/DistributedApi.h"
#define FLB200_HAVE_DISTRIBUTED_API 1
#else
#define FLB200_HAVE_DISTRIBUTED_API 0
namespace fl {
void distributedInit(
    DistributedInit initMethod,
    int worldRank,
    int worldSize,
    const std::unordered_map<std::string, std::string>& params);
int getWorldRank();
int getWorldSize();
void allReduce(Tensor& arr, bool async);
void allReduceMultiple(std::vector<Tensor*> arrs, bool async, bool contiguous);
void syncDistributed();
} // namespace fl
#endif

namespace fl {

namespace {

// Status of the C ABI -> the exception the reference's NCCL backend throws in that situation.
void check(int status) {
  if (status == FLB200_OK) {
    return;
  }
  const std::string msg = flb200_dist_last_error();
  if (status == FLB200_INVALID_ARG) {
    // "distributed environment not initialized", "… of different types" and "Total coalesce
    // buffer size …" are std::runtime_error in the reference; only bad rendezvous parameters
    // are std::invalid_argument there.
    if (msg.rfind("invalid", 0) == 0 || msg.find("world rank") != std::string::npos) {
      throw std::invalid_argument(msg);
    }
    throw std::runtime_error(msg);
  }
  throw std::runtime_error(msg);
}

int distType(const Tensor& arr) {
  switch (arr.type()) {
    case fl::dtype::f16:
      return FLB200_F16;
    case fl::dtype::f32:
      return FLB200_F32;
    case fl::dtype::f64:
      return FLB200_DIST_F64;
    case fl::dtype::s32:
      return FLB200_DIST_I32;
    case fl::dtype::s64:
      return FLB200_DIST_I64;
    default:
      throw std::runtime_error("unsupported data type for allreduce with NCCL");
  }
}

void* streamOf(const Tensor& arr) {
  return arr.stream().impl<CUDAStream>().handle();
}

} // namespace

void distributedInit(
    DistributedInit initMethod,
    int worldRank,
    int worldSize,
    const std::unordered_map<std::string, std::string>& params) {
  if (initMethod != DistributedInit::FILE_SYSTEM) {
    throw std::runtime_error("unsupported distributed init method for the B200 backend");
  }
  auto filePath = params.find(DistributedConstants::kFilePath);
  auto maxDevicePerNode = params.find(DistributedConstants::kMaxDevicePerNode);
  if (filePath == params.end() || filePath->second.empty()) {
    throw std::invalid_argument("invalid FilePath for NCCL initWithFileSystem");
  }
  if (maxDevicePerNode == params.end()) {
    throw std::invalid_argument("invalid MaxDevicePerNode for NCCL initWithFileSystem");
  }
  const int perNode = std::stoi(maxDevicePerNode->second);
  if (perNode <= 0) {
    throw std::invalid_argument("invalid MaxDevicePerNode for NCCL initWithFileSystem");
  }
  double timeout = 600.0;
  auto limit = params.find("RENDEZVOUS_TIMEOUT_S"); // this backend's own, optional key
  if (limit != params.end()) {
    timeout = std::stod(limit->second);
  }
  check(flb200_dist_init_file(
      filePath->second.c_str(), worldRank, worldSize, worldRank % perNode, timeout));
#if FLB200_HAVE_DISTRIBUTED_API
  auto& info = detail::DistributedInfo::getInstance();
  info.initMethod_ = DistributedInit::FILE_SYSTEM;
  info.isInitialized_ = true;
  info.backend_ = DistributedBackend::NCCL;
#endif
}

int getWorldRank() {
  return flb200_dist_world_rank();
}

int getWorldSize() {
  return flb200_dist_world_size();
}

void allReduce(Tensor& arr, bool async /* = false */) {
  if (!flb200_dist_is_initialized()) {
    throw std::runtime_error("distributed environment not initialized");
  }
  const int type = distType(arr);
  DevicePtr ptr(arr);
  check(flb200_dist_all_reduce(
      ptr.get(), static_cast<int64_t>(arr.elements()), type, 1.0, async ? 1 : 0, streamOf(arr)));
}

void allReduceMultiple(
    std::vector<Tensor*> arrs,
    bool async /* = false */,
    bool contiguous /* = false */) {
  if (arrs.empty()) {
    return;
  }
  std::vector<DevicePtr> held;
  std::vector<void*> ptrs;
  std::vector<int64_t> counts;
  std::vector<int> types;
  held.reserve(arrs.size());
  for (auto* arr : arrs) {
    types.push_back(distType(*arr));
    counts.push_back(static_cast<int64_t>(arr->elements()));
    held.emplace_back(*arr);
    ptrs.push_back(held.back().get());
  }
  check(flb200_dist_all_reduce_multiple(
      ptrs.data(),
      counts.data(),
      types.data(),
      static_cast<int>(arrs.size()),
      1.0,
      async ? 1 : 0,
      contiguous ? 1 : 0,
      streamOf(*arrs[0])));
}

void syncDistributed() {
  // Every stream of the active device waits for the backend's streams
  // (DistributedBackend.cpp:233-245 does the same with its worker and reduction streams).
  const auto& device = DeviceManager::getInstance().getActiveDevice(DeviceType::CUDA);
  for (const auto& stream : device.getStreams()) {
    check(flb200_dist_sync(stream->impl<CUDAStream>().handle()));
  }
}

} // namespace fl
