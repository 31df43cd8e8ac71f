// Status handling, launch counter and cached device facts for the flb200 C ABI.
#include "common.cuh"

#include <mutex>

namespace flb200 {

std::atomic<long long> g_kernel_launches{0};

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return status;
}

const DeviceInfo& device_info() {
  // One slot per device ordinal; filled on first use with that device current.
  static DeviceInfo infos[64];
  static bool ready[64] = {false};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  std::lock_guard<std::mutex> lock(mu);
  if (!ready[dev]) {
    DeviceInfo di;
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
      di.sm_count = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess)
      di.max_smem_optin = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess)
      di.cc_major = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMinor, dev) == cudaSuccess)
      di.cc_minor = v;
    (void)cudaGetLastError();
    infos[dev] = di;
    ready[dev] = true;
  }
  return infos[dev];
}

}  // namespace flb200

extern "C" {

int flb200_abi_version(void) { return 2; }

const char* flb200_status_string(int status) {
  switch (status) {
    case FLB200_OK: return "ok";
    case FLB200_INVALID_ARG: return "invalid argument";
    case FLB200_UNSUPPORTED: return "unsupported";
    case FLB200_LAUNCH_FAILURE: return "CUDA launch failure";
    case FLB200_TIMEOUT: return "device-side wait timed out";
    case FLB200_WORKSPACE_TOO_SMALL: return "workspace too small";
    default: return "unknown status";
  }
}

const char* flb200_last_error(void) { return flb200::last_error_buffer(); }

long long flb200_kernel_launches(void) {
  return flb200::g_kernel_launches.load(std::memory_order_relaxed);
}

}  // extern "C"
