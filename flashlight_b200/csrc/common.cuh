// Shared host/device helpers of the flb200 kernel library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "flb200.h"

namespace flb200 {

// ---------------------------------------------------------------- errors
// One message buffer per host thread; the C ABI never throws.
char* last_error_buffer();
int fail(int status, const char* fmt, ...);
extern std::atomic<long long> g_kernel_launches;

// Device facts are read once per device (SM count, opt-in shared memory).
struct DeviceInfo {
  int sm_count = 148;
  int max_smem_optin = 0;
  int cc_major = 0;
  int cc_minor = 0;
};
const DeviceInfo& device_info();

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Checks the launch error of the kernel just issued and counts the launch.
#define FLB200_AFTER_LAUNCH(name)                                                      \
  do {                                                                                 \
    ::flb200::g_kernel_launches.fetch_add(1, std::memory_order_relaxed);               \
    cudaError_t e__ = cudaGetLastError();                                              \
    if (e__ != cudaSuccess)                                                            \
      return ::flb200::fail(FLB200_LAUNCH_FAILURE, "%s: %s", name, cudaGetErrorString(e__)); \
  } while (0)

#define FLB200_CUDA_CHECK(expr)                                                        \
  do {                                                                                 \
    cudaError_t e__ = (expr);                                                          \
    if (e__ != cudaSuccess)                                                            \
      return ::flb200::fail(FLB200_LAUNCH_FAILURE, "%s: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

#define FLB200_REQUIRE(cond, ...)                                                      \
  do {                                                                                 \
    if (!(cond)) return ::flb200::fail(FLB200_INVALID_ARG, __VA_ARGS__);               \
  } while (0)

// Grid for a grid-stride kernel: enough CTAs to cover `work_items` at
// `per_cta` items each, capped at `waves` full waves of the device
// (148 SMs x resident CTAs), so big tensors run as a few persistent waves.
inline int grid_for(long long work_items, int per_cta, int ctas_per_sm = 8, int waves = 4) {
  long long need = (work_items + per_cta - 1) / per_cta;
  long long cap = 1LL * device_info().sm_count * ctas_per_sm * waves;
  if (need < 1) need = 1;
  return static_cast<int>(need < cap ? need : cap);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------------------ device side
template <typename T> struct Num;
template <> struct Num<float> {
  __device__ static float to_f(float v) { return v; }
  __device__ static float from_f(float v) { return v; }
};
template <> struct Num<__half> {
  __device__ static float to_f(__half v) { return __half2float(v); }
  __device__ static __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Num<__nv_bfloat16> {
  __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// 16-byte vector of T (4 floats or 8 halves) moved with one 128-bit access.
template <typename T> struct alignas(16) Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename T>
__device__ __forceinline__ Vec16<T> load16(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <typename T>
__device__ __forceinline__ void store16(T* p, const Vec16<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a CTA of up to 1024 threads; every thread gets the result.
// `scratch` must hold 32 values of T and is reusable after the call returns.
template <typename T>
__device__ __forceinline__ T block_sum(T v, T* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  T r = (lane < nwarps) ? scratch[lane] : T(0);
  r = warp_sum(r);
  return r;
}

}  // namespace flb200
