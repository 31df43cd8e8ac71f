// Embedding lookup and its gradient (fl::embedding, flashlight/fl/autograd/Functions.cpp:1707-1749).
//
// Forward is a row gather.  The gradient is a scatter-add of the output-gradient rows into the
// table rows named by the token ids; the reference does it with atomicAdd
// (flashlight/fl/tensor/backend/af/AdvancedIndex.cu:28-79), whose summation order changes from
// run to run.  Here the kernel is output-stationary instead: one warp per table row scans the
// id list 32 entries at a time (ballot), and adds the matching gradient rows in increasing
// position order — no atomics, bit-reproducible, and the table gradient is fully written
// (zero rows included), so no clearing pass is needed.  Cost vocab x rows / 32 warp iterations:
// 4 M for a 32000-word vocabulary and 4096 tokens — which is why id lists shorter than the
// vocabulary go to the warp-per-position kernel further down (0.27 -> 0.06 ms + a memset there).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace flb200 {
namespace {

template <typename I>
__device__ __forceinline__ long long id_at(const void* ids, long long i) {
  return static_cast<long long>(static_cast<const I*>(ids)[i]);
}

template <typename T, typename I>
__global__ void __launch_bounds__(256)
embedding_forward_kernel(const T* __restrict__ table, const void* __restrict__ ids,
                         T* __restrict__ out, long long rows, long long dim, long long vocab) {
  const long long total = rows * dim;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const long long r = t / dim, c = t - r * dim;
    const long long v = id_at<I>(ids, r);
    out[t] = (v >= 0 && v < vocab) ? table[v * dim + c] : Num<T>::from_f(0.f);
  }
}

constexpr int kMaxPerLane = 32;  // dim <= 32 * 32 * kChunks handled in column chunks of 1024

template <typename T, typename I>
__global__ void __launch_bounds__(256)
embedding_backward_kernel(const T* __restrict__ grad_out, const void* __restrict__ ids,
                          float* __restrict__ grad_table, long long rows, long long dim,
                          long long vocab) {
  const int lane = threadIdx.x & 31;
  const long long v = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (v >= vocab) return;
  for (long long c0 = 0; c0 < dim; c0 += 32 * kMaxPerLane) {
    float acc[kMaxPerLane];
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) acc[j] = 0.f;
    for (long long base = 0; base < rows; base += 32) {
      const long long pos = base + lane;
      const bool hit = pos < rows && id_at<I>(ids, pos) == v;
      unsigned m = __ballot_sync(0xffffffffu, hit);
      while (m) {  // matching positions of this chunk, lowest first
        const int b = __ffs(m) - 1;
        m &= m - 1;
        const T* src = grad_out + (base + b) * dim + c0;
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
          const long long c = (long long)j * 32 + lane;
          if (c0 + c < dim) acc[j] += Num<T>::to_f(src[c]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const long long c = c0 + (long long)j * 32 + lane;
      if (c < dim) grad_table[v * dim + c] = acc[j];
    }
  }
}

// The same sums with a warp per POSITION, for id lists shorter than the vocabulary: the warp of
// the first position that holds an id owns that table row and adds the rows of the later
// positions with the same id in increasing order (so the sums are those of the kernel above,
// bit for bit); every other warp leaves after the scan that finds an earlier holder.  The scan
// work is rows^2 / 32 instead of vocab x rows / 32; rows no position names are cleared by a
// memset before the launch.
template <typename T, typename I>
__global__ void __launch_bounds__(256)
embedding_backward_by_position_kernel(const T* __restrict__ grad_out,
                                      const void* __restrict__ ids,
                                      float* __restrict__ grad_table, long long rows,
                                      long long dim, long long vocab) {
  const int lane = threadIdx.x & 31;
  const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= rows) return;
  const long long v = id_at<I>(ids, i);
  if (v < 0 || v >= vocab) return;
  for (long long base = 0; base < i; base += 32) {
    const long long pos = base + lane;
    const bool hit = pos < i && id_at<I>(ids, pos) == v;
    if (__ballot_sync(0xffffffffu, hit) != 0u) return;  // an earlier position owns the row
  }
  for (long long c0 = 0; c0 < dim; c0 += 32 * kMaxPerLane) {
    float acc[kMaxPerLane];
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) acc[j] = 0.f;
    for (long long base = i & ~31LL; base < rows; base += 32) {
      const long long pos = base + lane;
      const bool hit = pos >= i && pos < rows && id_at<I>(ids, pos) == v;
      unsigned m = __ballot_sync(0xffffffffu, hit);
      while (m) {
        const int b = __ffs(m) - 1;
        m &= m - 1;
        const T* src = grad_out + (base + b) * dim + c0;
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
          const long long c = (long long)j * 32 + lane;
          if (c0 + c < dim) acc[j] += Num<T>::to_f(src[c]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const long long c = c0 + (long long)j * 32 + lane;
      if (c < dim) grad_table[v * dim + c] = acc[j];
    }
  }
}

template <typename T>
int launch_fwd(const void* table, const void* ids, int ids64, void* out, long long rows,
               long long dim, long long vocab, cudaStream_t st) {
  const int grid = grid_for(rows * dim, 256);
  if (ids64)
    embedding_forward_kernel<T, long long><<<grid, 256, 0, st>>>(
        static_cast<const T*>(table), ids, static_cast<T*>(out), rows, dim, vocab);
  else
    embedding_forward_kernel<T, int><<<grid, 256, 0, st>>>(
        static_cast<const T*>(table), ids, static_cast<T*>(out), rows, dim, vocab);
  return FLB200_OK;
}
template <typename T>
int launch_bwd(const void* grad_out, const void* ids, int ids64, float* grad_table, long long rows,
               long long dim, long long vocab, cudaStream_t st) {
  if (rows < vocab) {
    FLB200_CUDA_CHECK(cudaMemsetAsync(grad_table, 0, (size_t)vocab * dim * sizeof(float), st));
    if (rows == 0) return FLB200_OK;
    const unsigned pgrid = (unsigned)((rows + 7) / 8);
    if (ids64)
      embedding_backward_by_position_kernel<T, long long><<<pgrid, 256, 0, st>>>(
          static_cast<const T*>(grad_out), ids, grad_table, rows, dim, vocab);
    else
      embedding_backward_by_position_kernel<T, int><<<pgrid, 256, 0, st>>>(
          static_cast<const T*>(grad_out), ids, grad_table, rows, dim, vocab);
    return FLB200_OK;
  }
  const unsigned grid = (unsigned)((vocab + 7) / 8);
  if (ids64)
    embedding_backward_kernel<T, long long><<<grid, 256, 0, st>>>(
        static_cast<const T*>(grad_out), ids, grad_table, rows, dim, vocab);
  else
    embedding_backward_kernel<T, int><<<grid, 256, 0, st>>>(
        static_cast<const T*>(grad_out), ids, grad_table, rows, dim, vocab);
  return FLB200_OK;
}

int check(const char* name, long long rows, long long dim, long long vocab, int ids_dtype) {
  FLB200_REQUIRE(rows >= 0 && dim >= 1 && vocab >= 1, "%s: bad extents", name);
  FLB200_REQUIRE(ids_dtype == FLB200_IDS_I32 || ids_dtype == FLB200_IDS_I64,
                 "%s: ids must be int32 or int64", name);
  return FLB200_OK;
}

}  // namespace
}  // namespace flb200

extern "C" {

int flb200_embedding_forward(const void* table, const void* ids, int ids_dtype, void* out,
                             int64_t rows, int64_t dim, int64_t vocab, int dtype, void* stream) {
  using namespace flb200;
  if (int st = check("embedding_forward", rows, dim, vocab, ids_dtype)) return st;
  if (rows == 0) return FLB200_OK;
  FLB200_REQUIRE(table && ids && out, "embedding_forward: null tensor");
  cudaStream_t st = as_stream(stream);
  const int i64 = ids_dtype == FLB200_IDS_I64;
  switch (dtype) {
    case FLB200_F32: launch_fwd<float>(table, ids, i64, out, rows, dim, vocab, st); break;
    case FLB200_F16: launch_fwd<__half>(table, ids, i64, out, rows, dim, vocab, st); break;
    case FLB200_BF16: launch_fwd<__nv_bfloat16>(table, ids, i64, out, rows, dim, vocab, st); break;
    default: return fail(FLB200_UNSUPPORTED, "embedding_forward: unknown dtype %d", dtype);
  }
  FLB200_AFTER_LAUNCH("embedding_forward");
  return FLB200_OK;
}

int flb200_embedding_backward(const void* grad_out, const void* ids, int ids_dtype,
                              float* grad_table, int64_t rows, int64_t dim, int64_t vocab,
                              int dtype, void* stream) {
  using namespace flb200;
  if (int st = check("embedding_backward", rows, dim, vocab, ids_dtype)) return st;
  FLB200_REQUIRE(grad_table && (rows == 0 || (grad_out && ids)), "embedding_backward: null tensor");
  // every table row scans the id list: keep the product within what one launch does in
  // well under a second
  FLB200_REQUIRE((double)vocab * (double)rows <= 6.9e10,
                 "embedding_backward: vocabulary x tokens too large for the scan kernel");
  cudaStream_t st = as_stream(stream);
  const int i64 = ids_dtype == FLB200_IDS_I64;
  switch (dtype) {
    case FLB200_F32: launch_bwd<float>(grad_out, ids, i64, grad_table, rows, dim, vocab, st); break;
    case FLB200_F16: launch_bwd<__half>(grad_out, ids, i64, grad_table, rows, dim, vocab, st); break;
    case FLB200_BF16:
      launch_bwd<__nv_bfloat16>(grad_out, ids, i64, grad_table, rows, dim, vocab, st);
      break;
    default: return fail(FLB200_UNSUPPORTED, "embedding_backward: unknown dtype %d", dtype);
  }
  FLB200_AFTER_LAUNCH("embedding_backward");
  return FLB200_OK;
}

}  // extern "C"
