// One LSTM time step as ONE kernel: the recurrent GEMM on the tensor cores, its split-K
// reduction inside a thread-block cluster, and the cell update as the epilogue.
//
//   pre[b][g*H + j] = gx[b][g*H + j] + sum_k W_hh[g*H + j][k] * h_prev[b][k]      g = i, f, g, o
//
// Work split: a cluster owns 32 hidden units (all four gates = the 128 rows of one UMMA tile,
// gate-major), its KS CTAs split K = H into slices of 256.  A CTA brings its whole operand
// slice (128 x 256 of W_hh, 32 x 256 of h_prev) with one burst of TMA loads (a barrier per k tile),
// issues 32 tcgen05.mma (M = 128, N = 32 batch columns, TF32), copies its 128 x 32 partial
// accumulator from tensor memory to shared memory, and after a cluster barrier each CTA sums
// the partials of 32 / KS units over the cluster's shared memories (DSMEM), adds the input
// projection, applies the gates and writes c, h and the activated gates (the tensors the
// backward pass reads).  Replaces three launches per step (contraction, split-K reduction,
// cell kernel).  Every wait is bounded; on expiry the device status flag is raised.
#include <cuda.h>
#include <cuda_runtime.h>

#include "rnn_step.cuh"
#include "tc_core.cuh"

namespace flb200 {
namespace {

using namespace tc;

constexpr int kSliceK = 256;                // K per CTA
constexpr int kStagesK = kSliceK / kBK;     // 8 tiles of 32 k
constexpr int kABytes = kBM * kBK * 4;      // 16 KB per k tile
constexpr int kBBytes = 32 * kBK * 4;       // 4 KB per k tile (32 batch rows)
constexpr int kPartStride = 33;             // floats per partial row (bank-conflict padding)
constexpr int kSmemBytes = kStagesK * (kABytes + kBBytes) + kBM * kPartStride * 4 + 128 + 1024;

struct StepArgs {
  float* gates;          // [B][4H]: input projection + biases in, activated gates out
  const float* c_prev;   // [B] rows of stride cp_stride
  long long cp_stride;
  float* c_out;          // [B][H]
  float* h_out;          // [B] rows of stride ho_stride
  long long ho_stride;
  int B, H, KS;
  int* status;
};

__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float sigmoid_(float v) { return 1.f / (1.f + expf(-v)); }

// A backward twin of this kernel (dh_prev = dgates * W_hh over clusters of 16 CTAs) was built
// and measured slower than the contraction + split-K reduction it replaced; it was removed.
__global__ void __launch_bounds__(kThreads)
lstm_step_kernel(const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_h, const StepArgs a) {
  extern __shared__ char smem_raw[];
  char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                        ~static_cast<uintptr_t>(1023));
  char* a_tiles = tiles;
  char* b_tiles = tiles + kStagesK * kABytes;
  float* part = reinterpret_cast<float*>(b_tiles + kStagesK * kBBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(part + kBM * kPartStride);  // [kStagesK]
  uint64_t* done_bar = full_bar + kStagesK;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();          // K slice
  const int group = blockIdx.x / a.KS;               // 32 hidden units
  const int H = a.H;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesK; ++s) mbar_init(&full_bar[s], 1);
    mbar_init(done_bar, 1);
    *failed = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 32);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // one barrier per k tile, so that the MMAs of tile 0 start while later tiles are in flight
    if (lane < kStagesK) mbar_expect_tx(&full_bar[lane], kABytes + kBBytes);
    __syncwarp();
    {  // 32 boxes of W_hh: k tile = lane / 4, gate = lane % 4
      const int s = lane >> 2, g = lane & 3;
      int c[2] = {rank * kSliceK + s * kBK, g * H + group * 32};
      tma_load(&map_w, &full_bar[s], a_tiles + s * kABytes + g * (32 * 128), 2, c);
    }
    if (lane < kStagesK) {  // 8 boxes of h_prev (rows past the batch are zero-filled)
      int c[2] = {rank * kSliceK + lane * kBK, 0};
      tma_load(&map_h, &full_bar[lane], b_tiles + lane * kBBytes, 2, c);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_tf32(32, 0, 0);
      const uint64_t a_desc0 = umma_desc(smem_u32(a_tiles), 16, 1024, 2);
      const uint64_t b_desc0 = umma_desc(smem_u32(b_tiles), 16, 1024, 2);
      for (int s = 0; s < kStagesK; ++s) {
        if (!mbar_wait(&full_bar[s], 0)) {
          *failed = 1;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < kBK / kUmmaK; ++j)
          umma_tf32(tmem_base, umma_desc_advance(a_desc0, s * kABytes + j * 32),
                    umma_desc_advance(b_desc0, s * kBBytes + j * 32), idesc, (s | j) ? 1u : 0u);
      }
      umma_commit(done_bar);  // arrives when every MMA issued above (possibly none) is done
    }
  } else {
    // warps 2..5: copy this CTA's partial accumulator to shared memory
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // gate = quarter, unit = lane
    if (!mbar_wait(done_bar, 0)) *failed = 2;
    tc_fence_after();
    float v[32];
    tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16), v);
#pragma unroll
    for (int j = 0; j < 32; ++j) part[row * kPartStride + j] = v[j];
    tc_fence_before();
  }
  __syncthreads();
  const int bad = *failed;
  cluster_sync_all();  // every CTA's partial tile is complete and visible in the cluster

  const uint32_t part_local = smem_u32(part);
  {
    // cell update of 32 / KS units x B batch rows by this CTA
    const int upc = 32 / a.KS;
    for (int idx = threadIdx.x; idx < upc * 32; idx += kThreads) {
      const int b = idx / upc, ul = rank * upc + (idx - b * upc);
      if (b >= a.B || bad) continue;
      float pre[4] = {0.f, 0.f, 0.f, 0.f};
      for (int q = 0; q < a.KS; ++q) {
        const uint32_t base = mapa_u32(part_local, (uint32_t)q);
#pragma unroll
        for (int g = 0; g < 4; ++g)
          pre[g] += ld_cluster_f32(base + (uint32_t)(((g * 32 + ul) * kPartStride + b) * 4));
      }
      const int j = group * 32 + ul;
      float* gp = a.gates + (long long)b * 4 * H + j;
      const float i = sigmoid_(pre[0] + gp[0]), f = sigmoid_(pre[1] + gp[H]);
      const float gg = tanhf(pre[2] + gp[2 * H]), o = sigmoid_(pre[3] + gp[3 * H]);
      const float c = f * a.c_prev[(long long)b * a.cp_stride + j] + i * gg;
      gp[0] = i; gp[H] = f; gp[2 * H] = gg; gp[3 * H] = o;
      a.c_out[(long long)b * H + j] = c;
      a.h_out[(long long)b * a.ho_stride + j] = o * tanhf(c);
    }
  }
  if (threadIdx.x == 0 && bad && a.status) atomicExch(a.status, 10 + bad);
  __syncthreads();
  cluster_sync_all();  // nobody leaves while a peer may still read its partial tile
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
}

}  // namespace

bool lstm_step_supported(int math_mode, int B, int H) {
  if (math_mode != FLB200_MATH_TF32 || !flb200_has_tensor_core_path()) return false;
  if (B < 1 || B > 32 || H % kSliceK != 0) return false;
  const int ks = H / kSliceK;
  return ks == 1 || ks == 2 || ks == 4 || ks == 8;
}

int lstm_step_weight_map(CUtensorMap* map, const float* w_hh, int H) {
  const uint64_t dims[2] = {(uint64_t)H, (uint64_t)4 * H};
  const uint64_t strides[1] = {(uint64_t)H * 4};
  const uint32_t box[2] = {32, 32};
  return tc::make_tensor_map(map, w_hh, 2, dims, strides, box, tc::kMapKMajor);
}

namespace {

int launch_step(const char* name, const CUtensorMap& map_w, const float* rhs, long long rhs_stride,
                long long K, StepArgs& a, unsigned clusters, cudaStream_t st) {
  FLB200_REQUIRE((rhs_stride % 4) == 0 && (reinterpret_cast<uintptr_t>(rhs) & 15) == 0,
                 "%s: right-hand rows must be 16-byte aligned", name);
  CUtensorMap map_h;
  const uint64_t dims[2] = {(uint64_t)K, (uint64_t)a.B};
  const uint64_t strides[1] = {(uint64_t)rhs_stride * 4};
  const uint32_t box[2] = {32, 32};
  if (int rc = tc::make_tensor_map(&map_h, rhs, 2, dims, strides, box, tc::kMapKMajor)) return rc;
  static bool configured[64] = {false};
  int dev = 0;
  FLB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    FLB200_CUDA_CHECK(cudaFuncSetAttribute(lstm_step_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured[dev] = true;
  }
  a.status = tc::status_ptr();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(clusters * (unsigned)a.KS);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)a.KS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FLB200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, lstm_step_kernel, map_w, map_h, a));
  FLB200_AFTER_LAUNCH(name);
  tc::count_tc_launch();
  return FLB200_OK;
}

}  // namespace

int lstm_step_forward(const CUtensorMap& map_w, const float* h_prev, long long hp_stride,
                      float* gates, const float* c_prev, long long cp_stride, float* c_out,
                      float* h_out, long long ho_stride, int B, int H, cudaStream_t st) {
  StepArgs a{};
  a.gates = gates; a.c_prev = c_prev; a.cp_stride = cp_stride; a.c_out = c_out;
  a.h_out = h_out; a.ho_stride = ho_stride; a.B = B; a.H = H; a.KS = H / kSliceK;
  return launch_step("lstm_step_forward", map_w, h_prev, hp_stride, H, a, (unsigned)(H / 32),
                        st);
}

}  // namespace flb200
