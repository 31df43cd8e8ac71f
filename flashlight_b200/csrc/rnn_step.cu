// (The sequence kernels further down run the LSTM and the GRU; this first part is the LSTM's
// single-step kernel.)
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


// ----------------------------------------------------------------------------------------
// The whole recurrence of one (layer, direction) as ONE persistent kernel.
//
// Same work split as lstm_step_kernel (a cluster per 32 hidden units, its KS CTAs splitting
// K = H into slices of 256), but every CTA loads its 128 x 256 slice of W_hh ONCE and keeps it
// in shared memory for all T steps; per step it only brings its 32 x 256 slice of h_{t-1}.
// Steps are separated by a grid-wide barrier (a monotonic counter in global memory: step s is
// released when it reaches (s + 1) * CTAs), because every CTA needs the h values all the others
// produced.  h_{t-1} was written by other SMs with ordinary stores in the same launch, so it
// is read with L1-bypassing loads and laid out in shared memory by the threads themselves in
// the 128-byte swizzle the UMMA descriptor expects (what TMA would have produced).
//
// All CTAs must be resident at once for the barrier to make progress: the host launches the
// kernel only after cudaOccupancyMaxActiveClusters has confirmed that the device takes all
// clusters at the same time, and falls back to one kernel per step otherwise.  Every wait is
// bounded by a clock budget: on expiry (or once the device status flag is seen raised by
// anybody) a CTA stops waiting, still walks through the remaining steps and their cluster
// barriers without blocking, and the host reports FLB200_TIMEOUT.
struct SeqArgs {
  float* gates;          // [T][B][G*H]: input projections + biases in, activated gates out
  float* cells;          // [T][B][H] (LSTM); GRU: q = U_n h + b_hn, the candidate's recurrent part
  const float* b_hn;     // GRU: the recurrent bias of the candidate gate [H]
  int act;               // G = 1: 0 relu, 1 tanh
  float* out;            // layer output [T][B][out_stride]; this direction's columns start at 0
  long long out_stride;
  const float* h0;       // [B][H] initial state (or zeros)
  const float* c0;       // (LSTM)
  unsigned* sync;        // grid barrier counter, zero at launch
  int* status;
  long long wait_budget; // clocks per wait
  int T, B, H, KS, reverse;
  int absent_cta;        // test hook: this CTA never arrives at the grid barrier (-1: none)
};

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_volatile_i32(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Phase accounting of CTA 0, thread 0 (build with -DFLB200_RNN_PROFILE): clocks spent waiting at
// the barrier, loading h, in the MMAs and the accumulator copy, at the cluster barrier, in the
// cell update and in the closing fence, summed over the steps and printed by the host.
#ifdef FLB200_RNN_PROFILE
static __device__ long long g_rnn_profile[8];
#define RNN_PROF_MARK(slot)                                   \
  if (blockIdx.x == 0 && threadIdx.x == 0) {                  \
    const long long now__ = clock64();                        \
    prof[slot] += now__ - prof_t;                             \
    prof_t = now__;                                           \
  }
#else
#define RNN_PROF_MARK(slot)
#endif

constexpr int kSeqThreads = 256;  // warp 0 loads W_hh, warp 1 issues MMAs, warps 2-5 copy the
                                  // accumulator; all eight warps load h and update cells

// G = 4: LSTM (gates i, f, g, o; the running state of a thread's pairs is c).  G = 3: GRU (gates
// r, z, n with n = tanh(x_n + r * (U_n h + b_hn)); the running state is h itself): the
// cluster's UMMA tile holds 96 live rows, the fourth gate's rows are zeros.  G = 1: the plain
// cells h = relu / tanh(x + U h): 32 live rows.
template <int KS, int G>
__global__ void __launch_bounds__(kSeqThreads)
rnn_sequence_kernel(const __grid_constant__ CUtensorMap map_w, const SeqArgs a) {
  constexpr int kUnits = 32 / KS;                       // hidden units this CTA updates
  constexpr int kItems = (kUnits * 32 + kSeqThreads - 1) / kSeqThreads;  // (unit, batch) per thread
  constexpr int kLoads = 32 * (kSliceK / 4) / kSeqThreads;               // float4 of h per thread
  extern __shared__ char smem_raw[];
  char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                        ~static_cast<uintptr_t>(1023));
  char* a_tiles = tiles;
  char* b_tiles = tiles + kStagesK * kABytes;
  float* part = reinterpret_cast<float*>(b_tiles + kStagesK * kBBytes);
  uint64_t* w_bar = reinterpret_cast<uint64_t*>(part + kBM * kPartStride);
  uint64_t* done_bar = w_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();
  const int group = blockIdx.x / KS;
  const int H = a.H, B = a.B;
  const unsigned n_ctas = gridDim.x;

  if (threadIdx.x == 0) {
    mbar_init(w_bar, 1);
    mbar_init(done_bar, 1);
    *failed = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 32);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {  // the resident slice of W_hh: 8 * G boxes, one barrier
    if (lane == 0) mbar_expect_tx(w_bar, kStagesK * G * (32 * 128));
    __syncwarp();
    const int s = lane >> 2, g = lane & 3;
    if (g < G) {
      int c[2] = {rank * kSliceK + s * kBK, g * H + group * 32};
      tma_load(&map_w, w_bar, a_tiles + s * kABytes + g * (32 * 128), 2, c);
    }
  }
  if (G < 4) {  // rows 32 G .. 127 of every k tile belong to no gate
    constexpr int kPerStage = (4 - G) * (32 * 128 / 16);
    for (int i = threadIdx.x; i < kStagesK * kPerStage; i += kSeqThreads) {
      const int s = i / kPerStage, rem = i - s * kPerStage;
      *reinterpret_cast<float4*>(a_tiles + s * kABytes + G * (32 * 128) + rem * 16) =
          make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  if (threadIdx.x == 0 && !mbar_wait(w_bar, 0)) *failed = 1;
  __syncthreads();

  const uint32_t idesc = umma_idesc_tf32(32, 0, 0);
  const uint64_t a_desc0 = umma_desc(smem_u32(a_tiles), 16, 1024, 2);
  const uint64_t b_desc0 = umma_desc(smem_u32(b_tiles), 16, 1024, 2);
  const uint32_t part_local = smem_u32(part);

  // The (unit, batch) pairs of this thread stay the same for all steps: the cell state lives
  // in a register, and the step's pre-activations are fetched before the barrier wait.
  int item_b[kItems], item_ul[kItems];
  float c_reg[kItems];
  bool item_live[kItems];
#pragma unroll
  for (int it = 0; it < kItems; ++it) {
    const int idx = threadIdx.x + it * kSeqThreads;
    item_b[it] = idx / kUnits;
    item_ul[it] = rank * kUnits + (idx - item_b[it] * kUnits);
    item_live[it] = idx < kUnits * 32 && item_b[it] < B;
    c_reg[it] = item_live[it] ? (G == 4 ? a.c0 : a.h0)[(long long)item_b[it] * H + group * 32 +
                                                          item_ul[it]]
                              : 0.f;
  }

#ifdef FLB200_RNN_PROFILE
  long long prof[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  long long prof_t = clock64();
#endif
  for (int step = 0; step < a.T; ++step) {
    const int t = a.reverse ? a.T - 1 - step : step;
    const int t_prev = a.reverse ? t + 1 : t - 1;
    // input projections of this step (written before the launch): in flight during the wait
    float* g_t = a.gates + (long long)t * B * G * H;
    float gin[kItems][G];
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      if (!item_live[it]) continue;
      const float* gp = g_t + (long long)item_b[it] * G * H + group * 32 + item_ul[it];
#pragma unroll
      for (int g = 0; g < G; ++g) gin[it][g] = __ldcg(gp + (long long)g * H);
    }
    // ---- wait until every CTA has published h of the previous step
    if (step > 0) {
      if (threadIdx.x == 0 && *failed == 0) {
        const unsigned target = (unsigned)step * n_ctas;
        const long long t0 = clock64();
        while (ld_acquire_u32(a.sync) < target) {
          if (clock64() - t0 > a.wait_budget || ld_volatile_i32(a.status) != 0) {
            *failed = 3;
            atomicExch(a.status, 13);
            break;
          }
        }
      }
      __syncthreads();
    }
    const bool dead = *failed != 0;
    RNN_PROF_MARK(0)
    // ---- this CTA's K slice of h_{t-1}: [32 batch rows][256 k] as 8 swizzled k tiles; all the
    // loads of a thread are issued before the first store
    {
      const float* hp = step == 0 ? a.h0 : a.out + (long long)t_prev * B * a.out_stride;
      const long long hs = step == 0 ? H : a.out_stride;
      float4 v[kLoads];
#pragma unroll
      for (int u = 0; u < kLoads; ++u) {
        const int i = threadIdx.x + u * kSeqThreads;
        const int b = i / (kSliceK / 4), q = i - b * (kSliceK / 4);
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < B && !dead)
          v[u] = __ldcg(reinterpret_cast<const float4*>(hp + (long long)b * hs + rank * kSliceK) + q);
      }
#pragma unroll
      for (int u = 0; u < kLoads; ++u) {
        const int i = threadIdx.x + u * kSeqThreads;
        const int b = i / (kSliceK / 4), q = i - b * (kSliceK / 4);
        const int s = q >> 3, chunk = q & 7;  // k tile, 16-byte chunk of the 128-byte row
        *reinterpret_cast<float4*>(b_tiles + s * kBBytes + b * 128 + ((chunk ^ (b & 7)) << 4)) = v[u];
      }
      fence_proxy_async();  // generic-proxy writes, read by the tensor core next
    }
    __syncthreads();
    RNN_PROF_MARK(1)
    if (warp == 1 && lane == 0) {
      tc_fence_after();
#pragma unroll 1
      for (int s = 0; s < kStagesK; ++s) {
#pragma unroll
        for (int j = 0; j < kBK / kUmmaK; ++j)
          umma_tf32(tmem_base, umma_desc_advance(a_desc0, s * kABytes + j * 32),
                    umma_desc_advance(b_desc0, s * kBBytes + j * 32), idesc, (s | j) ? 1u : 0u);
      }
      umma_commit(done_bar);
    } else if (warp >= 2 && warp < 6) {
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;
      if (!mbar_wait(done_bar, step & 1)) *failed = 2;
      tc_fence_after();
      float v[32];
      tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16), v);
#pragma unroll
      for (int j = 0; j < 32; ++j) part[row * kPartStride + j] = v[j];
      tc_fence_before();
    }
    __syncthreads();
    RNN_PROF_MARK(2)
    cluster_sync_all();  // the cluster's partial tiles are complete and visible
    RNN_PROF_MARK(3)
    if (*failed == 0) {
#pragma unroll
      for (int it = 0; it < kItems; ++it) {
        if (!item_live[it]) continue;
        const int b = item_b[it], ul = item_ul[it];
        float pr[KS][G];
#pragma unroll
        for (int q = 0; q < KS; ++q) {
          const uint32_t base = mapa_u32(part_local, (uint32_t)q);
#pragma unroll
          for (int g = 0; g < G; ++g)
            pr[q][g] = ld_cluster_f32(base + (uint32_t)(((g * 32 + ul) * kPartStride + b) * 4));
        }
        float pre[G];
#pragma unroll
        for (int g = 0; g < G; ++g) pre[g] = 0.f;
#pragma unroll
        for (int q = 0; q < KS; ++q)  // same order as lstm_step_kernel: bit-identical sums
#pragma unroll
          for (int g = 0; g < G; ++g) pre[g] += pr[q][g];
        const int j = group * 32 + ul;
        float* gp = g_t + (long long)b * G * H + j;
        if constexpr (G == 4) {
          const float i = sigmoid_(pre[0] + gin[it][0]), f = sigmoid_(pre[1] + gin[it][1]);
          const float gg = tanhf(pre[2] + gin[it][2]), o = sigmoid_(pre[3] + gin[it][3]);
          const float c = f * c_reg[it] + i * gg;
          c_reg[it] = c;
          gp[0] = i; gp[H] = f; gp[2 * H] = gg; gp[3 * H] = o;
          a.cells[((long long)t * B + b) * H + j] = c;
          a.out[((long long)t * B + b) * a.out_stride + j] = o * tanhf(c);
        } else if constexpr (G == 1) {
          const float v = pre[0] + gin[it][0];
          const float h = a.act == 0 ? fmaxf(v, 0.f) : tanhf(v);
          gp[0] = h;
          a.out[((long long)t * B + b) * a.out_stride + j] = h;
        } else {
          const float r = sigmoid_(pre[0] + gin[it][0]), z = sigmoid_(pre[1] + gin[it][1]);
          const float q = pre[2] + a.b_hn[j];
          const float n = tanhf(gin[it][2] + r * q);
          const float h = (1.f - z) * n + z * c_reg[it];
          c_reg[it] = h;
          gp[0] = r; gp[H] = z; gp[2 * H] = n;
          a.cells[((long long)t * B + b) * H + j] = q;
          a.out[((long long)t * B + b) * a.out_stride + j] = h;
        }
      }
    }
    RNN_PROF_MARK(4)
    __threadfence();
    __syncthreads();
    // the peers' reads of this CTA's partial tile are over once they arrive below, and the
    // tile is only rewritten after the next grid barrier
    if (threadIdx.x == 0 && (int)blockIdx.x != a.absent_cta) red_release_add(a.sync, 1u);
    RNN_PROF_MARK(5)
  }
#ifdef FLB200_RNN_PROFILE
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (int i = 0; i < 8; ++i) g_rnn_profile[i] = prof[i];
#endif
  __syncthreads();
  cluster_sync_all();  // nobody leaves while a peer may still read its partial tile
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
}

// ----------------------------------------------------------------------------------------
// The backward recurrence of one (layer, direction) as one persistent kernel.
//
// Per step (walking time against the forward direction):
//   dgates_t          = cell gradient of (dh_t + dy_t, dc_t)          (element-wise)
//   dh_{t-1}[b][k]    = sum_r dgates_t[b][r] * W_hh[r][k]             (r over the 4H gate rows)
// Work split: the H outputs k form H / 128 row tiles of one UMMA (M = 128 outputs, N = 32
// batch columns), the 4H gate rows are split into SL = H / 64 slices of 256; one CTA per
// (tile, slice), H / 128 * SL of them (128 at H = 1024), no clusters.  A CTA keeps its
// 256 x 128 block of W_hh resident in shared memory for all steps -- read straight from the
// forward weights as an MN-major operand (the output index k is the contiguous one), no
// transposed copy -- and per step loads its 32 x 256 slice of dgates_t, contracts, and writes
// its 128 x 32 partial tile to a small exchange buffer in global memory.  After a grid barrier
// every (batch, output) pair is finished by exactly one thread of the grid: it adds the SL
// partial sums in slice order and immediately runs the cell gradient of the next step (dh and
// dc of its pair live in registers for the whole sequence), writes the new dgates, and a
// second grid barrier releases the next contraction.  (Clusters that sum the partial tiles
// over distributed shared memory would save the first barrier, but at H = 1024 they would
// have to be 16 CTAs large and the device holds only 7 such clusters at a time.)
// Barrier, bounded waits and residency rule as in lstm_sequence_kernel.
struct SeqBwdArgs {
  const float* gates;    // [T][B][G*H] activated gates of the forward pass
  const float* cells;    // [T][B][H]; GRU: q, the candidate's recurrent part
  const float* c0;       // [B][H]; GRU: h0
  const float* out;      // GRU: the forward output (h of every step), this direction's columns
  long long out_stride;
  const float* dy;       // gradient of the layer output, this direction's first column, or null
  long long dy_stride;
  const float* dh0;      // [B][H] gradient of the final hidden / cell state, or null
  const float* dc0;
  float* dgates;         // [T][B][G*H] out: gate gradients (also the operand of the weight GEMMs)
  int act;               // G = 1: 0 relu, 1 tanh
  float* dgh;            // GRU: the gate gradients as the recurrent side sees them (dn * r for
                         // the candidate); LSTM: == dgates
  float* dh_out;         // [B][H] out: gradient of the initial hidden / cell state
  float* dc_out;
  float* xbuf;           // [SL][H][32] partial sums of one step
  unsigned* sync;
  int* status;
  long long wait_budget;
  int T, B, H, reverse;
};

// Arrives at the grid barrier and waits for barrier number `index` (0, 1, 2, ...) to complete.
// Called by every thread; returns with the CTA synchronised.
__device__ __forceinline__ void grid_barrier(unsigned* sync, unsigned index, unsigned n_ctas,
                                             long long budget, int* status, volatile int* failed,
                                             int code) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    red_release_add(sync, 1u);
    if (*failed == 0) {
      const unsigned target = (index + 1u) * n_ctas;
      const long long t0 = clock64();
      while (ld_acquire_u32(sync) < target) {
        if (clock64() - t0 > budget || ld_volatile_i32(status) != 0) {
          *failed = 3;
          atomicExch(status, code);
          break;
        }
      }
    }
  }
  __syncthreads();
}

// G as in rnn_sequence_kernel; SL = G * H / 256 slices of the gate rows.  GRU: the running dc
// of a pair is the direct part dh * z of its next dh.
template <int SL, int G>
__global__ void __launch_bounds__(kSeqThreads)
rnn_sequence_backward_kernel(const __grid_constant__ CUtensorMap map_w, const SeqBwdArgs a) {
  constexpr int kUnits = (kBM + SL - 1) / SL;                             // outputs per CTA
  constexpr int kItems = (kUnits * 32 + kSeqThreads - 1) / kSeqThreads;
  constexpr int kLoads = 32 * (kSliceK / 4) / kSeqThreads;
  extern __shared__ char smem_raw[];
  char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                        ~static_cast<uintptr_t>(1023));
  char* a_tiles = tiles;
  char* b_tiles = tiles + kStagesK * kABytes;
  float* part = reinterpret_cast<float*>(b_tiles + kStagesK * kBBytes);
  uint64_t* w_bar = reinterpret_cast<uint64_t*>(part + kBM * kPartStride);
  uint64_t* done_bar = w_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = blockIdx.x % SL;          // slice of the gate rows
  const int mt = blockIdx.x / SL;            // tile of 128 outputs
  const int H = a.H, B = a.B;
  const unsigned n_ctas = gridDim.x;

  if (threadIdx.x == 0) {
    mbar_init(w_bar, 1);
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
    // W_hh[r][k], r in this CTA's slice, k in this tile: stage s = gate rows 32 s .. 32 s + 31,
    // box j = outputs 32 j .. 32 j + 31 (the layout of an MN-major A tile)
    if (lane == 0) mbar_expect_tx(w_bar, kStagesK * kABytes);
    __syncwarp();
    const int s = lane >> 2, j = lane & 3;
    int c[2] = {mt * kBM + 32 * j, rank * kSliceK + s * kBK};
    tma_load(&map_w, w_bar, a_tiles + s * kABytes + j * (kBK * 128), 2, c);
  }
  if (threadIdx.x == 0 && !mbar_wait(w_bar, 0)) *failed = 1;
  __syncthreads();

  const uint32_t idesc = umma_idesc_tf32(32, 1, 0);
  const uint64_t a_desc0 = umma_desc(smem_u32(a_tiles), kBK * 128, 512, 1);
  const uint64_t b_desc0 = umma_desc(smem_u32(b_tiles), 16, 1024, 2);

  int item_b[kItems], item_k[kItems];
  float dh[kItems], dc[kItems];
  bool item_live[kItems];
#pragma unroll
  for (int it = 0; it < kItems; ++it) {
    const int idx = threadIdx.x + it * kSeqThreads;
    item_b[it] = idx / kUnits;
    const int unit = rank * kUnits + (idx - item_b[it] * kUnits);  // within the 128-output tile
    item_k[it] = mt * kBM + unit;                                  // output (hidden unit)
    item_live[it] = idx < kUnits * 32 && unit < kBM && item_b[it] < B;
    const long long at = (long long)item_b[it] * H + item_k[it];
    dh[it] = item_live[it] && a.dh0 ? a.dh0[at] : 0.f;
    dc[it] = G == 4 && item_live[it] && a.dc0 ? a.dc0[at] : 0.f;
  }

  unsigned barrier_index = 0;
  for (int sb = 0; sb < a.T; ++sb) {
    const int step = a.T - 1 - sb;                       // index in forward order
    const int t = a.reverse ? a.T - 1 - step : step;
    const int t_prev = a.reverse ? t + 1 : t - 1;        // the forward pass's previous time
    // ---- cell gradient of time t for this thread's (batch, unit) pairs
    if (*failed == 0) {
#pragma unroll
      for (int it = 0; it < kItems; ++it) {
        if (!item_live[it]) continue;
        const int b = item_b[it], j = item_k[it];
        const float* g = a.gates + ((long long)t * B + b) * G * H + j;
        float d = dh[it];
        if (a.dy) d += __ldcg(a.dy + ((long long)t * B + b) * a.dy_stride + j);
        float* o = a.dgates + ((long long)t * B + b) * G * H + j;
        if constexpr (G == 4) {
          const float gi = __ldcg(g), gf = __ldcg(g + H), gg = __ldcg(g + 2 * H), go = __ldcg(g + 3 * H);
          const float c = __ldcg(a.cells + ((long long)t * B + b) * H + j);
          const float cp = step == 0 ? __ldcg(a.c0 + (long long)b * H + j)
                                     : __ldcg(a.cells + ((long long)t_prev * B + b) * H + j);
          const float tc = tanhf(c);
          const float dct = dc[it] + d * go * (1.f - tc * tc);
          o[0] = dct * gg * gi * (1.f - gi);
          o[H] = dct * cp * gf * (1.f - gf);
          o[2 * H] = dct * gi * (1.f - gg * gg);
          o[3 * H] = d * tc * go * (1.f - go);
          dc[it] = dct * gf;
        } else if constexpr (G == 1) {
          const float h = __ldcg(g);
          o[0] = a.act == 0 ? (h > 0.f ? d : 0.f) : d * (1.f - h * h);
        } else {
          const float r = __ldcg(g), z = __ldcg(g + H), n = __ldcg(g + 2 * H);
          const float q = __ldcg(a.cells + ((long long)t * B + b) * H + j);
          const float hp = step == 0 ? __ldcg(a.c0 + (long long)b * H + j)
                                     : __ldcg(a.out + ((long long)t_prev * B + b) * a.out_stride + j);
          const float dn = d * (1.f - z) * (1.f - n * n);
          const float dz = d * (hp - n) * z * (1.f - z);
          const float dr = dn * q * r * (1.f - r);
          float* oh = a.dgh + ((long long)t * B + b) * G * H + j;
          o[0] = dr; o[H] = dz; o[2 * H] = dn;
          oh[0] = dr; oh[H] = dz; oh[2 * H] = dn * r;
          dc[it] = d * z;
        }
      }
    }
    // ---- every CTA's dgates_t must be complete before anybody contracts over them
    grid_barrier(a.sync, barrier_index++, n_ctas, a.wait_budget, a.status, failed, 14);
    const bool dead = *failed != 0;
    {
      const float* src = a.dgh + (long long)t * B * G * H + rank * kSliceK;
      float4 v[kLoads];
#pragma unroll
      for (int u = 0; u < kLoads; ++u) {
        const int i = threadIdx.x + u * kSeqThreads;
        const int b = i / (kSliceK / 4), q = i - b * (kSliceK / 4);
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < B && !dead)
          v[u] = __ldcg(reinterpret_cast<const float4*>(src + (long long)b * G * H) + q);
      }
#pragma unroll
      for (int u = 0; u < kLoads; ++u) {
        const int i = threadIdx.x + u * kSeqThreads;
        const int b = i / (kSliceK / 4), q = i - b * (kSliceK / 4);
        const int s = q >> 3, chunk = q & 7;
        *reinterpret_cast<float4*>(b_tiles + s * kBBytes + b * 128 + ((chunk ^ (b & 7)) << 4)) = v[u];
      }
      fence_proxy_async();
    }
    __syncthreads();
    if (warp == 1 && lane == 0) {
      tc_fence_after();
#pragma unroll 1
      for (int s = 0; s < kStagesK; ++s) {
#pragma unroll
        for (int j = 0; j < kBK / kUmmaK; ++j)
          umma_tf32(tmem_base, umma_desc_advance(a_desc0, s * kABytes + j * 1024),
                    umma_desc_advance(b_desc0, s * kBBytes + j * 32), idesc, (s | j) ? 1u : 0u);
      }
      umma_commit(done_bar);
    } else if (warp >= 2 && warp < 6) {
      // the partial tile of this CTA, [output][batch], straight to the exchange buffer
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;
      if (!mbar_wait(done_bar, sb & 1)) *failed = 2;
      tc_fence_after();
      float v[32];
      tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16), v);
      float4* dst = reinterpret_cast<float4*>(a.xbuf + ((long long)rank * H + mt * kBM + row) * 32);
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      tc_fence_before();
    }
    grid_barrier(a.sync, barrier_index++, n_ctas, a.wait_budget, a.status, failed, 15);
    // ---- dh_{t-1} of this thread's pairs: the SL partial sums, in slice order
    if (*failed == 0) {
#pragma unroll
      for (int it = 0; it < kItems; ++it) {
        if (!item_live[it]) continue;
        float pr[SL];
#pragma unroll
        for (int q = 0; q < SL; ++q)
          pr[q] = __ldcg(a.xbuf + ((long long)q * H + item_k[it]) * 32 + item_b[it]);
        float sum = 0.f;
#pragma unroll
        for (int q = 0; q < SL; ++q) sum += pr[q];
        dh[it] = G == 3 ? dc[it] + sum : sum;
      }
    }
    // (the exchange buffer is rewritten only after the next step's first barrier, which every
    // CTA reaches after these reads)
  }
  if (*failed == 0) {
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      if (!item_live[it]) continue;
      const long long at = (long long)item_b[it] * H + item_k[it];
      a.dh_out[at] = dh[it];
      if (G == 4) a.dc_out[at] = dc[it];
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
}

typedef void (*SeqBwdKernel)(const CUtensorMap, const SeqBwdArgs);
SeqBwdKernel sequence_backward_kernel_for(int sl, int G) {
  if (G == 1) {
    switch (sl) {
      case 1: return rnn_sequence_backward_kernel<1, 1>;
      case 2: return rnn_sequence_backward_kernel<2, 1>;
      default: return rnn_sequence_backward_kernel<4, 1>;
    }
  }
  if (G == 3) {
    switch (sl) {
      case 3: return rnn_sequence_backward_kernel<3, 3>;
      case 6: return rnn_sequence_backward_kernel<6, 3>;
      default: return rnn_sequence_backward_kernel<12, 3>;
    }
  }
  switch (sl) {
    case 4: return rnn_sequence_backward_kernel<4, 4>;
    case 8: return rnn_sequence_backward_kernel<8, 4>;
    default: return rnn_sequence_backward_kernel<16, 4>;
  }
}

typedef void (*SeqKernel)(const CUtensorMap, const SeqArgs);
SeqKernel sequence_kernel_for(int ks, int G) {
  if (G == 1) {
    switch (ks) {
      case 1: return rnn_sequence_kernel<1, 1>;
      case 2: return rnn_sequence_kernel<2, 1>;
      case 4: return rnn_sequence_kernel<4, 1>;
      default: return rnn_sequence_kernel<8, 1>;
    }
  }
  if (G == 3) {
    switch (ks) {
      case 1: return rnn_sequence_kernel<1, 3>;
      case 2: return rnn_sequence_kernel<2, 3>;
      case 4: return rnn_sequence_kernel<4, 3>;
      default: return rnn_sequence_kernel<8, 3>;
    }
  }
  switch (ks) {
    case 1: return rnn_sequence_kernel<1, 4>;
    case 2: return rnn_sequence_kernel<2, 4>;
    case 4: return rnn_sequence_kernel<4, 4>;
    default: return rnn_sequence_kernel<8, 4>;
  }
}

}  // namespace

bool lstm_step_supported(int math_mode, int B, int H) {
  if (math_mode != FLB200_MATH_TF32 || !flb200_has_tensor_core_path()) return false;
  if (B < 1 || B > 32 || H % kSliceK != 0) return false;
  const int ks = H / kSliceK;
  return ks == 1 || ks == 2 || ks == 4 || ks == 8;
}

int lstm_step_weight_map(CUtensorMap* map, const float* w_hh, int H, int G) {
  const uint64_t dims[2] = {(uint64_t)H, (uint64_t)G * H};
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

bool lstm_sequence_supported(int math_mode, int B, int H, int G) {
  if (!lstm_step_supported(math_mode, B, H) || (G != 1 && G != 3 && G != 4)) return false;
  // every CTA of the kernel has to be resident at the same time (grid-wide barrier per step)
  // (one answer per device and cluster size 1, 2, 4 or 8)
  static int max_clusters[64][12];
  static bool known[64][12] = {{false}};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  const int ks = H / kSliceK;
  const int slot = (ks == 1 ? 0 : (ks == 2 ? 1 : (ks == 4 ? 2 : 3))) + (G == 3 ? 4 : (G == 1 ? 8 : 0));
  if (!known[dev][slot]) {
    if (cudaFuncSetAttribute(sequence_kernel_for(ks, G), cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemBytes) != cudaSuccess) {
      (void)cudaGetLastError();
      return false;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(H / 32 * ks));
    cfg.blockDim = dim3(kSeqThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, sequence_kernel_for(ks, G), &cfg) != cudaSuccess) {
      (void)cudaGetLastError();
      return false;
    }
    max_clusters[dev][slot] = n;
    known[dev][slot] = true;
  }
  return max_clusters[dev][slot] >= H / 32;
}

int lstm_sequence_forward(const CUtensorMap& map_w, float* gates, float* cells, float* out,
                          long long out_stride, const float* h0, const float* c0, unsigned* sync,
                          int T, int B, int H, int reverse, long long wait_budget, int absent_cta,
                          cudaStream_t st, int G, const float* b_hn, int act) {
  FLB200_REQUIRE(G == 4 || G == 1 || (G == 3 && b_hn),
                 "rnn_sequence_forward: LSTM, a plain cell, or GRU with its bias");
  SeqArgs a{};
  a.b_hn = b_hn;
  a.act = act;
  a.gates = gates; a.cells = cells; a.out = out; a.out_stride = out_stride;
  a.h0 = h0; a.c0 = c0; a.sync = sync; a.status = tc::status_ptr();
  a.wait_budget = wait_budget > 0 ? wait_budget : tc::kWaitBudget;
  a.T = T; a.B = B; a.H = H; a.KS = H / kSliceK; a.reverse = reverse; a.absent_cta = absent_cta;
  FLB200_REQUIRE((out_stride % 4) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(h0) & 15) == 0,
                 "lstm_sequence_forward: rows must be 16-byte aligned");
  FLB200_CUDA_CHECK(cudaMemsetAsync(sync, 0, sizeof(unsigned), st));
  SeqKernel kernel = sequence_kernel_for(a.KS, G);
  FLB200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)(H / 32 * a.KS));
  cfg.blockDim = dim3(kSeqThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)a.KS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FLB200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, map_w, a));
  FLB200_AFTER_LAUNCH("lstm_sequence_forward");
  tc::count_tc_launch();
#ifdef FLB200_RNN_PROFILE
  {
    cudaStreamSynchronize(st);
    long long h[8];
    cudaMemcpyFromSymbol(h, g_rnn_profile, sizeof(h));
    fprintf(stderr,
            "lstm sequence profile T=%d: clocks per step: barrier wait %.0f, h load %.0f, mma + "
            "accumulator copy %.0f, cluster barrier %.0f, cell update %.0f, fence + arrive %.0f\n",
            T, (double)h[0] / T, (double)h[1] / T, (double)h[2] / T, (double)h[3] / T,
            (double)h[4] / T, (double)h[5] / T);
  }
#endif
  return FLB200_OK;
}

bool lstm_sequence_backward_supported(int math_mode, int B, int H, int G) {
  if (math_mode != FLB200_MATH_TF32 || !flb200_has_tensor_core_path()) return false;
  if (B < 1 || B > 32 || (H != 256 && H != 512 && H != 1024) || (G != 1 && G != 3 && G != 4))
    return false;
  // every CTA resident at once: one per SM (the resident weights fill its shared memory)
  static int per_sm[64][9];
  static bool known[64][9] = {{false}};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  const int slot = (H == 256 ? 0 : (H == 512 ? 1 : 2)) + (G == 3 ? 3 : (G == 1 ? 6 : 0));
  if (!known[dev][slot]) {
    SeqBwdKernel kernel = sequence_backward_kernel_for(G * H / kSliceK, G);
    int n = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
            cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kSeqThreads, kSmemBytes) !=
            cudaSuccess) {
      (void)cudaGetLastError();
      n = 0;
    }
    per_sm[dev][slot] = n;
    known[dev][slot] = true;
  }
  return (long long)per_sm[dev][slot] * device_info().sm_count >=
         (long long)(H / kBM) * (G * H / kSliceK);
}

size_t lstm_sequence_backward_scratch_bytes(int H) {
  return (size_t)(H / 64) * H * 32 * sizeof(float);  // the LSTM's 4H / 256 slices: the larger
}

int lstm_sequence_weight_map_transposed(CUtensorMap* map, const float* w_hh, int H, int G) {
  // W_hh [G*H][H] read as an MN-major operand: the output index (column of W_hh) is contiguous
  const uint64_t dims[2] = {(uint64_t)H, (uint64_t)G * H};
  const uint64_t strides[1] = {(uint64_t)H * 4};
  const uint32_t box[2] = {32, 32};
  return tc::make_tensor_map(map, w_hh, 2, dims, strides, box, tc::kMapMnMajor);
}

int lstm_sequence_backward(const CUtensorMap& map_wt, const float* gates, const float* cells,
                           const float* c0, const float* dy, long long dy_stride,
                           const float* dh0, const float* dc0, float* dgates, float* dh_out,
                           float* dc_out, float* xbuf, unsigned* sync, int T, int B, int H,
                           int reverse, cudaStream_t st, int G, float* dgh, const float* out,
                           long long out_stride, int act) {
  FLB200_REQUIRE(G == 4 || G == 1 || (G == 3 && dgh && out && c0),
                 "rnn_sequence_backward: LSTM, or GRU with its second gradient buffer, the "
                 "forward output and h0");
  SeqBwdArgs a{};
  a.dgh = G == 3 ? dgh : dgates; a.out = out; a.out_stride = out_stride; a.act = act;
  a.gates = gates; a.cells = cells; a.c0 = c0; a.dy = dy; a.dy_stride = dy_stride;
  a.dh0 = dh0; a.dc0 = dc0; a.dgates = dgates; a.dh_out = dh_out; a.dc_out = dc_out;
  a.xbuf = xbuf; a.sync = sync; a.status = tc::status_ptr(); a.wait_budget = tc::kWaitBudget;
  a.T = T; a.B = B; a.H = H; a.reverse = reverse;
  FLB200_REQUIRE((reinterpret_cast<uintptr_t>(dgates) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(xbuf) & 15) == 0,
                 "lstm_sequence_backward: buffers must be 16-byte aligned");
  FLB200_CUDA_CHECK(cudaMemsetAsync(sync, 0, sizeof(unsigned), st));
  const int sl = G * H / kSliceK;
  SeqBwdKernel kernel = sequence_backward_kernel_for(sl, G);
  FLB200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes));
  kernel<<<(unsigned)(H / kBM * sl), kSeqThreads, kSmemBytes, st>>>(map_wt, a);
  FLB200_AFTER_LAUNCH("lstm_sequence_backward");
  tc::count_tc_launch();
  return FLB200_OK;
}

}  // namespace flb200
