// tcgen05 / TMA / mbarrier primitives and the generic TF32 tensor-core
// contraction kernel for sm_100a.
//
//   D[z][m][n] = sum_k A[z](m,k) * B[z](k,n),   fp32 operands read as TF32,
//   fp32 accumulation in tensor memory (TMEM).
//
// One CTA computes one 128 x BN output tile over a range of K (split-K aware):
//   warp 0   : TMA producer (one lane issues cp.async.bulk.tensor loads, no multicast)
//   warp 1   : allocates TMEM, one lane issues tcgen05.mma and tcgen05.commit
//   warps 2-5: epilogue — tcgen05.ld the accumulator rows and store them
// A STAGES-deep ring of shared-memory tiles is handed between producer and MMA
// issuer with full/empty mbarriers; smem tiles use the 128-byte swizzle that both
// TMA and the UMMA shared-memory descriptors understand.
//
// Either operand may be K-major (k contiguous in memory) or MN-major (m or n
// contiguous): a K-major tile is ONE TMA box [32 k][rows]; an MN-major tile is
// rows/32 boxes [32 rows][32 k] laid side by side, each a column of 8x128-byte
// swizzle atoms.  K advances 32 elements (128 bytes) per stage and 8 per MMA.
//
// Every wait is bounded by a clock budget; a wait that runs out raises a flag in
// global memory, the CTA drains and returns, and the host reports FLB200_TIMEOUT.
#pragma once
#include "tc_gemm.cuh"

namespace flb200 {
namespace tc {

constexpr int kUmmaK = 8;       // K per tcgen05.mma for kind::tf32
constexpr int kThreads = 192;   // 6 warps
constexpr long long kWaitBudget = 4000000000LL;  // ~2 s of SM clocks

// ------------------------------------------------------------------ PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the clock budget ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitBudget) return false;
  }
  return true;
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load(const CUtensorMap* map, uint64_t* bar, void* dst,
                                         int rank, const int* c) {
  const uint32_t d = smem_u32(dst), b = smem_u32(bar);
  const uint64_t m = reinterpret_cast<uint64_t>(map);
  if (rank == 2) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4}], [%2];" ::"r"(d), "l"(m), "r"(b), "r"(c[0]), "r"(c[1])
        : "memory");
  } else if (rank == 3) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4, %5}], [%2];" ::"r"(d), "l"(m), "r"(b), "r"(c[0]), "r"(c[1]), "r"(c[2])
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4, %5, %6}], [%2];" ::"r"(d), "l"(m), "r"(b), "r"(c[0]), "r"(c[1]), "r"(c[2]),
        "r"(c[3])
        : "memory");
  }
}
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          smem_u32(bar))
      : "memory");
}
// 32 consecutive accumulator columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// UMMA shared-memory descriptor with the sm_100 version bit.
//   K-major tile : 128-byte swizzle of 16-byte chunks (layout type 2); rows of 128 bytes,
//                  8-row atoms 1024 bytes apart -> LBO 16 B (unused), SBO 1024 B
//   MN-major tile: TF32 operands whose m / n index is contiguous must use the 128-byte
//                  swizzle of 32-BYTE chunks (layout type 1, TMA SWIZZLE_128B_ATOM_32B):
//                  boxes of [32 k][128 B]; atoms along MN are `box_bytes` apart (LBO),
//                  4-k-row swizzle atoms inside a box 512 bytes apart (SBO)
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)layout_type << 61;  // 2 = SWIZZLE_128B, 1 = SWIZZLE_128B_BASE32B
  return d;
}
// Instruction descriptor for kind::tf32, fp32 accumulate, M = 128.
__host__ __device__ inline uint32_t umma_idesc_tf32(int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

__device__ __forceinline__ void operand_coords(const OperandPlan& p, int mn, int k_iter, int z,
                                               int* c) {
#pragma unroll
  for (int d = 0; d < 4; ++d) c[d] = p.base[d];
  int k_hi = 0, k_lo = k_iter;
  if (p.k_inner > 0) {
    k_hi = k_iter / p.k_inner;
    k_lo = k_iter - k_hi * p.k_inner;
  }
  c[p.mn_dim] += mn;
  c[p.k_dim] += k_lo * kBK;
  if (p.k2_dim >= 0) c[p.k2_dim] += k_hi * p.k2_scale;
  if (p.z_dim >= 0) c[p.z_dim] += z;
}

// Issues the TMA loads of one operand tile (ROWS = 128 for A, BN for B) into `dst`.
template <int ROWS>
__device__ __forceinline__ void load_operand(const CUtensorMap* map, const OperandPlan& p,
                                             uint64_t* bar, char* dst, int mn0, int k_iter, int z) {
  int c[4];
  if (p.mn_major) {
#pragma unroll
    for (int j = 0; j < ROWS / 32; ++j) {
      operand_coords(p, mn0 + 32 * j, k_iter, z, c);
      tma_load(map, bar, dst + j * (kBK * 128), p.rank, c);
    }
  } else {
    operand_coords(p, mn0, k_iter, z, c);
    tma_load(map, bar, dst, p.rank, c);
  }
}

__device__ __forceinline__ long long epi_off(int idx, int div, long long stride,
                                             long long outer) {
  if (div == 0) return (long long)idx * stride;
  const int hi = idx / div;
  return (long long)hi * outer + (long long)(idx - hi * div) * stride;
}

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int kABytes = kBM * kBK * 4;  // 16 KB
  static constexpr int kBBytes = BN * kBK * 4;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTileBytes = STAGES * kStageBytes;
  static constexpr int kBarBytes = 256;
  static constexpr int kTotal = kTileBytes + kBarBytes + 1024;  // + slack to align to 1024
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const KernelArgs args) {
  using SL = SmemLayout<BN, STAGES>;
  extern __shared__ char smem_raw[];
  char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                        ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + SL::kTileBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * BN;
  const int z = blockIdx.z / args.splits, split = blockIdx.z - z * args.splits;
  const int it0 = split * args.iters_per_split;
  int it1 = it0 + args.iters_per_split;
  if (it1 > args.k_iters) it1 = args.k_iters;
  const int n_iters = it1 > it0 ? it1 - it0 : 0;
  constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full_bar, 1);
    *failed = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < n_iters; ++i) {
        const int s = i % STAGES;
        const uint32_t round = i / STAGES;
        if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) {
          *failed = 1;
          break;
        }
        char* a_dst = tiles + s * SL::kStageBytes;
        char* b_dst = a_dst + SL::kABytes;
        mbar_expect_tx(&full_bar[s], SL::kStageBytes);
        load_operand<kBM>(&map_a, args.a, &full_bar[s], a_dst, m0, it0 + i, z);
        load_operand<BN>(&map_b, args.b, &full_bar[s], b_dst, n0, it0 + i, z);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_tf32(BN, args.a.mn_major, args.b.mn_major);
      bool ok = true;
      for (int i = 0; i < n_iters && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t round = i / STAGES;
        if (!mbar_wait(&full_bar[s], round & 1)) {
          *failed = 2;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + s * SL::kStageBytes);
        const uint32_t b_addr = a_addr + SL::kABytes;
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          // K-major: step 8 elements = 32 bytes inside the swizzled row;
          // MN-major: step 8 k-rows = one 1024-byte atom inside each box.
          const uint64_t ad = args.a.mn_major
                                  ? umma_desc(a_addr + k * 1024, kBK * 128, 512, 1)
                                  : umma_desc(a_addr + k * 32, 16, 1024, 2);
          const uint64_t bd = args.b.mn_major
                                  ? umma_desc(b_addr + k * 1024, kBK * 128, 512, 1)
                                  : umma_desc(b_addr + k * 32, 16, 1024, 2);
          umma_tf32(tmem_base, ad, bd, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
      }
      umma_commit(tmem_full_bar);    // accumulator complete (or nothing was issued)
    }
  } else {
    // epilogue warps 2..5 own TMEM lanes 32*(warp % 4) .. +31
    const int lane_base = (warp & 3) * 32;
    const int m = m0 + lane_base + lane;
    bool ok = mbar_wait(tmem_full_bar, 0);
    if (!ok) *failed = 3;
    tc_fence_after();
    ok = ok && (*failed == 0);
    const EpiloguePlan& ep = args.ep;
    const bool to_partial = args.splits > 1;
    float* out = to_partial ? args.partial + ((long long)blockIdx.z * args.M) * args.N : ep.out;
    const long long m_off = to_partial ? (long long)m * args.N
                                       : epi_off(m, ep.m_div, ep.m_stride, ep.m_outer) +
                                             (long long)z * ep.z_stride;
    const float bm = (!to_partial && ep.bias_m && m < args.M) ? ep.bias_m[m] : 0.f;
    // padding rows of a padded pixel axis are computed but never stored
    const bool row_live =
        m < args.M && (to_partial || ep.m_valid == 0 || ep.m_div == 0 || (m % ep.m_div) < ep.m_valid);
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (n0 + c0 >= args.N) break;  // uniform across the warp
        float v[32];
        if (n_iters > 0) {
          tmem_ld32(tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)c0, v);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        if (row_live) {
          if (to_partial) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int n = n0 + c0 + j;
              if (n < args.N) out[m_off + n] = v[j];
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int n = n0 + c0 + j;
              if (n < args.N) {
                float* dst = out + m_off + epi_off(n, ep.n_div, ep.n_stride, ep.n_outer);
                float r = ep.alpha * v[j] + bm + (ep.bias_n ? ep.bias_n[n] : 0.f);
                if (ep.beta != 0.f) r += ep.beta * *dst;
                *dst = r;
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *failed != 0 && args.status) atomicExch(args.status, *failed);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Sums split-K partial tiles in split order, then applies the epilogue.
__global__ void __launch_bounds__(256)
tc_splitk_reduce_kernel(const float* __restrict__ partial, EpiloguePlan ep, int M, int N, int Z,
                        int splits) {
  const long long mn = (long long)M * N;
  const long long total = mn * Z;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int z = (int)(i / mn);
    const long long r = i - (long long)z * mn;
    const int m = (int)(r / N), n = (int)(r - (long long)m * N);
    if (ep.m_valid != 0 && ep.m_div != 0 && (m % ep.m_div) >= ep.m_valid) continue;
    float s = 0.f;
    for (int sp = 0; sp < splits; ++sp) s += partial[((long long)z * splits + sp) * mn + r];
    float* dst = ep.out + epi_off(m, ep.m_div, ep.m_stride, ep.m_outer) +
                 epi_off(n, ep.n_div, ep.n_stride, ep.n_outer) + (long long)z * ep.z_stride;
    float v = ep.alpha * s + (ep.bias_m ? ep.bias_m[m] : 0.f) + (ep.bias_n ? ep.bias_n[n] : 0.f);
    if (ep.beta != 0.f) v += ep.beta * *dst;
    *dst = v;
  }
}

}  // namespace tc
}  // namespace flb200
