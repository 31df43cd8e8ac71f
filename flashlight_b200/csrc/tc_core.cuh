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
// Adds to the barrier's pending byte count without arriving; the phase cannot complete before
// the arrival that follows.
__device__ __forceinline__ void mbar_expect_tx_only(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
// Byte count of one sub-block of a stage: the last sub-block of the stage also arrives.
__device__ __forceinline__ void mbar_post_tx(uint64_t* bar, uint32_t bytes, bool last) {
  if (last) mbar_expect_tx(bar, bytes);
  else mbar_expect_tx_only(bar, bytes);
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
// TMA store of a 3-D box from shared memory (bulk-group completion); elements outside the
// tensor are clipped by the hardware.  c[0] is the contiguous coordinate (16-byte rule applies).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int c0,
                                             int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(map)),
      "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Waits until at most N of this thread's bulk groups still READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
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
  } else if (rank == 4) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4, %5, %6}], [%2];" ::"r"(d), "l"(m), "r"(b), "r"(c[0]), "r"(c[1]), "r"(c[2]),
        "r"(c[3])
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4, %5, %6, %7}], [%2];" ::"r"(d), "l"(m), "r"(b), "r"(c[0]), "r"(c[1]), "r"(c[2]),
        "r"(c[3]), "r"(c[4])
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
// bf16 operands (kind::f16), fp32 accumulate; K = 16 per instruction.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
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
// The descriptor of the same layout `bytes` further into shared memory.  The start-address
// field is the low 14 bits (address / 16); any address inside the CTA's shared memory fits, so
// the addition never carries into the neighbouring field and touches the low word only.
// Building a descriptor from scratch costs the single issuing thread tens of dependent
// instructions; measured, an MMA loop that rebuilds both descriptors per instruction issues one
// tcgen05.mma per ~220 clocks, one that offsets two prebuilt descriptors one per ~50 clocks
// (the shared-memory read time of a 128 x 64 x 8 TF32 MMA).
__device__ __forceinline__ uint64_t umma_desc_advance(uint64_t desc, uint32_t bytes) {
  const uint32_t lo = (uint32_t)desc + (bytes >> 4);
  return (desc & 0xffffffff00000000ull) | lo;
}
// Instruction descriptor for kind::tf32, fp32 accumulate, M = 128.
__host__ __device__ inline uint32_t umma_idesc_tf32(int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

// Instruction descriptor for kind::f16 with bf16 operands (format 1), fp32 accumulate, M = 128.
__host__ __device__ inline uint32_t umma_idesc_bf16(int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

// Coordinates of one operand box: every term is a multiply-add with per-dimension
// multipliers prepared on the host (zero where a term does not apply), so that the single
// producer thread needs no divisions, no branches and no indexed local arrays per stage.
__device__ __forceinline__ void operand_coords(const OperandCoords& p, int mn, int k_lo, int k_hi,
                                               int z, int* c) {
#pragma unroll
  for (int d = 0; d < 4; ++d)
    c[d] = p.base[d] + (mn >> p.mn_shift) * p.mn_mul[d] + k_lo * p.k_mul[d] +
           k_hi * p.k2_mul[d] + z * p.z_mul[d];
}

// ------------------------------------------------------ CTA pairs (cta_group::2)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `saddr` (a shared::cta address) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa_u32(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// TMA load into this CTA's shared memory whose bytes complete on a barrier given by its
// shared::cluster address (the leader's).  No multicast.
__device__ __forceinline__ void tma_load_pair(const CUtensorMap* map, uint32_t bar_cluster_addr,
                                              void* dst, int rank, const int* c) {
  const uint32_t d = smem_u32(dst);
  const uint64_t m = reinterpret_cast<uint64_t>(map);
  if (rank == 2) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(d),
        "l"(m), "r"(bar_cluster_addr), "r"(c[0]), "r"(c[1])
        : "memory");
  } else if (rank == 3) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(d),
        "l"(m), "r"(bar_cluster_addr), "r"(c[0]), "r"(c[1]), "r"(c[2])
        : "memory");
  } else if (rank == 4) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(d),
        "l"(m), "r"(bar_cluster_addr), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3])
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(d),
        "l"(m), "r"(bar_cluster_addr), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]), "r"(c[4])
        : "memory");
  }
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair once every
// MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)),
      "h"(mask)
      : "memory");
}
// kind::tf32, fp32 accumulate, M = 256 across the pair.
__host__ __device__ inline uint32_t umma_idesc_tf32_pair(int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)((2 * kBM) >> 4) << 24);
}

__device__ __forceinline__ long long epi_off(int idx, int div, long long stride,
                                             long long outer) {
  if (div == 0) return (long long)idx * stride;
  const int hi = idx / div;
  return (long long)hi * outer + (long long)(idx - hi * div) * stride;
}

}  // namespace tc
}  // namespace flb200
