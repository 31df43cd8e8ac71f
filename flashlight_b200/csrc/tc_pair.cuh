// The persistent tcgen05 contraction on CTA PAIRS (tcgen05 cta_group::2).
//
// Two CTAs of a 2-CTA cluster (two SMs) compute one 256 x BN output tile: each CTA owns
// 128 rows of it (its own accumulator in its own TMEM) and brings its own 128 x 32 A tile,
// but only HALF of the 32 x BN B tile per stage; the tensor cores of both SMs read both
// halves.  Per SM and stage that is 16 KB + BN * 64 bytes instead of 16 KB + BN * 128:
// at BN = 256 a third less TMA traffic for the same math, and six stages fit in the ring
// instead of four.  One tcgen05.mma.cta_group::2 issued by the leader CTA (cluster rank 0)
// drives both SMs.
//
// Hand-offs (every wait bounded as in tc_kernel.cuh):
//   full[s]    leader's barrier; the TMA loads of BOTH CTAs complete their bytes on it
//              (cp.async.bulk.tensor .cta_group::2, plain loads: nothing is multicast)
//   empty[s]   one per CTA; tcgen05.commit.cta_group::2 arrives on both when the MMAs that
//              read stage s are done
//   tfull[a]   one per CTA; tcgen05.commit arrives on both when accumulator a is complete
//   tempty[a]  leader's barrier; the 8 epilogue warps of each CTA arrive on it (the peer's
//              through a remote mbarrier.arrive) once they have drained accumulator a
// The cluster synchronises after barrier initialisation and before TMEM is freed, so no CTA
// signals a barrier of a peer that has not started or has already left.
//
// A policy used here adds to the interface of tc_kernel.cuh:
//   __device__ int  num_pair_tiles() const;
//   __device__ void decode_pair(int pair_tile, int rank, Tile&) const;  // this CTA's half
//   __device__ void load_pair(const CUtensorMap* a, const CUtensorMap* b, const Tile&, LoadState&,
//                             uint32_t full_bar_cluster_addr, char* a_dst, char* b_dst,
//                             int rank, int lane) const;
//                             // called by the whole producer warp; lane i issues copy i.
//                             // A: this CTA's 128 rows; B: rows n0 + rank * BN/2 ...
#pragma once
#include <cuda_runtime.h>

#include "tc_kernel.cuh"

namespace flb200 {
namespace tc {

template <int BN, int STAGES>
struct PairSmemLayout {
  static constexpr int kABytes = kBM * kBK * 4;         // 16 KB: this CTA's 128 rows
  static constexpr int kBBytes = (BN / 2) * kBK * 4;    // this CTA's half of the columns
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTileBytes = STAGES * kStageBytes;
  static constexpr int kBarBytes = 512;
  static constexpr int kStagingBytes = 8 * kEpiStageBytes;  // one staging tile per epilogue warp
  static constexpr int kTotal = kTileBytes + kBarBytes + kStagingBytes + 1024;
};
constexpr int pair_stages_for(int bn) { return bn >= 256 ? 6 : 8; }

// Threads: the six warps of tc_kernel.cuh plus, for policies whose stage is several copies, a
// second producer warp (warp 6) that issues every other copy.
// ... and a second group of four epilogue warps (see tc_kernel.cuh) behind them.
template <class P>
constexpr int pair_second_epilogue_first_warp() { return P::kWarpProducer ? 7 : 6; }
template <class P>
constexpr int pair_threads_for() { return (pair_second_epilogue_first_warp<P>() + 4) * 32; }

template <class P, int BN, int STAGES, int KSUB = 2>
__global__ void __launch_bounds__(pair_threads_for<P>(), 1)
tc_pair_kernel(const __grid_constant__ CUtensorMap map_a,
               const __grid_constant__ CUtensorMap map_b, const P prob, int* status) {
  using SL = PairSmemLayout<BN, STAGES>;
  static_assert(BN >= 64 && BN % 64 == 0, "each CTA holds BN/2 columns in 32-column boxes");
  // the ring's sub-stages change hands in groups of KSUB (see tc_kernel.cuh)
  static_assert(STAGES % KSUB == 0, "ring must be whole groups");
  constexpr int NG = STAGES / KSUB;
  extern __shared__ char smem_raw[];
  char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                        ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + SL::kTileBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  constexpr uint32_t kTmemCols = 2 * BN;
  const int n_tiles = prob.num_pair_tiles();

  if (threadIdx.x == 0) {
    for (int s = 0; s < NG; ++s) {
      mbar_init(&full_bar[s], 1);   // leader: its own arrive.expect_tx for both CTAs' bytes
      mbar_init(&empty_bar[s], 1);  // one tcgen05.commit arrival
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 16);  // leader: 8 epilogue warps of each CTA
    }
    *failed = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  constexpr bool kTwoProducers = P::kWarpProducer;
  if (warp == 0 || (kTwoProducers && warp == 6)) {
    // The whole warp walks the loop (see tc_kernel.cuh): lane 0 owns the barriers, lane i
    // issues copy i * parts + part of the stage; the leader's part 0 posts the byte count.
    const int part = warp == 0 ? 0 : 1;
    constexpr int parts = kTwoProducers ? 2 : 1;
    uint32_t s = 0, round = 0;
    typename P::Tile t;
    typename P::LoadState ls;
    bool live = true;
    TC_PROF_VAR(p_wait);
    TC_PROF_NOW(p_t0);
    for (int tile = pair; live && tile < n_tiles; tile += n_pairs) {
      int stop = 0;
      if (lane == 0) stop = *failed;
      if (__shfl_sync(0xffffffffu, stop, 0) != 0) {
        live = false;
        break;
      }
      prob.decode_pair(tile, (int)rank, t);
      prob.load_begin(t, ls, lane * parts + part);
      const int k1 = prob.k_end(t);
      for (int k = prob.k_begin(t); k < k1; k += KSUB) {
        const int kn = min(KSUB, k1 - k);
        int ok = 1;
        TC_PROF_NOW(w0);
        if (lane == 0) {
          if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) {
            *failed = 1;
            ok = 0;
          } else if (rank == 0 && part == 0) {
            mbar_expect_tx(&full_bar[s], kn * 2 * SL::kStageBytes);
          }
        }
        TC_PROF_ADD(p_wait, w0);
        if (__shfl_sync(0xffffffffu, ok, 0) == 0) {
          live = false;
          break;
        }
        const uint32_t full_leader = mapa_u32(smem_u32(&full_bar[s]), 0);
#pragma unroll
        for (int sub = 0; sub < KSUB; ++sub) {
          if (sub >= kn) break;
          char* a_dst = tiles + (s * KSUB + sub) * SL::kStageBytes;
          prob.load_pair(&map_a, &map_b, t, ls, full_leader, a_dst, a_dst + SL::kABytes,
                         (int)rank, lane * parts + part);
        }
        if (++s == NG) { s = 0; ++round; }
      }
    }
#ifdef FLB200_TC_PROFILE
    if (lane == 0 && part == 0) { TC_PROF_PUT(0, p_wait); TC_PROF_PUT(1, clock64() - p_t0); }
#endif
    // The leader's last commits still arrive on this CTA's empty barriers: wait for them
    // so that the CTA does not leave while they are in flight.
    if (live && lane == 0 && part == 0 && *failed == 0) {
      for (int i = 0; i < NG; ++i) {
        const uint32_t fills = round + (static_cast<uint32_t>(i) < s ? 1u : 0u);
        if (fills > 0 && !mbar_wait(&empty_bar[i], (fills - 1) & 1)) {
          *failed = 1;
          break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc_tf32_pair(BN, prob.a_mn_major, prob.b_mn_major);
      // descriptors of the ring's first stage; every MMA offsets them
      const uint32_t ring = smem_u32(tiles);
      const uint64_t a_desc0 = prob.a_mn_major ? umma_desc(ring, kBK * 128, 512, 1)
                                               : umma_desc(ring, 16, 1024, 2);
      const uint64_t b_desc0 = prob.b_mn_major
                                   ? umma_desc(ring + SL::kABytes, kBK * 128, 512, 1)
                                   : umma_desc(ring + SL::kABytes, 16, 1024, 2);
      const uint32_t a_jstep = prob.a_mn_major ? 1024 : 32, b_jstep = prob.b_mn_major ? 1024 : 32;
      uint32_t s = 0, round = 0, nt = 0;
      typename P::Tile t;
      TC_PROF_VAR(m_full);
      TC_PROF_VAR(m_acc);
      TC_PROF_NOW(m_t0);
      for (int tile = pair; tile < n_tiles && *failed == 0; tile += n_pairs, ++nt) {
        prob.decode_pair(tile, 0, t);
        const uint32_t acc = nt & 1, around = nt >> 1;
        TC_PROF_NOW(w0);
        if (around > 0 && !mbar_wait(&tempty_bar[acc], (around - 1) & 1)) {
          *failed = 4;
          break;
        }
        TC_PROF_ADD(m_acc, w0);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int k0 = prob.k_begin(t), k1 = prob.k_end(t);
        for (int k = k0; k < k1; k += KSUB) {
          const int kn = min(KSUB, k1 - k);
          TC_PROF_NOW(w1);
          if (!mbar_wait(&full_bar[s], round & 1)) {
            *failed = 2;
            break;
          }
          TC_PROF_ADD(m_full, w1);
          tc_fence_after();
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            if (sub >= kn) break;
            const uint32_t off = (s * KSUB + sub) * SL::kStageBytes;
#pragma unroll
            for (int j = 0; j < kBK / kUmmaK; ++j) {
              const uint64_t ad = umma_desc_advance(a_desc0, off + j * a_jstep);
              const uint64_t bd = umma_desc_advance(b_desc0, off + j * b_jstep);
              umma_tf32_pair(d_tmem, ad, bd, idesc, (k > k0 || sub > 0 || j > 0) ? 1u : 0u);
            }
          }
          umma_commit_pair(&empty_bar[s]);  // frees the group in both CTAs
          if (++s == NG) { s = 0; ++round; }
        }
        umma_commit_pair(&tfull_bar[acc]);  // both CTAs' halves of the accumulator complete
      }
#ifdef FLB200_TC_PROFILE
      TC_PROF_PUT(2, m_full); TC_PROF_PUT(3, m_acc); TC_PROF_PUT(4, clock64() - m_t0);
#endif
    }
  } else if ((warp >= 2 && warp < 6) || (warp >= pair_second_epilogue_first_warp<P>() &&
                                        warp < pair_second_epilogue_first_warp<P>() + 4)) {
    // two groups of four epilogue warps: group 0 drains the even 32-column chunks, group 1 the
    // odd ones; a warp owns TMEM lanes 32 * (warp % 4) .. + 31
    const int group = warp < 6 ? 0 : 1;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    float* stage = reinterpret_cast<float*>(
        tiles + SL::kTileBytes + SL::kBarBytes +
        (group * 4 + (warp < 6 ? warp - 2 : warp - pair_second_epilogue_first_warp<P>())) *
            kEpiStageBytes);
    uint32_t nt = 0;
    typename P::Tile t;
    TC_PROF_VAR(e_wait);
    TC_PROF_VAR(e_store);
    TC_PROF_NOW(e_t0);
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++nt) {
      prob.decode_pair(tile, (int)rank, t);
      const uint32_t acc = nt & 1, around = nt >> 1;
      if (*failed != 0) break;
      TC_PROF_NOW(w0);
      if (!mbar_wait(&tfull_bar[acc], around & 1)) {
        *failed = 3;
        break;
      }
      TC_PROF_ADD(e_wait, w0);
      TC_PROF_NOW(w1);
      tc_fence_after();
      if (*failed != 0) break;
#pragma unroll 1
      for (int c0 = 32 * group; c0 < BN; c0 += 64) {
        if (!prob.chunk_live(t, c0)) continue;
        float v[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + (uint32_t)c0, v);
        prob.store(t, row, c0, v, stage, lane);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty_bar[acc]), 0));
      TC_PROF_ADD(e_store, w1);
    }
#ifdef FLB200_TC_PROFILE
    if (threadIdx.x == 64) { TC_PROF_PUT(5, e_wait); TC_PROF_PUT(6, e_store); TC_PROF_PUT(7, clock64() - e_t0); }
#endif
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *failed != 0 && status) atomicExch(status, *failed);
  cluster_sync_all();  // the peer is done with this CTA's barriers and tensor memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// KSUB = 2 pays where the operands come out of L2 and the producer's barrier chain is the
// limit (the patch convolution); contractions that stream both operands from DRAM keep single
// sub-stages: coarser hand-overs cost them bytes in flight (measured both ways).
template <class P, int BN, int KSUB = 1>
int launch_pair_problem(const char* name, const CUtensorMap& ma, const CUtensorMap& mb,
                        const P& prob, long long pair_tiles, cudaStream_t st) {
  constexpr int STAGES = pair_stages_for(BN);
  using SL = PairSmemLayout<BN, STAGES>;
  if (pair_tiles <= 0) return FLB200_OK;
  static bool configured[64] = {false};
  int dev = 0;
  FLB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    FLB200_CUDA_CHECK(cudaFuncSetAttribute(tc_pair_kernel<P, BN, STAGES, KSUB>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SL::kTotal));
    configured[dev] = true;
  }
  const long long pairs = device_info().sm_count / 2;
  const unsigned grid = 2u * (unsigned)(pair_tiles < pairs ? pair_tiles : pairs);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(pair_threads_for<P>());
  cfg.dynamicSmemBytes = SL::kTotal;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FLB200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, tc_pair_kernel<P, BN, STAGES, KSUB>, ma, mb, prob,
                                       status_ptr()));
  FLB200_AFTER_LAUNCH(name);
  count_tc_launch();
#ifdef FLB200_TC_PROFILE
  {
    cudaStreamSynchronize(st);
    static long long h[256 * 8];
    cudaMemcpyFromSymbol(h, g_tc_profile, sizeof(h));
    double a[8] = {0};  // leaders (even CTAs) only: the MMA slots of the peers are never written
    unsigned n = 0;
    for (unsigned c = 0; c < grid && c < 256; c += 2, ++n)
      for (int i = 0; i < 8; ++i) a[i] += (double)h[c * 8 + i];
    for (int i = 0; i < 8; ++i) a[i] /= n ? n : 1;
    fprintf(stderr,
            "tc profile %s (pairs) BN=%d stages=%d ksub=%d tiles=%lld grid=%u | producer wait %.0f of %.0f | "
            "mma wait full %.0f, accumulator %.0f of %.0f | epilogue wait %.0f, store %.0f of %.0f "
            "(mean clocks per leader CTA)\n",
            name, BN, STAGES, KSUB, pair_tiles, grid, a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7]);
  }
#endif
  return FLB200_OK;
}

}  // namespace tc
}  // namespace flb200
