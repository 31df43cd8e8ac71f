// Persistent tcgen05 contraction kernel for sm_100a and the "problem" policies that feed it.
//
//   D = sum_k A(m,k) * B(k,n),  fp32 operands read as TF32, fp32 accumulation in TMEM.
//
// One CTA per SM walks a static list of 128 x BN output tiles:
//   warp 0   : TMA producer — issues cp.async.bulk.tensor loads (never multicast) into a
//              STAGES-deep ring of 128-byte-swizzled shared-memory tiles and runs ahead into
//              the next output tile while the current one drains.  Lane 0 owns the
//              barriers; every lane issues at most one copy per stage, so the boxes of a
//              stage go out together.  Per-stage work is a handful of multiply-adds:
//              coordinates advance incrementally.
//   warp 1   : allocates TMEM (2 accumulators of BN columns); one lane issues tcgen05.mma
//              for each ready stage and tcgen05.commit to free the stage / publish the tile
//   warps 6-9: only in the 3xTF32 instantiation (fp32-grade products): split every landed
//              operand element into a TF32-exact high part and the remainder, so that the MMA
//              warp can issue a_lo*b_hi + a_hi*b_lo + a_hi*b_hi
//   warps 2-5 (and four more behind the producers for tiles of 128+ columns, each group
//              taking every other 32-column chunk):
//              epilogue — tcgen05.ld the finished accumulator (32 lanes each) and store it
//              from registers (coalesced 128-byte rows when the row index is contiguous in
//              memory, 16-byte vectors when the column index is) while the MMA warp already
//              fills the other accumulator
// Hand-offs: full/empty mbarriers per stage, full/empty mbarriers per accumulator.
// Every wait is bounded by a clock budget; a wait that runs out raises a flag, all roles
// drain and the CTA frees its TMEM and returns (the host then reports FLB200_TIMEOUT).
//
// A problem policy P tells the skeleton what a tile is:
//   int  a_mn_major, b_mn_major;
//   static constexpr bool kWarpProducer;  // load() is called by the whole warp (else lane 0)
//   static constexpr int kMinBlocks;      // second argument of tc_persistent_kernel's launch
//                                         // bounds: 1 = the register allocator may use the whole
//                                         // file for the one resident CTA, 0 = its own choice
//   struct Tile;  struct LoadState;
//   __device__ int  num_tiles() const;
//   __device__ void decode(int tile, Tile&) const;
//   __device__ int  k_begin(const Tile&) const;  __device__ int k_end(const Tile&) const;
//   __device__ void load_begin(const Tile&, LoadState&, int copy) const;   // once per tile;
//                        // copy = index of the stage's copy this lane will issue
//   __device__ void load(const CUtensorMap* a, const CUtensorMap* b, const Tile&, LoadState&,
//                        uint64_t* bar, char* a_dst, char* b_dst, int lane) const;
//                        // one stage, called by the whole warp: lane 0 posts the byte count,
//                        // lane i issues copy i; every lane advances its LoadState
//   __device__ bool chunk_live(const Tile&, int c0) const;                // warp-uniform
//   __device__ void store(const Tile&, int row, int c0, const float* v, float* stage,
//                         int lane) const;   // 32 columns of row `row`; called by all 32 lanes
//                         // of an epilogue warp (rows row - lane .. + 31), `stage` is the
//                         // warp's 4 KB staging tile for policies that store through it
#pragma once
#include <cuda_bf16.h>

#include "tc_core.cuh"

namespace flb200 {
namespace tc {

// Staging tile of one epilogue warp and the transposing store through it.  The accumulator
// arrives with one row per lane (32 consecutive columns in registers).  Written to a row-major
// output as it is, every store instruction touches 32 rows at 16 bytes each (32 memory sectors,
// half filled); staged through shared memory, an instruction stores 4 whole 128-byte rows.
// Layout: row r, 16-byte chunk q at chunk (q ^ (r & 7)) of row r: conflict-free both ways.
constexpr int kEpiStageBytes = 32 * 128;
__device__ __forceinline__ void epi_stage_write(float* stage, int lane, const float* v) {
  float4* rowp = reinterpret_cast<float4*>(stage) + lane * 8;
#pragma unroll
  for (int q = 0; q < 8; ++q)
    rowp[q ^ (lane & 7)] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  __syncwarp();
}
// The float4 that lane `lane` stores in step k (0..7): row 4 * k + lane / 8, columns
// 4 * (lane % 8) .. + 3 of the chunk.
__device__ __forceinline__ float4 epi_stage_read(const float* stage, int lane, int k) {
  const int r = 4 * k + (lane >> 3), q = lane & 7;
  return reinterpret_cast<const float4*>(stage)[r * 8 + (q ^ (r & 7))];
}

// Batch-norm statistics of a convolution's output taken from its accumulators: while a warp
// stores its 32 x 32 chunk through the staging tile, every lane adds up the values (and their
// squares) it holds — 4 channels of 8 rows — and the four row groups are added through the
// staging tile; lanes 0..7 then write them, 128 contiguous bytes each for sums and squares,
// into row `group` of a [groups][2 * channels] matrix (sums first, then squares).  Its column
// sums are the per-channel totals; no atomics, so the result does not depend on timing.
struct EpiStats {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f, q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
  __device__ __forceinline__ void add(float4 v) {
    s0 += v.x; s1 += v.y; s2 += v.z; s3 += v.w;
    q0 = fmaf(v.x, v.x, q0); q1 = fmaf(v.y, v.y, q1);
    q2 = fmaf(v.z, v.z, q2); q3 = fmaf(v.w, v.w, q3);
  }
  // `stage`: the warp's staging tile, free again once every lane has read its values out of
  // it (the caller's loop is done); the four row groups of a chunk (lane / 8) meet through it.
  __device__ __forceinline__ void flush(float* stats, long long group, int channels, int c0,
                                        int lane, float* stage) {
    __syncwarp();
    float4* slot = reinterpret_cast<float4*>(stage);
    slot[2 * lane] = make_float4(s0, s1, s2, s3);
    slot[2 * lane + 1] = make_float4(q0, q1, q2, q3);
    __syncwarp();
    if (lane < 8) {
#pragma unroll
      for (int g = 1; g < 4; ++g) {
        const float4 a = slot[2 * (lane + 8 * g)], b = slot[2 * (lane + 8 * g) + 1];
        s0 += a.x; s1 += a.y; s2 += a.z; s3 += a.w;
        q0 += b.x; q1 += b.y; q2 += b.z; q3 += b.w;
      }
      float* row = stats + group * (2LL * channels) + c0 + 4 * lane;
      *reinterpret_cast<float4*>(row) = make_float4(s0, s1, s2, s3);
      *reinterpret_cast<float4*>(row + channels) = make_float4(q0, q1, q2, q3);
    }
  }
};

// gelu in the tanh form of flashlight/fl/autograd/Functions.cpp:1791-1796 (the constants of
// flb200_gelu_forward)
// tanh(u) = 1 - 2 / (1 + exp(2u)) from the fast exponential: branch-free (no library call inside
// the store loop of the contraction kernels), absolute error below 1e-6
__device__ __forceinline__ float epi_gelu(float x) {
  const float u = 0.7978845608f * (x + 0.044715f * x * x * x);
  const float t = 1.f - __fdividef(2.f, 1.f + __expf(2.f * u));
  return 0.5f * x * (1.f + t);
}

// X3 = 1: every stage also holds the low-order tiles of the 3xTF32 split (see the kernel).
template <int BN, int STAGES, int X3 = 0>
struct SmemLayout {
  static constexpr int kABytes = kBM * kBK * 4;  // 16 KB
  static constexpr int kBBytes = BN * kBK * 4;
  static constexpr int kLoOffset = kABytes + kBBytes;  // low-order A tile, then low-order B tile
  static constexpr int kStageBytes = (X3 ? 2 : 1) * (kABytes + kBBytes);
  static constexpr int kTileBytes = STAGES * kStageBytes;
  static constexpr int kBarBytes = 512;
  // 4 KB per epilogue warp: a 32 x 32 accumulator chunk is turned from "one row per lane" into
  // "128 contiguous bytes per 8 lanes" through it before it is stored to a row-major output
  static constexpr int kStagingBytes = ((X3 == 0 && BN >= 128) ? 8 : 4) * kEpiStageBytes;
  static constexpr int kTotal = kTileBytes + kBarBytes + kStagingBytes + 1024;  // + slack to align
};

// ~200 KB of tiles per CTA
constexpr int stages_for(int bn) { return bn >= 256 ? 4 : (bn >= 128 ? 6 : (bn >= 64 ? 8 : 10)); }
constexpr int stages_for_x3(int bn) { return bn >= 256 ? 2 : (bn >= 128 ? 3 : (bn >= 64 ? 4 : 5)); }
constexpr int kThreadsX3 = kThreads + 128;  // four more warps split the operands
// Policies whose stage is several copies get a second producer warp (warp 6): issuing one TMA
// copy costs the issuing warp ~110-130 clocks and copies issued from different lanes of one
// warp still go out one after the other, so a stage of 5 to 12 copies took 650 to 1500 clocks
// to issue against ~500 clocks of MMAs; two warps issue the even and the odd copies.
// Tiles of 128 or more columns get a second group of four epilogue warps (each group drains
// every other 32-column chunk of the accumulator): with one group, shapes with a short K loop
// and a large output (1x1 layers on 56x56 planes: 2 K blocks per 128 KB tile) were bound by the
// time four warps need to store a tile.
template <int X3, int BN>
constexpr int epilogue_groups() { return (X3 == 0 && BN >= 128) ? 2 : 1; }
template <class P, int X3>
constexpr int second_epilogue_first_warp() { return P::kWarpProducer && X3 == 0 ? 7 : 6; }
template <class P, int X3, int BN>
constexpr int threads_for() {
  if (X3) return kThreadsX3;
  if (epilogue_groups<X3, BN>() == 2) return (second_epilogue_first_warp<P, X3>() + 4) * 32;
  return P::kWarpProducer ? kThreads + 32 : kThreads;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Stall accounting, compiled in with -DFLB200_TC_PROFILE only (FLB200_NVCC_EXTRA of the build
// script): every role of every CTA sums the clocks it spends in each of its waits, and the
// host prints the means after each launch.  Slots: producer {wait empty, total}, MMA issuer
// {wait full, wait accumulator free, total}, epilogue warp 2 {wait accumulator full, store, total}.
#ifdef FLB200_TC_PROFILE
static __device__ long long g_tc_profile[256 * 8];
#define TC_PROF_VAR(x) long long x = 0
#define TC_PROF_NOW(t) const long long t = clock64()
#define TC_PROF_ADD(x, t) x += clock64() - t
#define TC_PROF_PUT(slot, v) g_tc_profile[(blockIdx.x & 255) * 8 + (slot)] = (v)
#else
#define TC_PROF_VAR(x)
#define TC_PROF_NOW(t)
#define TC_PROF_ADD(x, t)
#define TC_PROF_PUT(slot, v)
#endif

template <class P, int BN, int STAGES, int X3 = 0, int KSUB = 1>
__global__ void __launch_bounds__(threads_for<P, X3, BN>(), P::kMinBlocks)
tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                     const __grid_constant__ CUtensorMap map_b, const P prob, int* status) {
  using SL = SmemLayout<BN, STAGES, X3>;
  // The ring's STAGES sub-stages (one 128-byte-wide K block of both operands each) are handed
  // over in groups of KSUB: one pair of barriers, one wait and one commit per group.  A
  // hand-off costs each side a chain of dependent barrier instructions (measured: ~270 clocks
  // for wait + arrive alone, ~400 with one copy issued), which a narrow tile's four MMAs do
  // not cover; a group amortises it over 4 * KSUB MMAs.
  static_assert(STAGES % KSUB == 0 && (X3 == 0 || KSUB == 1), "ring must be whole groups");
  constexpr int NG = STAGES / KSUB;
  extern __shared__ char smem_raw[];
  char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                        ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + SL::kTileBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;   // [2] accumulator ready for the epilogue
  uint64_t* tempty_bar = tfull_bar + 2;       // [2] accumulator drained, MMA may overwrite
  uint64_t* split_bar = tempty_bar + 2;       // [STAGES] X3: low-order tiles of the stage written
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(split_bar + STAGES);
  volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  const int n_tiles = prob.num_tiles();

  if (threadIdx.x == 0) {
    for (int s = 0; s < NG; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
      mbar_init(&split_bar[s], 4);  // one arrival per splitting warp
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4 * epilogue_groups<X3, BN>());  // one arrival per epilogue warp
    }
    *failed = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  constexpr bool kTwoProducers = P::kWarpProducer && X3 == 0;
  if (warp == 0 || (kTwoProducers && warp == 6)) {
    uint32_t s = 0, round = 0;
    typename P::Tile t;
    typename P::LoadState ls;
    // part / parts: this warp issues the copies whose index is congruent to part mod parts;
    // part 0 also posts the stage's byte count
    const int part = warp == 0 ? 0 : 1;
    constexpr int parts = kTwoProducers ? 2 : 1;
    if constexpr (P::kWarpProducer) {
      // All 32 lanes walk the loop: lane 0 waits for the stage to be free and posts the byte
      // count, then each lane issues one of the stage's copies (a single instruction for
      // the warp), so a stage made of many boxes costs the same issue time as a small one.
      bool live = true;
      TC_PROF_VAR(p_wait);
      TC_PROF_NOW(p_t0);
      for (int tile = blockIdx.x; live && tile < n_tiles; tile += gridDim.x) {
        int stop = 0;
        if (lane == 0) stop = *failed;
        if (__shfl_sync(0xffffffffu, stop, 0) != 0) break;
        prob.decode(tile, t);
        prob.load_begin(t, ls, lane * parts + part);  // the index of the copy this lane issues
        const int k1 = prob.k_end(t);
        for (int k = prob.k_begin(t); k < k1; k += KSUB) {
          int ok = 1;
          TC_PROF_NOW(w0);
          if (lane == 0 && round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) {
            *failed = 1;
            ok = 0;
          }
          TC_PROF_ADD(p_wait, w0);
          if (__shfl_sync(0xffffffffu, ok, 0) == 0) {
            live = false;
            break;
          }
          const int kn = min(KSUB, k1 - k);
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            if (sub >= kn) break;
            char* a_dst = tiles + (s * KSUB + sub) * SL::kStageBytes;
            prob.load(&map_a, &map_b, t, ls, &full_bar[s], a_dst, a_dst + SL::kABytes, lane,
                      sub == kn - 1, part, parts);
          }
          if (++s == NG) { s = 0; ++round; }
        }
      }
#ifdef FLB200_TC_PROFILE
      if (lane == 0 && part == 0) { TC_PROF_PUT(0, p_wait); TC_PROF_PUT(1, clock64() - p_t0); }
#endif
    } else if (lane == 0) {
      // Two copies per stage: one lane does everything and the loop has no warp exchange.
      TC_PROF_VAR(p_wait);
      TC_PROF_NOW(p_t0);
      for (int tile = blockIdx.x; tile < n_tiles && *failed == 0; tile += gridDim.x) {
        prob.decode(tile, t);
        prob.load_begin(t, ls, 0);
        const int k1 = prob.k_end(t);
        for (int k = prob.k_begin(t); k < k1; k += KSUB) {
          TC_PROF_NOW(w0);
          if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) {
            *failed = 1;
            break;
          }
          TC_PROF_ADD(p_wait, w0);
          const int kn = min(KSUB, k1 - k);
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            if (sub >= kn) break;
            char* a_dst = tiles + (s * KSUB + sub) * SL::kStageBytes;
            prob.load(&map_a, &map_b, t, ls, &full_bar[s], a_dst, a_dst + SL::kABytes, 0,
                      sub == kn - 1, 0, 1);
          }
          if (++s == NG) { s = 0; ++round; }
        }
      }
#ifdef FLB200_TC_PROFILE
      TC_PROF_PUT(0, p_wait); TC_PROF_PUT(1, clock64() - p_t0);
#endif
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool bf16 = false;
      if constexpr (P::kBf16Capable) bf16 = prob.bf16 != 0;
      const uint32_t idesc = bf16 ? umma_idesc_bf16(BN, prob.a_mn_major, prob.b_mn_major)
                                  : umma_idesc_tf32(BN, prob.a_mn_major, prob.b_mn_major);
      // MN-major tiles: fp32 in 32 x 32 boxes with the 32-byte-chunk swizzle (4 KB apart, k
      // atoms 512 B apart, 8 k-rows = 1 KB per MMA); bf16 in 64 x 64 boxes with the plain
      // 128-byte swizzle (8 KB apart, k atoms 1 KB apart, 16 k-rows = 2 KB per MMA)
      const uint32_t mn_lbo = bf16 ? 8192 : kBK * 128, mn_sbo = bf16 ? 1024 : 512;
      const uint32_t mn_step = bf16 ? 2048 : 1024, mn_layout = bf16 ? 2 : 1;
      // descriptors of the ring's first sub-stage; every MMA offsets them (umma_desc_advance)
      const uint32_t ring = smem_u32(tiles);
      const uint64_t a_desc0 = prob.a_mn_major ? umma_desc(ring, mn_lbo, mn_sbo, mn_layout)
                                               : umma_desc(ring, 16, 1024, 2);
      const uint64_t b_desc0 = prob.b_mn_major
                                   ? umma_desc(ring + SL::kABytes, mn_lbo, mn_sbo, mn_layout)
                                   : umma_desc(ring + SL::kABytes, 16, 1024, 2);
      // K-major: step 8 elements = 32 bytes inside the swizzled row;
      // MN-major: step 8 (bf16: 16) k-rows = 1024 (2048) bytes inside each box.
      const uint32_t a_jstep = prob.a_mn_major ? mn_step : 32;
      const uint32_t b_jstep = prob.b_mn_major ? mn_step : 32;
      uint32_t s = 0, round = 0, nt = 0;
      typename P::Tile t;
      TC_PROF_VAR(m_full);
      TC_PROF_VAR(m_acc);
      TC_PROF_NOW(m_t0);
      for (int tile = blockIdx.x; tile < n_tiles && *failed == 0; tile += gridDim.x, ++nt) {
        prob.decode(tile, t);
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
          TC_PROF_NOW(w1);
          if (!mbar_wait(X3 ? &split_bar[s] : &full_bar[s], round & 1)) {
            *failed = 2;
            break;
          }
          TC_PROF_ADD(m_full, w1);
          tc_fence_after();
          if constexpr (X3 != 0) {
            // a * b ~ a_hi * b_hi + a_lo * b_hi + a_hi * b_lo with x = x_hi + x_lo, x_hi exact
            // in TF32: fp32-grade products out of three tensor-core passes
            const uint32_t off = s * SL::kStageBytes;
#pragma unroll
            for (int j = 0; j < kBK / kUmmaK; ++j) {
              const uint64_t ah = umma_desc_advance(a_desc0, off + j * a_jstep);
              const uint64_t bh = umma_desc_advance(b_desc0, off + j * b_jstep);
              const uint64_t al = umma_desc_advance(a_desc0, off + SL::kLoOffset + j * a_jstep);
              const uint64_t bl = umma_desc_advance(b_desc0, off + SL::kLoOffset + j * b_jstep);
              umma_tf32(d_tmem, al, bh, idesc, (k > k0 || j > 0) ? 1u : 0u);
              umma_tf32(d_tmem, ah, bl, idesc, 1u);
              umma_tf32(d_tmem, ah, bh, idesc, 1u);
            }
            umma_commit(&empty_bar[s]);
            if (++s == NG) { s = 0; ++round; }
            continue;
          }
          const int kn = min(KSUB, k1 - k);
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            if (sub >= kn) break;
            const uint32_t off = (s * KSUB + sub) * SL::kStageBytes;
#pragma unroll
            for (int j = 0; j < kBK / kUmmaK; ++j) {
              const uint64_t ad = umma_desc_advance(a_desc0, off + j * a_jstep);
              const uint64_t bd = umma_desc_advance(b_desc0, off + j * b_jstep);
              const uint32_t accumulate = (k > k0 || sub > 0 || j > 0) ? 1u : 0u;
              if (bf16) umma_bf16(d_tmem, ad, bd, idesc, accumulate);
              else umma_tf32(d_tmem, ad, bd, idesc, accumulate);
            }
          }
          umma_commit(&empty_bar[s]);  // frees the group once these MMAs have read it
          if (++s == NG) { s = 0; ++round; }
        }
        umma_commit(&tfull_bar[acc]);  // accumulator complete
      }
#ifdef FLB200_TC_PROFILE
      TC_PROF_PUT(2, m_full); TC_PROF_PUT(3, m_acc); TC_PROF_PUT(4, clock64() - m_t0);
#endif
    }
  } else if (X3 != 0 && warp >= 6) {
    // splitting warps (X3 only): once a stage has landed, rewrite every operand element x in
    // place as x_hi (low 13 mantissa bits cleared: exact in TF32 however the tensor core
    // converts) and write x_lo = x - x_hi at the same offset of the stage's low-order tiles;
    // elementwise at equal offsets, so the swizzled layout carries over unchanged.
    const int t128 = threadIdx.x - 6 * 32;
    uint32_t s = 0, round = 0;
    typename P::Tile t;
    bool live = true;
    for (int tile = blockIdx.x; live && tile < n_tiles; tile += gridDim.x) {
      prob.decode(tile, t);
      const int k0 = prob.k_begin(t), k1 = prob.k_end(t);
      for (int k = k0; k < k1; ++k) {
        if (*failed != 0 || !mbar_wait(&full_bar[s], round & 1)) {
          if (*failed == 0) *failed = 5;
          live = false;
          break;
        }
        float4* hi = reinterpret_cast<float4*>(tiles + s * SL::kStageBytes);
        float4* lo = reinterpret_cast<float4*>(tiles + s * SL::kStageBytes + SL::kLoOffset);
        constexpr int kVec = SL::kLoOffset / 16;
#pragma unroll 4
        for (int i = t128; i < kVec; i += 128) {
          const float4 v = hi[i];
          float4 h;
          h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
          h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
          h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
          h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
          hi[i] = h;
          lo[i] = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
        }
        fence_proxy_async();  // these generic-proxy writes are read by the tensor core next
        __syncwarp();
        if (lane == 0) mbar_arrive(&split_bar[s]);
        if (++s == NG) { s = 0; ++round; }
      }
    }
  } else if ((warp >= 2 && warp < 6) ||
             (epilogue_groups<X3, BN>() == 2 && warp >= second_epilogue_first_warp<P, X3>() &&
              warp < second_epilogue_first_warp<P, X3>() + 4)) {
    // an epilogue warp owns TMEM lanes 32*(warp % 4) .. +31; group 0 = warps 2..5 drains the
    // even 32-column chunks (all of them when there is one group), group 1 the odd ones
    constexpr int kGroups = epilogue_groups<X3, BN>();
    const int group = warp < 6 ? 0 : 1;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    float* stage = reinterpret_cast<float*>(tiles + SL::kTileBytes + SL::kBarBytes +
                                            (group * 4 + (warp < 6 ? warp - 2
                                                                   : warp - second_epilogue_first_warp<P, X3>())) *
                                                kEpiStageBytes);
    uint32_t nt = 0;
    typename P::Tile t;
    TC_PROF_VAR(e_wait);
    TC_PROF_VAR(e_store);
    TC_PROF_NOW(e_t0);
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++nt) {
      prob.decode(tile, t);
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
      for (int c0 = 32 * group; c0 < BN; c0 += 32 * kGroups) {
        if (!prob.chunk_live(t, c0)) continue;  // uniform across the warp; need not be a prefix
        float v[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + (uint32_t)c0, v);
        prob.store(t, row, c0, v, stage, lane);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      TC_PROF_ADD(e_store, w1);
    }
#ifdef FLB200_TC_PROFILE
    if (threadIdx.x == 64) { TC_PROF_PUT(5, e_wait); TC_PROF_PUT(6, e_store); TC_PROF_PUT(7, clock64() - e_t0); }
#endif
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *failed != 0 && status) atomicExch(status, *failed);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------ plain GEMM
// Tiles ordered split-fastest, then n, then m, then batch, so that CTAs running
// together share the (large) A tile through L2.
template <int BN>
struct GemmProblem {
  static constexpr bool kWarpProducer = true;
  static constexpr int kMinBlocks = 0;
  static constexpr bool kBf16Capable = true;
  int bf16;  // operands are bf16 (64 elements per stage), else fp32 read as TF32
  OperandCoords a, b;
  EpiloguePlan ep;
  int a_mn_major, b_mn_major;
  int M, N, k_iters, splits, iters_per_split;
  int tiles_m, tiles_n, Z;
  int pair_n_fast;  // order of the pair tiles: column tiles of one row pair next to each other
  float* partial;  // split-K scratch [z*splits + s][M][N]

  struct Tile { int m0, n0, z, split, k0, k1; };
  struct LoadState { int a_lo, a_hi, b_lo, b_hi; };

  __device__ __forceinline__ int num_tiles() const { return tiles_m * tiles_n * Z * splits; }
  __device__ __forceinline__ void decode(int tile, Tile& t) const {
    int r = tile;
    t.split = r % splits; r /= splits;
    t.n0 = (r % tiles_n) * BN; r /= tiles_n;
    t.m0 = (r % tiles_m) * kBM; r /= tiles_m;
    t.z = r;
    t.k0 = t.split * iters_per_split;
    t.k1 = min(t.k0 + iters_per_split, k_iters);
  }
  __device__ __forceinline__ int k_begin(const Tile& t) const { return t.k0; }
  __device__ __forceinline__ int k_end(const Tile& t) const { return t.k1; }
  __device__ __forceinline__ void load_begin(const Tile& t, LoadState& ls, int) const {
    ls.a_hi = a.k_inner > 0 ? t.k0 / a.k_inner : 0;
    ls.a_lo = t.k0 - ls.a_hi * a.k_inner;
    ls.b_hi = b.k_inner > 0 ? t.k0 / b.k_inner : 0;
    ls.b_lo = t.k0 - ls.b_hi * b.k_inner;
  }
  __device__ __forceinline__ void load(const CUtensorMap* ma, const CUtensorMap* mb,
                                       const Tile& t, LoadState& ls, uint64_t* bar, char* a_dst,
                                       char* b_dst, int lane, bool last, int part,
                                       int parts) const {
    if (lane == 0 && part == 0) mbar_post_tx(bar, (kBM + BN) * kBK * 4, last);
    __syncwarp();
    // a K-major operand is one box, an MN-major one a box per 32 rows: copies [0, na) are A,
    // [na, na + nb) are B; copy i is issued by lane i / parts of producer warp i % parts
    const int box_mn = bf16 ? 64 : 32, box_bytes = bf16 ? 8192 : kBK * 128;
    const int na = a_mn_major && !a.mn_shift ? kBM / box_mn : 1;
    const int nb = b_mn_major && !b.mn_shift ? BN / box_mn : 1;  // grouped: one copy
    const int copy = lane * parts + part;
    if (copy < na) {
      int c[4];
      operand_coords(a, t.m0 + box_mn * copy, ls.a_lo, ls.a_hi, t.z, c);
      tma_load(ma, bar, a_dst + copy * box_bytes, a.rank, c);
    } else if (copy < na + nb) {
      const int j = copy - na;
      int c[4];
      operand_coords(b, t.n0 + box_mn * j, ls.b_lo, ls.b_hi, t.z, c);
      tma_load(mb, bar, b_dst + j * box_bytes, b.rank, c);
    }
    if (++ls.a_lo == a.k_inner) { ls.a_lo = 0; ++ls.a_hi; }
    if (++ls.b_lo == b.k_inner) { ls.b_lo = 0; ++ls.b_hi; }
  }
  // CTA pairs (tc_pair.cuh): the halves of a pair tile are two consecutive 128-row blocks of
  // the same column block, batch and K slice; row blocks run fastest, then splits, columns,
  // batches.  With an odd number of row blocks the last pair has a phantom half past M
  // (zero-filled loads, masked stores).
  __device__ __forceinline__ int num_pair_tiles() const {
    return ((tiles_m + 1) >> 1) * splits * tiles_n * Z;
  }
  __device__ __forceinline__ void decode_pair(int tile, int rank, Tile& t) const {
    const int pairs_m = (tiles_m + 1) >> 1;
    int r = tile;
    if (pair_n_fast) {
      t.n0 = (r % tiles_n) * BN; r /= tiles_n;
      t.split = r % splits; r /= splits;
      t.m0 = (2 * (r % pairs_m) + rank) * kBM; r /= pairs_m;
    } else {
      t.m0 = (2 * (r % pairs_m) + rank) * kBM; r /= pairs_m;
      t.split = r % splits; r /= splits;
      t.n0 = (r % tiles_n) * BN; r /= tiles_n;
    }
    t.z = r;
    t.k0 = t.split * iters_per_split;
    t.k1 = min(t.k0 + iters_per_split, k_iters);
  }
  __device__ __forceinline__ void load_pair(const CUtensorMap* ma, const CUtensorMap* mb,
                                            const Tile& t, LoadState& ls, uint32_t full_bar,
                                            char* a_dst, char* b_dst, int rank, int copy) const {
    // this CTA's 128 rows of A and its BN/2 columns of B; `copy` = which of the stage's copies
    // the calling lane issues
    const int na = a_mn_major ? kBM / 32 : 1, nb = b_mn_major ? BN / 64 : 1;
    if (copy < na) {
      int c[4];
      operand_coords(a, t.m0 + 32 * copy, ls.a_lo, ls.a_hi, t.z, c);
      tma_load_pair(ma, full_bar, a_dst + copy * (kBK * 128), a.rank, c);
    } else if (copy < na + nb) {
      const int j = copy - na;
      int c[4];
      operand_coords(b, t.n0 + rank * (BN / 2) + 32 * j, ls.b_lo, ls.b_hi, t.z, c);
      tma_load_pair(mb, full_bar, b_dst + j * (kBK * 128), b.rank, c);
    }
    if (++ls.a_lo == a.k_inner) { ls.a_lo = 0; ++ls.a_hi; }
    if (++ls.b_lo == b.k_inner) { ls.b_lo = 0; ++ls.b_hi; }
  }
  __device__ __forceinline__ bool chunk_live(const Tile& t, int c0) const {
    return t.n0 + c0 < N;
  }

  // Rows 4k + lane / 8 (k = 0..7) of the warp's staged 32 x 32 chunk to a row-major output,
  // 16 bytes per lane.  MODE 0: the values as staged; 1: + bias_n; 2: + bias_n, then gelu, the
  // pre-activation kept in ep.pre when that is set.  STATS: per-channel sums of the stored
  // values into row `group` of ep.stats.
  template <int MODE, bool STATS>
  __device__ __forceinline__ void staged_rows(float* stage, int lane, int m_first, float* out_row,
                                              long long ld, int nb, long long group) const {
    float4 bq = make_float4(0.f, 0.f, 0.f, 0.f);
    if (MODE != 0 && ep.bias_n)
      bq = *reinterpret_cast<const float4*>(ep.bias_n + nb + 4 * (lane & 7));
    float* pre_row = nullptr;
    if (MODE == 2 && ep.pre)
      pre_row = static_cast<float*>(ep.pre) + (out_row - ep.out);
    EpiStats acc;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int mr = m_first + 4 * k + (lane >> 3);
      float4 val = epi_stage_read(stage, lane, k);
      if (MODE != 0) { val.x += bq.x; val.y += bq.y; val.z += bq.z; val.w += bq.w; }
      if (mr < M) {
        const long long off = (long long)mr * ld;
        if (MODE == 2) {
          if (pre_row) *reinterpret_cast<float4*>(pre_row + off) = val;
          val = make_float4(epi_gelu(val.x), epi_gelu(val.y), epi_gelu(val.z), epi_gelu(val.w));
        }
        *reinterpret_cast<float4*>(out_row + off) = val;
        if (STATS) acc.add(val);
      }
    }
    if (STATS) acc.flush(ep.stats, group, N, nb, lane, stage);
  }

  __device__ __forceinline__ void store(const Tile& t, int row, int c0, const float* v,
                                        float* stage, int lane) const {
    const int m = t.m0 + row;
    const int nb = t.n0 + c0;
    // Row-major fp32 output with nothing but alpha to apply (a linear layer's product, a 1 x 1
    // convolution over channels-last tensors, split-K partial sums): through the staging tile,
    // whole 128-byte rows per store instruction.  The condition is uniform across the warp.
    {
      float* base = nullptr;
      long long ld = 0;
      float scale = 1.f;
      if (splits > 1) {
        if ((N & 3) == 0) {
          base = partial + ((long long)(t.z * splits + t.split) * M) * N;
          ld = N;
        }
      } else if (!ep.out_bf16 && ep.beta == 0.f && ep.n_div == 0 && ep.m_div == 0 &&
                 ep.n_stride == 1 && ep.bias_m == nullptr &&
                 (ep.m_stride & 3) == 0 && ((ep.z_stride * t.z) & 3) == 0 &&
                 (reinterpret_cast<uintptr_t>(ep.out) & 15) == 0) {
        base = ep.out + (long long)t.z * ep.z_stride;
        ld = ep.m_stride;
        scale = ep.alpha;
      }
      if (base != nullptr && nb + 32 <= N) {
        float w[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = scale * v[j];
        epi_stage_write(stage, lane, w);
        const int m_first = m - lane;  // first row of this warp
        // The flags are uniform across the grid: each combination has its own copy of the
        // store loop, so the plain one stays eight loads followed by eight stores.
        const bool fused = splits == 1 && (ep.bias_n != nullptr || ep.act != 0);
        const bool stats = splits == 1 && ep.stats != nullptr;
        float* out_row = base + nb + 4 * (lane & 7);
        const long long group = (long long)(t.m0 >> 7) * 4 + (row >> 5);
        if (!fused) {
          if (!stats) staged_rows<0, false>(stage, lane, m_first, out_row, ld, nb, group);
          else staged_rows<0, true>(stage, lane, m_first, out_row, ld, nb, group);
        } else if (ep.act == 0) {
          if (!stats) staged_rows<1, false>(stage, lane, m_first, out_row, ld, nb, group);
          else staged_rows<1, true>(stage, lane, m_first, out_row, ld, nb, group);
        } else {
          if (!stats) staged_rows<2, false>(stage, lane, m_first, out_row, ld, nb, group);
          else staged_rows<2, true>(stage, lane, m_first, out_row, ld, nb, group);
        }
        __syncwarp();  // the tile is rewritten by the next chunk
        return;
      }
    }
    if (m >= M) return;
    if (splits > 1) {
      float* dst = partial + ((long long)(t.z * splits + t.split) * M + m) * N + nb;
      if (nb + 32 <= N && (N & 3) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (nb + j < N) dst[j] = v[j];
      }
      return;
    }
    if (ep.m_valid != 0 && ep.m_div != 0 && (m % ep.m_div) >= ep.m_valid) return;
    const long long m_off =
        epi_off(m, ep.m_div, ep.m_stride, ep.m_outer) + (long long)t.z * ep.z_stride;
    const float bm = ep.bias_m ? ep.bias_m[m] : 0.f;
    if (ep.out_bf16) {
      __nv_bfloat16* outb = reinterpret_cast<__nv_bfloat16*>(ep.out);
      if (ep.beta == 0.f && ep.n_div == 0 && ep.n_stride == 1 && nb + 32 <= N &&
          ((m_off + nb) & 7) == 0 && (reinterpret_cast<uintptr_t>(ep.out) & 15) == 0) {
        uint4* dst = reinterpret_cast<uint4*>(outb + m_off + nb);
        uint4* dpre = ep.act && ep.pre
                          ? reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(ep.pre) + m_off + nb)
                          : nullptr;
        const float* bn = ep.bias_n ? ep.bias_n + nb : nullptr;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          float r[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) r[q] = ep.alpha * v[j + q] + bm + (bn ? bn[j + q] : 0.f);
          __nv_bfloat162 h[4];
          if (ep.act) {
            if (dpre) {
#pragma unroll
              for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(r[2 * q], r[2 * q + 1]);
              dpre[j >> 3] = *reinterpret_cast<uint4*>(h);
            }
            // the activation sees the value the pre-activation tensor holds (rounded to bf16),
            // as the unfused chain does
#pragma unroll
            for (int q = 0; q < 8; ++q) r[q] = epi_gelu(__bfloat162float(__float2bfloat16(r[q])));
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(r[2 * q], r[2 * q + 1]);
          dst[j >> 3] = *reinterpret_cast<uint4*>(h);
        }
        return;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int n = nb + j;
        if (n < N) {
          __nv_bfloat16* dst = outb + m_off + epi_off(n, ep.n_div, ep.n_stride, ep.n_outer);
          float r = ep.alpha * v[j] + bm + (ep.bias_n ? ep.bias_n[n] : 0.f);
          if (ep.beta != 0.f) r += ep.beta * __bfloat162float(*dst);
          *dst = __float2bfloat16(r);
        }
      }
      return;
    }
    const bool simple = ep.beta == 0.f && ep.n_div == 0;
    if (simple && nb + 32 <= N && ep.bias_n != nullptr) {
      // strided columns with a per-column bias (convolution output planes)
      float* dst = ep.out + m_off + (long long)nb * ep.n_stride;
      const long long ns = ep.n_stride;
      const float* bn = ep.bias_n + nb;
#pragma unroll
      for (int j = 0; j < 32; ++j) dst[j * ns] = ep.alpha * v[j] + bm + bn[j];
      return;
    }
    if (simple && nb + 32 <= N) {
      float* dst = ep.out + m_off + (long long)nb * ep.n_stride;
      if (ep.n_stride == 1 && ((m_off + nb) & 3) == 0 &&
          (reinterpret_cast<uintptr_t>(ep.out) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) =
              make_float4(ep.alpha * v[j] + bm, ep.alpha * v[j + 1] + bm,
                          ep.alpha * v[j + 2] + bm, ep.alpha * v[j + 3] + bm);
      } else {
        const long long ns = ep.n_stride;
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[j * ns] = ep.alpha * v[j] + bm;
      }
      return;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int n = nb + j;
      if (n < N) {
        float* dst = ep.out + m_off + epi_off(n, ep.n_div, ep.n_stride, ep.n_outer);
        float r = ep.alpha * v[j] + bm + (ep.bias_n ? ep.bias_n[n] : 0.f);
        if (ep.beta != 0.f) r += ep.beta * *dst;
        *dst = r;
      }
    }
  }
};

// ------------------------------------------------------------- host launch
// Launches the persistent kernel for problem P: one CTA per SM (fewer when there are fewer tiles).
template <class P, int BN, int STAGES, int X3, int KSUB = 1>
int launch_problem_as(const char* name, const CUtensorMap& ma, const CUtensorMap& mb, const P& prob,
                      long long tiles, cudaStream_t st) {
  using SL = SmemLayout<BN, STAGES, X3>;
  static bool configured[64] = {false};
  int dev = 0;
  FLB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    FLB200_CUDA_CHECK(cudaFuncSetAttribute(tc_persistent_kernel<P, BN, STAGES, X3, KSUB>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SL::kTotal));
    configured[dev] = true;
  }
  const long long sms = device_info().sm_count;
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  tc_persistent_kernel<P, BN, STAGES, X3, KSUB><<<grid, threads_for<P, X3, BN>(), SL::kTotal, st>>>(
      ma, mb, prob, status_ptr());
  FLB200_AFTER_LAUNCH(name);
  count_tc_launch();
#ifdef FLB200_TC_PROFILE
  {
    cudaStreamSynchronize(st);
    static long long h[256 * 8];
    cudaMemcpyFromSymbol(h, g_tc_profile, sizeof(h));
    double a[8] = {0};
    for (unsigned c = 0; c < grid && c < 256; ++c)
      for (int i = 0; i < 8; ++i) a[i] += (double)h[c * 8 + i] / (grid < 256 ? grid : 256);
    fprintf(stderr,
            "tc profile %s BN=%d stages=%d ksub=%d tiles=%lld grid=%u | producer wait %.0f of %.0f | "
            "mma wait full %.0f, accumulator %.0f of %.0f | epilogue wait %.0f, store %.0f of %.0f "
            "(mean clocks per CTA)\n",
            name, BN, STAGES, KSUB, tiles, grid, a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7]);
  }
#endif
  return FLB200_OK;
}

template <class P, int BN>
int launch_problem(const char* name, const CUtensorMap& ma, const CUtensorMap& mb, const P& prob,
                   long long tiles, cudaStream_t st) {
  if (tiles <= 0) return FLB200_OK;
  if (x3_enabled())
    return launch_problem_as<P, BN, stages_for_x3(BN), 1>(name, ma, mb, prob, tiles, st);
  // Narrow tiles hand the ring over in groups of two sub-stages (measured 5-10 % faster than
  // single sub-stages, no further gain from four); 256-column tiles keep four single stages.
  constexpr int kS = stages_for(BN);
  if constexpr (BN <= 128)
    return launch_problem_as<P, BN, kS, 0, 2>(name, ma, mb, prob, tiles, st);
  else
    return launch_problem_as<P, BN, kS, 0, 1>(name, ma, mb, prob, tiles, st);
}

}  // namespace tc
}  // namespace flb200
