// fp32-FMA tiled contraction used by the STRICT (fp32 parity) mode of matmul and
// of the three convolution passes.  One kernel template; the operands are
// described by small "loader" functors, so a plain strided matrix, an im2col
// view of an NCHW image or a transposed filter are all the same main loop.
//
//   C[z][m][n] = sum_k A[z](m,k) * B[z](k,n)
//
// Loader concept (operand A indexes rows by m, operand B by n):
//   static constexpr bool kAlongK;  // consecutive k are adjacent in memory
//   struct Row; struct Kk;
//   __device__ Row  row(int r, int z) const;        // r may be out of range
//   __device__ Kk   kk(long long k, int z) const;   // k always in range
//   __device__ float load(const Row&, const Kk&) const;  // 0 when out of range
// The thread->element map of the global loads follows kAlongK so that a warp
// always reads along the contiguous direction of the operand.
//
// Epilogue concept:
//   struct Row; struct Col;
//   __device__ Row row(int m, int z) const;  __device__ Col col(int n, int z) const;
//   __device__ void store(const Row&, const Col&, float acc) const;
//
// Split-K (deterministic): each split writes raw partial tiles to scratch and a
// second kernel adds the splits in a fixed order before calling the epilogue.
#pragma once
#include "common.cuh"

namespace flb200 {

constexpr int kGemmThreads = 256;
constexpr int kGemmBK = 16;

template <int BM, int BN, class AL, class BL, class EP>
__global__ void __launch_bounds__(kGemmThreads)
simt_gemm_kernel(AL al, BL bl, EP ep, int M, int N, long long K, int splits,
                 long long k_per_split, float* __restrict__ partial) {
  constexpr int BK = kGemmBK;
  constexpr int TM = BM / 16, TN = BN / 16;
  constexpr int PA = BM * BK / kGemmThreads;  // loads of A per thread per tile
  constexpr int PB = BN * BK / kGemmThreads;
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];

  const int t = threadIdx.x;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  const int z = blockIdx.z / splits, split = blockIdx.z - z * splits;
  const long long kbeg = (long long)split * k_per_split;
  long long kend = kbeg + k_per_split;
  if (kend > K) kend = K;

  // ---- per-thread load slots
  // along-K map: lane k = t % BK, rows t / BK + (256/BK) * pass
  // along-row map: row = t % BM, k = t / BM + (256/BM) * pass
  typename AL::Row a_rows[AL::kAlongK ? PA : 1];
  typename BL::Row b_rows[BL::kAlongK ? PB : 1];
  if (AL::kAlongK) {
#pragma unroll
    for (int p = 0; p < PA; ++p) a_rows[p] = al.row(m0 + t / BK + (kGemmThreads / BK) * p, z);
  } else {
    a_rows[0] = al.row(m0 + t % BM, z);
  }
  if (BL::kAlongK) {
#pragma unroll
    for (int p = 0; p < PB; ++p) b_rows[p] = bl.row(n0 + t / BK + (kGemmThreads / BK) * p, z);
  } else {
    b_rows[0] = bl.row(n0 + t % BN, z);
  }

  float ra[PA], rb[PB];
  auto fetch = [&](long long kt) {
    if (AL::kAlongK) {
      const long long k = kt + t % BK;
      const bool kv = k < kend;
      const typename AL::Kk ks = al.kk(kv ? k : kbeg, z);
#pragma unroll
      for (int p = 0; p < PA; ++p) ra[p] = kv ? al.load(a_rows[p], ks) : 0.f;
    } else {
#pragma unroll
      for (int p = 0; p < PA; ++p) {
        const long long k = kt + t / BM + (kGemmThreads / BM) * p;
        const bool kv = k < kend;
        const typename AL::Kk ks = al.kk(kv ? k : kbeg, z);
        ra[p] = kv ? al.load(a_rows[0], ks) : 0.f;
      }
    }
    if (BL::kAlongK) {
      const long long k = kt + t % BK;
      const bool kv = k < kend;
      const typename BL::Kk ks = bl.kk(kv ? k : kbeg, z);
#pragma unroll
      for (int p = 0; p < PB; ++p) rb[p] = kv ? bl.load(b_rows[p], ks) : 0.f;
    } else {
#pragma unroll
      for (int p = 0; p < PB; ++p) {
        const long long k = kt + t / BN + (kGemmThreads / BN) * p;
        const bool kv = k < kend;
        const typename BL::Kk ks = bl.kk(kv ? k : kbeg, z);
        rb[p] = kv ? bl.load(b_rows[0], ks) : 0.f;
      }
    }
  };
  auto stash = [&]() {
    if (AL::kAlongK) {
#pragma unroll
      for (int p = 0; p < PA; ++p) As[t % BK][t / BK + (kGemmThreads / BK) * p] = ra[p];
    } else {
#pragma unroll
      for (int p = 0; p < PA; ++p) As[t / BM + (kGemmThreads / BM) * p][t % BM] = ra[p];
    }
    if (BL::kAlongK) {
#pragma unroll
      for (int p = 0; p < PB; ++p) Bs[t % BK][t / BK + (kGemmThreads / BK) * p] = rb[p];
    } else {
#pragma unroll
      for (int p = 0; p < PB; ++p) Bs[t / BN + (kGemmThreads / BN) * p][t % BN] = rb[p];
    }
  };

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  const int tx = t % 16, ty = t / 16;
  if (kbeg < kend) {
    fetch(kbeg);
    stash();
    __syncthreads();
    for (long long kt = kbeg; kt < kend; kt += BK) {
      const bool more = kt + BK < kend;
      if (more) fetch(kt + BK);
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        float a[TM], b[TN];
#pragma unroll
        for (int i = 0; i < TM / 4; ++i) {
          const float4 v = *reinterpret_cast<const float4*>(&As[kk][i * 64 + ty * 4]);
          a[i * 4 + 0] = v.x; a[i * 4 + 1] = v.y; a[i * 4 + 2] = v.z; a[i * 4 + 3] = v.w;
        }
#pragma unroll
        for (int j = 0; j < TN / 4; ++j) {
          const float4 v = *reinterpret_cast<const float4*>(&Bs[kk][j * 64 + tx * 4]);
          b[j * 4 + 0] = v.x; b[j * 4 + 1] = v.y; b[j * 4 + 2] = v.z; b[j * 4 + 3] = v.w;
        }
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
      if (more) {
        stash();
        __syncthreads();
      }
    }
  }

  // ---- epilogue
  if (splits == 1) {
    typename EP::Col cols[TN];
#pragma unroll
    for (int j = 0; j < TN; ++j) cols[j] = ep.col(n0 + (j / 4) * 64 + tx * 4 + (j % 4), z);
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const int m = m0 + (i / 4) * 64 + ty * 4 + (i % 4);
      if (m >= M) continue;
      const typename EP::Row r = ep.row(m, z);
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const int n = n0 + (j / 4) * 64 + tx * 4 + (j % 4);
        if (n < N) ep.store(r, cols[j], acc[i][j]);
      }
    }
  } else {
    float* base = partial + ((long long)blockIdx.z * M) * N;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const int m = m0 + (i / 4) * 64 + ty * 4 + (i % 4);
      if (m >= M) continue;
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const int n = n0 + (j / 4) * 64 + tx * 4 + (j % 4);
        if (n < N) base[(long long)m * N + n] = acc[i][j];
      }
    }
  }
}

// Adds the split-K partial tiles in split order and hands the sum to the epilogue.
template <class EP>
__global__ void __launch_bounds__(256)
simt_splitk_reduce_kernel(const float* __restrict__ partial, EP ep, int M, int N, int Z,
                          int splits) {
  const long long mn = (long long)M * N;
  const long long total = mn * Z;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int z = (int)(i / mn);
    const long long r = i - (long long)z * mn;
    const int m = (int)(r / N), n = (int)(r - (long long)m * N);
    float s = 0.f;
    for (int sp = 0; sp < splits; ++sp) s += partial[((long long)(z * splits + sp)) * mn + r];
    ep.store(ep.row(m, z), ep.col(n, z), s);
  }
}

// A(row, k) = p[row*row_stride + k*k_stride + z*z_stride]; rows beyond `rows` read as 0.
template <bool ALONG_K>
struct StridedLoader {
  static constexpr bool kAlongK = ALONG_K;
  const float* p;
  long long row_stride, k_stride, z_stride;
  int rows;
  struct Row { long long off; };
  struct Kk { long long off; };
  __device__ Row row(int r, int z) const {
    return Row{r < rows ? (long long)r * row_stride + (long long)z * z_stride : -1};
  }
  __device__ Kk kk(long long k, int) const { return Kk{k * k_stride}; }
  __device__ float load(const Row& r, const Kk& k) const {
    return r.off >= 0 ? p[r.off + k.off] : 0.f;
  }
};

struct StridedEpilogue {
  float* c;
  long long row_stride, col_stride, z_stride;
  float alpha, beta;
  struct Row { long long off; };
  struct Col { long long off; };
  __device__ Row row(int m, int z) const {
    return Row{(long long)m * row_stride + (long long)z * z_stride};
  }
  __device__ Col col(int n, int) const { return Col{(long long)n * col_stride}; }
  __device__ void store(const Row& r, const Col& cc, float acc) const {
    float* dst = c + r.off + cc.off;
    *dst = beta == 0.f ? alpha * acc : alpha * acc + beta * *dst;
  }
};

struct SimtPlan {
  int bm, bn;
  int splits;
  long long k_per_split;
  size_t workspace_bytes;
};

inline SimtPlan plan_simt(long long M, long long N, long long K, long long Z) {
  SimtPlan p;
  p.bm = M <= 64 ? 64 : 128;
  p.bn = N <= 64 ? 64 : 128;
  const long long tiles = ((M + p.bm - 1) / p.bm) * ((N + p.bn - 1) / p.bn) * Z;
  const long long target = 4LL * device_info().sm_count;
  long long splits = 1;
  if (tiles < target && K >= 1024) {
    splits = (target + tiles - 1) / tiles;
    const long long max_by_k = K / 256;
    if (splits > max_by_k) splits = max_by_k;
    if (splits > 512) splits = 512;
    if (Z * splits > 65535) splits = 65535 / Z;
    if (splits < 1) splits = 1;
  }
  long long kps = (K + splits - 1) / splits;
  kps = (kps + kGemmBK - 1) / kGemmBK * kGemmBK;
  if (kps < kGemmBK) kps = kGemmBK;
  splits = (K + kps - 1) / kps;
  if (splits < 1) splits = 1;
  p.splits = (int)splits;
  p.k_per_split = kps;
  p.workspace_bytes = splits > 1 ? (size_t)(Z * splits * M * N) * sizeof(float) : 0;
  return p;
}

template <class AL, class BL, class EP>
int launch_simt_gemm(const char* name, const AL& al, const BL& bl, const EP& ep, long long M,
                     long long N, long long K, long long Z, void* workspace,
                     size_t workspace_bytes, cudaStream_t st) {
  if (M <= 0 || N <= 0 || Z <= 0) return FLB200_OK;
  FLB200_REQUIRE(M < 0x7fffffffLL && N < 0x7fffffffLL && K >= 0, "%s: extent out of range", name);
  SimtPlan p = plan_simt(M, N, K, Z);
  if (p.splits > 1 && (!workspace || workspace_bytes < p.workspace_bytes)) {
    // No scratch from the caller: run the whole K extent in one CTA per tile.
    p.splits = 1;
    p.k_per_split = (K + kGemmBK - 1) / kGemmBK * kGemmBK;
    if (p.k_per_split < kGemmBK) p.k_per_split = kGemmBK;
  }
  FLB200_REQUIRE(Z * p.splits <= 65535, "%s: too many batches", name);
  float* partial = static_cast<float*>(workspace);
  dim3 grid((unsigned)((N + p.bn - 1) / p.bn), (unsigned)((M + p.bm - 1) / p.bm),
            (unsigned)(Z * p.splits));
  FLB200_REQUIRE(grid.y <= 65535, "%s: M too large for the fp32 path", name);
#define FLB200_SIMT_LAUNCH(BM_, BN_)                                                    \
  simt_gemm_kernel<BM_, BN_, AL, BL, EP><<<grid, kGemmThreads, 0, st>>>(                \
      al, bl, ep, (int)M, (int)N, K, p.splits, p.k_per_split, partial)
  if (p.bm == 128 && p.bn == 128) FLB200_SIMT_LAUNCH(128, 128);
  else if (p.bm == 64 && p.bn == 128) FLB200_SIMT_LAUNCH(64, 128);
  else if (p.bm == 128 && p.bn == 64) FLB200_SIMT_LAUNCH(128, 64);
  else FLB200_SIMT_LAUNCH(64, 64);
#undef FLB200_SIMT_LAUNCH
  FLB200_AFTER_LAUNCH(name);
  if (p.splits > 1) {
    const int rgrid = grid_for(M * N * Z, 256);
    simt_splitk_reduce_kernel<EP><<<rgrid, 256, 0, st>>>(partial, ep, (int)M, (int)N, (int)Z,
                                                         p.splits);
    FLB200_AFTER_LAUNCH("splitk_reduce");
  }
  return FLB200_OK;
}

}  // namespace flb200
