// Fused attention backward (flash style): dq, dk, dv of  o = softmax(scale * q k^T [+ causal
// mask]) v  without materialising the T x T score tensors in device memory.  The reference
// builds the chain out of whole-tensor operators and keeps the probabilities for the gradient
// (flashlight/fl/autograd/Functions.cpp:1828-1891, 1021-1042); here the forward pass keeps only
// the row-wise log-sum-exp of the scaled scores, and this kernel recomputes the probabilities of
// one 128 x 128 block at a time in tensor memory.
//
// bf16 tensors [batch * heads][T][64], T a multiple of 128.  One CTA per (batch-head, block of
// 128 keys): K_j and V_j stay in shared memory, the CTA walks the query blocks i (i >= j with
// the causal mask) and per block issues five tcgen05 contractions with fp32 accumulators in
// tensor memory:
//     S  = Q_i K_j^T                    (128 x 128, K = 64)   columns   0..127
//     dP = dO_i V_j^T                   (128 x 128, K = 64)   columns 128..255
//     dV_j += P^T dO_i                  (128 x  64, K = 128)  columns 256..319   (kept over i)
//     dK_j += dS^T Q_i                  (128 x  64, K = 128)  columns 320..383   (kept over i)
//     dQ_i  = dS K_j                    (128 x  64, K = 128)  columns 384..447
// with P = exp(scale * S - lse), dS = scale * P * (dP - D) and D = rowsum(dO * O) from a small
// pre-pass, computed by the row threads (two per query row, half of the columns each) between
// the two groups of contractions and written to shared memory as bf16
// operand tiles.  One storage order serves every role a tile plays: row r of a tile is 128
// bytes (64 bf16) at r * 128 with its 16-byte chunks XOR-swizzled by r & 7 — read as a K-major
// operand (rows = m or n, 64 k per row) or as an MN-major operand (rows = k, 64 m or n per
// row), so Q_i, dO_i and K_j are used as TMA delivered them, and P / dS (two 64-key halves,
// 16 KB apart) feed both the transposed products and dS K_j.  dQ blocks of different CTAs are
// summed with fp32 atomics into scratch and rounded to bf16 by a second small kernel.
// Every mbarrier wait is bounded (tc_core.cuh): a wait that runs out raises the library's status
// flag and the CTA finishes its loop without waiting again.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "flb200.h"
#include "tc_core.cuh"
#include "tc_gemm.cuh"

namespace flb200 {
namespace {

using namespace tc;

constexpr int kAttnThreads = 288;      // warps 0..7: two threads per query row (each half of the
                                       // columns); warp 8: TMA + MMA
constexpr int kTile = 128 * 128;       // bytes of a [128 rows][64 bf16] tile
constexpr int kAttnSmem = 4 * kTile + 2 * 2 * kTile + 1024 + 256;  // K V Q dO, P dS, align, bars

struct AttnArgs {
  const float* dsum;  // rowsum(dO * O), from attention_dsum_kernel
  const float* lse;
  float* dq_acc;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int T, causal;
  float scale;
  int* status;
};

// byte offset of the 16-byte chunk holding keys key0 .. key0 + 7 of query row r in a P / dS tile
__device__ __forceinline__ uint32_t score_chunk(int r, int key0) {
  return (uint32_t)(key0 >> 6) * kTile + (uint32_t)r * 128 +
         ((((uint32_t)(key0 & 63) >> 3) ^ ((uint32_t)r & 7)) << 4);
}

// four consecutive fp32 sums in one reduction instruction (16-byte aligned address)
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// two 32-column loads of this thread's tensor-memory lane in flight together
__device__ __forceinline__ void tmem_ld32_pair(uint32_t ta, float* a, uint32_t tb, float* b) {
  uint32_t x[32], y[32];
#define FLB200_LD32(addr, r)                                                                     \
  asm volatile(                                                                                  \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                  \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                  \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"  \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),      \
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),  \
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),            \
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),            \
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])             \
      : "r"(addr)                                                                                \
      : "memory")
  FLB200_LD32(ta, x);
  FLB200_LD32(tb, y);
#undef FLB200_LD32
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    a[i] = __uint_as_float(x[i]);
    b[i] = __uint_as_float(y[i]);
  }
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(kAttnThreads)
attention_backward_kernel(const __grid_constant__ CUtensorMap map_q,
                          const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v,
                          const __grid_constant__ CUtensorMap map_do, const AttnArgs a) {
  extern __shared__ __align__(1024) char smem_raw[];
  char* base = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                       ~static_cast<uintptr_t>(1023));
  char* sK = base;
  char* sV = base + kTile;
  char* sQ = base + 2 * kTile;
  char* sDO = base + 3 * kTile;
  char* sP = base + 4 * kTile;   // two 64-key halves
  char* sDS = base + 6 * kTile;  // two 64-key halves
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + 8 * kTile);
  uint64_t* bar_kv = bars;      // K_j, V_j landed
  uint64_t* bar_q = bars + 1;   // Q_i, dO_i landed
  uint64_t* bar_s = bars + 2;   // S and dP complete
  uint64_t* bar_o = bars + 3;   // dV, dK, dQ contractions complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  int* failed = reinterpret_cast<int*>(bars + 5);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = a.T / 128;
  const int j = blockIdx.x % nblk;        // key block
  const int bh = blockIdx.x / nblk;       // batch * heads index
  const long long row0 = (long long)bh * a.T;  // first row of this head in the [BH * T][64] views

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(bar_q, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *failed = 0;
    fence_barrier_init();
  }
  if (warp == 8) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const bool issuer = warp == 8 && lane == 0;
  const bool row_thread = warp < 8;
  const int r = (warp & 3) * 32 + lane;  // query row inside the block (row threads)
  const int half = warp >> 2;            // which half of the columns this row thread handles

  // operand descriptors (see the file comment): K-major tiles step 32 bytes per 16 k,
  // MN-major tiles step 16 rows = 2048 bytes per 16 k
  const uint64_t dK_k = umma_desc(smem_u32(sK), 16, 1024, 2);
  const uint64_t dV_k = umma_desc(smem_u32(sV), 16, 1024, 2);
  const uint64_t dQ_k = umma_desc(smem_u32(sQ), 16, 1024, 2);
  const uint64_t dDO_k = umma_desc(smem_u32(sDO), 16, 1024, 2);
  const uint64_t dP_mn = umma_desc(smem_u32(sP), kTile, 1024, 2);    // 64-key boxes 16 KB apart
  const uint64_t dDS_mn = umma_desc(smem_u32(sDS), kTile, 1024, 2);
  const uint64_t dDS_k = umma_desc(smem_u32(sDS), 16, 1024, 2);
  const uint64_t dDO_mn = umma_desc(smem_u32(sDO), 8192, 1024, 2);   // one box of 64 d
  const uint64_t dQ_mn = umma_desc(smem_u32(sQ), 8192, 1024, 2);
  const uint64_t dK_mn = umma_desc(smem_u32(sK), 8192, 1024, 2);
  const uint32_t id_s = umma_idesc_bf16(128, 0, 0);   // S, dP
  const uint32_t id_t = umma_idesc_bf16(64, 1, 1);    // dV, dK: both operands MN-major
  const uint32_t id_q = umma_idesc_bf16(64, 0, 1);    // dQ: dS K-major, K_j MN-major

  if (issuer) {
    mbar_expect_tx(bar_kv, 2 * kTile);
    int c[2] = {0, (int)(row0 + (long long)j * 128)};
    tma_load(&map_k, bar_kv, sK, 2, c);
    tma_load(&map_v, bar_kv, sV, 2, c);
  }

#ifdef FLB200_ATTN_PROFILE
  long long pc[6] = {0, 0, 0, 0, 0, 0};
#define ATTN_MARK(k, t) pc[k] += clock64() - t; t = clock64()
  long long tp = clock64();
#else
#define ATTN_MARK(k, t)
#endif
  const int i_first = a.causal ? j : 0;
  uint32_t it = 0;
  for (int i = i_first; i < nblk; ++i, ++it) {
    const uint32_t ph = it & 1;
    const long long qrow = row0 + (long long)i * 128;
    if (issuer) {
      mbar_expect_tx(bar_q, 2 * kTile);
      int c[2] = {0, (int)qrow};
      tma_load(&map_q, bar_q, sQ, 2, c);
      tma_load(&map_do, bar_q, sDO, 2, c);
      if (it == 0 && *failed == 0 && !mbar_wait(bar_kv, 0)) *failed = 1;
      if (*failed == 0 && !mbar_wait(bar_q, ph)) *failed = 2;
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)  // K = 64 d in steps of 16
        umma_bf16(tmem, umma_desc_advance(dQ_k, kk * 32), umma_desc_advance(dK_k, kk * 32), id_s,
                  kk > 0);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem + 128, umma_desc_advance(dDO_k, kk * 32), umma_desc_advance(dV_k, kk * 32),
                  id_s, kk > 0);
      umma_commit(bar_s);
    }
    float lse = 0.f, dsum = 0.f;
    if (row_thread) {
      dsum = a.dsum[qrow + r];
      lse = a.lse[qrow + r];
      ATTN_MARK(0, tp);
      if (*failed == 0 && !mbar_wait(bar_s, ph)) *failed = 3;
      tc_fence_after();
      ATTN_MARK(1, tp);
      const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
      const int q_pos = i * 128 + r;
#pragma unroll 1
      for (int c0 = 64 * half; c0 < 64 * half + 64; c0 += 32) {
        float s[32], dp[32];
        tmem_ld32_pair(lane_addr + (uint32_t)c0, s, lane_addr + 128u + (uint32_t)c0, dp);
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const bool masked = a.causal && (j * 128 + c0 + e > q_pos);
          const float p = masked ? 0.f : __expf(a.scale * s[e] - lse);
          s[e] = p;
          dp[e] = a.scale * p * (dp[e] - dsum);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t off = score_chunk(r, c0 + 8 * u);
          *reinterpret_cast<uint4*>(sP + off) =
              make_uint4(pack_bf16(s[8 * u], s[8 * u + 1]), pack_bf16(s[8 * u + 2], s[8 * u + 3]),
                         pack_bf16(s[8 * u + 4], s[8 * u + 5]), pack_bf16(s[8 * u + 6], s[8 * u + 7]));
          *reinterpret_cast<uint4*>(sDS + off) = make_uint4(
              pack_bf16(dp[8 * u], dp[8 * u + 1]), pack_bf16(dp[8 * u + 2], dp[8 * u + 3]),
              pack_bf16(dp[8 * u + 4], dp[8 * u + 5]), pack_bf16(dp[8 * u + 6], dp[8 * u + 7]));
        }
      }
      fence_proxy_async();  // the tensor core reads these generic-proxy writes next
      ATTN_MARK(2, tp);
    }
    tc_fence_before();
    __syncthreads();
    if (issuer) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {  // K = 128 query rows in steps of 16
        umma_bf16(tmem + 256, umma_desc_advance(dP_mn, kk * 2048),
                  umma_desc_advance(dDO_mn, kk * 2048), id_t, (it > 0 || kk > 0) ? 1u : 0u);
        umma_bf16(tmem + 320, umma_desc_advance(dDS_mn, kk * 2048),
                  umma_desc_advance(dQ_mn, kk * 2048), id_t, (it > 0 || kk > 0) ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)  // K = 128 keys: two 64-key halves of dS, 16 key rows of K_j
        umma_bf16(tmem + 384, umma_desc_advance(dDS_k, (kk >> 2) * kTile + (kk & 3) * 32),
                  umma_desc_advance(dK_mn, kk * 2048), id_q, kk > 0);
      umma_commit(bar_o);
    }
    if (*failed == 0 && !mbar_wait(bar_o, ph)) *failed = 4;
    tc_fence_after();
    if (row_thread) {
      ATTN_MARK(3, tp);
      float* dst = a.dq_acc + (qrow + r) * 64 + 32 * half;
      float v[32];
      tmem_ld32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + 384u + 32u * half, v);
#pragma unroll
      for (int e = 0; e < 32; e += 4) red_add_v4(dst + e, v[e], v[e + 1], v[e + 2], v[e + 3]);
      ATTN_MARK(4, tp);
    }
    // the next block's loads and contractions overwrite Q_i, dO_i, S, dP, P, dS and dQ
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
#ifdef FLB200_ATTN_PROFILE
    if (row_thread) { ATTN_MARK(5, tp); }
#endif
  }
#ifdef FLB200_ATTN_PROFILE
  if (blockIdx.x == 0 && threadIdx.x == 0)
    printf("attention profile (CTA 0, %u blocks): D+lse %lld | wait S,dP %lld | softmax %lld | wait dV dK dQ %lld | atomics %lld | sync %lld\n",
           it, pc[0], pc[1], pc[2], pc[3], pc[4], pc[5]);
#endif

  if (row_thread) {
    // the first half of the row threads stores dV_j, the second dK_j
    const long long krow = row0 + (long long)j * 128 + r;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + 256u + 64u * half;
    __nv_bfloat16* out = (half == 0 ? a.dv : a.dk) + krow * 64;
#pragma unroll 1
    for (int c0 = 0; c0 < 64; c0 += 32) {
      float v[32];
      tmem_ld32(lane_addr + (uint32_t)c0, v);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        *reinterpret_cast<uint4*>(out + c0 + 8 * u) =
            make_uint4(pack_bf16(v[8 * u], v[8 * u + 1]), pack_bf16(v[8 * u + 2], v[8 * u + 3]),
                       pack_bf16(v[8 * u + 4], v[8 * u + 5]), pack_bf16(v[8 * u + 6], v[8 * u + 7]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *failed != 0 && a.status) atomicExch(a.status, *failed);
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// D[row] = sum_d dO[row][d] * O[row][d]: eight lanes per row, one 16-byte load each
__global__ void attention_dsum_kernel(const __nv_bfloat16* __restrict__ o,
                                      const __nv_bfloat16* __restrict__ d_o,
                                      float* __restrict__ dsum, long long rows) {
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long row = t >> 3;
  float acc = 0.f;
  if (row < rows) {
    const uint4 vo = reinterpret_cast<const uint4*>(o)[t];
    const uint4 vg = reinterpret_cast<const uint4*>(d_o)[t];
    const __nv_bfloat162* ho = reinterpret_cast<const __nv_bfloat162*>(&vo);
    const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&vg);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 fo = __bfloat1622float2(ho[e]), fg = __bfloat1622float2(hg[e]);
      acc += fo.x * fg.x + fo.y * fg.y;
    }
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  if (row < rows && (threadIdx.x & 7) == 0) dsum[row] = acc;
}

__global__ void narrow_dq_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                 long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 lo = reinterpret_cast<const float4*>(acc)[2 * i];
    const float4 hi = reinterpret_cast<const float4*>(acc)[2 * i + 1];
    reinterpret_cast<uint4*>(dq)[i] = make_uint4(pack_bf16(lo.x, lo.y), pack_bf16(lo.z, lo.w),
                                                 pack_bf16(hi.x, hi.y), pack_bf16(hi.z, hi.w));
  }
}

}  // namespace
}  // namespace flb200

using namespace flb200;

extern "C" {

size_t flb200_attention_backward_workspace_bytes(int64_t batch_heads, int64_t seq_len,
                                                 int64_t head_dim) {
  if (batch_heads <= 0 || seq_len <= 0 || head_dim <= 0) return 0;
  // fp32 sums of dq, then rowsum(dO * O)
  return (size_t)batch_heads * seq_len * head_dim * sizeof(float) +
         (size_t)batch_heads * seq_len * sizeof(float);
}

int flb200_attention_backward_supported(int64_t seq_len, int64_t head_dim, int dtype) {
  return flb200_has_tensor_core_path() && dtype == FLB200_BF16 && head_dim == 64 && seq_len > 0 &&
                 seq_len % 128 == 0
             ? 1
             : 0;
}

int flb200_attention_backward(const void* q, const void* k, const void* v, const void* o,
                              const void* grad_o, const float* lse, void* grad_q, void* grad_k,
                              void* grad_v, int64_t batch_heads, int64_t seq_len,
                              int64_t head_dim, float scale, int causal, int dtype,
                              void* workspace, size_t workspace_bytes, void* stream) {
  FLB200_REQUIRE(q && k && v && o && grad_o && lse && grad_q && grad_k && grad_v,
                 "attention_backward: null tensor");
  FLB200_REQUIRE(batch_heads > 0, "attention_backward: empty batch");
  if (!flb200_attention_backward_supported(seq_len, head_dim, dtype))
    return fail(FLB200_UNSUPPORTED,
                "attention_backward: built for bf16, head dimension 64 and a sequence length that "
                "is a multiple of 128 (got dtype %d, head %lld, length %lld)",
                dtype, (long long)head_dim, (long long)seq_len);
  const long long rows = (long long)batch_heads * seq_len;
  FLB200_REQUIRE(rows < 0x7fffffffLL, "attention_backward: too many rows");
  const size_t need = flb200_attention_backward_workspace_bytes(batch_heads, seq_len, head_dim);
  if (!workspace || workspace_bytes < need)
    return fail(FLB200_WORKSPACE_TOO_SMALL, "attention_backward: workspace %zu < %zu",
                workspace_bytes, need);
  const void* ptrs[] = {q, k, v, o, grad_o, grad_q, grad_k, grad_v, workspace};
  for (const void* p : ptrs)
    FLB200_REQUIRE(aligned16(p), "attention_backward: tensors must be 16-byte aligned");
  cudaStream_t st = as_stream(stream);
  CUtensorMap mq, mk, mv, mg;
  const uint64_t dims[2] = {64, (uint64_t)rows};
  const uint64_t strides[1] = {128};
  const uint32_t box[2] = {64, 128};
  if (int rc = tc::make_tensor_map(&mq, q, 2, dims, strides, box, tc::kMapKMajor, nullptr, true)) return rc;
  if (int rc = tc::make_tensor_map(&mk, k, 2, dims, strides, box, tc::kMapKMajor, nullptr, true)) return rc;
  if (int rc = tc::make_tensor_map(&mv, v, 2, dims, strides, box, tc::kMapKMajor, nullptr, true)) return rc;
  if (int rc = tc::make_tensor_map(&mg, grad_o, 2, dims, strides, box, tc::kMapKMajor, nullptr, true)) return rc;
  static bool configured[64] = {false};
  int dev = 0;
  FLB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    FLB200_CUDA_CHECK(cudaFuncSetAttribute(attention_backward_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem));
    configured[dev] = true;
  }
  const size_t acc_bytes = (size_t)rows * 64 * sizeof(float);
  FLB200_CUDA_CHECK(cudaMemsetAsync(workspace, 0, acc_bytes, st));
  float* dsum = reinterpret_cast<float*>(static_cast<char*>(workspace) + acc_bytes);
  attention_dsum_kernel<<<(unsigned)((rows * 8 + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(grad_o), dsum, rows);
  FLB200_AFTER_LAUNCH("attention_dsum");
  AttnArgs a{};
  a.dsum = dsum;
  a.lse = lse;
  a.dq_acc = static_cast<float*>(workspace);
  a.dk = static_cast<__nv_bfloat16*>(grad_k);
  a.dv = static_cast<__nv_bfloat16*>(grad_v);
  a.T = (int)seq_len;
  a.causal = causal ? 1 : 0;
  a.scale = scale;
  a.status = tc::status_ptr();
  const unsigned grid = (unsigned)(batch_heads * (seq_len / 128));
  attention_backward_kernel<<<grid, kAttnThreads, kAttnSmem, st>>>(mq, mk, mv, mg, a);
  FLB200_AFTER_LAUNCH("attention_backward");
  tc::count_tc_launch();
  const long long n8 = rows * 64 / 8;
  narrow_dq_kernel<<<(unsigned)std::min<long long>((n8 + 255) / 256, 148 * 8), 256, 0, st>>>(
      a.dq_acc, static_cast<__nv_bfloat16*>(grad_q), n8);
  FLB200_AFTER_LAUNCH("attention_narrow_dq");
  return FLB200_OK;
}

}  // extern "C"
