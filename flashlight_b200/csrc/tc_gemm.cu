// Host side of the tcgen05 contraction: turns a strided matmul description into
// TMA tensor maps + operand plans, picks the tile width and the split-K factor,
// and launches tc_gemm_kernel (tc_core.cuh).  Used by flb200_matmul / the linear
// gradients in TF32 mode, by the convolution paths in tc_conv.cu and by rnn.cu.
#include <cuda_bf16.h>

#include "tc_gemm.cuh"

#include <cstdlib>
#include <mutex>

#include "tc_pair.cuh"

namespace flb200 {
namespace tc {

// ------------------------------------------------------- driver entry point
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    (void)cudaGetLastError();
  });
  return fn;
}

// fp32 tensor map; dims[0] is the contiguous dimension, strides_bytes[i] belongs to
// dims[i+1], box[0] must be 32 elements (128 bytes).  K-major operand tiles use the
// 128-byte swizzle of 16-byte chunks, MN-major ones the swizzle of 32-byte chunks.
int make_tensor_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, int mode,
                    const uint32_t* elem_strides, bool bf16) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(FLB200_UNSUPPORTED, "cuTensorMapEncodeTiled is not available");
  cuuint64_t gd[5];
  cuuint64_t gs[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = elem_strides ? elem_strides[i] : 1;
    if (i > 0) gs[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                  (cuuint32_t)rank, const_cast<void*>(base),
                  gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  mode == kMapStaging ? CU_TENSOR_MAP_SWIZZLE_NONE
                                      : (mode == kMapMnMajor ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                             : CU_TENSOR_MAP_SWIZZLE_128B),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(FLB200_INVALID_ARG, "cuTensorMapEncodeTiled failed with code %d (rank %d)", (int)r,
                rank);
  return FLB200_OK;
}

namespace {
thread_local bool t_x3 = false;
}
bool x3_enabled() { return t_x3; }
X3Scope::X3Scope(bool on) : prev(t_x3) { t_x3 = on; }
X3Scope::~X3Scope() { t_x3 = prev; }

std::atomic<long long> g_tc_launches{0};
void count_tc_launch() { g_tc_launches.fetch_add(1, std::memory_order_relaxed); }

// ------------------------------------------------------------ status flag
__device__ int g_tc_status = 0;

int* status_ptr() {
  // one address per device, looked up with that device current
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_tc_status) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

// ---------------------------------------------------------------- launch
// Sums split-K partial tiles in split order, then applies the epilogue.
static __global__ void __launch_bounds__(256)
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
    const long long off = epi_off(m, ep.m_div, ep.m_stride, ep.m_outer) +
                          epi_off(n, ep.n_div, ep.n_stride, ep.n_outer) + (long long)z * ep.z_stride;
    float v = ep.alpha * s + (ep.bias_m ? ep.bias_m[m] : 0.f) + (ep.bias_n ? ep.bias_n[n] : 0.f);
    if (ep.out_bf16) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(ep.out) + off;
      if (ep.beta != 0.f) v += ep.beta * __bfloat162float(*dst);
      *dst = __float2bfloat16(v);
    } else {
      float* dst = ep.out + off;
      if (ep.beta != 0.f) v += ep.beta * *dst;
      *dst = v;
    }
  }
}

// The same for a row-major result (unit column stride, no row / column regrouping) of a
// multiple of 4 columns: four columns per thread, 16-byte loads of every split's partial sums.
static __global__ void __launch_bounds__(256)
tc_splitk_reduce_vec_kernel(const float4* __restrict__ partial, EpiloguePlan ep, int M, int N4,
                            int Z, int splits) {
  const long long mn4 = (long long)M * N4;
  const long long total = mn4 * Z;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int z = (int)(i / mn4);
    const long long r = i - (long long)z * mn4;
    const int m = (int)(r / N4), n = 4 * (int)(r - (long long)m * N4);
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp = 0; sp < splits; ++sp) {
      const float4 p = partial[((long long)z * splits + sp) * mn4 + r];
      s.x += p.x; s.y += p.y; s.z += p.z; s.w += p.w;
    }
    const long long off = (long long)m * ep.m_stride + n + (long long)z * ep.z_stride;
    const float bm = ep.bias_m ? ep.bias_m[m] : 0.f;
    float v[4] = {ep.alpha * s.x + bm, ep.alpha * s.y + bm, ep.alpha * s.z + bm,
                  ep.alpha * s.w + bm};
    if (ep.bias_n) {
      const float4 b = *reinterpret_cast<const float4*>(ep.bias_n + n);
      v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
    }
    if (ep.out_bf16) {
      __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(
          reinterpret_cast<__nv_bfloat16*>(ep.out) + off);
      if (ep.beta != 0.f) {
        const float2 d0 = __bfloat1622float2(dst[0]), d1 = __bfloat1622float2(dst[1]);
        v[0] += ep.beta * d0.x; v[1] += ep.beta * d0.y;
        v[2] += ep.beta * d1.x; v[3] += ep.beta * d1.y;
      }
      __nv_bfloat162 h[2] = {__floats2bfloat162_rn(v[0], v[1]), __floats2bfloat162_rn(v[2], v[3])};
      *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<uint2*>(h);
    } else {
      float4* dst = reinterpret_cast<float4*>(ep.out + off);
      if (ep.beta != 0.f) {
        const float4 d = *dst;
        v[0] += ep.beta * d.x; v[1] += ep.beta * d.y; v[2] += ep.beta * d.z; v[3] += ep.beta * d.w;
      }
      *dst = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
}

static long long env_ll(const char* name, long long dflt) {
  const char* v = getenv(name);
  return v && *v ? atoll(v) : dflt;
}

template <int BN>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const OperandPlan& pa,
                       const OperandPlan& pb, const EpiloguePlan& ep, long long M, long long N,
                       long long k_iters, long long Z, const Launch& L, float* partial,
                       cudaStream_t st, bool bf16) {
  GemmProblem<BN> p;
  p.bf16 = bf16 ? 1 : 0;
  p.a = make_coords(pa); p.b = make_coords(pb); p.ep = ep;
  p.a_mn_major = pa.mn_major; p.b_mn_major = pb.mn_major;
  p.M = (int)M; p.N = (int)N; p.k_iters = (int)k_iters;
  p.splits = L.splits; p.iters_per_split = L.iters_per_split;
  p.tiles_m = (int)((M + kBM - 1) / kBM);
  // Pair tiles walk the column tiles of one pair of row tiles first: the row operand (the
  // large one of a tall product) is then fetched from DRAM once and found in L2 by the other
  // column tiles, instead of being streamed once per column tile with the output written in
  // between (1 x 1 layers that widen 4x: 11-15 % faster; FLB200_PAIR_N_FAST=0: rows first).
  static const long long n_fast = env_ll("FLB200_PAIR_N_FAST", 1);
  p.pair_n_fast = (int)n_fast;
  p.tiles_n = (int)((N + BN - 1) / BN);
  p.Z = (int)Z;
  p.partial = partial;
  const long long tiles = (long long)p.tiles_m * p.tiles_n * Z * L.splits;
  FLB200_REQUIRE(tiles < 0x7fffffffLL, "tc_gemm: too many tiles");
  if constexpr (BN >= 128) {
    if (!bf16 && !x3_enabled() &&
        gemm_uses_pairs(M, N, k_iters, pa.mn_major != 0, pb.mn_major != 0)) {
      const long long pair_tiles = (long long)((p.tiles_m + 1) / 2) * p.tiles_n * Z * L.splits;
      return launch_pair_problem<GemmProblem<BN>, BN>("tc_gemm_pair", ma, mb, p, pair_tiles, st);
    }
  }
  return launch_problem<GemmProblem<BN>, BN>("tc_gemm", ma, mb, p, tiles, st);
}

// Wider tiles re-read the 128-row operand less often (the contraction is fed from L2):
// 256 columns as soon as there are enough of them to fill most of such a tile.
int pick_bn(long long N) {
  if (N <= 32) return 32;
  if (N <= 64) return 64;
  if (N < 192) return 128;
  return 256;
}

bool gemm_uses_pairs(long long M, long long N, long long k_iters, bool a_mn_major,
                     bool b_mn_major) {
  if (x3_enabled()) return false;  // the CTA-pair kernel has no 3xTF32 instantiation
  // 1x1 forward layers (activation planes MN-major, filter K-major): 5-9 % faster on pairs
  // with 256-column tiles; with both operands MN-major (1x1 backward data: 8 copies per CTA
  // and stage) pairs measured between 7 % faster and 11 % slower and are not used.
  if (a_mn_major && !b_mn_major) return pick_bn(N) >= 256 && M > kBM && k_iters >= 8;
  if (a_mn_major || b_mn_major) return false;
  // both K-major: long K loops (backward-filter of 1 x 1 layers) ...
  if (pick_bn(N) >= 128 && M > kBM && k_iters >= 64) return true;
  // ... and tall products with wide rows (1 x 1 layers over channels-last tensors, linear
  // layers): every 128-row tile re-reads the whole B panel out of L2, a pair halves that
  static const long long min_k = env_ll("FLB200_PAIR_MIN_K", 4);
  static const long long min_bn = env_ll("FLB200_PAIR_MIN_BN", 256);
  return pick_bn(N) >= min_bn && M >= 8 * kBM && k_iters >= min_k;
}
int b_box_rows(long long M, long long N, long long k_iters, bool a_mn_major, bool b_mn_major) {
  const int bn = pick_bn(N);
  return gemm_uses_pairs(M, N, k_iters, a_mn_major, b_mn_major) ? bn / 2 : bn;
}

void plan_splits(long long tiles, long long k_iters, long long min_ips, int* splits_out,
                 int* ips_out) {
  // The persistent grid hands tile i to CTA i % grid, so the launch lasts
  // ceil(tiles * splits / SMs) rounds of one tile each.  Pick the split count with the
  // shortest critical path, charging every tile a fixed cost (pipeline fill, writing and
  // re-reading its partial sums) expressed in stage iterations.
  const long long sm = device_info().sm_count > 0 ? device_info().sm_count : 148;
  if (tiles < 1) tiles = 1;
  if (k_iters < 1) k_iters = 1;
  long long smax = k_iters / (min_ips > 0 ? min_ips : 1);
  const long long by_waves = (4 * sm + tiles - 1) / tiles;
  if (smax > by_waves) smax = by_waves;
  if (smax > 1024) smax = 1024;
  if (smax < 1) smax = 1;
  long long best_s = 1, best_ips = k_iters, best_cost = -1;
  for (long long s = 1; s <= smax; ++s) {
    const long long ips = (k_iters + s - 1) / s;
    const long long se = (k_iters + ips - 1) / ips;
    const long long rounds = (tiles * se + sm - 1) / sm;
    const long long cost = rounds * (ips + (se > 1 ? 16 : 4));
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best_s = se;
      best_ips = ips;
    }
  }
  *splits_out = (int)best_s;
  *ips_out = (int)best_ips;
}

Launch plan_launch(long long M, long long N, long long k_iters, long long Z) {
  Launch L;
  L.bn = pick_bn(N);
  const long long tiles = ((M + kBM - 1) / kBM) * ((N + L.bn - 1) / L.bn) * Z;
  plan_splits(tiles, k_iters, 8, &L.splits, &L.iters_per_split);
  L.workspace_bytes = L.splits > 1 ? (size_t)(Z * L.splits * M * N) * sizeof(float) : 0;
  return L;
}

int run(const CUtensorMap& ma, const CUtensorMap& mb, const OperandPlan& pa, const OperandPlan& pb,
        const EpiloguePlan& ep, long long M, long long N, long long k_iters, long long Z, void* ws,
        size_t ws_bytes, cudaStream_t st, bool bf16) {
  Launch L = plan_launch(M, N, k_iters, Z);
  // an MN-major bf16 B tile is made of 64-column boxes: no narrower tile than one box
  if (bf16 && pb.mn_major && L.bn < 64) L.bn = 64;
  // split-K partials are written with 16-byte vectors: an unaligned workspace is not used
  // (nor are the column statistics of the output taken from partial sums)
  if (L.splits > 1 && (!ws || !aligned16(ws) || ws_bytes < L.workspace_bytes || ep.stats || ep.act ||
                       ep.pre)) {
    L.splits = 1;
    L.iters_per_split = (int)k_iters;
  }
  float* partial = static_cast<float*>(ws);
  int rc;
  if (L.bn == 32) rc = launch_gemm<32>(ma, mb, pa, pb, ep, M, N, k_iters, Z, L, partial, st, bf16);
  else if (L.bn == 64) rc = launch_gemm<64>(ma, mb, pa, pb, ep, M, N, k_iters, Z, L, partial, st, bf16);
  else if (L.bn == 128) rc = launch_gemm<128>(ma, mb, pa, pb, ep, M, N, k_iters, Z, L, partial, st, bf16);
  else rc = launch_gemm<256>(ma, mb, pa, pb, ep, M, N, k_iters, Z, L, partial, st, bf16);
  if (rc) return rc;
  if (L.splits > 1) {
    const uintptr_t out_addr = reinterpret_cast<uintptr_t>(ep.out);
    const bool rows_of_4 = ep.m_div == 0 && ep.n_div == 0 && ep.m_valid == 0 && ep.n_stride == 1 &&
                           N % 4 == 0 && ep.m_stride % 4 == 0 && ep.z_stride % 4 == 0 &&
                           out_addr % (ep.out_bf16 ? 8 : 16) == 0 &&
                           (!ep.bias_n || aligned16(ep.bias_n));
    if (rows_of_4) {
      const int rgrid = grid_for(M * (N / 4) * Z, 256);
      tc_splitk_reduce_vec_kernel<<<rgrid, 256, 0, st>>>(reinterpret_cast<const float4*>(partial),
                                                         ep, (int)M, (int)(N / 4), (int)Z,
                                                         L.splits);
    } else {
      const int rgrid = grid_for(M * N * Z, 256);
      tc_splitk_reduce_kernel<<<rgrid, 256, 0, st>>>(partial, ep, (int)M, (int)N, (int)Z,
                                                     L.splits);
    }
    FLB200_AFTER_LAUNCH("tc_splitk_reduce");
  }
  return FLB200_OK;
}

}  // namespace tc

// ----------------------------------------------------- strided matmul entry
namespace {

struct Side {
  bool ok, mn_major;
  long long ld;  // stride (elements) of the non-contiguous dimension
};

// op(r, k) at base[r*row + k*col]: decide the major and the leading dimension.
// `vec` = elements per 16 bytes (4 for fp32, 8 for bf16): leading dimensions must keep every
// row 16-byte aligned.
Side classify(long long row, long long col, long long rows, long long K, long long vec) {
  Side s{false, false, 0};
  if (col == 1 && (row % vec == 0 || rows == 1) && row >= 1) {
    s = Side{true, false, rows == 1 ? (K + vec - 1) / vec * vec : row};
  } else if (row == 1 && (col % vec == 0 || K == 1) && col >= 1) {
    s = Side{true, true, K == 1 ? (rows + vec - 1) / vec * vec : col};
  }
  return s;
}

struct Prepared {
  bool ok = false;
  bool swap = false;
  Side a, b;
};

Prepared prepare(const flb200_matmul_desc* d, const void* a, const void* b, const void* c) {
  Prepared p;
  const bool bf16 = d->dtype == FLB200_BF16;
  if ((d->dtype != FLB200_F32 && !bf16) || d->m < 1 || d->n < 1 || d->k < 1) return p;
  const long long vec = bf16 ? 8 : 4;
  if (!aligned16(a) || !aligned16(b) || !c) return p;
  if (d->batch > 1 && (d->a_batch % vec != 0 || d->b_batch % vec != 0)) return p;
  // too little work to pay for a tensor-core launch: leave it to the fp32 kernel (bf16 has
  // no other kernel and always comes here)
  if (!bf16 && (double)d->m * (double)d->n * (double)d->k < 262144.0) return p;
  p.a = classify(d->a_row, d->a_col, d->m, d->k, vec);
  // B(k, n): "row" of the operand is n with stride b_col; k stride is b_row
  p.b = classify(d->b_col, d->b_row, d->n, d->k, vec);
  if (!p.a.ok || !p.b.ok) return p;
  p.swap = d->m < 64 && d->n > d->m;  // put the long extent on the 128-row side of the MMA
  p.ok = true;
  return p;
}

// Tensor map + plan of one operand: rows x K matrix (+ batch).
int build_operand(const Side& s, const void* base, long long rows, long long K, long long batch,
                  long long batch_stride, int tile_rows, CUtensorMap* map, tc::OperandPlan* plan,
                  bool bf16) {
  const uint32_t kstage = bf16 ? 64 : tc::kBK;   // elements of K per stage (128 bytes)
  const uint64_t esize = bf16 ? 2 : 4;
  uint64_t dims[3], strides[2];
  uint32_t box[3];
  *plan = tc::OperandPlan{};
  plan->k_inner = 0;
  plan->k2_dim = -1;
  if (s.mn_major) {
    dims[0] = (uint64_t)rows; dims[1] = (uint64_t)K;
    box[0] = bf16 ? 64 : 32; box[1] = kstage;
    plan->mn_major = 1; plan->mn_dim = 0; plan->k_dim = 1;
  } else {
    dims[0] = (uint64_t)K; dims[1] = (uint64_t)rows;
    box[0] = kstage; box[1] = (uint32_t)tile_rows;
    plan->mn_major = 0; plan->mn_dim = 1; plan->k_dim = 0;
  }
  plan->k_elems = (int)kstage;
  strides[0] = (uint64_t)s.ld * esize;
  int rank = 2;
  plan->z_dim = -1;
  if (batch > 1) {
    dims[2] = (uint64_t)batch;
    strides[1] = (uint64_t)batch_stride * esize;
    box[2] = 1;
    rank = 3;
    plan->z_dim = 2;
  }
  plan->rank = rank;
  // bf16 tiles use the plain 128-byte swizzle for both majors
  return tc::make_tensor_map(map, base, rank, dims, strides, box,
                             s.mn_major && !bf16 ? tc::kMapMnMajor : tc::kMapKMajor, nullptr,
                             bf16);
}

}  // namespace

bool tc_gemm_supported(const flb200_matmul_desc* d, const void* a, const void* b, const void* c) {
  if (device_info().cc_major != 10) return false;
  if (!tc::encode_tiled_fn()) return false;
  return prepare(d, a, b, c).ok;
}

size_t tc_gemm_workspace_bytes(const flb200_matmul_desc* d) {
  if (!d || d->m < 1 || d->n < 1 || d->k < 1) return 0;
  const long long kstage = d->dtype == FLB200_BF16 ? 64 : tc::kBK;
  const long long k_iters = (d->k + kstage - 1) / kstage;
  // the swapped orientation has the same M*N; take the larger split count of both
  const size_t w1 = tc::plan_launch(d->m, d->n, k_iters, d->batch).workspace_bytes;
  const size_t w2 = tc::plan_launch(d->n, d->m, k_iters, d->batch).workspace_bytes;
  return w1 > w2 ? w1 : w2;
}

int tc_gemm_run(const flb200_matmul_desc* d, const void* a, const void* b, void* c, void* ws,
                size_t ws_bytes, cudaStream_t st, const float* bias_n, int act, void* pre) {
  const Prepared p = prepare(d, a, b, c);
  if (!p.ok) return fail(FLB200_UNSUPPORTED, "tc_gemm: layout not covered");
  const bool fused = bias_n != nullptr || act != 0 || pre != nullptr;
  if (fused && (p.swap || d->c_col != 1 || d->beta != 0.f || d->n % 32 != 0 || d->batch != 1 ||
                (d->c_row & 7) != 0 || !aligned16(c) || (pre && !aligned16(pre))))
    return fail(FLB200_UNSUPPORTED,
                "tc_gemm: bias / activation are fused only into a row-major, 16-byte aligned "
                "result of a multiple of 32 columns");
  const bool bf16 = d->dtype == FLB200_BF16;
  const long long kstage = bf16 ? 64 : tc::kBK;
  const long long k_iters = (d->k + kstage - 1) / kstage;
  CUtensorMap ma, mb;
  tc::OperandPlan pa, pb;
  tc::EpiloguePlan ep{};
  ep.out = static_cast<float*>(c);
  ep.out_bf16 = bf16 ? 1 : 0;
  ep.alpha = d->alpha;
  ep.beta = d->beta;
  ep.z_stride = d->c_batch;
  ep.bias_n = bias_n;
  ep.act = act;
  ep.pre = pre;
  long long M, N;
  if (!p.swap) {
    M = d->m; N = d->n;
    const int bn = tc::pick_bn(N);
    if (int rc = build_operand(p.a, a, d->m, d->k, d->batch, d->a_batch, tc::kBM, &ma, &pa, bf16)) return rc;
    if (int rc = build_operand(p.b, b, d->n, d->k, d->batch, d->b_batch,
                               bf16 ? bn : tc::b_box_rows(M, N, k_iters, p.a.mn_major, p.b.mn_major), &mb,
                               &pb, bf16)) return rc;
    ep.m_stride = d->c_row;
    ep.n_stride = d->c_col;
  } else {
    // C^T = B^T A^T: the kernel's rows are the caller's columns
    M = d->n; N = d->m;
    const int bn = tc::pick_bn(N);
    if (int rc = build_operand(p.b, b, d->n, d->k, d->batch, d->b_batch, tc::kBM, &ma, &pa, bf16)) return rc;
    if (int rc = build_operand(p.a, a, d->m, d->k, d->batch, d->a_batch,
                               bf16 ? bn : tc::b_box_rows(M, N, k_iters, p.b.mn_major, p.a.mn_major), &mb,
                               &pb, bf16)) return rc;
    ep.m_stride = d->c_col;
    ep.n_stride = d->c_row;
  }
  return tc::run(ma, mb, pa, pb, ep, M, N, k_iters, d->batch, ws, ws_bytes, st, bf16);
}

}  // namespace flb200

extern "C" {

int flb200_has_tensor_core_path(void) {
  return flb200::device_info().cc_major == 10 && flb200::tc::encode_tiled_fn() != nullptr ? 1 : 0;
}

long long flb200_tc_kernel_launches(void) {
  return flb200::tc::g_tc_launches.load(std::memory_order_relaxed);
}

// Reads (and clears) the device flag that a bounded wait inside a tensor-core kernel raises when
// it runs out.  Synchronises the stream.  Returns FLB200_TIMEOUT if the flag was set.
int flb200_tc_poll_status(void* stream) {
  using namespace flb200;
  int* p = tc::status_ptr();
  if (!p) return FLB200_OK;
  int v = 0;
  cudaStream_t st = as_stream(stream);
  FLB200_CUDA_CHECK(cudaMemcpyAsync(&v, p, sizeof(int), cudaMemcpyDeviceToHost, st));
  FLB200_CUDA_CHECK(cudaStreamSynchronize(st));
  if (v != 0) {
    FLB200_CUDA_CHECK(cudaMemsetAsync(p, 0, sizeof(int), st));
    return fail(FLB200_TIMEOUT, "a tensor-core kernel gave up waiting (stage %d)", v);
  }
  return FLB200_OK;
}

}  // extern "C"
