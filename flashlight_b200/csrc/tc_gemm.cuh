// Host interface of the tcgen05 (tensor-core) contraction — fp32 operands read as TF32, or
// bf16 operands — with fp32 accumulation: the plan structs that describe how operands are
// fetched by TMA and how the accumulator is stored, and the entry points used by matmul, the
// convolution paths and the RNN.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace flb200 {

// True when the tensor-core kernel covers this problem (layout, alignment, size).
bool tc_gemm_supported(const flb200_matmul_desc* d, const void* a, const void* b, const void* c);
size_t tc_gemm_workspace_bytes(const flb200_matmul_desc* d);
// bias_n / act / pre: per-column bias, activation and pre-activation copy fused into the store
// (EpiloguePlan); only for products whose result is stored row-major as the caller's C
// (FLB200_UNSUPPORTED otherwise, so that the caller can run the operators one by one).
int tc_gemm_run(const flb200_matmul_desc* d, const void* a, const void* b, void* c, void* ws,
                size_t ws_bytes, cudaStream_t st, const float* bias_n = nullptr, int act = 0,
                void* pre = nullptr);

namespace tc {

constexpr int kBM = 128;  // rows of one output tile (UMMA M)
constexpr int kBK = 32;   // fp32 elements per pipeline stage along K (= 128 bytes)

// How one operand's TMA coordinates advance.  coord[d] for dimension d of the
// tensor map is  base[d] + mn * (d == mn_dim) + k_lo * (d == k_dim)
//                + k_hi * k2_scale * (d == k2_dim) + z * (d == z_dim)
// where k = k_hi * k_inner + k_lo walks the contraction (k_lo in elements).  k2_dim may
// equal k_dim (a flat pixel axis made of images of k2_scale pixels each).
struct OperandPlan {
  int rank;      // tensor-map rank, 2..4
  int mn_major;  // 1: m (or n) is the contiguous dimension
  int mn_dim, k_dim, k2_dim, z_dim;  // -1 = unused
  int k_inner;   // stage iterations per k2 step (ceil(extent of k_dim / kBK)); 0 = single level
  int k2_scale;  // coordinate step per k_hi
  int base[4];
  int k_elems;   // elements per stage along K: 0 = kBK (fp32), 64 for 2-byte operands
  // MN-major fp32 operand whose m / n extent is a multiple of 32: the map splits that index
  // into (32 contiguous, group of 32) and mn_dim is the GROUP dimension, so ONE copy of
  // `tile rows / 32` groups lands as the same consecutive 32 x 32 boxes as one copy per box.
  int mn_grouped;
};

// The same plan flattened for the device: per-dimension multipliers of the tile offset, the
// two levels of the k walk and the batch index.
struct OperandCoords {
  int rank, mn_major, k_inner;
  int base[4], mn_mul[4], k_mul[4], k2_mul[4], z_mul[4];
  int mn_shift;  // 5 for a grouped MN-major operand (the coordinate counts groups of 32), else 0
};
inline OperandCoords make_coords(const OperandPlan& p) {
  OperandCoords c{};
  c.rank = p.rank; c.mn_major = p.mn_major; c.k_inner = p.k_inner;
  c.mn_shift = p.mn_grouped ? 5 : 0;
  for (int d = 0; d < 4; ++d) {
    c.base[d] = p.base[d];
    c.mn_mul[d] = d == p.mn_dim ? 1 : 0;
    c.k_mul[d] = d == p.k_dim ? (p.k_elems ? p.k_elems : kBK) : 0;
    c.k2_mul[d] = d == p.k2_dim ? p.k2_scale : 0;
    c.z_mul[d] = d == p.z_dim ? 1 : 0;
  }
  return c;
}

struct EpiloguePlan {
  float* out;
  // offset(m) = (m / m_div) * m_outer + (m % m_div) * m_stride   (m_div == 0: m * m_stride);
  // rows with (m % m_div) >= m_valid are padding and are not stored (m_valid == 0: all valid)
  long long m_stride, m_outer, n_stride, n_outer, z_stride;
  int m_div, n_div, m_valid;
  const float* bias_m;  // added per row (may be null)
  const float* bias_n;  // added per column (may be null)
  float alpha, beta;
  int out_bf16;         // `out` points at __nv_bfloat16 (offsets are in elements either way)
  int act;              // 0 none, 1 GELU (tanh form): applied after alpha and the biases, on the
                        // row-major fp32 (staged) and bf16 (vector) store paths only
  void* pre;            // with act: where the value BEFORE the activation goes too (same type
                        // and layout as `out`; what the activation's gradient needs), or null
  float* stats;         // EpiStats matrix [ceil(M / 128) * 4][2 * N] (tc_kernel.cuh) or null:
                        // per-column sums and sums of squares of a row-major fp32 output
};

struct Launch {
  int bn, splits, iters_per_split;
  size_t workspace_bytes;
};

int pick_bn(long long N);
// Whether an M x N contraction runs on CTA pairs (two SMs per 256 x BN tile, each loading half
// of the B tile), and the number of rows a K-major B map must put in one box accordingly.
// Pairs pay off when both operands are K-major single boxes and the K loop is long (the
// backward-filter shapes), and for an MN-major A with a K-major B at 256 columns (the 1x1
// forward layers); tiles with a short K loop lose more to the cross-CTA hand-offs per tile
// than they gain (measured).  Every K-major B map must take its box rows from b_box_rows.
bool gemm_uses_pairs(long long M, long long N, long long k_iters, bool a_mn_major,
                     bool b_mn_major);
int b_box_rows(long long M, long long N, long long k_iters, bool a_mn_major, bool b_mn_major);
// Tile width, split-K factor and scratch size for an M x N output over k_iters stages, Z batches.
Launch plan_launch(long long M, long long N, long long k_iters, long long Z);
// Split-K factor for `tiles` output tiles of k_iters stage iterations each, at least min_ips
// iterations per split, chosen so that tiles * splits fills whole rounds of the persistent grid.
void plan_splits(long long tiles, long long k_iters, long long min_ips, int* splits, int* ips);

// fp32 tensor map; dims[0] is the contiguous dimension, strides_bytes[i] belongs to
// dims[i+1]; box[0] must be 32 elements.  mode: K-major operand tile (128-byte swizzle of
// 16-byte chunks), MN-major operand tile (TF32 operands with a contiguous m / n index need
// the swizzle of 32-byte chunks), or an unswizzled staging tile for TMA stores.
// elem_strides (optional) samples every s-th element of a dimension; the box extent of that
// dimension is then given in source elements (count * s).
enum { kMapKMajor = 0, kMapMnMajor = 1, kMapStaging = 2 };
int make_tensor_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, int mode,
                    const uint32_t* elem_strides = nullptr, bool bf16 = false);

// 3xTF32 ("fp32-grade") mode of the current host thread: set by the C entry points around a
// call (X3Scope), read where kernels are launched.
bool x3_enabled();
struct X3Scope {
  explicit X3Scope(bool on);
  ~X3Scope();
  bool prev;
};

// Address of the device flag that bounded waits raise (per device), and the launch counter.
int* status_ptr();
void count_tc_launch();

// Launches the contraction (and the split-K reduction when the plan splits K).  Without
// enough scratch the contraction runs unsplit.
int run(const CUtensorMap& ma, const CUtensorMap& mb, const OperandPlan& pa, const OperandPlan& pb,
        const EpiloguePlan& ep, long long M, long long N, long long k_iters, long long Z, void* ws,
        size_t ws_bytes, cudaStream_t st, bool bf16 = false);

}  // namespace tc
}  // namespace flb200
