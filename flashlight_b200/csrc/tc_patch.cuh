// Problem policies that turn the persistent tcgen05 kernel (tc_kernel.cuh) into implicit-GEMM
// convolutions over a channels-last (NHWC) copy of the activations.
//
// Why channels-last: a filter tap shifts the window by whole pixels.  In NCHW the shifted
// pixel is the contiguous index, which breaks TMA's 16-byte start rule; in NHWC the shift
// lands on the w / h coordinates of the tensor map (any value, negative = zero padding for
// free) and the contiguous coordinate is the channel, always a multiple of 32 here.
//
//  PatchConvProblem  (forward, and backward-data with transposed taps)
//     rows  m = output pixels of a rectangular patch  NB images x PH rows x QW columns = 128
//     cols  n = output channels
//     k     = taps x 32-channel chunks:  A = one TMA box [32 c][QW][PH][NB] of the source at
//             the tap's offset (element strides implement the convolution stride),
//             B = packed filter [tap][n][c] (K-major)
//     out   = NCHW, optionally strided (the parity classes of a strided backward-data);
//             lanes of a warp hold consecutive pixels of a row, so each column is stored
//             as one coalesced run per patch row
//
//  PatchWgradProblem (backward-filter), one GEMM per group of taps:
//     rows  m = output channels (A = dy in NHWC, MN-major boxes [32 co][32 pixels])
//     cols  n = (tap of the group, input channel)  (B = x in NHWC at each tap's offset,
//             MN-major); layers with few input channels put several taps side by side so
//             that the dy tile is loaded once for all of them
//     k     = 32-pixel patches (QW x PH) of every image; split over CTAs, partial sums are
//             reduced in a fixed order by a second kernel.
#pragma once
#include "tc_pair.cuh"

namespace flb200 {
namespace tc {

// The taps a launch walks form a grid: tap (i, j) reads the source at offset
// (dh0 + i*dh_step, dw0 + j*dw_step) and uses filter element (r0 + i*r_step, s0 + j*s_step).
// Forward: every (r, s).  A parity class of a strided backward-data: the arithmetic
// progressions of r and s whose offsets divide by the stride.
struct TapGrid {
  int ni, nj;
  int dh0, dh_step, dw0, dw_step;
  int r0, r_step, s0, s_step, kW;
};

// One parity class of a launch (a forward pass has a single class): its taps and where its
// pixels land in the output.
struct PatchClass {
  TapGrid taps;
  int ntaps, oh_add, ow_add;
};
constexpr int kMaxPatchClasses = 4;

template <int BN>
struct PatchConvProblem {
  static constexpr bool kWarpProducer = false;
  static constexpr int kMinBlocks = 1;
  static constexpr bool kBf16Capable = false;
  int a_mn_major, b_mn_major;  // 0, 0
  // patch geometry (all powers of two, NB * PH * QW == 128)
  int QW, PH, NB, qw_shift, ph_shift;
  int tiles_q, tiles_p, tiles_b, tiles_n;
  int pix_w, pix_h, images;  // extent of the pixel grid the rows walk over
  int n_out;                 // number of output channels (columns)
  // K loop
  int cchunks;
  int a_w_mul, a_h_mul;      // A box origin = (q0 * a_w_mul + dw, p0 * a_h_mul + dh)
  // Parity classes served by this launch (strided backward-data with equal class extents: the
  // classes of one pixel patch are consecutive tiles, so that the interleaved stores of the
  // classes meet in L2 instead of reaching DRAM as half-written sectors of separate launches).
  int ncls;
  PatchClass cls[kMaxPatchClasses];
  // output: out[img][co][oh][ow], oh = p * oh_mul + oh_add, ow = q * ow_mul + ow_add
  float* out;
  const float* bias;
  int out_H, out_W, out_C;
  int oh_mul, ow_mul;
  int fill_cell;  // see store()
  int out_cl;     // output stored channels-last: out[img][oh][ow][co]
  float* stats;   // EpiStats matrix [pixel tiles * 4][2 * n_out] (tc_kernel.cuh), or null

  struct Tile { int q0, p0, b0, n0, c; };
  struct LoadState { int i, j, cc, aw, ah, wtap, c; };

  __device__ __forceinline__ int num_tiles() const {
    return tiles_q * tiles_p * tiles_b * tiles_n * ncls;
  }
  __device__ __forceinline__ void decode(int tile, Tile& t) const {
    int r = tile;
    t.c = r % ncls; r /= ncls;
    t.n0 = (r % tiles_n) * BN; r /= tiles_n;
    t.q0 = (r % tiles_q) * QW; r /= tiles_q;
    t.p0 = (r % tiles_p) * PH; r /= tiles_p;
    t.b0 = r * NB;
  }
  // CTA pairs: the two halves of a pair tile are consecutive pixel patches that share the
  // column block n0 (hence the whole B tile and the K loop).  Patches are enumerated fastest,
  // column blocks slowest; an odd patch count leaves the last pair a phantom half whose image
  // index is out of range (its loads are zero-filled, its stores masked).
  __device__ __forceinline__ int num_pair_tiles() const {
    return ((tiles_q * tiles_p * tiles_b + 1) >> 1) * tiles_n * ncls;
  }
  __device__ __forceinline__ void decode_pair(int tile, int rank, Tile& t) const {
    const int pairs_m = (tiles_q * tiles_p * tiles_b + 1) >> 1;
    t.c = tile % ncls;
    tile /= ncls;
    const int nt = tile / pairs_m;
    int r = 2 * (tile - nt * pairs_m) + rank;
    t.n0 = nt * BN;
    t.q0 = (r % tiles_q) * QW; r /= tiles_q;
    t.p0 = (r % tiles_p) * PH; r /= tiles_p;
    t.b0 = r * NB;
  }
  __device__ __forceinline__ void load_pair(const CUtensorMap* ma, const CUtensorMap* mb,
                                            const Tile& t, LoadState& ls, uint32_t full_bar,
                                            char* a_dst, char* b_dst, int rank, int lane) const {
    if (lane == 0) {
      int ca[4] = {ls.cc * kBK, ls.aw, ls.ah, t.b0};
      tma_load_pair(ma, full_bar, a_dst, 4, ca);
    } else if (lane == 1) {
      int cb[4] = {ls.cc * kBK, t.n0 + rank * (BN / 2), ls.wtap, 0};  // this CTA's half of B
      tma_load_pair(mb, full_bar, b_dst, 3, cb);
    }
    advance(ls);
  }
  __device__ __forceinline__ void advance(LoadState& ls) const {
    if (++ls.cc == cchunks) {  // next tap: j fastest
      const TapGrid& taps = cls[ls.c].taps;
      ls.cc = 0;
      ls.aw += taps.dw_step;
      ls.wtap += taps.s_step;
      if (++ls.j == taps.nj) {
        ls.j = 0;
        ++ls.i;
        ls.aw -= taps.nj * taps.dw_step;
        ls.ah += taps.dh_step;
        ls.wtap += taps.r_step * taps.kW - taps.nj * taps.s_step;
      }
    }
  }
  __device__ __forceinline__ int k_begin(const Tile&) const { return 0; }
  __device__ __forceinline__ int k_end(const Tile& t) const { return cls[t.c].ntaps * cchunks; }
  __device__ __forceinline__ void load_begin(const Tile& t, LoadState& ls, int) const {
    ls.i = 0;
    ls.j = 0;
    ls.cc = 0;
    const TapGrid& taps = cls[t.c].taps;
    ls.c = t.c;
    ls.aw = t.q0 * a_w_mul + taps.dw0;
    ls.ah = t.p0 * a_h_mul + taps.dh0;
    ls.wtap = taps.r0 * taps.kW + taps.s0;
  }
  __device__ __forceinline__ void load(const CUtensorMap* ma, const CUtensorMap* mb,
                                       const Tile& t, LoadState& ls, uint64_t* bar, char* a_dst,
                                       char* b_dst, int, bool last, int, int) const {
    mbar_post_tx(bar, (kBM + BN) * kBK * 4, last);  // NB*PH*QW == 128 rows of 128 bytes + B tile
    int ca[4] = {ls.cc * kBK, ls.aw, ls.ah, t.b0};
    tma_load(ma, bar, a_dst, 4, ca);
    int cb[4] = {ls.cc * kBK, t.n0, ls.wtap, 0};
    tma_load(mb, bar, b_dst, 3, cb);
    advance(ls);
  }
  __device__ __forceinline__ bool chunk_live(const Tile& t, int c0) const {
    return t.n0 + c0 < n_out;
  }
  // output address of row `r` of the tile (channels-last output, class offsets applied), or
  // null for a row outside the image
  __device__ __forceinline__ float* cl_row(const Tile& t, int r) const {
    const int q = t.q0 + (r & (QW - 1));
    const int p = t.p0 + ((r >> qw_shift) & (PH - 1));
    const int img = t.b0 + (r >> (qw_shift + ph_shift));
    if (q >= pix_w || p >= pix_h || img >= images) return nullptr;
    const int oh_add = fill_cell ? 0 : cls[t.c].oh_add, ow_add = fill_cell ? 0 : cls[t.c].ow_add;
    return out + (((long long)img * out_H + p * oh_mul + oh_add) * out_W + q * ow_mul + ow_add) *
                     out_C;
  }
  // Pixel rows 4k + lane / 8 (k = 0..7) of the warp's staged chunk, 16 bytes per lane, bias
  // added; STATS (uniform across the grid, so a copy of the loop each): per-channel sums of
  // the stored values into the statistics matrix.  FILL: the strided backward-data whose only
  // class with taps is (0, 0) — every pixel also writes the zeros of its cell, whole 128-byte
  // rows like its own values, so the tensor needs no clearing pass.
  template <bool STATS, bool FILL>
  __device__ __forceinline__ void staged_pixels(const Tile& t, int row, int nb, float* stage,
                                                int lane) const {
    float4 bq = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias) bq = *reinterpret_cast<const float4*>(bias + nb + 4 * (lane & 7));
    const int r_first = row - lane;
    EpiStats acc;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float* dst = cl_row(t, r_first + 4 * k + (lane >> 3));
      float4 val = epi_stage_read(stage, lane, k);
      val.x += bq.x; val.y += bq.y; val.z += bq.z; val.w += bq.w;
      if (dst) {
        *reinterpret_cast<float4*>(dst + nb + 4 * (lane & 7)) = val;
        if (STATS) acc.add(val);
        if (FILL) {
          // this pixel owns its whole oh_mul x ow_mul cell: the other pixels receive zeros
          const int r = r_first + 4 * k + (lane >> 3);
          const int ow0 = (t.q0 + (r & (QW - 1))) * ow_mul;
          const int oh0 = (t.p0 + ((r >> qw_shift) & (PH - 1))) * oh_mul;
          for (int a = 0; a < oh_mul && oh0 + a < out_H; ++a)
            for (int b = a == 0 ? 1 : 0; b < ow_mul && ow0 + b < out_W; ++b)
              *reinterpret_cast<float4*>(dst + ((long long)a * out_W + b) * out_C + nb +
                                         4 * (lane & 7)) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    }
    if (STATS) {
      const long long tile_m = ((long long)(t.b0 >> (7 - qw_shift - ph_shift)) * tiles_p +
                                (t.p0 >> ph_shift)) * tiles_q + (t.q0 >> qw_shift);
      acc.flush(stats, tile_m * 4 + (row >> 5), n_out, nb, lane, stage);
    }
  }
  __device__ __forceinline__ void store(const Tile& t, int row, int c0, const float* v,
                                        float* stage, int lane) const {
    const int nb = t.n0 + c0;
    if (out_cl && nb + 32 <= n_out && (out_C & 3) == 0) {
      // channels-last output: through the warp's staging tile, 4 whole 128-byte pixel rows per
      // store instruction (see tc_kernel.cuh)
      epi_stage_write(stage, lane, v);
      if (fill_cell) staged_pixels<false, true>(t, row, nb, stage, lane);
      else if (stats) staged_pixels<true, false>(t, row, nb, stage, lane);
      else staged_pixels<false, false>(t, row, nb, stage, lane);
      __syncwarp();
      return;
    }
    // row -> (image, p, q) inside the patch
    const int q = t.q0 + (row & (QW - 1));
    const int p = t.p0 + ((row >> qw_shift) & (PH - 1));
    const int img = t.b0 + (row >> (qw_shift + ph_shift));
    if (q >= pix_w || p >= pix_h || img >= images) return;
    if (out_cl) {
      // channels-last: the 32 columns of this chunk are 128 contiguous bytes of one pixel
      const int oh0 = p * oh_mul + (fill_cell ? 0 : cls[t.c].oh_add);
      const int ow0 = q * ow_mul + (fill_cell ? 0 : cls[t.c].ow_add);
      const int cell_h = fill_cell ? oh_mul : 1, cell_w = fill_cell ? ow_mul : 1;
      for (int a = 0; a < cell_h; ++a) {
        if (oh0 + a >= out_H) break;
        for (int b = 0; b < cell_w; ++b) {
          if (ow0 + b >= out_W) break;
          float* dst = out + (((long long)img * out_H + oh0 + a) * out_W + ow0 + b) * out_C + nb;
          const bool mine = a == 0 && b == 0;  // the other pixels of a cell receive zeros
          if (nb + 32 <= n_out && (out_C & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
              if (mine) {
                val = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (bias) {
                  val.x += bias[nb + j]; val.y += bias[nb + j + 1];
                  val.z += bias[nb + j + 2]; val.w += bias[nb + j + 3];
                }
              }
              *reinterpret_cast<float4*>(dst + j) = val;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nb + j < n_out) dst[j] = mine ? v[j] + (bias ? bias[nb + j] : 0.f) : 0.f;
          }
        }
      }
      return;
    }
    const long long plane = (long long)out_H * out_W;
    if (fill_cell) {
      // Strided backward-data whose only class with taps is (0, 0): this pixel owns the whole
      // oh_mul x ow_mul cell and writes its zeros too, so the tensor needs no separate
      // clearing pass and every 32-byte sector is written whole.
      float* cell = out + ((long long)img * out_C + nb) * plane +
                    (long long)(p * oh_mul) * out_W + q * ow_mul;
      const bool pair = ow_mul == 2 && (out_W & 1) == 0;
      for (int a = 0; a < oh_mul; ++a) {
        if (p * oh_mul + a >= out_H) break;
        float* rowp = cell + (long long)a * out_W;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (nb + j >= n_out) break;
          const float val = a == 0 ? v[j] : 0.f;
          if (pair) {
            *reinterpret_cast<float2*>(rowp + j * plane) = make_float2(val, 0.f);
          } else {
            for (int b = 0; b < ow_mul; ++b)
              if (q * ow_mul + b < out_W) rowp[j * plane + b] = b == 0 ? val : 0.f;
          }
        }
      }
      return;
    }
    float* dst = out + ((long long)img * out_C + nb) * plane +
                 (long long)(p * oh_mul + cls[t.c].oh_add) * out_W + (q * ow_mul + cls[t.c].ow_add);
    if (nb + 32 <= n_out) {
      if (bias) {
        const float* bn = bias + nb;
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[j * plane] = v[j] + bn[j];
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[j * plane] = v[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (nb + j < n_out) dst[j * plane] = v[j] + (bias ? bias[nb + j] : 0.f);
    }
  }
};

template <int BN>
struct PatchWgradProblem {
  static constexpr bool kWarpProducer = true;
  static constexpr int kMinBlocks = 1;
  static constexpr bool kBf16Capable = false;
  int a_mn_major, b_mn_major;  // 1, 1
  int QW, PH;                  // 32-pixel patch: QW * PH == 32
  int tiles_q, tiles_p, images;
  int tiles_m, tiles_n, M, N;  // M = output channels, N = input channels
  // The BN columns of a tile are tg taps x (1 << cn_shift) boxes of 32 input channels, so a
  // narrow layer shares one load of dy between several taps.
  int ntaps, tap_groups, tg, cn_shift;
  int a_nbox;                  // 32-channel boxes of dy per copy: min(4, ceil(M / 32))
  int splits, iters_per_split, k_iters;  // k_iters = images * tiles_p * tiles_q
  int b_w_mul, b_h_mul;        // B box origin = (q0 * b_w_mul + dw, p0 * b_h_mul + dh)
  int kW, dil_x, dil_y, pad_x, pad_y;  // tap t = (r, s) = (t / kW, t % kW): dw = s*dil_x - pad_x
  float* partial;              // [split][tap][M][N]

  struct Tile { int m0, n0, tap0, ntap, cn_live, split, k0, k1; };
  struct LoadState { int qi, pi, img, dw, dh; };

  __device__ __forceinline__ int num_tiles() const {
    return tiles_m * tiles_n * tap_groups * splits;
  }
  __device__ __forceinline__ void decode(int tile, Tile& t) const {
    int r = tile;
    t.split = r % splits; r /= splits;
    t.n0 = (r % tiles_n) * BN; r /= tiles_n;
    t.m0 = (r % tiles_m) * kBM; r /= tiles_m;
    t.tap0 = r * tg;
    t.ntap = min(tg, ntaps - t.tap0);
    t.cn_live = min(1 << cn_shift, (N - t.n0 + 31) >> 5);
    t.k0 = t.split * iters_per_split;
    t.k1 = min(t.k0 + iters_per_split, k_iters);
  }
  __device__ __forceinline__ int k_begin(const Tile& t) const { return t.k0; }
  __device__ __forceinline__ int k_end(const Tile& t) const { return t.k1; }
  __device__ __forceinline__ void load_begin(const Tile& t, LoadState& ls, int copy) const {
    int r = t.k0;
    ls.qi = r % tiles_q; r /= tiles_q;
    ls.pi = r % tiles_p; r /= tiles_p;
    ls.img = r;
    // copy 0 is dy, copy j >= 1 the x box of tap tap0 + j - 1
    const int tap = t.tap0 + max(copy - 1, 0);
    const int tr = tap / kW, ts = tap - tr * kW;
    ls.dw = ts * dil_x - pad_x;
    ls.dh = tr * dil_y - pad_y;
  }
  __device__ __forceinline__ void load(const CUtensorMap* ma, const CUtensorMap* mb,
                                       const Tile& t, LoadState& ls, uint64_t* bar, char* a_dst,
                                       char* b_dst, int lane, bool last, int part,
                                       int parts) const {
    const int q0 = ls.qi * QW, p0 = ls.pi * PH;
    const int copy = lane * parts + part;
    // The channel index is split into (32 contiguous channels, group of 32) in both maps, so
    // one copy brings every 32 x 32 box of an operand: a_nbox boxes of dy, and per tap
    // 1 << cn_shift boxes of x.  Boxes past the last channel are zero-filled or hold a
    // neighbouring pixel's channels; they only reach accumulator rows / columns that the
    // epilogue never stores.
    if (lane == 0 && part == 0)
      mbar_post_tx(bar, (a_nbox + (t.ntap << cn_shift)) * (kBK * 128), last);
    __syncwarp();
    if (copy == 0) {
      int ca[5] = {0, q0, p0, ls.img, t.m0 >> 5};
      tma_load(ma, bar, a_dst, 5, ca);
    } else if (copy <= t.ntap) {
      int cb[5] = {0, q0 * b_w_mul + ls.dw, p0 * b_h_mul + ls.dh, ls.img, t.n0 >> 5};
      tma_load(mb, bar, b_dst + ((copy - 1) << cn_shift) * (kBK * 128), 5, cb);
    }
    if (++ls.qi == tiles_q) {
      ls.qi = 0;
      if (++ls.pi == tiles_p) { ls.pi = 0; ++ls.img; }
    }
  }
  __device__ __forceinline__ bool chunk_live(const Tile& t, int c0) const {
    const int j = c0 >> 5;
    return (j >> cn_shift) < t.ntap && (j & ((1 << cn_shift) - 1)) < t.cn_live;
  }
  __device__ __forceinline__ void store(const Tile& t, int row, int c0, const float* v, float*,
                                        int) const {
    const int m = t.m0 + row;
    if (m >= M) return;
    const int j = c0 >> 5;
    const int tap = t.tap0 + (j >> cn_shift);
    const int nb = t.n0 + ((j & ((1 << cn_shift) - 1)) << 5);
    float* dst = partial + (((long long)t.split * ntaps + tap) * M + m) * N + nb;
    if (nb + 32 <= N && (N & 3) == 0) {
#pragma unroll
      for (int jj = 0; jj < 32; jj += 4)
        *reinterpret_cast<float4*>(dst + jj) =
            make_float4(v[jj], v[jj + 1], v[jj + 2], v[jj + 3]);
    } else {
#pragma unroll
      for (int jj = 0; jj < 32; ++jj)
        if (nb + jj < N) dst[jj] = v[jj];
    }
  }
};

}  // namespace tc
}  // namespace flb200
