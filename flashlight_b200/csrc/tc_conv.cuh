// Convolution geometry shared by the fp32 and the tensor-core paths, and the
// interface of the tcgen05 implicit-GEMM convolution used by TF32 mode.
#pragma once
#include "common.cuh"

namespace flb200 {

struct ConvGeo {
  int W, H, C, N;
  int kW, kH, Cout;
  int sx, sy, px, py, dx, dy, groups;
  int Wo, Ho, Cg, Coutg;
  int HW, HoWo, RS;
  // Memory layout of the activations: x / grad_x and y / grad_y are [N][C][H][W] (fl's own
  // order) or channels-last [N][H][W][C].  Element (img, c, pixel) of x sits at
  // img * C * HW + c * x_cs + pixel * x_ps; likewise y with Cout, HoWo, y_cs, y_ps.
  int x_cl, y_cl;
  int x_cs, x_ps, y_cs, y_ps;
};

int make_conv_geo(const char* name, const flb200_conv2d_desc* d, ConvGeo* g);

// which: 0 forward, 1 backward-data, 2 backward-filter.
bool tc_conv_supported(const ConvGeo& g, int which, size_t workspace_bytes);
size_t tc_conv_workspace_bytes(const ConvGeo& g, int which);
// Size of the channels-last copy of x (which 0) or grad_y (which 1) that can be kept between
// the calls of one convolution; 0 for routes that make no such copy.
size_t tc_conv_cache_bytes(const ConvGeo& g, int which);
// Per-channel statistics of the output, taken in the forward pass's epilogue (EpiStats,
// tc_kernel.cuh): `matrix` receives tc_conv_stats_groups(g) rows of 2 * Cout floats whose column
// sums are, per output channel, the sum and the sum of squares of y.
struct ConvStats {
  float* matrix;
};
// Number of rows the forward pass of this geometry writes, 0 where it cannot (output not stored
// channels-last, Cout not a multiple of 32, or a route without the staged epilogue).
long long tc_conv_stats_groups(const ConvGeo& g);
int tc_conv_forward(const ConvGeo& g, const float* x, const float* w, const float* bias, float* y,
                    void* ws, size_t ws_bytes, cudaStream_t st,
                    flb200_conv2d_cache* cache = nullptr, const ConvStats* stats = nullptr);
int tc_conv_backward_data(const ConvGeo& g, const float* gy, const float* w, float* gx, void* ws,
                          size_t ws_bytes, cudaStream_t st,
    flb200_conv2d_cache* cache = nullptr);
int tc_conv_backward_filter(const ConvGeo& g, const float* gy, const float* x, float* gw, void* ws,
                            size_t ws_bytes, cudaStream_t st,
    flb200_conv2d_cache* cache = nullptr);

// Channels-last implicit-GEMM route (tc_conv_patch.cu): no im2col matrix, one NHWC copy of the
// activation operand per pass.
bool patch_conv_supported(const ConvGeo& g);
size_t patch_conv_workspace_bytes(const ConvGeo& g, int which);
size_t patch_conv_cache_bytes(const ConvGeo& g, int which);
long long patch_conv_stats_groups(const ConvGeo& g);
int patch_conv_forward(const ConvGeo& g, const float* x, const float* w, const float* bias,
                       float* y, void* ws, size_t ws_bytes, cudaStream_t st,
                       flb200_conv2d_cache* cache = nullptr, const ConvStats* stats = nullptr);
int patch_conv_backward_data(const ConvGeo& g, const float* gy, const float* w, float* gx,
                             void* ws, size_t ws_bytes, cudaStream_t st,
    flb200_conv2d_cache* cache = nullptr);
int patch_conv_backward_filter(const ConvGeo& g, const float* gy, const float* x, float* gw,
                               void* ws, size_t ws_bytes, cudaStream_t st,
    flb200_conv2d_cache* cache = nullptr);

// Few-channel "row window" route (<= 4 input channels, e.g. the ResNet stem): forward and
// backward-filter only; returns a non-zero status without launching anything if the driver
// refuses the overlapping tensor map, so that the caller can take another route.
bool window_conv_supported(const ConvGeo& g);
size_t window_conv_workspace_bytes(const ConvGeo& g, int which);
size_t window_conv_cache_bytes(const ConvGeo& g, int which);
int window_conv_forward(const ConvGeo& g, const float* x, const float* w, const float* bias,
                        float* y, void* ws, size_t ws_bytes, cudaStream_t st,
                        flb200_conv2d_cache* cache = nullptr, const ConvStats* stats = nullptr);
int window_conv_backward_filter(const ConvGeo& g, const float* gy, const float* x, float* gw,
                                void* ws, size_t ws_bytes, cudaStream_t st,
    flb200_conv2d_cache* cache = nullptr);

}  // namespace flb200
