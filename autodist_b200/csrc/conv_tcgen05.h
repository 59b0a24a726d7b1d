// Host-side interface of the implicit-GEMM convolution on tcgen05 (see conv_tcgen05.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace adb200 {

enum ConvMode { CONV_FPROP = 0, CONV_DGRAD = 1, CONV_WGRAD = 2 };

constexpr int kMaxConvTaps = 49;      // 7 x 7
constexpr int kMaxStatChannels = 2048;

// One filter tap of the contraction: which activation map it reads, the pixel offset of that read relative to the
// tile's own pixel, and which tap of the weight tensor multiplies it.
struct ConvTap {
  short dw, dh;
  short wtap;
  short amap;
};

// Activations are channels-last bf16 [N, H, W, C]; the weight is [Cout, taps, Cin] bf16.
//
// A tile of the "pixel" modes (forward, input gradient) is a patch of tw x th x tn pixels (at most 128) of one pixel
// grid GW x GH x GN; one TMA box (64 channels, tw, th, tn) per tap and 64-channel block fetches the patch shifted by the
// tap's offset, zero-filled outside the tensor, straight into the swizzled K-major layout the MMA reads. Strided
// convolutions read parity sub-grids of the input (one tensor map per parity class, chosen per tap), so no traversal
// stride is needed. The weight-gradient mode contracts over pixels: its K blocks are patches of exactly 64 pixels of
// dY (A operand) and of the shifted input (B operand), both MN-major, split over `ksplit` CTAs per output tile.
struct ConvParams {
  int mode;
  int tw, th, tn;                 // patch extents
  int wsplit;                     // 1: one box per patch column (row-tap view of an input with 8 padded channels)
  int xstep;                      // wsplit: inner-dimension elements between neighbouring output columns
  int tiles_w, tiles_h, tiles_n;  // patches per dimension of the pixel grid
  int GW, GH, GN;                 // pixel grid the patches tile
  int Nc;                         // GEMM N extent: Cout (forward), Cin (input / weight gradient)
  int Kc;                         // channels contracted per tap (forward: Cin, input gradient: Cout)
  int Mc;                         // weight gradient: Cout
  int ntaps;
  int ksplit;                     // weight gradient: CTAs sharing one output tile
  void* out;                      // pixel modes: bf16 [N, OH, OW, ldc]; weight gradient: fp32 [Cout, ldc]
  long long ldc;
  int OH, OW, os, oh0, ow0;       // pixel (i, j) of the grid is written to (i * os + oh0, j * os + ow0)
  int wtap_stride;                // weight gradient: elements between taps inside one output row
  int accumulate;                 // weight gradient: add into `out` (atomics) instead of overwriting it
  const float* bias;              // forward: per output channel, or null
  int relu;                       // forward: clamp at zero after the bias
  float* stats;                   // forward: [2, Nc] fp32, per-channel sum and sum of squares are added here, or null
  const __nv_bfloat16* addend;    // pixel modes: tensor of the output's shape added to the result before it is stored, or null
  int* error_flag;
  long long* trace;               // optional tuning aid: [grid, 8] clock64 marks per CTA (see conv_kernel), or null
  ConvTap taps[kMaxConvTaps];
};

struct ConvMaps {
  CUtensorMap act[4];             // input (forward / weight gradient) or dY (input gradient), per parity class
  CUtensorMap w;                  // weight
  CUtensorMap dy;                 // weight gradient: dY
};

cudaError_t launch_conv(const ConvMaps& maps, const ConvParams& p, int bn, int num_sms, cudaStream_t stream);

}  // namespace adb200
