// Which kernel route a convolution descriptor takes; shared by the kernel library, which
// plans it, and the program planner, which must know what the library accepts.
#pragma once

#include "pmlb_kernels.h"

namespace pmlb {

// Packed-row route: thin inputs (first layers of image networks: few channels, wide filters).
// A filter row's s taps times the channel count (padded to a multiple of 8) fit one 128-byte
// operand row, so each filter row is one k-block and the filter-column taps cost nothing,
// where the im2col route would spend a whole k-block on every tap.
inline int conv_padded_channels(const pmlb_conv_desc& d) { return (d.c + 7) / 8 * 8; }

inline bool conv_takes_packed_rows(const pmlb_conv_desc& d) {
  const int cp = conv_padded_channels(d);
  return (d.in_dtype == PMLB_BF16 || d.in_dtype == PMLB_F16) && cp <= 32 && d.s > 1 &&
         d.s * cp <= 64 && d.k <= 64 && d.dil_h == 1 && d.dil_w == 1 && d.stride_h <= d.r &&
         d.r <= 7 && !(d.epilogue & PMLB_EPI_ROWMAX);
}

// Width in pixels of the padded activation rows of the packed-row route.
inline int conv_packed_row_width(const pmlb_conv_desc& d) {
  int wp = d.pad_w + d.w;
  const int reach = (d.q - 1) * d.stride_w + d.s;
  if (reach > wp) wp = reach;
  const int unit = d.stride_w * 2;   // keeps every row pitch a multiple of the window stride
  return (wp + unit - 1) / unit * unit;
}

// Halo route: stride-1, undilated convolutions on whole 64-channel blocks into exactly 64 output
// channels whose weights fit beside the pixel ring (the 3x3 convolutions of a network's first
// stage): every tap is a row-shifted window of one fetched pixel buffer, so the activation
// crosses from L2 to shared memory about 1.3 times instead of r * s times.
// Shared memory the halo route has for weights plus pixel buffers (the kernel instance's operand
// ring and its unused output staging area).
constexpr int kHaloSmemBytes = 212992;

inline bool conv_takes_halo(const pmlb_conv_desc& d) {
  if (!(d.in_dtype == PMLB_BF16 || d.in_dtype == PMLB_F16)) return false;
  if (d.stride_h != 1 || d.stride_w != 1 || d.dil_h != 1 || d.dil_w != 1) return false;
  if (d.k != 64 || d.c % 64 != 0 || d.r * d.s < 2) return false;
  const int wp = d.w + 2 * d.pad_w;
  if (wp > 128 || d.q != wp - d.s + 1 || d.p != d.h + 2 * d.pad_h - d.r + 1) return false;
  const int th = 128 / wp < d.p ? 128 / wp : d.p;
  if (th < 1) return false;
  // at least 3/4 of the 128 accumulator rows must be real outputs
  if (th * d.q * 4 < 128 * 3) return false;
  const int wts = d.r * d.s * (d.c / 64) * 64 * 128;
  const int stage = (wp * (th + d.r - 1) * 128 + 1023) / 1024 * 1024;
  return wts + 2 * stage + 8192 <= kHaloSmemBytes && (d.epilogue & PMLB_EPI_ROWMAX) == 0;
}

// Space-to-depth route: stride-2 convolutions of thin inputs (at most 4 channels: the first layer
// of an image network) into at most 64 channels.  The 2 x 2 pixel phases become channels, which
// turns the r x s / 2 convolution into a stride-1 one with ceil(r / 2) x ceil(s / 2) taps over
// 16-channel (32-byte) pixels; the kernel then works as the halo route does, with the 32-byte
// k-steps of its 128-byte operand rows being four neighbouring pixels.
struct S2dShape {
  int pe_h, pe_w;   // padding before the first row / column, rounded up to even
  int dh, dw;       // pe - pad: filter tap fr sits at row fr + dh of the 2 x 2 phase grid
  int r2, s2;       // taps of the stride-1 convolution
  int h2, wp;       // rows and (padded to a multiple of 32) pixels per row of the packed activation
  int stage_px;     // pixels a 512-position tile reads (a multiple of 32)
};

inline S2dShape conv_s2d_shape(const pmlb_conv_desc& d) {
  S2dShape g;
  g.pe_h = (d.pad_h + 1) & ~1;
  g.pe_w = (d.pad_w + 1) & ~1;
  g.dh = g.pe_h - d.pad_h;
  g.dw = g.pe_w - d.pad_w;
  g.r2 = (d.r + g.dh + 1) / 2;
  g.s2 = (d.s + g.dw + 1) / 2;
  g.h2 = d.p + g.r2 - 1;
  g.wp = (d.q + g.s2 - 1 + 31) / 32 * 32;
  g.stage_px = (512 + (g.r2 - 1) * g.wp + g.s2 - 1 + 31) / 32 * 32;
  return g;
}

// Shared memory the route has for weights plus pixel buffers (the operand ring of the 64-wide
// instance with two epilogue groups).
constexpr int kS2dSmemBytes = 147456;

// packed weights: one 64-row block of 128-byte rows per tap row and four tap columns
inline int conv_s2d_weight_bytes(const S2dShape& g) { return g.r2 * ((g.s2 + 3) / 4) * 8192; }

inline int conv_s2d_stage_bytes(const S2dShape& g) { return g.stage_px * 32; }

inline bool conv_takes_s2d(const pmlb_conv_desc& d) {
  if (!(d.in_dtype == PMLB_BF16 || d.in_dtype == PMLB_F16)) return false;
  if (d.stride_h != 2 || d.stride_w != 2 || d.dil_h != 1 || d.dil_w != 1) return false;
  // (the output map addresses columns as (column % 4, column / 4): whole groups of four only)
  if (d.c > 4 || d.k > 64 || d.k % 8 != 0 || d.q % 4 != 0 || d.r * d.s < 2) return false;
  if (d.epilogue & (PMLB_EPI_ROWMAX | PMLB_EPI_RESIDUAL)) return false;
  const S2dShape g = conv_s2d_shape(d);
  return conv_s2d_weight_bytes(g) + 2 * conv_s2d_stage_bytes(g) <= kS2dSmemBytes;
}

// The space-to-depth route fused with the 3 x 3 / 2 max pool (one pixel of padding) that follows the layer:
// a 7-wide filter (four tap columns in the stride-1 form) on rows of exactly 128 packed positions, 64
// output channels, a 16-bit output, whole tiles of four output rows.  The output tensor is then
// [n][p / 2][q / 2][64].
inline bool conv_takes_s2d_pool(const pmlb_conv_desc& d) {
  if (!conv_takes_s2d(d)) return false;
  if (d.k != 64 || d.p % 4 != 0 || !(d.out_dtype == PMLB_BF16 || d.out_dtype == PMLB_F16)) return false;
  if (d.epilogue & ~(PMLB_EPI_BIAS | PMLB_EPI_RELU)) return false;
  const S2dShape g = conv_s2d_shape(d);
  return g.s2 == 4 && g.r2 <= 4 && g.wp == 128;
}

}  // namespace pmlb
