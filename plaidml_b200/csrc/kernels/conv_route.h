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

}  // namespace pmlb
