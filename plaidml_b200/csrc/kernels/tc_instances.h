// The instantiations of the tensor-core contraction kernel, as X-macro lists shared by the
// files that compile them and the dispatcher that selects one.
// X(element bytes, tile N, operand split, A mode (0 tiled, 1 im2col, 2 packed rows), B stored [k][n],
//   output bytes, epilogue groups)
// A modes: 0 tiled, 1 im2col, 2 packed rows, 3 halo rows
#pragma once

#define PMLB_TC_LIST_H16(X, G)      \
  X(2, 64, 1, false, false, 4, G)   \
  X(2, 64, 1, false, false, 2, G)   \
  X(2, 128, 1, false, false, 4, G)  \
  X(2, 128, 1, false, false, 2, G)  \
  X(2, 256, 1, false, false, 4, G)  \
  X(2, 256, 1, false, false, 2, G)  \
  X(2, 64, 1, false, true, 4, G)    \
  X(2, 64, 1, false, true, 2, G)    \
  X(2, 128, 1, false, true, 4, G)   \
  X(2, 128, 1, false, true, 2, G)   \
  X(2, 256, 1, false, true, 4, G)   \
  X(2, 256, 1, false, true, 2, G)   \
  X(2, 64, 1, true, false, 4, G)    \
  X(2, 64, 1, true, false, 2, G)    \
  X(2, 128, 1, true, false, 4, G)   \
  X(2, 128, 1, true, false, 2, G)   \
  X(2, 256, 1, true, false, 4, G)   \
  X(2, 256, 1, true, false, 2, G)

#define PMLB_TC_LIST_MISC(X)        \
  X(2, 64, 1, 3, false, 2, 2)       \
  X(2, 64, 1, 3, false, 4, 2)       \
  X(2, 64, 1, 4, false, 2, 2)       \
  X(2, 64, 1, 4, false, 4, 2)       \
  X(2, 64, 1, 2, false, 2, 1)       \
  X(2, 64, 1, 2, false, 4, 1)       \
  X(1, 64, 1, false, false, 4, 1)   \
  X(1, 128, 1, false, false, 4, 1)  \
  X(1, 256, 1, false, false, 4, 1)  \
  X(1, 128, 1, false, true, 4, 1)   \
  X(1, 256, 1, false, true, 4, 1)   \
  X(1, 64, 1, false, false, 4, 2)   \
  X(1, 128, 1, false, false, 4, 2)  \
  X(1, 128, 1, false, true, 4, 2)   \
  X(4, 64, 2, false, false, 4, 1)   \
  X(4, 128, 2, false, false, 4, 1)  \
  X(4, 64, 2, false, false, 4, 2)   \
  X(4, 64, 2, 1, false, 4, 1)       \
  X(4, 128, 2, 1, false, 4, 1)      \
  X(4, 64, 2, 1, false, 4, 2)

// CTA-pair instances (two CTAs per 256 x 256 tile, cta_group::2 MMAs): plain GEMMs with long
// main loops; same columns, always one epilogue group per CTA.
#define PMLB_TC_LIST_PAIR(X)        \
  X(2, 256, 1, 0, false, 4, 1)      \
  X(2, 256, 1, 0, false, 2, 1)      \
  X(2, 256, 1, 0, true, 4, 1)       \
  X(2, 256, 1, 0, true, 2, 1)       \
  X(1, 256, 1, 0, false, 4, 1)      \
  X(1, 256, 1, 0, true, 4, 1)       \
  X(2, 256, 1, 1, false, 4, 1)      \
  X(2, 256, 1, 1, false, 2, 1)      \
  X(2, 128, 1, 1, false, 4, 1)      \
  X(2, 128, 1, 1, false, 2, 1)
