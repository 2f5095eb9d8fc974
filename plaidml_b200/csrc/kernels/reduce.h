// Launchers of the bandwidth-bound aggregation kernels.
#pragma once

#include <cuda_runtime.h>

#include "pmlb_kernels.h"

namespace pmlb {

struct PoolGeom {
  int agg;
  int n, h, w, c;
  int r, s;
  int p, q;
  int stride_h, stride_w;
  int pad_h, pad_w;
  int average;
  int include_padding;
};

bool reduce_supported(int agg, int dtype, int out_dtype);
// `scale` applies to float sums only: positive = factor, negative = minus the divisor, 1 = none.
cudaError_t launch_reduce(int agg, int dtype, int out_dtype, const void* in, void* out,
                          long long outer, long long red, long long inner, float scale,
                          cudaStream_t stream);

bool pool_supported(int agg, int dtype);
cudaError_t launch_pool(const PoolGeom& g, int dtype, const void* in, void* out,
                        cudaStream_t stream);

}  // namespace pmlb
