// Host-side entry and launch parameters of the fused first-layer kernel (s2d_pool_kernel.cuh): a 7-wide
// stride-2 convolution on at most 4 channels into 64, bias, ReLU and the 3 x 3 / 2 max pool behind it.
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

namespace pmlb {

struct S2dPoolParams {
  const void* px;        // packed activation [n][h2][128][16], pre-swizzled (s2d_pack_kernel)
  const void* wts;       // weights [4 tap columns, descending][64][tap row][16], pre-swizzled: 32 KB
  const float* bias;     // 64 values, or null
  void* out;             // pooled output [n][pool_p][pool_q][64], 16-bit
  int* status;
  int total_tiles;       // n * tiles_per_img
  int tiles_per_img;     // conv_p / 4
  int img_px;            // pixels per packed image = h2 * 128
  int stage_load;        // bytes copied per tile
  int stage_bytes;       // the same rounded up to 1024
  int stages;            // pixel buffers (2 .. 6)
  int r2;                // tap rows of the stride-1 form (<= 4)
  int conv_q;            // columns of the convolution's output (a multiple of 4, <= 124)
  int pool_p, pool_q;    // rows and columns of the pooled output = half of the convolution's
  int relu;
  int wait_limit_us;
  uint32_t idesc[4];     // instruction descriptors of 128 x N x 16 MMAs, N = 64, 128, 192, 256
};

// Pixel buffers of `stage_bytes` that fit (at most 6; fewer than 2 = the kernel cannot run).
int s2d_pool_stages(int stage_bytes);

// (fills idesc itself; in_f16: operands are f16, else bf16; out_bf16: the output is bf16, else f16)
cudaError_t launch_s2d_pool(const S2dPoolParams& p, int grid, bool in_f16, bool out_bf16, cudaStream_t stream);

}  // namespace pmlb
