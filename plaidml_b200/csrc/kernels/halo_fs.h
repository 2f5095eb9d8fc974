// Host-side entry of the filter-column-merged halo convolution (halo_fs_kernel.cuh).
#pragma once

#include <cuda_runtime.h>

#include "tc_gemm.cuh"

namespace pmlb {

// Pixel buffers that fit beside `weight_bytes` of resident weights (at most 8).
int halo_fs_stages(int weight_bytes, int stage_bytes);
// Bytes of shared memory behind the last pixel buffer (what a tap window may read past its buffer).
int halo_fs_tail_bytes();
// p: the halo fields of TcParams filled as for the general kernel, halo_stages from halo_fs_stages,
// idesc for a 128 x 128 MMA, idesc_half for a 128 x 64 one (pair: 256 rows high both).
// pair: clusters of two CTAs on two neighbouring tiles (grid even; maps.b1 = the weights with a 32-row box, and
// halo_fs_stages was asked with half the weight bytes).
// dependent_launch: the kernel's set-up may overlap the tail of the kernel before it in the stream.
cudaError_t launch_halo_fs(const TcMaps& maps, const TcParams& p, int grid, int out_bytes, bool pair, bool dependent_launch,
                           cudaStream_t stream);

}  // namespace pmlb
