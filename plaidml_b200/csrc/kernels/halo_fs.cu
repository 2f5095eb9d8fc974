// Compiles and launches the filter-column-merged halo convolution kernel.
#include "halo_fs_kernel.cuh"

#include "halo_fs.h"

namespace pmlb {

int halo_fs_stages(int weight_bytes, int stage_bytes) {
  if (stage_bytes <= 0) return 0;
  const int room = kFsSmemLimit - 1024 - weight_bytes - kFsTailBytes;
  const int n = room / stage_bytes;
  return n > kFsMaxStages ? kFsMaxStages : n;
}

int halo_fs_tail_bytes() { return kFsTailBytes; }

cudaError_t launch_halo_fs(const TcMaps& maps, const TcParams& p, int grid, int out_bytes, cudaStream_t stream) {
  const int smem = 1024 + p.conv_r * 3 * 8192 + p.halo_stages * p.halo_stage_bytes + kFsTailBytes;
  if (out_bytes == 2) {
    cudaError_t e = cudaFuncSetAttribute(conv_halo_fs_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    conv_halo_fs_kernel<2><<<grid, kFsThreads, smem, stream>>>(maps, p);
  } else {
    cudaError_t e = cudaFuncSetAttribute(conv_halo_fs_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    conv_halo_fs_kernel<4><<<grid, kFsThreads, smem, stream>>>(maps, p);
  }
  return cudaGetLastError();
}

}  // namespace pmlb
