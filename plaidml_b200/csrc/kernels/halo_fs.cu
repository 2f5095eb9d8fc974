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

cudaError_t launch_halo_fs(const TcMaps& maps, const TcParams& p, int grid, int out_bytes, bool dependent_launch,
                           cudaStream_t stream) {
  const int smem = 1024 + p.conv_r * 3 * 8192 + p.halo_stages * p.halo_stage_bytes + kFsTailBytes;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kFsThreads, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int na = 0;
  if (dependent_launch) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (out_bytes == 2) {
    cudaError_t e = cudaFuncSetAttribute(conv_halo_fs_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    return cudaLaunchKernelEx(&cfg, conv_halo_fs_kernel<2>, maps, p);
  }
  cudaError_t e = cudaFuncSetAttribute(conv_halo_fs_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  return cudaLaunchKernelEx(&cfg, conv_halo_fs_kernel<4>, maps, p);
}

}  // namespace pmlb
