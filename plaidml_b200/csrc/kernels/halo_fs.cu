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

cudaError_t launch_halo_fs(const TcMaps& maps, const TcParams& p, int grid, int out_bytes, bool pair, bool dependent_launch,
                           cudaStream_t stream) {
  const int wts = p.conv_r * (pair ? 12288 : 24576);
  const int smem = 1024 + wts + p.halo_stages * p.halo_stage_bytes + kFsTailBytes;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kFsThreads, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pair) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 2;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (dependent_launch) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  auto go = [&](auto kernel) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    return cudaLaunchKernelEx(&cfg, kernel, maps, p);
  };
  if (pair) return out_bytes == 2 ? go(conv_halo_fs_kernel<2, 2>) : go(conv_halo_fs_kernel<4, 2>);
  return out_bytes == 2 ? go(conv_halo_fs_kernel<2, 1>) : go(conv_halo_fs_kernel<4, 1>);
}

}  // namespace pmlb
