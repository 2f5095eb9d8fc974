// Compiles and launches the fused first-layer kernel (convolution + bias + ReLU + max pool).
#include "s2d_pool_kernel.cuh"

#include "s2d_pool.h"

#include <cstdlib>

namespace pmlb {

int s2d_pool_stages(int stage_bytes) {
  if (stage_bytes <= 0) return 0;
  const int room = kSpSmemLimit - 1024 - kSpWeightBytes - kSpHbufBytes - kSpTailBytes;
  const int n = room / stage_bytes;
  return n > kSpMaxStages ? kSpMaxStages : n;
}

namespace {

// 128 x n x 16 MMA on 16-bit operands with an f32 accumulator, both operands K-major
uint32_t mma_desc(bool is_f16, int n) {
  const uint32_t fmt = is_f16 ? 0u : 1u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

bool dependent_launch() {
  static const bool on = [] {
    const char* v = std::getenv("PMLB_TC_DEPENDENT_LAUNCH");
    return v && v[0] == '1';
  }();
  return on;
}

}  // namespace

cudaError_t launch_s2d_pool(const S2dPoolParams& params, int grid, bool in_f16, bool out_bf16, cudaStream_t stream) {
  S2dPoolParams p = params;
  for (int i = 0; i < 4; ++i) p.idesc[i] = mma_desc(in_f16, 64 * (i + 1));
  const bool bf16 = out_bf16;
  const bool dependent_launch_on = dependent_launch();
  const int smem = 1024 + kSpWeightBytes + kSpHbufBytes + p.stages * p.stage_bytes + kSpTailBytes;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kSpThreads, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int na = 0;
  if (dependent_launch_on) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (bf16) {
    cudaError_t e = cudaFuncSetAttribute(conv_s2d_pool_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    return cudaLaunchKernelEx(&cfg, conv_s2d_pool_kernel<true>, p);
  }
  cudaError_t e = cudaFuncSetAttribute(conv_s2d_pool_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  return cudaLaunchKernelEx(&cfg, conv_s2d_pool_kernel<false>, p);
}

}  // namespace pmlb
