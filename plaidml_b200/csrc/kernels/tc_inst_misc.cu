// Compiles the int8 and split-fp32 instances of the tensor-core kernel.
#include "tc_gemm_kernel.cuh"
#include "tc_instances.h"

namespace pmlb {
#define PMLB_TC_DEFINE(EB, BN, NS, IM, MN, OB, G)                                              \
  template cudaError_t launch_cfg<TcCfg<EB, BN, NS, IM, MN, OB, G>>(                            \
      const TcMaps&, const TcParams&, int, cudaStream_t);
PMLB_TC_LIST_MISC(PMLB_TC_DEFINE)
#undef PMLB_TC_DEFINE
}  // namespace pmlb
