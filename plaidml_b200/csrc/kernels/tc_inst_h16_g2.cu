// Compiles the 16-bit-operand instances of the tensor-core kernel with 2 epilogue group(s).
#include "tc_gemm_kernel.cuh"
#include "tc_instances.h"

namespace pmlb {
#define PMLB_TC_DEFINE(EB, BN, NS, IM, MN, OB, G)                                              \
  template cudaError_t launch_cfg<TcCfg<EB, BN, NS, IM, MN, OB, G>>(                            \
      const TcMaps&, const TcParams&, int, cudaStream_t);
PMLB_TC_LIST_H16(PMLB_TC_DEFINE, 2)
#undef PMLB_TC_DEFINE
}  // namespace pmlb
