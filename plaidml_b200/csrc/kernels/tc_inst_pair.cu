// Compiles the CTA-pair instances of the tensor-core kernel.
#include "tc_gemm_kernel.cuh"
#include "tc_instances.h"

namespace pmlb {
#define PMLB_TC_DEFINE(EB, BN, NS, IM, MN, OB, G)                                              \
  template cudaError_t launch_cfg<TcCfg<EB, BN, NS, IM, MN, OB, G, 2>>(                         \
      const TcMaps&, const TcParams&, int, cudaStream_t);
PMLB_TC_LIST_PAIR(PMLB_TC_DEFINE)
#undef PMLB_TC_DEFINE
template int max_resident_pairs<TcCfg<2, 256, 1, 0, false, 2, 1, 2>>();
}  // namespace pmlb
