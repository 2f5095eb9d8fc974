// Parameter blocks of the general contraction and element-wise kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "pmlb_kernels.h"

namespace pmlb {

enum : int { kClassF32 = 0, kClassF64 = 1, kClassI64 = 2, kClassU64 = 3 };

// Compute class of an element type, -1 if unknown.
int dtype_class(int dtype);

struct GAccess {
  int dtype;
  int rank;
  long long sizes[PMLB_MAX_RANK];
  long long strides[PMLB_MAX_RANK];
  long long off[PMLB_MAX_RANK];
  int den[PMLB_MAX_RANK];
  int coef[PMLB_MAX_RANK][PMLB_MAX_IDX];
};

struct GenericParams {
  int agg, combo, n_idx, n_src, n_cons, has_init;
  int direct;                    // 1: out_var[d] names the index variable of output dim d
  int out_var[PMLB_MAX_RANK];
  int n_loop;                    // variables the thread iterates over
  int loop_var[PMLB_MAX_IDX];
  // Without `direct`: variable solve_var[s] follows from output dim solve_dim[s] once the loop variables and
  // the variables of earlier entries are set (its coefficient there is non-zero), so it is not iterated over.
  int n_solve;
  int solve_dim[PMLB_MAX_RANK];
  int solve_var[PMLB_MAX_RANK];
  long long range[PMLB_MAX_IDX];
  GAccess out, init;
  GAccess src[3];
  int cons_coef[PMLB_MAX_CONS][PMLB_MAX_IDX];
  long long cons_off[PMLB_MAX_CONS];
  long long cons_range[PMLB_MAX_CONS];
  const void* srcp[3];
  const void* initp;
  void* outp;
  long long out_elems;
};

enum : int {
  kEwIdent = 0, kEwAdd, kEwSub, kEwMul, kEwDiv, kEwMod, kEwMax, kEwMin, kEwNeg, kEwAbs, kEwRelu,
  kEwSign, kEwSelect, kEwCmpEq, kEwCmpNe, kEwCmpLt, kEwCmpLe, kEwCmpGt, kEwCmpGe, kEwLogicalAnd,
  kEwLogicalOr, kEwLogicalXor, kEwLogicalNot, kEwExp, kEwLog, kEwSqrt, kEwRsqrt, kEwTanh,
  kEwSigmoid, kEwSin, kEwCos, kEwTan, kEwSinh, kEwCosh, kEwAsin, kEwAcos, kEwAtan, kEwAsinh,
  kEwAcosh, kEwAtanh, kEwErf, kEwPow, kEwFloor, kEwCeil, kEwRound, kEwBitAnd, kEwBitOr, kEwBitXor,
  kEwBitNot, kEwBitShl, kEwBitShr, kEwCount
};

struct EltwiseParams {
  int op;
  int n_in;
  int rank;
  int out_dtype;
  int in_dtype[3];
  int compute_class;   // kClass*
  int arith_dtype;     // element type the arithmetic is carried out in
  int narrow_inputs;   // convert operands to arith_dtype first (a cast's source is not)
  int narrow_result;
  long long sizes[PMLB_MAX_RANK];
  long long in_strides[3][PMLB_MAX_RANK];
  const void* in[3];
  void* out;
  long long elems;
};

cudaError_t launch_contract(const GenericParams& p, cudaStream_t stream);
cudaError_t launch_eltwise(const EltwiseParams& p, cudaStream_t stream);
cudaError_t launch_fill_f32(float* out, long long n, float value, cudaStream_t stream);

}  // namespace pmlb
