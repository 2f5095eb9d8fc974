// Parameter blocks of the gather / scatter / argsort / prng kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "pmlb_kernels.h"

namespace pmlb {

struct GatherParams {
  int dtype, idx_dtype, elem_bytes;
  int nd;  // 0: along one axis, 1: the last dim of indices addresses several dims
  int copies;  // set by the launcher: elements are copied (no interpolation)
  long long out_elems;
  // along one axis: the tensor seen as [outer][axis_len][inner], the indices as a flat list of n_idx
  long long axis_len, inner, n_idx;
  // nd: the tensor seen as [batch][dims[0]]..[dims[k-1]][inner]; index rows of k entries, rows_per_batch of them
  // per batch entry
  int k;
  long long dims[PMLB_MAX_RANK];
  long long rows_per_batch;
  int interpolation, nearest, out_of_bounds;
  double cube_coeff;
  const void* tensor;
  const void* indices;
  void* out;
};

struct ScatterParams {
  int dtype, idx_dtype, elem_bytes, mode, axis, rank, idx_rank, upd_rank;
  long long sizes[PMLB_MAX_RANK], idx_sizes[PMLB_MAX_RANK], upd_sizes[PMLB_MAX_RANK];
  long long upd_elems;
  const void* indices;
  const void* updates;
  void* out;
};

struct ArgsortParams {
  int dtype, descending;
  long long outer, n, inner;  // the tensor seen as [outer][n][inner], sorted along n
  const void* tensor;
};

// The jump table holds, per generator word and power-of-two step count, the step matrix as eight 16-entry tables (one
// per 4-bit group of the state word): applying it is eight look-ups and exclusive-ors.
enum : int { kPrngChunk = 64, kPrngLevels = 32, kPrngNibbleWords = 8 * 16, kPrngTableWords = 3 * kPrngLevels * kPrngNibbleWords };

cudaError_t launch_gather(const GatherParams& p, cudaStream_t stream);
cudaError_t launch_scatter(const ScatterParams& p, cudaStream_t stream);
// `scratch` holds as many int32 as the tensor has elements.
cudaError_t launch_argsort(const ArgsortParams& p, int32_t* out, int32_t* scratch, cudaStream_t stream);
// `table` is prng_jump_table() on the device.
cudaError_t launch_prng(const uint32_t* state, long long state_elems, float* out, long long count, uint32_t* new_state,
                        const uint32_t* table, cudaStream_t stream);
// The three step matrices raised to the powers 2^0 .. 2^31: table[c][level][4-bit group][value].
void prng_jump_table(uint32_t* table);

}  // namespace pmlb
