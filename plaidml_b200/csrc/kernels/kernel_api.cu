// extern "C" surface of the kernel library: validates descriptors, owns plan scratch,
// sequences the preparation kernels and the main kernel of each plan.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>

#include "generic.h"
#include "pmlb_kernels.h"
#include "prepass.h"
#include "reduce.h"
#include "s2d_pool.h"
#include "special.h"
#include "tc_gemm.cuh"
#include "conv_route.h"
#include "tc_launch.h"

namespace {

thread_local std::string g_last_error;

pmlb_status fail(pmlb_status code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

}  // namespace

// Lets the other translation units of the library report through pmlb_last_error().
void pmlb_set_last_error_message(const std::string& msg) { g_last_error = msg; }

namespace {

pmlb_status cuda_fail(cudaError_t e, const char* what) {
  return fail(PMLB_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

int elem_bytes_of(int dtype) {
  switch (dtype) {
    case PMLB_BOOL:
    case PMLB_I8:
    case PMLB_U8: return 1;
    case PMLB_I16:
    case PMLB_U16:
    case PMLB_F16:
    case PMLB_BF16: return 2;
    case PMLB_I32:
    case PMLB_U32:
    case PMLB_F32: return 4;
    case PMLB_I64:
    case PMLB_U64:
    case PMLB_F64: return 8;
    default: return 0;
  }
}

long long round_up(long long v, long long m) { return (v + m - 1) / m * m; }

bool have_sm100(std::string* why) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    cudaGetLastError();
    *why = "no CUDA device is visible; this library has no CPU path";
    return false;
  }
  int dev = 0;
  cudaGetDevice(&dev);
  int major = 0;
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (major != 10) {
    *why = "the current CUDA device is not compute capability 10.x (sm_100a kernels only)";
    return false;
  }
  return true;
}

// Debugging aid (see pmlb_debug_set_trace): device buffer that CTA 0 of the next tensor-core
// launches logs its pipeline timeline to.
long long* g_trace_buffer = nullptr;

enum PlanKind { kPlanGemm, kPlanConv, kPlanReduce, kPlanPool, kPlanContract, kPlanEltwise, kPlanSpecial };

}  // namespace

struct pmlb_plan {
  PlanKind kind;
  const char* kind_name = "";
  int device = 0;
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  int* status = nullptr;  // device word shared by the plan's tensor-core launches
  bool owns_status = true;

  pmlb_gemm_desc gemm;
  long long kpad = 0;       // fp32 path: padded K of the split copies
  bool transpose_b = false; // 8/16-bit path: B goes through [n][k] scratch
  bool split = false;
  int armed_wait_us = 0;    // > 0: the next invoke runs the time-out test (see pmlb_plan_arm_timeout_test)
  int ksplit = 1;           // parts of the K range (two-pass split-K), each of kslice elements
  long long kslice = 0;

  pmlb_conv_desc conv;
  bool filter_set = false;
  bool halo = false;             // conv: halo route (scratch = weights as for im2col)
  bool packed_rows = false;      // conv: packed-row route (scratch = weights, then the padded activation)
  bool s2d = false;              // conv: space-to-depth route (scratch = weights, then the packed activation)
  bool s2d_pool = false;         // ... fused with the 3 x 3 / 2 max pool behind it
  size_t packed_input_off = 0;   // byte offset of the padded activation inside scratch

  pmlb_reduce_desc reduce;
  pmlb_pool_desc pool;
  pmlb::GenericParams generic;
  pmlb::EltwiseParams eltwise;
  pmlb_special_desc special;
};

namespace {

pmlb_status alloc_plan_memory(pmlb_plan* plan, size_t scratch_bytes, bool need_status) {
  cudaGetDevice(&plan->device);
  if (scratch_bytes > 0) {
    cudaError_t e = cudaMalloc(&plan->scratch, scratch_bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(plan scratch)");
    plan->scratch_bytes = scratch_bytes;
  }
  if (need_status) {
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&plan->status), sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(plan status)");
    e = cudaMemset(plan->status, 0, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(plan status)");
  }
  return PMLB_OK;
}

int ew_opcode(const char* name) {
  static const struct {
    const char* name;
    int code;
  } table[] = {
      {"ident", pmlb::kEwIdent}, {"assign", pmlb::kEwIdent}, {"cast", pmlb::kEwIdent},
      {"add", pmlb::kEwAdd}, {"sub", pmlb::kEwSub}, {"mul", pmlb::kEwMul}, {"div", pmlb::kEwDiv},
      {"mod", pmlb::kEwMod}, {"max", pmlb::kEwMax}, {"min", pmlb::kEwMin}, {"neg", pmlb::kEwNeg},
      {"abs", pmlb::kEwAbs}, {"relu", pmlb::kEwRelu}, {"sign", pmlb::kEwSign},
      {"select", pmlb::kEwSelect}, {"cmp_eq", pmlb::kEwCmpEq}, {"cmp_ne", pmlb::kEwCmpNe},
      {"cmp_lt", pmlb::kEwCmpLt}, {"cmp_le", pmlb::kEwCmpLe}, {"cmp_gt", pmlb::kEwCmpGt},
      {"cmp_ge", pmlb::kEwCmpGe}, {"logical_and", pmlb::kEwLogicalAnd},
      {"logical_or", pmlb::kEwLogicalOr}, {"logical_xor", pmlb::kEwLogicalXor},
      {"logical_not", pmlb::kEwLogicalNot}, {"exp", pmlb::kEwExp}, {"log", pmlb::kEwLog},
      {"sqrt", pmlb::kEwSqrt}, {"rsqrt", pmlb::kEwRsqrt}, {"tanh", pmlb::kEwTanh},
      {"sigmoid", pmlb::kEwSigmoid}, {"sin", pmlb::kEwSin}, {"cos", pmlb::kEwCos},
      {"tan", pmlb::kEwTan}, {"sinh", pmlb::kEwSinh}, {"cosh", pmlb::kEwCosh},
      {"asin", pmlb::kEwAsin}, {"acos", pmlb::kEwAcos}, {"atan", pmlb::kEwAtan},
      {"asinh", pmlb::kEwAsinh}, {"acosh", pmlb::kEwAcosh}, {"atanh", pmlb::kEwAtanh},
      {"erf", pmlb::kEwErf}, {"pow", pmlb::kEwPow}, {"floor", pmlb::kEwFloor},
      {"ceil", pmlb::kEwCeil}, {"round", pmlb::kEwRound}, {"bit_and", pmlb::kEwBitAnd},
      {"bit_or", pmlb::kEwBitOr}, {"bit_xor", pmlb::kEwBitXor}, {"bit_not", pmlb::kEwBitNot},
      {"bit_shl", pmlb::kEwBitShl}, {"bit_shr", pmlb::kEwBitShr},
  };
  for (const auto& e : table) {
    if (std::strcmp(e.name, name) == 0) return e.code;
  }
  return -1;
}

bool is_compare(int op) {
  return (op >= pmlb::kEwCmpEq && op <= pmlb::kEwLogicalNot);
}

void copy_access(const pmlb_access& in, pmlb::GAccess* out, int n_idx) {
  std::memset(out, 0, sizeof(*out));
  out->dtype = in.dtype;
  out->rank = in.rank;
  for (int d = 0; d < in.rank; ++d) {
    out->sizes[d] = in.sizes[d];
    out->strides[d] = in.strides[d];
    out->off[d] = in.off[d];
    out->den[d] = in.den[d] >= 1 ? in.den[d] : 1;
    for (int i = 0; i < n_idx; ++i) out->coef[d][i] = in.coef[d][i];
  }
}

}  // namespace

extern "C" {

const char* pmlb_last_error(void) { return g_last_error.c_str(); }

const char* pmlb_version(void) { return "plaidml-b200 kernels 0.1 (sm_100a)"; }

int pmlb_device_count(void) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  int good = 0;
  for (int d = 0; d < count; ++d) {
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d);
    if (major == 10) ++good;
  }
  return good;
}

void pmlb_debug_set_trace(void* device_buffer) {
  g_trace_buffer = static_cast<long long*>(device_buffer);
}

void pmlb_plan_free(pmlb_plan* plan) {
  if (!plan) return;
  if (plan->scratch) cudaFree(plan->scratch);
  if (plan->status && plan->owns_status) cudaFree(plan->status);
  delete plan;
}

pmlb_status pmlb_plan_share_status(pmlb_plan* plan, int* device_word) {
  if (!plan || !device_word) return fail(PMLB_ERR_INVALID, "null argument");
  if (plan->status && plan->owns_status) cudaFree(plan->status);
  plan->status = device_word;
  plan->owns_status = false;
  return PMLB_OK;
}

size_t pmlb_plan_scratch_bytes(const pmlb_plan* plan) { return plan ? plan->scratch_bytes : 0; }

const char* pmlb_plan_kind(const pmlb_plan* plan) { return plan ? plan->kind_name : ""; }

int pmlb_plan_split_k(const pmlb_plan* plan) { return plan ? plan->ksplit : 1; }

pmlb_status pmlb_plan_arm_timeout_test(pmlb_plan* plan, int wait_limit_ms) {
  if (!plan || plan->kind != kPlanGemm) return fail(PMLB_ERR_INVALID, "the time-out test takes a gemm plan");
  if (wait_limit_ms < 1 || wait_limit_ms > 100) return fail(PMLB_ERR_INVALID, "wait limit must be 1..100 ms");
  if (plan->gemm.in_dtype == PMLB_F32 || plan->ksplit > 1) {
    return fail(PMLB_ERR_UNSUPPORTED, "the time-out test takes a single-pass 8/16-bit gemm plan");
  }
  plan->armed_wait_us = wait_limit_ms * 1000;
  return PMLB_OK;
}

pmlb_status pmlb_plan_check(pmlb_plan* plan, void* stream) {
  if (!plan) return fail(PMLB_ERR_INVALID, "null plan");
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
  if (!plan->status) return PMLB_OK;
  int code = 0;
  e = cudaMemcpy(&code, plan->status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(status)");
  if (code != 0) {
    cudaMemset(plan->status, 0, sizeof(int));
    return fail(PMLB_ERR_TIMEOUT,
                "a device-side pipeline wait gave up (role code " + std::to_string(code) + ")");
  }
  return PMLB_OK;
}

// ------------------------------------------------------------------ GEMM

pmlb_status pmlb_gemm_dispatch(const pmlb_gemm_desc* d, pmlb_plan** out) {
  if (!d || !out) return fail(PMLB_ERR_INVALID, "null argument");
  *out = nullptr;
  std::string why;
  if (!have_sm100(&why)) return fail(PMLB_ERR_UNSUPPORTED, why);
  if (d->m <= 0 || d->n <= 0 || d->k <= 0 || d->batch <= 0) {
    return fail(PMLB_ERR_INVALID, "gemm: m, n, k and batch must be positive");
  }
  const int in = d->in_dtype, od = d->out_dtype;
  const bool f32 = in == PMLB_F32;
  const bool h16 = in == PMLB_BF16 || in == PMLB_F16;
  const bool i8 = in == PMLB_I8;
  if (f32) {
    if (od != PMLB_F32) return fail(PMLB_ERR_UNSUPPORTED, "gemm: f32 inputs produce f32");
  } else if (h16) {
    if (od != PMLB_F32 && od != PMLB_BF16 && od != PMLB_F16) {
      return fail(PMLB_ERR_UNSUPPORTED, "gemm: 16-bit inputs produce f32, bf16 or f16");
    }
  } else if (i8) {
    if (od != PMLB_I32 && od != PMLB_I8) {
      return fail(PMLB_ERR_UNSUPPORTED, "gemm: int8 inputs produce int32 or int8");
    }
    if (d->epilogue & PMLB_EPI_ROWMAX) {
      return fail(PMLB_ERR_UNSUPPORTED, "gemm: row max is a float epilogue");
    }
  } else {
    return fail(PMLB_ERR_UNSUPPORTED, "gemm: input type must be f32, bf16, f16 or int8");
  }
  if ((d->epilogue & PMLB_EPI_ROWMAX) && (d->epilogue & ~PMLB_EPI_ROWMAX)) {
    return fail(PMLB_ERR_UNSUPPORTED, "gemm: row max cannot be combined with other epilogue steps");
  }
  const int eb = elem_bytes_of(in);
  if (d->k_first < 0 || d->k_first >= d->k) return fail(PMLB_ERR_INVALID, "gemm: k_first outside (0, k)");
  if (d->k_first > 0) {
    if (f32 || d->batch != 1 || (d->k_first * eb) % 128 != 0 || (d->epilogue & PMLB_EPI_ROWMAX)) {
      return fail(PMLB_ERR_UNSUPPORTED, "gemm: A in two parts needs 8/16-bit inputs, one matrix, whole k-blocks in the first part");
    }
    if (d->a2_stride < 0) return fail(PMLB_ERR_INVALID, "gemm: negative a2_stride");
    if (d->a2_stride == 0 && (d->lda2 < d->k - d->k_first || (d->lda2 * eb) % 16 != 0)) {
      return fail(PMLB_ERR_INVALID, "gemm: lda2 smaller than the second part's width, or rows not 16-byte aligned");
    }
    if (d->a2_stride > 0) {
      const long long pp = (d->a2_h + d->a2_stride - 1) / d->a2_stride, qq = (d->a2_w + d->a2_stride - 1) / d->a2_stride;
      if (d->a2_n <= 0 || d->a2_h <= 0 || d->a2_w <= 0 || d->a2_n * pp * qq != d->m || d->a2_stride > 8 ||
          ((d->k - d->k_first) * eb) % 16 != 0) {
        return fail(PMLB_ERR_UNSUPPORTED, "gemm: the second part's pixels do not match m, or its channels are not whole 16-byte groups");
      }
    }
  }
  const long long min_lda = d->k_first > 0 ? d->k_first : d->k;
  const long long min_ldb = d->b_is_nk ? d->k : d->n;
  if (d->lda < min_lda || d->ldb < min_ldb || d->ldc < d->n) {
    return fail(PMLB_ERR_INVALID, "gemm: leading dimension smaller than the row length");
  }
  pmlb_plan* plan = new (std::nothrow) pmlb_plan();
  if (!plan) return fail(PMLB_ERR_INVALID, "out of host memory");
  plan->kind = kPlanGemm;
  plan->kind_name = "tc_gemm";
  plan->gemm = *d;
  size_t scratch = 0;
  if (f32) {
    plan->split = true;
    plan->kpad = round_up(d->k, 4);
    const long long a_mats = d->stride_a != 0 ? d->batch : 1;
    const long long b_mats = d->stride_b != 0 ? d->batch : 1;
    scratch = static_cast<size_t>(2 * 4 * plan->kpad * (a_mats * d->m + b_mats * d->n));
  } else {
    if ((d->lda * eb) % 16 != 0 || (d->stride_a * eb) % 16 != 0) {
      delete plan;
      return fail(PMLB_ERR_UNSUPPORTED, "gemm: A rows must start on 16-byte boundaries");
    }
    const bool b_aligned = (d->ldb * eb) % 16 == 0 && (d->stride_b * eb) % 16 == 0;
    if (d->b_is_nk) {
      if (!b_aligned) {
        delete plan;
        return fail(PMLB_ERR_UNSUPPORTED, "gemm: B rows must start on 16-byte boundaries");
      }
    } else if ((d->flags & PMLB_GEMM_TRANSPOSE_B) || !b_aligned) {
      plan->transpose_b = true;
      plan->kpad = round_up(d->k, 16 / eb);
      const long long b_mats = d->stride_b != 0 ? d->batch : 1;
      scratch = static_cast<size_t>(b_mats * d->n * plan->kpad * eb);
    }
  }
  // Split K?  (8/16-bit inputs read in place, one matrix, no row maxima: see PMLB_GEMM_NO_SPLIT_K)
  const char* split_env = std::getenv("PMLB_SPLIT_K");   // "0": never split (sums then never depend on the tile count)
  const bool split_allowed = !(split_env && split_env[0] == '0') || (d->flags & PMLB_GEMM_SPLIT_K);
  if (!f32 && !plan->transpose_b && d->batch == 1 && !(d->epilogue & PMLB_EPI_ROWMAX) && d->k_first == 0 &&
      !(d->flags & PMLB_GEMM_NO_SPLIT_K) && split_allowed) {
    const int bk = 128 / eb;
    int dev = 0, num_sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    const long long bn = d->n <= 64 ? 64 : 128;
    const long long tiles = static_cast<long long>((d->m + 127) / 128) * ((d->n + bn - 1) / bn);
    const int num_kb = d->k / bk;
    const bool forced = (d->flags & PMLB_GEMM_SPLIT_K) != 0;
    if (d->k % bk == 0 && ((tiles * 2 <= num_sms && num_kb >= 8) || forced)) {
      const long long room = forced ? 8 : num_sms / tiles;            // CTAs per tile that still fit one wave
      int parts = 1;
      for (int s = 2; s <= 8; ++s) {
        if (s <= room && num_kb % s == 0 && (forced || num_kb / s >= 4)) parts = s;
      }
      if (parts > 1) {
        plan->ksplit = parts;
        plan->kslice = static_cast<long long>(num_kb / parts) * bk;
        scratch = static_cast<size_t>(parts) * d->m * d->n * 4;
      }
    }
  }
  pmlb_status st = alloc_plan_memory(plan, scratch, true);
  if (st != PMLB_OK) {
    pmlb_plan_free(plan);
    return st;
  }
  if (plan->transpose_b && plan->scratch) {
    // the K tail of the transposed copy must read as zero
    cudaMemset(plan->scratch, 0, plan->scratch_bytes);
  }
  *out = plan;
  return PMLB_OK;
}

pmlb_status pmlb_gemm_invoke(pmlb_plan* plan, void* stream_v, const void* a, const void* b, void* c,
                             const void* bias, const void* residual, float* rowmax) {
  return pmlb_gemm_invoke_two(plan, stream_v, a, nullptr, b, c, bias, residual, rowmax);
}

pmlb_status pmlb_gemm_invoke_two(pmlb_plan* plan, void* stream_v, const void* a, const void* a2, const void* b, void* c,
                                 const void* bias, const void* residual, float* rowmax) {
  if (!plan || plan->kind != kPlanGemm) return fail(PMLB_ERR_INVALID, "not a gemm plan");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const pmlb_gemm_desc& d = plan->gemm;
  if (!a || !b) return fail(PMLB_ERR_INVALID, "gemm: null operand");
  if ((d.k_first > 0) != (a2 != nullptr)) {
    return fail(PMLB_ERR_INVALID, d.k_first > 0 ? "gemm: the second part of A is missing (pmlb_gemm_invoke_two)"
                                                : "gemm: this plan takes A in one part");
  }
  if ((d.epilogue & PMLB_EPI_BIAS) && !bias) return fail(PMLB_ERR_INVALID, "gemm: bias missing");
  if ((d.epilogue & PMLB_EPI_RESIDUAL) && !residual) return fail(PMLB_ERR_INVALID, "gemm: residual missing");
  if ((d.epilogue & PMLB_EPI_ROWMAX) && !rowmax) return fail(PMLB_ERR_INVALID, "gemm: rowmax missing");
  if (!(d.epilogue & PMLB_EPI_ROWMAX) && !c) return fail(PMLB_ERR_INVALID, "gemm: null output");

  pmlb::TcLaunch L;
  L.elem_bytes = elem_bytes_of(d.in_dtype);
  L.is_f16 = d.in_dtype == PMLB_F16;
  L.m = d.m;
  L.n = d.n;
  L.k = d.k;
  L.batch = d.batch;
  L.out = c;
  L.ldc = d.ldc;
  L.out_batch_stride = d.stride_c;
  L.out_dtype = d.out_dtype;
  L.epi_flags = d.epilogue;
  L.bias = bias;
  L.residual = residual;
  L.ldr = d.ldr;
  L.res_batch_stride = d.stride_r;
  L.rowmax = rowmax;
  L.status = plan->status;
  L.bn_override = d.tile_n;
  L.k_first = d.k_first;
  L.lda_second = d.lda2;
  pmlb::ConvGeom second_pixels;
  if (d.k_first > 0 && d.a2_stride > 0) {
    second_pixels = pmlb::ConvGeom{};
    second_pixels.n = d.a2_n; second_pixels.h = d.a2_h; second_pixels.w = d.a2_w; second_pixels.c = d.k - d.k_first;
    second_pixels.r = second_pixels.s = 1;
    second_pixels.p = (d.a2_h + d.a2_stride - 1) / d.a2_stride;
    second_pixels.q = (d.a2_w + d.a2_stride - 1) / d.a2_stride;
    second_pixels.stride_h = second_pixels.stride_w = d.a2_stride;
    second_pixels.pad_h = second_pixels.pad_w = 0;
    second_pixels.dil_h = second_pixels.dil_w = 1;
    L.a_second_pixels = &second_pixels;
  }
  L.force_slow_epilogue = (d.flags & PMLB_GEMM_PLAIN_STORES) != 0;
  L.residual_from_global = (d.flags & PMLB_GEMM_PLAIN_RESIDUAL) != 0;
  if (d.flags & PMLB_GEMM_CTA_PAIRS) L.pair_override = 1;
  if (d.flags & PMLB_GEMM_NO_CTA_PAIRS) L.pair_override = 0;
  if (d.flags & PMLB_GEMM_NO_TAIL_SPLIT) L.split_tail = 0;
  L.trace = g_trace_buffer;
  if (plan->armed_wait_us > 0) {
    // one launch whose first operand load of CTA 0 never happens: the wait for it gives up after the armed
    // limit, every role of that CTA leaves through the tear-down and the status word reports it
    L.wait_limit_us = plan->armed_wait_us;
    L.test_drop_load = true;
    L.pair_override = 0;
    plan->armed_wait_us = 0;
  }

  if (plan->split) {
    const long long kp = plan->kpad;
    const long long a_mats = d.stride_a != 0 ? d.batch : 1;
    const long long b_mats = d.stride_b != 0 ? d.batch : 1;
    float* a_hi = static_cast<float*>(plan->scratch);
    float* a_lo = a_hi + a_mats * d.m * kp;
    float* b_hi = a_lo + a_mats * d.m * kp;
    float* b_lo = b_hi + b_mats * d.n * kp;
    pmlb::SplitTf32Args sa{static_cast<const float*>(a), d.lda, d.stride_a, a_hi, a_lo, kp,
                           static_cast<long long>(d.m) * kp, d.m, d.k, static_cast<int>(a_mats), false};
    pmlb::SplitTf32Args sb{static_cast<const float*>(b), d.ldb, d.stride_b, b_hi, b_lo, kp,
                           static_cast<long long>(d.n) * kp, d.b_is_nk ? d.n : d.k, d.b_is_nk ? d.k : d.n,
                           static_cast<int>(b_mats), !d.b_is_nk};
    cudaError_t e = pmlb::launch_split_tf32_pair(sa, sb, stream);
    if (e != cudaSuccess) return cuda_fail(e, "split(A, B)");
    L.nsplit = 2;
    L.a0 = a_hi;
    L.a1 = a_lo;
    L.lda = kp;
    L.a_batch_stride = d.stride_a != 0 ? static_cast<long long>(d.m) * kp : 0;
    L.b0 = b_hi;
    L.b1 = b_lo;
    L.ldb = kp;
    L.b_batch_stride = d.stride_b != 0 ? static_cast<long long>(d.n) * kp : 0;
    L.b_mn = false;
  } else {
    L.a0 = a;
    L.a1 = a2;   // (second part of A, plans with k_first > 0)
    L.lda = d.lda;
    L.a_batch_stride = d.stride_a;
    if (plan->transpose_b) {
      const long long kp = plan->kpad;
      const long long b_mats = d.stride_b != 0 ? d.batch : 1;
      cudaError_t e = pmlb::launch_transpose(b, d.ldb, d.stride_b, plan->scratch, kp,
                                             static_cast<long long>(d.n) * kp, d.k, d.n,
                                             static_cast<int>(b_mats), L.elem_bytes, stream);
      if (e != cudaSuccess) return cuda_fail(e, "transpose(B)");
      L.b0 = plan->scratch;
      L.ldb = kp;
      L.b_batch_stride = d.stride_b != 0 ? static_cast<long long>(d.n) * kp : 0;
      L.b_mn = false;
    } else {
      L.b0 = b;
      L.ldb = d.ldb;
      L.b_batch_stride = d.stride_b;
      L.b_mn = !d.b_is_nk;
    }
  }
  if (d.epilogue & PMLB_EPI_ROWMAX) {
    cudaError_t e = pmlb::launch_fill_f32(rowmax, static_cast<long long>(d.batch) * d.m,
                                          -__builtin_inff(), stream);
    if (e != cudaSuccess) return cuda_fail(e, "fill(rowmax)");
  }
  if (plan->ksplit > 1) {
    // pass 1: part s multiplies columns [s * kslice, (s + 1) * kslice) of A with the matching rows of B,
    // as entry s of a batch, into partial products in plan scratch; no epilogue
    const bool is_int = d.in_dtype == PMLB_I8;
    L.batch = plan->ksplit;
    L.k = static_cast<int>(plan->kslice);
    L.a_batch_stride = plan->kslice;
    L.b_batch_stride = d.b_is_nk ? plan->kslice : plan->kslice * d.ldb;
    L.out = plan->scratch;
    L.ldc = d.n;
    L.out_batch_stride = static_cast<long long>(d.m) * d.n;
    L.out_dtype = is_int ? PMLB_I32 : PMLB_F32;
    L.epi_flags = 0;
    L.bias = nullptr;
    L.residual = nullptr;
    std::string err1;
    const int rc1 = pmlb::tc_launch(L, stream, &err1);
    if (rc1 != 0) return fail(static_cast<pmlb_status>(rc1), "gemm (split K): " + err1);
    // pass 2: the parts summed in order, then the epilogue
    cudaError_t e = pmlb::launch_splitk_combine(plan->scratch, is_int, plan->ksplit, d.m, d.n, c, d.out_dtype, d.ldc,
                                                d.epilogue, bias, residual, d.ldr, stream);
    if (e != cudaSuccess) return cuda_fail(e, "split-K combine");
    return PMLB_OK;
  }
  std::string err;
  const int rc = pmlb::tc_launch(L, stream, &err);
  if (rc != 0) return fail(static_cast<pmlb_status>(rc), "gemm: " + err);
  return PMLB_OK;
}

// ------------------------------------------------------------------ convolution

pmlb_status pmlb_conv_dispatch(const pmlb_conv_desc* d, pmlb_plan** out) {
  if (!d || !out) return fail(PMLB_ERR_INVALID, "null argument");
  *out = nullptr;
  std::string why;
  if (!have_sm100(&why)) return fail(PMLB_ERR_UNSUPPORTED, why);
  if (d->in_dtype != PMLB_BF16 && d->in_dtype != PMLB_F16 && d->in_dtype != PMLB_F32) {
    return fail(PMLB_ERR_UNSUPPORTED, "conv: activations must be bf16, f16 or f32");
  }
  if (d->out_dtype != PMLB_F32 && d->out_dtype != PMLB_BF16 && d->out_dtype != PMLB_F16) {
    return fail(PMLB_ERR_UNSUPPORTED, "conv: output must be f32, bf16 or f16");
  }
  const bool f32 = d->in_dtype == PMLB_F32;
  if (f32 && d->out_dtype != PMLB_F32) return fail(PMLB_ERR_UNSUPPORTED, "conv: f32 activations produce f32");
  if (f32 && (d->flags & PMLB_CONV_MAX_POOL_3X3_S2)) {
    return fail(PMLB_ERR_UNSUPPORTED, "conv: this shape does not take the fused max pool");
  }
  if (d->n <= 0 || d->h <= 0 || d->w <= 0 || d->c <= 0 || d->r <= 0 || d->s <= 0 || d->k <= 0 ||
      d->p <= 0 || d->q <= 0 || d->stride_h <= 0 || d->stride_w <= 0 || d->dil_h <= 0 ||
      d->dil_w <= 0 || d->pad_h < 0 || d->pad_w < 0) {
    return fail(PMLB_ERR_INVALID, "conv: bad geometry");
  }
  const bool s2d = pmlb::conv_takes_s2d(*d) && (d->flags & PMLB_CONV_NO_S2D) == 0;
  const bool pooled = (d->flags & PMLB_CONV_MAX_POOL_3X3_S2) != 0;
  if (pooled && !(s2d && pmlb::conv_takes_s2d_pool(*d))) {
    return fail(PMLB_ERR_UNSUPPORTED, "conv: this shape does not take the fused max pool");
  }
  const bool packed =
      !s2d && pmlb::conv_takes_packed_rows(*d) && (d->flags & PMLB_CONV_NO_PACKED_ROWS) == 0;
  if (!f32 && !packed && !s2d && d->c % 8 != 0) {
    return fail(PMLB_ERR_UNSUPPORTED, "conv: channel count must be a multiple of 8");
  }
  // every output pixel's first tap must lie inside the im2col bounding box
  const int upper_w = (d->q - 1) * d->stride_w + 1 - d->pad_w - d->w;
  const int upper_h = (d->p - 1) * d->stride_h + 1 - d->pad_h - d->h;
  if (d->pad_w > 128 || d->pad_h > 128 || upper_w < -128 || upper_w > 127 || upper_h < -128 ||
      upper_h > 127 || d->stride_w > 8 || d->stride_h > 8) {
    return fail(PMLB_ERR_UNSUPPORTED, "conv: geometry outside the im2col descriptor range");
  }
  if (d->epilogue & PMLB_EPI_ROWMAX) return fail(PMLB_ERR_UNSUPPORTED, "conv: no row max");
  pmlb_plan* plan = new (std::nothrow) pmlb_plan();
  if (!plan) return fail(PMLB_ERR_INVALID, "out of host memory");
  plan->kind = kPlanConv;
  plan->kind_name = "tc_conv";
  plan->conv = *d;
  size_t scratch = static_cast<size_t>(d->k) * d->r * d->s * d->c * 2;
  if (f32) {
    // fp32: three TF32 products per term (as the fp32 GEMM): the filter and, per call, the activation are split
    // into high and low TF32 parts, channels padded to whole 16-byte groups; scratch = [w hi][w lo][x hi][x lo]
    plan->split = true;
    plan->kpad = round_up(d->c, 4);
    plan->kind_name = "tc_conv";
    const size_t wts = static_cast<size_t>(d->k) * d->r * d->s * plan->kpad * 4;
    const size_t act = static_cast<size_t>(d->n) * d->h * d->w * plan->kpad * 4;
    plan->packed_input_off = (2 * wts + 255) / 256 * 256;
    scratch = plan->packed_input_off + 2 * ((act + 255) / 256 * 256);
  }
  if (s2d) {
    const pmlb::S2dShape g = pmlb::conv_s2d_shape(*d);
    plan->s2d = true;
    plan->s2d_pool = pooled;
    plan->kind_name = pooled ? "tc_conv_s2d_pool" : "tc_conv_s2d";
    const size_t wts = static_cast<size_t>(pmlb::conv_s2d_weight_bytes(g));
    plan->packed_input_off = (wts + 255) / 256 * 256;
    // (a tile's copy may run past the last image: keep that much readable behind it)
    scratch = plan->packed_input_off + static_cast<size_t>(d->n) * g.h2 * g.wp * 32 +
              static_cast<size_t>(g.stage_px) * 32;
  }
  if (!packed && !s2d && pmlb::conv_takes_halo(*d) && (d->flags & PMLB_CONV_NO_HALO) == 0) {
    plan->halo = true;
    plan->kind_name = "tc_conv_halo";
  }
  if (packed) {
    plan->packed_rows = true;
    plan->kind_name = "tc_conv_rows";
    const size_t wts = static_cast<size_t>(d->k) * d->r * 64 * 2;
    plan->packed_input_off = (wts + 255) / 256 * 256;
    scratch = plan->packed_input_off + static_cast<size_t>(d->n) * d->h *
                                           pmlb::conv_packed_row_width(*d) *
                                           pmlb::conv_padded_channels(*d) * 2;
  }
  pmlb_status st = alloc_plan_memory(plan, scratch, true);
  if (st != PMLB_OK) {
    pmlb_plan_free(plan);
    return st;
  }
  *out = plan;
  return PMLB_OK;
}

pmlb_status pmlb_conv_set_filter(pmlb_plan* plan, void* stream, const void* filter, int32_t dtype) {
  if (!plan || plan->kind != kPlanConv) return fail(PMLB_ERR_INVALID, "not a conv plan");
  if (!filter) return fail(PMLB_ERR_INVALID, "conv: null filter");
  if (dtype != PMLB_F32 && dtype != PMLB_BF16 && dtype != PMLB_F16) {
    return fail(PMLB_ERR_UNSUPPORTED, "conv: filter must be f32, bf16 or f16");
  }
  const pmlb_conv_desc& d = plan->conv;
  cudaError_t e;
  if (plan->split) {
    const size_t wts = static_cast<size_t>(d.k) * d.r * d.s * plan->kpad;   // elements of one part
    e = pmlb::launch_filter_relayout_split(filter, dtype, static_cast<float*>(plan->scratch),
                                           static_cast<float*>(plan->scratch) + wts, d.r * d.s, d.c,
                                           static_cast<int>(plan->kpad), d.k, static_cast<cudaStream_t>(stream));
  } else if (plan->s2d) {
    const pmlb::S2dShape g = pmlb::conv_s2d_shape(d);
    e = plan->s2d_pool ? pmlb::launch_filter_s2d_merged(filter, dtype, plan->scratch, d.in_dtype, d.r, d.s, d.c, d.k,
                                                        g.r2, g.s2, g.dh, g.dw, static_cast<cudaStream_t>(stream))
                       : pmlb::launch_filter_s2d(filter, dtype, plan->scratch, d.in_dtype, d.r, d.s, d.c, d.k, g.r2,
                                                 g.s2, g.dh, g.dw, static_cast<cudaStream_t>(stream));
  } else if (plan->packed_rows) {
    e = pmlb::launch_filter_pack_rows(filter, dtype, plan->scratch, d.in_dtype, d.r, d.s, d.c,
                                      pmlb::conv_padded_channels(d), d.k,
                                      static_cast<cudaStream_t>(stream));
  } else {
    e = pmlb::launch_filter_relayout(filter, dtype, plan->scratch, d.in_dtype, d.r * d.s, d.c, d.k,
                                     static_cast<cudaStream_t>(stream));
  }
  if (e != cudaSuccess) return cuda_fail(e, "filter relayout");
  plan->filter_set = true;
  return PMLB_OK;
}

pmlb_status pmlb_conv_invoke(pmlb_plan* plan, void* stream, const void* input, void* output,
                             const void* bias, const void* residual) {
  if (!plan || plan->kind != kPlanConv) return fail(PMLB_ERR_INVALID, "not a conv plan");
  if (!plan->filter_set) return fail(PMLB_ERR_INVALID, "conv: pmlb_conv_set_filter not called");
  if (!input || !output) return fail(PMLB_ERR_INVALID, "conv: null tensor");
  const pmlb_conv_desc& d = plan->conv;
  if ((d.epilogue & PMLB_EPI_BIAS) && !bias) return fail(PMLB_ERR_INVALID, "conv: bias missing");
  if ((d.epilogue & PMLB_EPI_RESIDUAL) && !residual) return fail(PMLB_ERR_INVALID, "conv: residual missing");
  if (plan->s2d) {
    const pmlb::S2dShape sh = pmlb::conv_s2d_shape(d);
    void* packed = static_cast<char*>(plan->scratch) + plan->packed_input_off;
    cudaError_t e = pmlb::launch_s2d_pack(input, packed, d.n, d.h, d.w, d.c, sh.h2, sh.wp, sh.pe_h,
                                          sh.pe_w, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "activation space-to-depth packing");
    if (plan->s2d_pool) {
      pmlb::S2dPoolParams sp = {};
      sp.px = packed;
      sp.wts = plan->scratch;
      sp.bias = (d.epilogue & PMLB_EPI_BIAS) ? static_cast<const float*>(bias) : nullptr;
      sp.out = output;
      sp.status = plan->status;
      sp.tiles_per_img = d.p / 4;
      sp.total_tiles = d.n * sp.tiles_per_img;
      sp.img_px = sh.h2 * sh.wp;
      sp.stage_load = sh.stage_px * 32;
      sp.stage_bytes = (sp.stage_load + 1023) / 1024 * 1024;
      sp.stages = pmlb::s2d_pool_stages(sp.stage_bytes);
      sp.r2 = sh.r2;
      sp.conv_q = d.q;
      sp.pool_p = d.p / 2;
      sp.pool_q = d.q / 2;
      sp.relu = (d.epilogue & PMLB_EPI_RELU) ? 1 : 0;
      sp.wait_limit_us = 0;
      if (sp.stages < 2) return fail(PMLB_ERR_UNSUPPORTED, "conv (space to depth + pool): pixel buffers do not fit");
      int dev = 0, num_sms = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
      const int grid = std::min(num_sms, sp.total_tiles);
      e = pmlb::launch_s2d_pool(sp, grid, d.in_dtype == PMLB_F16, d.out_dtype == PMLB_BF16, static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) return cuda_fail(e, "conv (space to depth + pool)");
      return PMLB_OK;
    }
    pmlb::S2dGeom g;
    g.n = d.n; g.p = d.p; g.q = d.q;
    g.r2 = sh.r2; g.s2 = sh.s2; g.h2 = sh.h2; g.wp = sh.wp; g.stage_px = sh.stage_px;
    pmlb::TcLaunch L;
    L.elem_bytes = 2;
    L.is_f16 = d.in_dtype == PMLB_F16;
    L.m = d.n * d.p * d.q;
    L.n = d.k;
    L.k = sh.r2 * sh.s2 * 16;
    L.batch = 1;
    L.a0 = packed;
    L.b0 = plan->scratch;
    L.s2d = &g;
    L.out = output;
    L.ldc = d.k;
    L.out_dtype = d.out_dtype;
    L.epi_flags = d.epilogue;
    L.bias = bias;
    L.status = plan->status;
    L.trace = g_trace_buffer;
    std::string err;
    const int rc = pmlb::tc_launch(L, static_cast<cudaStream_t>(stream), &err);
    if (rc != 0) return fail(static_cast<pmlb_status>(rc), "conv (space to depth): " + err);
    return PMLB_OK;
  }
  if (plan->packed_rows) {
    const int cp = pmlb::conv_padded_channels(d);
    const int wp = pmlb::conv_packed_row_width(d);
    void* padded = static_cast<char*>(plan->scratch) + plan->packed_input_off;
    cudaError_t e = pmlb::launch_pack_rows(input, padded, d.n, d.h, d.w, d.c, wp, cp, d.pad_w,
                                           static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "activation row packing");
    pmlb::WinGeom g;
    g.n = d.n; g.h = d.h; g.wp = wp; g.cp = cp;
    g.r = d.r; g.s = d.s; g.p = d.p; g.q = d.q;
    g.stride_h = d.stride_h; g.stride_w = d.stride_w;
    g.pad_h = d.pad_h;
    pmlb::TcLaunch L;
    L.elem_bytes = 2;
    L.is_f16 = d.in_dtype == PMLB_F16;
    L.m = d.q;
    L.n = d.k;
    L.k = d.r * 64;
    L.batch = d.n * d.p;
    L.a0 = padded;
    L.b0 = plan->scratch;
    L.window = &g;
    L.out = output;
    L.ldc = d.k;
    L.out_batch_stride = static_cast<long long>(d.q) * d.k;
    L.out_dtype = d.out_dtype;
    L.epi_flags = d.epilogue;
    L.bias = bias;
    L.residual = residual;
    L.ldr = d.k;
    L.res_batch_stride = static_cast<long long>(d.q) * d.k;
    L.status = plan->status;
    L.trace = g_trace_buffer;
    std::string err;
    const int rc = pmlb::tc_launch(L, static_cast<cudaStream_t>(stream), &err);
    if (rc != 0) return fail(static_cast<pmlb_status>(rc), "conv (packed rows): " + err);
    return PMLB_OK;
  }
  pmlb::ConvGeom g;
  g.n = d.n; g.h = d.h; g.w = d.w; g.c = d.c;
  g.r = d.r; g.s = d.s; g.p = d.p; g.q = d.q;
  g.stride_h = d.stride_h; g.stride_w = d.stride_w;
  g.pad_h = d.pad_h; g.pad_w = d.pad_w;
  g.dil_h = d.dil_h; g.dil_w = d.dil_w;
  pmlb::TcLaunch L;
  L.elem_bytes = 2;
  L.is_f16 = d.in_dtype == PMLB_F16;
  L.m = d.n * d.p * d.q;
  L.n = d.k;
  L.k = d.r * d.s * d.c;
  L.batch = 1;
  L.a0 = input;
  L.b0 = plan->scratch;
  if (plan->split) {
    // the activation's high and low TF32 parts, one image per z block of the pre-pass, channels padded
    const int cp = static_cast<int>(plan->kpad);
    const size_t wts = static_cast<size_t>(d.k) * d.r * d.s * cp;
    const size_t act = (static_cast<size_t>(d.n) * d.h * d.w * cp * 4 + 255) / 256 * 256;
    float* x_hi = reinterpret_cast<float*>(static_cast<char*>(plan->scratch) + plan->packed_input_off);
    float* x_lo = reinterpret_cast<float*>(static_cast<char*>(plan->scratch) + plan->packed_input_off + act);
    const long long img = static_cast<long long>(d.h) * d.w;
    for (int n0 = 0; n0 < d.n; n0 += 32768) {
      const int nb = d.n - n0 < 32768 ? d.n - n0 : 32768;
      cudaError_t e = pmlb::launch_split_tf32(static_cast<const float*>(input) + n0 * img * d.c, d.c, img * d.c,
                                              x_hi + n0 * img * cp, x_lo + n0 * img * cp, cp, img * cp, static_cast<int>(img),
                                              d.c, nb, false, static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) return cuda_fail(e, "split(activation)");
    }
    g.c = cp;
    L.elem_bytes = 4;
    L.nsplit = 2;
    L.k = d.r * d.s * cp;
    L.a0 = x_hi;
    L.a1 = x_lo;
    L.b0 = plan->scratch;
    L.b1 = static_cast<float*>(plan->scratch) + wts;
  }
  pmlb::HaloGeom hg;
  if (plan->halo) {
    hg.conv = g;
    L.halo = &hg;
  } else {
    L.conv = &g;
  }
  L.out = output;
  L.ldc = d.k;
  L.out_dtype = d.out_dtype;
  L.epi_flags = d.epilogue;
  L.bias = bias;
  L.residual = residual;
  L.ldr = d.k;
  L.status = plan->status;
  L.bn_override = d.tile_n;
  if (d.flags & PMLB_CONV_CTA_PAIRS) L.pair_override = 1;
  if (d.flags & PMLB_CONV_NO_CTA_PAIRS) L.pair_override = 0;
  if (d.flags & PMLB_CONV_NO_COLUMN_MERGE) L.halo_merge_columns = 0;
  L.trace = g_trace_buffer;
  std::string err;
  const int rc = pmlb::tc_launch(L, static_cast<cudaStream_t>(stream), &err);
  if (rc != 0) return fail(static_cast<pmlb_status>(rc), "conv: " + err);
  return PMLB_OK;
}

// ------------------------------------------------------------------ reductions

pmlb_status pmlb_reduce_dispatch(const pmlb_reduce_desc* d, pmlb_plan** out) {
  if (!d || !out) return fail(PMLB_ERR_INVALID, "null argument");
  *out = nullptr;
  std::string why;
  if (!have_sm100(&why)) return fail(PMLB_ERR_UNSUPPORTED, why);
  if (d->outer < 0 || d->reduce < 0 || d->inner <= 0) return fail(PMLB_ERR_INVALID, "reduce: bad extents");
  if (!pmlb::reduce_supported(d->agg, d->dtype, d->out_dtype)) {
    return fail(PMLB_ERR_UNSUPPORTED, "reduce: aggregation / type combination not covered");
  }
  pmlb_plan* plan = new (std::nothrow) pmlb_plan();
  if (!plan) return fail(PMLB_ERR_INVALID, "out of host memory");
  plan->kind = kPlanReduce;
  plan->kind_name = d->inner == 1 ? "row_reduce" : "strided_reduce";
  plan->reduce = *d;
  cudaGetDevice(&plan->device);
  *out = plan;
  return PMLB_OK;
}

pmlb_status pmlb_reduce_invoke(pmlb_plan* plan, void* stream, const void* in, void* outp) {
  if (!plan || plan->kind != kPlanReduce) return fail(PMLB_ERR_INVALID, "not a reduce plan");
  if (!in || !outp) return fail(PMLB_ERR_INVALID, "reduce: null tensor");
  const pmlb_reduce_desc& d = plan->reduce;
  float scale = d.scale == 0.0 ? 1.f : static_cast<float>(d.scale);
  if (d.divide != 0) {
    if (!(scale > 0.f)) return fail(PMLB_ERR_INVALID, "reduce: a divisor must be positive");
    scale = -scale;   // (the kernels' encoding of a divisor)
  }
  cudaError_t e = pmlb::launch_reduce(d.agg, d.dtype, d.out_dtype, in, outp, d.outer, d.reduce,
                                      d.inner, scale, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "reduce launch");
  return PMLB_OK;
}

pmlb_status pmlb_pool_dispatch(const pmlb_pool_desc* d, pmlb_plan** out) {
  if (!d || !out) return fail(PMLB_ERR_INVALID, "null argument");
  *out = nullptr;
  std::string why;
  if (!have_sm100(&why)) return fail(PMLB_ERR_UNSUPPORTED, why);
  if (!pmlb::pool_supported(d->agg, d->dtype)) {
    return fail(PMLB_ERR_UNSUPPORTED, "pool: aggregation / type combination not covered");
  }
  if (d->n <= 0 || d->h <= 0 || d->w <= 0 || d->c <= 0 || d->r <= 0 || d->s <= 0 || d->p <= 0 ||
      d->q <= 0 || d->stride_h <= 0 || d->stride_w <= 0) {
    return fail(PMLB_ERR_INVALID, "pool: bad geometry");
  }
  pmlb_plan* plan = new (std::nothrow) pmlb_plan();
  if (!plan) return fail(PMLB_ERR_INVALID, "out of host memory");
  plan->kind = kPlanPool;
  plan->kind_name = "nhwc_pool";
  plan->pool = *d;
  cudaGetDevice(&plan->device);
  *out = plan;
  return PMLB_OK;
}

pmlb_status pmlb_pool_invoke(pmlb_plan* plan, void* stream, const void* in, void* outp) {
  if (!plan || plan->kind != kPlanPool) return fail(PMLB_ERR_INVALID, "not a pool plan");
  if (!in || !outp) return fail(PMLB_ERR_INVALID, "pool: null tensor");
  const pmlb_pool_desc& d = plan->pool;
  pmlb::PoolGeom g;
  g.agg = d.agg;
  g.n = d.n; g.h = d.h; g.w = d.w; g.c = d.c;
  g.r = d.r; g.s = d.s; g.p = d.p; g.q = d.q;
  g.stride_h = d.stride_h; g.stride_w = d.stride_w;
  g.pad_h = d.pad_h; g.pad_w = d.pad_w;
  g.average = d.average;
  g.include_padding = d.include_padding;
  cudaError_t e = pmlb::launch_pool(g, d.dtype, in, outp, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "pool launch");
  return PMLB_OK;
}

// ------------------------------------------------------------------ general contraction

pmlb_status pmlb_contract_dispatch(const pmlb_contract_desc* d, pmlb_plan** out) {
  if (!d || !out) return fail(PMLB_ERR_INVALID, "null argument");
  *out = nullptr;
  std::string why;
  if (!have_sm100(&why)) return fail(PMLB_ERR_UNSUPPORTED, why);
  if (d->n_idx < 0 || d->n_idx > PMLB_MAX_IDX || d->n_src < 1 || d->n_src > 3 || d->n_cons < 0 ||
      d->n_cons > PMLB_MAX_CONS || d->out.rank < 0 || d->out.rank > PMLB_MAX_RANK) {
    return fail(PMLB_ERR_INVALID, "contract: descriptor counts out of range");
  }
  const int need_src = d->combo == PMLB_COMBO_NONE ? 1 : (d->combo == PMLB_COMBO_COND ? 3 : 2);
  if (d->n_src != need_src) return fail(PMLB_ERR_INVALID, "contract: operand count does not match the combination");
  if (pmlb::dtype_class(d->out.dtype) < 0) return fail(PMLB_ERR_INVALID, "contract: bad output type");
  for (int s = 0; s < d->n_src; ++s) {
    if (d->src[s].rank < 0 || d->src[s].rank > PMLB_MAX_RANK || pmlb::dtype_class(d->src[s].dtype) < 0) {
      return fail(PMLB_ERR_INVALID, "contract: bad operand");
    }
  }
  pmlb_plan* plan = new (std::nothrow) pmlb_plan();
  if (!plan) return fail(PMLB_ERR_INVALID, "out of host memory");
  plan->kind = kPlanContract;
  plan->kind_name = "generic_contract";
  pmlb::GenericParams& p = plan->generic;
  std::memset(&p, 0, sizeof(p));
  p.agg = d->agg;
  p.combo = d->combo;
  p.n_idx = d->n_idx;
  p.n_src = d->n_src;
  p.n_cons = d->n_cons;
  p.has_init = d->has_init;
  for (int i = 0; i < d->n_idx; ++i) p.range[i] = d->range[i];
  copy_access(d->out, &p.out, d->n_idx);
  for (int s = 0; s < d->n_src; ++s) copy_access(d->src[s], &p.src[s], d->n_idx);
  if (d->has_init) {
    copy_access(d->init, &p.init, 0);
    p.init.rank = d->out.rank;
  }
  for (int c = 0; c < d->n_cons; ++c) {
    for (int i = 0; i < d->n_idx; ++i) p.cons_coef[c][i] = d->cons_coef[c][i];
    p.cons_off[c] = d->cons_off[c];
    p.cons_range[c] = d->cons_range[c];
  }
  long long elems = 1;
  for (int dd = 0; dd < d->out.rank; ++dd) elems *= d->out.sizes[dd];
  p.out_elems = elems;
  // direct mode: each output dim is exactly one distinct index variable
  bool direct = true;
  bool used[PMLB_MAX_IDX] = {false};
  for (int dd = 0; dd < d->out.rank && direct; ++dd) {
    int var = -1;
    for (int i = 0; i < d->n_idx; ++i) {
      if (d->out.coef[dd][i] != 0) {
        if (var >= 0 || d->out.coef[dd][i] != 1) direct = false;
        var = i;
      }
    }
    if (var < 0 || p.out.den[dd] != 1 || used[var]) direct = false;
    if (direct) {
      used[var] = true;
      p.out_var[dd] = var;
    }
  }
  p.direct = direct ? 1 : 0;
  p.n_loop = 0;
  p.n_solve = 0;
  bool solvable = !direct;
  for (int dd = 0; dd < d->out.rank; ++dd) {
    if (p.out.den[dd] != 1) solvable = false;
  }
  if (solvable) {
    // Output dims that mix variables (a transposed convolution's `s*x + i - pad`, a resize's `f*y + j`): per
    // dim, the not yet fixed variable of the widest range is solved for from the element's coordinate and the
    // others are iterated over, so a thread visits the taps of its element instead of the whole index box.
    bool fixed[PMLB_MAX_IDX] = {false};
    for (int dd = 0; dd < d->out.rank; ++dd) {
      int pivot = -1;
      for (int i = 0; i < d->n_idx; ++i) {
        if (d->out.coef[dd][i] == 0 || fixed[i]) continue;
        if (pivot < 0 || d->range[i] > d->range[pivot]) pivot = i;
      }
      if (pivot < 0) continue;
      for (int i = 0; i < d->n_idx; ++i) {
        if (d->out.coef[dd][i] == 0 || fixed[i] || i == pivot) continue;
        fixed[i] = true;
        p.loop_var[p.n_loop++] = i;
      }
      fixed[pivot] = true;
      p.solve_dim[p.n_solve] = dd;
      p.solve_var[p.n_solve] = pivot;
      ++p.n_solve;
    }
    for (int i = 0; i < d->n_idx; ++i) {
      if (!fixed[i]) p.loop_var[p.n_loop++] = i;
    }
  } else {
    for (int i = 0; i < d->n_idx; ++i) {
      if (!direct || !used[i]) p.loop_var[p.n_loop++] = i;
    }
  }
  cudaGetDevice(&plan->device);
  *out = plan;
  return PMLB_OK;
}

pmlb_status pmlb_contract_invoke(pmlb_plan* plan, void* stream, const void* src0, const void* src1,
                                 const void* src2, const void* init, void* outp) {
  if (!plan || plan->kind != kPlanContract) return fail(PMLB_ERR_INVALID, "not a contraction plan");
  pmlb::GenericParams p = plan->generic;
  p.srcp[0] = src0;
  p.srcp[1] = src1;
  p.srcp[2] = src2;
  p.initp = init;
  p.outp = outp;
  if (!outp || !src0 || (p.n_src > 1 && !src1) || (p.n_src > 2 && !src2) || (p.has_init && !init)) {
    return fail(PMLB_ERR_INVALID, "contract: null tensor");
  }
  cudaError_t e = pmlb::launch_contract(p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "contract launch");
  return PMLB_OK;
}

// ------------------------------------------------------------------ element-wise

pmlb_status pmlb_eltwise_dispatch(const pmlb_eltwise_desc* d, pmlb_plan** out) {
  if (!d || !out) return fail(PMLB_ERR_INVALID, "null argument");
  *out = nullptr;
  std::string why;
  if (!have_sm100(&why)) return fail(PMLB_ERR_UNSUPPORTED, why);
  char name[25];
  std::memcpy(name, d->op, 24);
  name[24] = 0;
  const int op = ew_opcode(name);
  if (op < 0) return fail(PMLB_ERR_UNSUPPORTED, std::string("eltwise: unknown operation '") + name + "'");
  if (d->n_in < 1 || d->n_in > 3 || d->rank < 0 || d->rank > PMLB_MAX_RANK) {
    return fail(PMLB_ERR_INVALID, "eltwise: descriptor counts out of range");
  }
  if (pmlb::dtype_class(d->out_dtype) < 0) return fail(PMLB_ERR_INVALID, "eltwise: bad output type");
  pmlb_plan* plan = new (std::nothrow) pmlb_plan();
  if (!plan) return fail(PMLB_ERR_INVALID, "out of host memory");
  plan->kind = kPlanEltwise;
  plan->kind_name = "eltwise";
  pmlb::EltwiseParams& p = plan->eltwise;
  std::memset(&p, 0, sizeof(p));
  p.op = op;
  p.n_in = d->n_in;
  p.rank = d->rank;
  p.out_dtype = d->out_dtype;
  long long elems = 1;
  for (int i = 0; i < d->rank; ++i) {
    p.sizes[i] = d->sizes[i];
    elems *= d->sizes[i];
    for (int s = 0; s < 3; ++s) p.in_strides[s][i] = d->in_strides[s][i];
  }
  p.elems = elems;
  bool any_float = false, all_unsigned = true, any_f64 = false;
  for (int s = 0; s < d->n_in; ++s) {
    p.in_dtype[s] = d->in_dtype[s];
    const int cls = pmlb::dtype_class(d->in_dtype[s]);
    if (cls < 0) {
      delete plan;
      return fail(PMLB_ERR_INVALID, "eltwise: bad operand type");
    }
    if (cls == pmlb::kClassF32 || cls == pmlb::kClassF64) any_float = true;
    if (cls == pmlb::kClassF64) any_f64 = true;
    if (cls != pmlb::kClassU64) all_unsigned = false;
  }
  (void)any_f64;
  const bool is_cast = std::strcmp(name, "cast") == 0 || std::strcmp(name, "ident") == 0 ||
                       std::strcmp(name, "assign") == 0;
  if (is_compare(op)) {
    // compare in a class wide enough for every operand; the result is 0 / 1
    p.compute_class = any_float ? pmlb::kClassF64 : (all_unsigned ? pmlb::kClassU64 : pmlb::kClassI64);
    p.arith_dtype = any_float ? PMLB_F64 : (all_unsigned ? PMLB_U64 : PMLB_I64);
    p.narrow_inputs = 0;
    p.narrow_result = 0;
  } else if (is_cast) {
    p.compute_class = pmlb::dtype_class(d->out_dtype);
    if (d->out_dtype == PMLB_BOOL && any_float) p.compute_class = pmlb::kClassF64;
    p.arith_dtype = d->out_dtype;
    p.narrow_inputs = 0;
    p.narrow_result = 0;
  } else {
    p.compute_class = pmlb::dtype_class(d->out_dtype);
    p.arith_dtype = d->out_dtype;
    p.narrow_inputs = 1;
    p.narrow_result = 1;
  }
  cudaGetDevice(&plan->device);
  *out = plan;
  return PMLB_OK;
}

pmlb_status pmlb_eltwise_invoke(pmlb_plan* plan, void* stream, const void* in0, const void* in1,
                                const void* in2, void* outp) {
  if (!plan || plan->kind != kPlanEltwise) return fail(PMLB_ERR_INVALID, "not an eltwise plan");
  pmlb::EltwiseParams p = plan->eltwise;
  p.in[0] = in0;
  p.in[1] = in1;
  p.in[2] = in2;
  p.out = outp;
  if (!outp || !in0 || (p.n_in > 1 && !in1) || (p.n_in > 2 && !in2)) {
    return fail(PMLB_ERR_INVALID, "eltwise: null tensor");
  }
  cudaError_t e = pmlb::launch_eltwise(p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "eltwise launch");
  return PMLB_OK;
}

// ------------------------------------------------------------------ gather / scatter / argsort / prng

namespace {

int special_elem_bytes(int dtype) {
  switch (dtype) {
    case PMLB_BOOL:
    case PMLB_I8:
    case PMLB_U8: return 1;
    case PMLB_I16:
    case PMLB_U16:
    case PMLB_F16:
    case PMLB_BF16: return 2;
    case PMLB_I32:
    case PMLB_U32:
    case PMLB_F32: return 4;
    case PMLB_I64:
    case PMLB_U64:
    case PMLB_F64: return 8;
    default: return 0;
  }
}

bool special_is_float(int dtype) {
  return dtype == PMLB_F16 || dtype == PMLB_BF16 || dtype == PMLB_F32 || dtype == PMLB_F64;
}

long long product(const int64_t* v, int from, int to) {
  long long r = 1;
  for (int i = from; i < to; ++i) r *= v[i];
  return r;
}

// Empty string if the descriptor is consistent, else what is wrong with it.
std::string special_problem(const pmlb_special_desc* d) {
  auto ranks_ok = [](int r) { return r >= 0 && r <= PMLB_MAX_RANK; };
  if (!ranks_ok(d->rank) || !ranks_ok(d->idx_rank) || !ranks_ok(d->upd_rank)) return "rank out of range";
  for (int i = 0; i < d->rank; ++i) {
    if (d->sizes[i] < 0) return "negative size";
  }
  switch (d->op) {
    case PMLB_SPECIAL_GATHER: {
      if (special_elem_bytes(d->dtype) == 0 || special_elem_bytes(d->idx_dtype) == 0) return "gather: bad element type";
      if (d->rank < 1) return "gather: the tensor needs at least one dimension";
      if (d->mode == 0) {
        if (d->axis < 0 || d->axis >= d->rank) return "gather: axis outside the tensor's dimensions";
        if (special_is_float(d->idx_dtype) && special_is_float(d->dtype)) {
          if (d->interpolation < 0 || d->interpolation > 2) return "gather: float indices need an interpolation mode";
          if (d->interpolation == 0 && (d->nearest < 0 || d->nearest > 4)) return "gather: unknown rounding rule";
        }
        if (d->out_of_bounds < 0 || d->out_of_bounds > 1) return "gather: unknown out-of-bounds rule";
        return "";
      }
      if (d->mode != 1) return "gather: unknown mode";
      if (special_is_float(d->idx_dtype)) return "gather: nd mode requires indices elements to be integers";
      if (d->idx_rank < 1) return "gather: nd mode needs indices of at least one dimension";
      const long long k = d->idx_sizes[d->idx_rank - 1];
      if (d->batch_dims < 0 || d->batch_dims > d->idx_rank - 1 || k < 0 || k + d->batch_dims > d->rank) {
        return "gather: indices address more dimensions than the tensor has";
      }
      for (int i = 0; i < d->batch_dims; ++i) {
        if (d->idx_sizes[i] != d->sizes[i]) return "gather: batch dimensions of tensor and indices differ";
      }
      return "";
    }
    case PMLB_SPECIAL_SCATTER: {
      if (special_elem_bytes(d->dtype) == 0) return "scatter: bad element type";
      if (d->idx_dtype != PMLB_I32 && d->idx_dtype != PMLB_U32) return "scatter: indices must be 32-bit integers";
      if (d->rank < 1 || d->idx_rank < 1) return "scatter: data and indices need at least one dimension";
      if (d->mode < 0 || d->mode > 3) return "scatter: unknown mode";
      int dst_rank;
      if (d->mode == 3) {
        if (d->upd_rank < d->idx_rank - 1) return "scatter: updates have fewer dimensions than the indices address";
        dst_rank = static_cast<int>(d->idx_sizes[d->idx_rank - 1]) + d->upd_rank - (d->idx_rank - 1);
        for (int i = 0; i < d->idx_rank - 1; ++i) {
          if (d->upd_sizes[i] > d->idx_sizes[i]) return "scatter: updates run past the indices";
        }
      } else {
        if (d->axis < 0 || d->axis >= d->rank) return "scatter: axis outside the data's dimensions";
        const int first = d->mode == 1 ? d->axis : 0;
        if (first + d->idx_rank > d->upd_rank) return "scatter: updates have fewer dimensions than the indices";
        for (int i = 0; i < d->idx_rank; ++i) {
          if (d->upd_sizes[first + i] > d->idx_sizes[i]) return "scatter: updates run past the indices";
        }
        dst_rank = d->mode == 1 ? d->upd_rank - d->idx_rank + 1 : d->upd_rank;
      }
      if (dst_rank != d->rank) return "scatter: updates and indices do not address the data's dimensions";
      return "";
    }
    case PMLB_SPECIAL_ARGSORT: {
      if (special_elem_bytes(d->dtype) == 0) return "argsort: bad element type";
      if (d->rank < 1 || d->axis < 0 || d->axis >= d->rank) return "argsort: axis outside the tensor's dimensions";
      if (d->mode < 0 || d->mode > 1) return "argsort: unknown direction";
      if (d->sizes[d->axis] > 2147483647LL) return "argsort: positions do not fit 32 bits";
      return "";
    }
    case PMLB_SPECIAL_PRNG: {
      if (d->state_elems < 3) return "prng: the state needs three words";
      if (product(d->sizes, 0, d->rank) >= (1LL << 32)) return "prng: more than 2^32 elements";
      return "";
    }
    default: return "unknown operation";
  }
}

}  // namespace

int64_t pmlb_special_out_elems(const pmlb_special_desc* d) {
  if (!d || !special_problem(d).empty()) return 0;
  switch (d->op) {
    case PMLB_SPECIAL_GATHER:
      if (d->mode == 0) {
        return product(d->sizes, 0, d->axis) * product(d->idx_sizes, 0, d->idx_rank) *
               product(d->sizes, d->axis + 1, d->rank);
      }
      return product(d->idx_sizes, 0, d->idx_rank - 1) *
             product(d->sizes, static_cast<int>(d->idx_sizes[d->idx_rank - 1]) + d->batch_dims, d->rank);
    default: return product(d->sizes, 0, d->rank);
  }
}

pmlb_status pmlb_special_dispatch(const pmlb_special_desc* d, pmlb_plan** out) {
  if (!d || !out) return fail(PMLB_ERR_INVALID, "null argument");
  *out = nullptr;
  std::string why;
  if (!have_sm100(&why)) return fail(PMLB_ERR_UNSUPPORTED, why);
  const std::string problem = special_problem(d);
  if (!problem.empty()) return fail(PMLB_ERR_INVALID, problem);
  pmlb_plan* plan = new (std::nothrow) pmlb_plan();
  if (!plan) return fail(PMLB_ERR_INVALID, "out of host memory");
  plan->kind = kPlanSpecial;
  static const char* const names[] = {"gather", "scatter", "argsort", "prng"};
  plan->kind_name = names[d->op];
  plan->special = *d;
  size_t scratch = 0;
  if (d->op == PMLB_SPECIAL_ARGSORT) scratch = static_cast<size_t>(product(d->sizes, 0, d->rank)) * sizeof(int32_t);
  if (d->op == PMLB_SPECIAL_PRNG) scratch = pmlb::kPrngTableWords * sizeof(uint32_t);
  pmlb_status st = alloc_plan_memory(plan, scratch, false);
  if (st == PMLB_OK && d->op == PMLB_SPECIAL_PRNG) {
    static uint32_t table[pmlb::kPrngTableWords];
    static const bool filled = (pmlb::prng_jump_table(table), true);
    (void)filled;
    cudaError_t e = cudaMemcpy(plan->scratch, table, sizeof(table), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) st = cuda_fail(e, "cudaMemcpy(prng table)");
  }
  if (st != PMLB_OK) {
    pmlb_plan_free(plan);
    return st;
  }
  *out = plan;
  return PMLB_OK;
}

pmlb_status pmlb_special_invoke(pmlb_plan* plan, void* stream_, const void* in0, const void* in1, const void* in2,
                                void* out0, void* out1) {
  if (!plan || plan->kind != kPlanSpecial) return fail(PMLB_ERR_INVALID, "not a gather / scatter / argsort / prng plan");
  const pmlb_special_desc& d = plan->special;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaSuccess;
  switch (d.op) {
    case PMLB_SPECIAL_GATHER: {
      if (!in0 || !in1 || !out0) return fail(PMLB_ERR_INVALID, "gather: null tensor");
      pmlb::GatherParams p{};
      p.dtype = d.dtype;
      p.idx_dtype = d.idx_dtype;
      p.elem_bytes = special_elem_bytes(d.dtype);
      p.nd = d.mode;
      p.out_elems = pmlb_special_out_elems(&d);
      p.interpolation = d.interpolation;
      p.nearest = d.nearest;
      p.out_of_bounds = d.out_of_bounds;
      p.cube_coeff = d.cube_coeff;
      if (d.mode == 0) {
        p.axis_len = d.sizes[d.axis];
        p.inner = product(d.sizes, d.axis + 1, d.rank);
        p.n_idx = product(d.idx_sizes, 0, d.idx_rank);
        if (p.axis_len == 0 && p.out_elems > 0) return fail(PMLB_ERR_INVALID, "gather: nothing to gather from");
      } else {
        p.k = static_cast<int>(d.idx_sizes[d.idx_rank - 1]);
        for (int i = 0; i < p.k; ++i) {
          p.dims[i] = d.sizes[d.batch_dims + i];
          if (p.dims[i] == 0 && p.out_elems > 0) return fail(PMLB_ERR_INVALID, "gather: nothing to gather from");
        }
        p.inner = product(d.sizes, d.batch_dims + p.k, d.rank);
        p.rows_per_batch = product(d.idx_sizes, d.batch_dims, d.idx_rank - 1);
      }
      p.tensor = in0;
      p.indices = in1;
      p.out = out0;
      e = pmlb::launch_gather(p, stream);
      break;
    }
    case PMLB_SPECIAL_SCATTER: {
      if (!in0 || !in1 || !in2 || !out0) return fail(PMLB_ERR_INVALID, "scatter: null tensor");
      pmlb::ScatterParams p{};
      p.dtype = d.dtype;
      p.idx_dtype = d.idx_dtype;
      p.elem_bytes = special_elem_bytes(d.dtype);
      p.mode = d.mode;
      p.axis = d.axis;
      p.rank = d.rank;
      p.idx_rank = d.idx_rank;
      p.upd_rank = d.upd_rank;
      for (int i = 0; i < PMLB_MAX_RANK; ++i) {
        p.sizes[i] = d.sizes[i];
        p.idx_sizes[i] = d.idx_sizes[i];
        p.upd_sizes[i] = d.upd_sizes[i];
      }
      p.upd_elems = product(d.upd_sizes, 0, d.upd_rank);
      p.indices = in1;
      p.updates = in2;
      p.out = out0;
      const size_t bytes = static_cast<size_t>(product(d.sizes, 0, d.rank)) * p.elem_bytes;
      if (bytes > 0 && out0 != in0) {
        e = cudaMemcpyAsync(out0, in0, bytes, cudaMemcpyDeviceToDevice, stream);
        if (e != cudaSuccess) return cuda_fail(e, "scatter copy");
      }
      e = pmlb::launch_scatter(p, stream);
      break;
    }
    case PMLB_SPECIAL_ARGSORT: {
      if (!in0 || !out0) return fail(PMLB_ERR_INVALID, "argsort: null tensor");
      pmlb::ArgsortParams p{};
      p.dtype = d.dtype;
      p.descending = d.mode;
      p.outer = product(d.sizes, 0, d.axis);
      p.n = d.sizes[d.axis];
      p.inner = product(d.sizes, d.axis + 1, d.rank);
      p.tensor = in0;
      e = pmlb::launch_argsort(p, static_cast<int32_t*>(out0), static_cast<int32_t*>(plan->scratch), stream);
      break;
    }
    default: {
      // either result may be left out: the numbers alone, or only the state after them
      if (!in0 || (!out0 && !out1)) return fail(PMLB_ERR_INVALID, "prng: null tensor");
      e = pmlb::launch_prng(static_cast<const uint32_t*>(in0), d.state_elems, static_cast<float*>(out0),
                            product(d.sizes, 0, d.rank), static_cast<uint32_t*>(out1),
                            static_cast<const uint32_t*>(plan->scratch), stream);
      break;
    }
  }
  if (e != cudaSuccess) return cuda_fail(e, "gather / scatter / argsort / prng launch");
  return PMLB_OK;
}

}  // extern "C"
