/*
 * tile_oracle.c -- CPU restatement of PlaidML's Tile contraction semantics.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA kernels: tests, the
 * smoke test and the bench's CPU-baseline leg call it; nothing under plaidml_b200/ links,
 * loads or imports it.
 *
 * What it restates (paths inside the plaidml/plaidml repository, branch plaidml-v1):
 *   - the meaning of a contraction: every integer point of the index box contributes
 *     iff all tensor accesses are in range, all constraints hold and all index expressions
 *     are integral (docs/usage/edsl_ops.rst:19-66; pmlc/dialect/tile/transforms/
 *     contraction.cc:229-260,657-681);
 *   - the arithmetic: combination then aggregation in the result element type, integers
 *     wrapping, max/min as `cmp(acc, v) ? acc : v` with ordered / signed / unsigned compares
 *     (pmlc/conversion/tile_to_linalg/tile_to_linalg.cc:485-544, 681-861);
 *   - initial values: the init tensor broadcast to the output, else the aggregation's
 *     identity (pmlc/ast/builder.cc:366-401, pmlc/dialect/tile/ir/util.cc:217-274);
 *   - casts between element types (pmlc/conversion/tile_to_linalg/utils.cc:35-91);
 *   - ReLU as select(x < 0, 0, x) (pmlc/conversion/pxa_to_affine/pxa_to_affine.cc:312-332).
 *
 * The loops visit the index box in lexicographic order with the last index fastest and
 * accumulate straight into the output buffer, i.e. the textbook order of the definition,
 * not the order of any GPU kernel.
 *
 * Parity status: pinned against the known-answer vectors the reference's own tests hold
 * for this path (tests/golden/, taken from plaidml/edsl/examples/gemm.cc, plaidml/edsl/
 * tests/edsl_test.cc and edsl_test.py, pmlc/target/x86/tests/xsmm_call.mlir).  The
 * reference itself cannot be built in this environment (its LLVM/MLIR fork and libxsmm are
 * fetched at configure time), so it was never run here.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_MAX_IDX 10
#define ORC_MAX_RANK 8
#define ORC_MAX_CONS 8

enum {
  DT_BOOL = 4, DT_I8 = 5, DT_U8 = 6, DT_I16 = 7, DT_U16 = 8, DT_I32 = 9, DT_U32 = 10,
  DT_I64 = 11, DT_U64 = 12, DT_F16 = 13, DT_F32 = 14, DT_F64 = 15, DT_BF16 = 16
};
enum { AGG_NONE = 0, AGG_SUM, AGG_MAX, AGG_MIN, AGG_PROD, AGG_ASSIGN };
enum { COMBO_NONE = 0, COMBO_MUL, COMBO_ADD, COMBO_EQ, COMBO_COND };

/* Same field layout as pmlb_access / pmlb_contract_desc so that one Python structure
 * drives both the kernel library and this checker. */
typedef struct {
  int32_t dtype;
  int32_t rank;
  int64_t sizes[ORC_MAX_RANK];
  int64_t strides[ORC_MAX_RANK];
  int32_t coef[ORC_MAX_RANK][ORC_MAX_IDX];
  int64_t off[ORC_MAX_RANK];
  int32_t den[ORC_MAX_RANK];
} orc_access;

typedef struct {
  int32_t agg;
  int32_t combo;
  int32_t n_idx;
  int32_t n_src;
  int64_t range[ORC_MAX_IDX];
  orc_access out;
  orc_access src[3];
  int32_t n_cons;
  int32_t has_init;
  int32_t cons_coef[ORC_MAX_CONS][ORC_MAX_IDX];
  int64_t cons_off[ORC_MAX_CONS];
  int64_t cons_range[ORC_MAX_CONS];
  orc_access init;
} orc_contract_desc;

/* ------------------------------------------------------------------ 16-bit floats */

static float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static uint16_t f32_to_bf16(float f) { /* round to nearest even, NaN kept quiet */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static float f16_to_f32(uint16_t h) {
  _Float16 x;
  memcpy(&x, &h, 2);
  return (float)x;
}

static uint16_t f32_to_f16(float f) {
  _Float16 x = (_Float16)f;
  uint16_t h;
  memcpy(&h, &x, 2);
  return h;
}

/* ------------------------------------------------------------------ scalar model
 * A value is carried as one of three machine classes and re-narrowed to the element
 * type after every operation. */
typedef struct {
  int cls; /* 0 = float (f16/bf16/f32 carried in f32), 1 = f64, 2 = integer (64-bit pattern) */
  float f;
  double d;
  uint64_t u;
} val;

static int is_float_dt(int dt) { return dt == DT_F16 || dt == DT_BF16 || dt == DT_F32 || dt == DT_F64; }
static int is_signed_dt(int dt) { return dt == DT_I8 || dt == DT_I16 || dt == DT_I32 || dt == DT_I64; }
static int class_of(int dt) { return dt == DT_F64 ? 1 : (is_float_dt(dt) ? 0 : 2); }

static size_t dt_size(int dt) {
  switch (dt) {
    case DT_BOOL: case DT_I8: case DT_U8: return 1;
    case DT_I16: case DT_U16: case DT_F16: case DT_BF16: return 2;
    case DT_I32: case DT_U32: case DT_F32: return 4;
    default: return 8;
  }
}

/* wrap / round `v` (of class class_of(dt)) to what `dt` can hold */
static val narrow(val v, int dt) {
  switch (dt) {
    case DT_F16: v.f = f16_to_f32(f32_to_f16(v.f)); break;
    case DT_BF16: v.f = bf16_to_f32(f32_to_bf16(v.f)); break;
    case DT_BOOL: v.u = v.u != 0; break;
    case DT_I8: v.u = (uint64_t)(int64_t)(int8_t)v.u; break;
    case DT_U8: v.u = (uint8_t)v.u; break;
    case DT_I16: v.u = (uint64_t)(int64_t)(int16_t)v.u; break;
    case DT_U16: v.u = (uint16_t)v.u; break;
    case DT_I32: v.u = (uint64_t)(int64_t)(int32_t)v.u; break;
    case DT_U32: v.u = (uint32_t)v.u; break;
    default: break;
  }
  return v;
}

/* read element i of a tensor of type `dt`, converted (cast) to the class/type `to` */
static val load_cast(const void* p, int dt, int64_t i, int to) {
  val v;
  memset(&v, 0, sizeof v);
  v.cls = class_of(to);
  double as_d = 0;
  int64_t as_i = 0;
  uint64_t as_u = 0;
  int src_float = is_float_dt(dt);
  switch (dt) {
    case DT_BOOL: case DT_U8: as_u = ((const uint8_t*)p)[i]; break;
    case DT_I8: as_i = ((const int8_t*)p)[i]; break;
    case DT_I16: as_i = ((const int16_t*)p)[i]; break;
    case DT_U16: as_u = ((const uint16_t*)p)[i]; break;
    case DT_I32: as_i = ((const int32_t*)p)[i]; break;
    case DT_U32: as_u = ((const uint32_t*)p)[i]; break;
    case DT_I64: as_i = ((const int64_t*)p)[i]; break;
    case DT_U64: as_u = ((const uint64_t*)p)[i]; break;
    case DT_F16: as_d = f16_to_f32(((const uint16_t*)p)[i]); break;
    case DT_BF16: as_d = bf16_to_f32(((const uint16_t*)p)[i]); break;
    case DT_F32: as_d = ((const float*)p)[i]; break;
    case DT_F64: as_d = ((const double*)p)[i]; break;
    default: break;
  }
  if (src_float) {
    if (v.cls == 0) v.f = (float)as_d;
    else if (v.cls == 1) v.d = as_d;
    else v.u = is_signed_dt(to) ? (uint64_t)(int64_t)as_d : (uint64_t)as_d;
  } else if (is_signed_dt(dt)) {
    if (v.cls == 0) v.f = (float)as_i;
    else if (v.cls == 1) v.d = (double)as_i;
    else v.u = (uint64_t)as_i;
  } else {
    if (v.cls == 0) v.f = (float)as_u;
    else if (v.cls == 1) v.d = (double)as_u;
    else v.u = as_u;
  }
  return narrow(v, to);
}

static void store_val(void* p, int dt, int64_t i, val v) {
  switch (dt) {
    case DT_BOOL: ((uint8_t*)p)[i] = v.u != 0; break;
    case DT_I8: case DT_U8: ((uint8_t*)p)[i] = (uint8_t)v.u; break;
    case DT_I16: case DT_U16: ((uint16_t*)p)[i] = (uint16_t)v.u; break;
    case DT_I32: case DT_U32: ((uint32_t*)p)[i] = (uint32_t)v.u; break;
    case DT_I64: case DT_U64: ((uint64_t*)p)[i] = v.u; break;
    case DT_F16: ((uint16_t*)p)[i] = f32_to_f16(v.f); break;
    case DT_BF16: ((uint16_t*)p)[i] = f32_to_bf16(v.f); break;
    case DT_F32: ((float*)p)[i] = v.f; break;
    case DT_F64: ((double*)p)[i] = v.d; break;
    default: break;
  }
}

static val identity_val(int agg, int dt) {
  val v;
  memset(&v, 0, sizeof v);
  v.cls = class_of(dt);
  if (agg == AGG_PROD) { v.f = 1.f; v.d = 1.0; v.u = 1; }
  if (agg == AGG_MAX) {
    v.f = -INFINITY; v.d = -INFINITY;
    switch (dt) {
      case DT_I8: v.u = (uint64_t)(int64_t)INT8_MIN; break;
      case DT_I16: v.u = (uint64_t)(int64_t)INT16_MIN; break;
      case DT_I32: v.u = (uint64_t)(int64_t)INT32_MIN; break;
      case DT_I64: v.u = (uint64_t)INT64_MIN; break;
      default: v.u = 0; break;
    }
  }
  if (agg == AGG_MIN) {
    v.f = INFINITY; v.d = INFINITY;
    switch (dt) {
      case DT_BOOL: v.u = 1; break;
      case DT_I8: v.u = INT8_MAX; break;
      case DT_U8: v.u = UINT8_MAX; break;
      case DT_I16: v.u = INT16_MAX; break;
      case DT_U16: v.u = UINT16_MAX; break;
      case DT_I32: v.u = INT32_MAX; break;
      case DT_U32: v.u = UINT32_MAX; break;
      case DT_I64: v.u = INT64_MAX; break;
      default: v.u = UINT64_MAX; break;
    }
  }
  return v;
}

static val v_mul(val a, val b, int dt) {
  a.f *= b.f; a.d *= b.d; a.u *= b.u;
  return narrow(a, dt);
}
static val v_add(val a, val b, int dt) {
  a.f += b.f; a.d += b.d; a.u += b.u;
  return narrow(a, dt);
}
static int v_gt(val a, val b, int dt) {
  if (a.cls == 0) return a.f > b.f;
  if (a.cls == 1) return a.d > b.d;
  return is_signed_dt(dt) ? ((int64_t)a.u > (int64_t)b.u) : (a.u > b.u);
}
static int v_lt(val a, val b, int dt) {
  if (a.cls == 0) return a.f < b.f;
  if (a.cls == 1) return a.d < b.d;
  return is_signed_dt(dt) ? ((int64_t)a.u < (int64_t)b.u) : (a.u < b.u);
}

/* T1 == T2 in the wider of the two operand types */
static int src_equal(const void* p0, int dt0, int64_t i0, const void* p1, int dt1, int64_t i1) {
  if (is_float_dt(dt0) || is_float_dt(dt1)) {
    return load_cast(p0, dt0, i0, DT_F64).d == load_cast(p1, dt1, i1, DT_F64).d;
  }
  return load_cast(p0, dt0, i0, DT_I64).u == load_cast(p1, dt1, i1, DT_I64).u;
}

/* ------------------------------------------------------------------ contraction */

static int eval_access(const orc_access* a, int n_idx, const int64_t* x, int64_t* coords) {
  for (int d = 0; d < a->rank; ++d) {
    int64_t num = a->off[d];
    for (int i = 0; i < n_idx; ++i) num += (int64_t)a->coef[d][i] * x[i];
    int den = a->den[d] >= 1 ? a->den[d] : 1;
    if (num % den != 0) return 0;
    int64_t c = num / den;
    if (c < 0 || c >= a->sizes[d]) return 0;
    coords[d] = c;
  }
  return 1;
}

static int64_t flat(const orc_access* a, const int64_t* coords) {
  int64_t o = 0;
  for (int d = 0; d < a->rank; ++d) o += coords[d] * a->strides[d];
  return o;
}

int orc_contract(const orc_contract_desc* d, const void* s0, const void* s1, const void* s2,
                 const void* init, void* out) {
  const void* sp[3] = {s0, s1, s2};
  const int odt = d->out.dtype;
  /* 1. initial value of every output element */
  int64_t oc[ORC_MAX_RANK] = {0};
  int64_t total = 1;
  for (int k = 0; k < d->out.rank; ++k) total *= d->out.sizes[k];
  for (int64_t e = 0; e < total; ++e) {
    int64_t rem = e, ioff = 0;
    for (int k = d->out.rank - 1; k >= 0; --k) {
      oc[k] = rem % d->out.sizes[k];
      rem /= d->out.sizes[k];
      ioff += oc[k] * d->init.strides[k];
    }
    val v = d->has_init ? load_cast(init, d->init.dtype, ioff, odt) : identity_val(d->agg, odt);
    store_val(out, odt, flat(&d->out, oc), v);
  }
  /* 2. visit the index box */
  for (int i = 0; i < d->n_idx; ++i) {
    if (d->range[i] <= 0) return 0;
  }
  int64_t x[ORC_MAX_IDX] = {0};
  for (;;) {
    int ok = 1;
    int64_t co[ORC_MAX_RANK], cs[3][ORC_MAX_RANK];
    for (int c = 0; c < d->n_cons && ok; ++c) {
      int64_t v = d->cons_off[c];
      for (int i = 0; i < d->n_idx; ++i) v += (int64_t)d->cons_coef[c][i] * x[i];
      if (v < 0 || v >= d->cons_range[c]) ok = 0;
    }
    if (ok) ok = eval_access(&d->out, d->n_idx, x, co);
    for (int s = 0; s < d->n_src && ok; ++s) ok = eval_access(&d->src[s], d->n_idx, x, cs[s]);
    if (ok) {
      int64_t so[3] = {0, 0, 0};
      for (int s = 0; s < d->n_src; ++s) so[s] = flat(&d->src[s], cs[s]);
      val v;
      switch (d->combo) {
        case COMBO_MUL:
          v = v_mul(load_cast(sp[0], d->src[0].dtype, so[0], odt),
                    load_cast(sp[1], d->src[1].dtype, so[1], odt), odt);
          break;
        case COMBO_ADD:
          v = v_add(load_cast(sp[0], d->src[0].dtype, so[0], odt),
                    load_cast(sp[1], d->src[1].dtype, so[1], odt), odt);
          break;
        case COMBO_EQ:
          memset(&v, 0, sizeof v);
          v.cls = class_of(odt);
          if (src_equal(sp[0], d->src[0].dtype, so[0], sp[1], d->src[1].dtype, so[1])) {
            v.f = 1.f; v.d = 1.0; v.u = 1;
          }
          break;
        case COMBO_COND:
          if (src_equal(sp[0], d->src[0].dtype, so[0], sp[1], d->src[1].dtype, so[1])) {
            v = load_cast(sp[2], d->src[2].dtype, so[2], odt);
          } else {
            memset(&v, 0, sizeof v);
            v.cls = class_of(odt);
          }
          break;
        default:
          v = load_cast(sp[0], d->src[0].dtype, so[0], odt);
          break;
      }
      const int64_t oo = flat(&d->out, co);
      val acc = load_cast(out, odt, oo, odt);
      switch (d->agg) {
        case AGG_SUM: acc = v_add(acc, v, odt); break;
        case AGG_PROD: acc = v_mul(acc, v, odt); break;
        case AGG_MAX: acc = v_gt(acc, v, odt) ? acc : v; break;
        case AGG_MIN: acc = v_lt(acc, v, odt) ? acc : v; break;
        default: acc = v; break;
      }
      store_val(out, odt, oo, acc);
    }
    int j = d->n_idx - 1;
    while (j >= 0) {
      if (++x[j] < d->range[j]) break;
      x[j] = 0;
      --j;
    }
    if (j < 0) break;
  }
  return 0;
}

/* ------------------------------------------------------------------ dense fast paths
 * The same definition written as the plain loop nests a CPU backend would run, threaded
 * over output rows with OpenMP; used for sizes the generic walker cannot finish in seconds
 * and as the timed CPU baseline. Accumulation order: reduction index ascending. */

/* C[b,i,j] = sum_k A[b,i,k] * B[b,k,j] (b_is_nk == 0) or B[b,j,k] (b_is_nk == 1), f32. */
void orc_gemm_f32(const float* a, const float* b, float* c, int batch, int m, int n, int k,
                  int64_t lda, int64_t ldb, int64_t ldc, int64_t sa, int64_t sb, int64_t sc,
                  int b_is_nk) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int bb = 0; bb < batch; ++bb) {
    for (int i = 0; i < m; ++i) {
      const float* ar = a + bb * sa + (int64_t)i * lda;
      float* cr = c + bb * sc + (int64_t)i * ldc;
      const float* bm = b + bb * sb;
      if (b_is_nk) {
        for (int j = 0; j < n; ++j) {
          const float* br = bm + (int64_t)j * ldb;
          float acc = 0.f;
          for (int kk = 0; kk < k; ++kk) acc += ar[kk] * br[kk];
          cr[j] = acc;
        }
      } else {
        for (int j = 0; j < n; ++j) cr[j] = 0.f;
        for (int kk = 0; kk < k; ++kk) {
          const float av = ar[kk];
          const float* br = bm + (int64_t)kk * ldb;
          for (int j = 0; j < n; ++j) cr[j] += av * br[j];
        }
      }
    }
  }
}

/* Same with f64 accumulation: the yardstick that attributes fp32 error. */
void orc_gemm_f32_acc64(const float* a, const float* b, double* c, int batch, int m, int n, int k,
                        int64_t lda, int64_t ldb, int64_t ldc, int64_t sa, int64_t sb, int64_t sc,
                        int b_is_nk) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int bb = 0; bb < batch; ++bb) {
    for (int i = 0; i < m; ++i) {
      const float* ar = a + bb * sa + (int64_t)i * lda;
      double* cr = c + bb * sc + (int64_t)i * ldc;
      const float* bm = b + bb * sb;
      for (int j = 0; j < n; ++j) cr[j] = 0.0;
      for (int kk = 0; kk < k; ++kk) {
        const double av = ar[kk];
        if (b_is_nk) {
          for (int j = 0; j < n; ++j) cr[j] += av * (double)bm[(int64_t)j * ldb + kk];
        } else {
          const float* br = bm + (int64_t)kk * ldb;
          for (int j = 0; j < n; ++j) cr[j] += av * (double)br[j];
        }
      }
    }
  }
}

/* int8 x int8 -> int32 (operands sign-extended first, as cast(A, INT32) does). */
void orc_gemm_i8_i32(const int8_t* a, const int8_t* b, int32_t* c, int batch, int m, int n, int k,
                     int64_t lda, int64_t ldb, int64_t ldc, int64_t sa, int64_t sb, int64_t sc,
                     int b_is_nk) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int bb = 0; bb < batch; ++bb) {
    for (int i = 0; i < m; ++i) {
      const int8_t* ar = a + bb * sa + (int64_t)i * lda;
      int32_t* cr = c + bb * sc + (int64_t)i * ldc;
      const int8_t* bm = b + bb * sb;
      if (b_is_nk) {
        for (int j = 0; j < n; ++j) {
          const int8_t* br = bm + (int64_t)j * ldb;
          uint32_t acc = 0;
          for (int kk = 0; kk < k; ++kk) acc += (uint32_t)((int32_t)ar[kk] * (int32_t)br[kk]);
          cr[j] = (int32_t)acc;
        }
      } else {
        for (int j = 0; j < n; ++j) cr[j] = 0;
        for (int kk = 0; kk < k; ++kk) {
          const int32_t av = ar[kk];
          const int8_t* br = bm + (int64_t)kk * ldb;
          for (int j = 0; j < n; ++j) cr[j] = (int32_t)((uint32_t)cr[j] + (uint32_t)(av * (int32_t)br[j]));
        }
      }
    }
  }
}

/* 16-bit float inputs (is_f16: IEEE half, else bfloat16) widened exactly to f32,
 * f32 accumulate, f32 result: the DotF16_AccF32 pattern of plaidml/edsl/tests/edsl_test.cc:509-545. */
void orc_gemm_h16_f32(const uint16_t* a, const uint16_t* b, float* c, int is_f16, int batch, int m,
                      int n, int k, int64_t lda, int64_t ldb, int64_t ldc, int64_t sa, int64_t sb,
                      int64_t sc, int b_is_nk) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int bb = 0; bb < batch; ++bb) {
    for (int i = 0; i < m; ++i) {
      const uint16_t* ar = a + bb * sa + (int64_t)i * lda;
      float* cr = c + bb * sc + (int64_t)i * ldc;
      const uint16_t* bm = b + bb * sb;
      for (int j = 0; j < n; ++j) cr[j] = 0.f;
      for (int kk = 0; kk < k; ++kk) {
        const float av = is_f16 ? f16_to_f32(ar[kk]) : bf16_to_f32(ar[kk]);
        for (int j = 0; j < n; ++j) {
          const uint16_t bv = b_is_nk ? bm[(int64_t)j * ldb + kk] : bm[(int64_t)kk * ldb + j];
          cr[j] += av * (is_f16 ? f16_to_f32(bv) : bf16_to_f32(bv));
        }
      }
    }
  }
}

/* NHWC convolution, filter [r][s][c][k], the contraction of plaidml/op/lib/ops.cc:1351-1446:
 * O[n,y,x,ko] += I[n, sh*y + dh*fr - ph, sw*x + dw*fs - pw, ci] * F[fr,fs,ci,ko], taps outside
 * the image skipped.  f32 in / f32 accumulate; optional bias[k] added and ReLU applied after
 * the sum, the order of networks/oplib/resnet50.cc:26-57. */
void orc_conv2d_nhwc_f32(const float* in, const float* flt, const float* bias, const float* residual,
                         float* out, int n, int h, int w, int c, int r, int s, int k, int p, int q,
                         int sh, int sw, int ph, int pw, int dh, int dw, int relu) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int nn = 0; nn < n; ++nn) {
    for (int y = 0; y < p; ++y) {
      float* acc = (float*)malloc(sizeof(float) * (size_t)k);
      for (int x = 0; x < q; ++x) {
        for (int ko = 0; ko < k; ++ko) acc[ko] = 0.f;
        for (int fr = 0; fr < r; ++fr) {
          const int iy = sh * y + dh * fr - ph;
          if (iy < 0 || iy >= h) continue;
          for (int fs = 0; fs < s; ++fs) {
            const int ix = sw * x + dw * fs - pw;
            if (ix < 0 || ix >= w) continue;
            const float* ip = in + (((int64_t)nn * h + iy) * w + ix) * c;
            const float* fp = flt + ((int64_t)fr * s + fs) * c * k;
            for (int ci = 0; ci < c; ++ci) {
              const float iv = ip[ci];
              const float* fk = fp + (int64_t)ci * k;
              for (int ko = 0; ko < k; ++ko) acc[ko] += iv * fk[ko];
            }
          }
        }
        float* op = out + (((int64_t)nn * p + y) * q + x) * k;
        const float* rp = residual ? residual + (((int64_t)nn * p + y) * q + x) * k : 0;
        for (int ko = 0; ko < k; ++ko) {
          float v = acc[ko];
          if (bias) v += bias[ko];
          if (rp) v += rp[ko];
          if (relu) v = v < 0.f ? 0.f : v;
          op[ko] = v;
        }
      }
      free(acc);
    }
  }
}

/* NHWC window pooling, plaidml/op/lib/ops.cc:2562-2703: agg over in-range taps. */
void orc_pool2d_nhwc_f32(const float* in, float* out, int agg, int n, int h, int w, int c, int r,
                         int s, int p, int q, int sh, int sw, int ph, int pw, int average,
                         int include_padding) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int nn = 0; nn < n; ++nn) {
    for (int y = 0; y < p; ++y) {
      for (int x = 0; x < q; ++x) {
        for (int ch = 0; ch < c; ++ch) {
          float acc = agg == AGG_MAX ? -INFINITY : (agg == AGG_MIN ? INFINITY : 0.f);
          int taps = 0;
          for (int fr = 0; fr < r; ++fr) {
            const int iy = sh * y + fr - ph;
            if (iy < 0 || iy >= h) continue;
            for (int fs = 0; fs < s; ++fs) {
              const int ix = sw * x + fs - pw;
              if (ix < 0 || ix >= w) continue;
              const float v = in[(((int64_t)nn * h + iy) * w + ix) * c + ch];
              ++taps;
              if (agg == AGG_MAX) acc = (acc > v) ? acc : v;
              else if (agg == AGG_MIN) acc = (acc < v) ? acc : v;
              else acc += v;
            }
          }
          if (average) acc = acc / (float)(include_padding ? r * s : (taps ? taps : 1));
          out[(((int64_t)nn * p + y) * q + x) * c + ch] = acc;
        }
      }
    }
  }
}

/* out[o, i] = agg_r in[o, r, i] in f32. */
void orc_reduce_f32(const float* in, float* out, int agg, int64_t outer, int64_t red, int64_t inner) {
#pragma omp parallel for schedule(static)
  for (int64_t o = 0; o < outer; ++o) {
    for (int64_t i = 0; i < inner; ++i) {
      float acc = agg == AGG_MAX ? -INFINITY : (agg == AGG_MIN ? INFINITY : 0.f);
      for (int64_t r = 0; r < red; ++r) {
        const float v = in[(o * red + r) * inner + i];
        if (agg == AGG_MAX) acc = (acc > v) ? acc : v;
        else if (agg == AGG_MIN) acc = (acc < v) ? acc : v;
        else acc += v;
      }
      out[o * inner + i] = acc;
    }
  }
}

/* exact widening / RNE narrowing helpers exported for the Python side */
void orc_bf16_to_f32(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = bf16_to_f32(in[i]);
}
void orc_f32_to_bf16(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]);
}
