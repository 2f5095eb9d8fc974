// General Tile contraction and element-wise kernels: complete but unspecialised.
//
// contraction  one thread per output element.  When every output coordinate is a single
//              index variable (the usual case) those variables are read off the element's
//              position and the thread loops over the remaining (reduction) variables;
//              otherwise, per output dim that mixes variables (`s*x + i`), one variable is
//              solved for from the element's coordinate and the others are looped over, and
//              only with a rational output coordinate does the thread walk the whole index
//              box and keep the points that land on its element.  A point contributes only
//              if every tensor access is in range, every constraint holds and every rational
//              index is integral.
// eltwise      one thread per output element, operands read through broadcast strides.
//
// Arithmetic happens in the contraction's element type: integers wrap (computed in 64
// bits and truncated on store), f16 / bf16 round after every operation, max / min are a
// compare-and-select with an ordered compare.
#include "generic.h"
#include "typed_access.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

namespace pmlb {

namespace {

template <class T>
__device__ __forceinline__ T agg_identity(int agg, int dtype) {
  constexpr bool is_float = static_cast<T>(0.5) != T(0);
  if (agg == PMLB_AGG_PROD) return T(1);
  if (agg == PMLB_AGG_MAX) {
    if constexpr (is_float) return static_cast<T>(-INFINITY);
    switch (dtype) {
      case PMLB_I8: return static_cast<T>(-128);
      case PMLB_I16: return static_cast<T>(-32768);
      case PMLB_I32: return static_cast<T>(-2147483647 - 1);
      case PMLB_I64: return static_cast<T>(-9223372036854775807LL - 1);
      default: return T(0);
    }
  }
  if (agg == PMLB_AGG_MIN) {
    if constexpr (is_float) return static_cast<T>(INFINITY);
    switch (dtype) {
      case PMLB_BOOL: return T(1);
      case PMLB_I8: return static_cast<T>(127);
      case PMLB_U8: return static_cast<T>(255);
      case PMLB_I16: return static_cast<T>(32767);
      case PMLB_U16: return static_cast<T>(65535);
      case PMLB_I32: return static_cast<T>(2147483647);
      case PMLB_U32: return static_cast<T>(4294967295LL);
      case PMLB_I64: return static_cast<T>(9223372036854775807LL);
      default: return static_cast<T>(~0ULL);
    }
  }
  return T(0);
}

__device__ __forceinline__ long long floor_div_exact(long long num, int den, bool* integral) {
  if (den == 1) return num;
  const long long q = num / den;
  if (q * den != num) *integral = false;
  return q;
}

// ------------------------------------------------------------------ contraction

template <class T>
__global__ void __launch_bounds__(256) contract_kernel(const __grid_constant__ GenericParams p) {
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= p.out_elems) return;

  long long oc[PMLB_MAX_RANK];
  long long rem = e;
  long long out_off = 0, init_off = 0;
  for (int d = p.out.rank - 1; d >= 0; --d) {
    oc[d] = rem % p.out.sizes[d];
    rem /= p.out.sizes[d];
    out_off += oc[d] * p.out.strides[d];
    init_off += oc[d] * p.init.strides[d];
  }

  long long x[PMLB_MAX_IDX];
  for (int i = 0; i < PMLB_MAX_IDX; ++i) x[i] = 0;
  bool alive = true;
  if (p.direct) {
    for (int d = 0; d < p.out.rank; ++d) {
      const int v = p.out_var[d];
      const long long xv = oc[d] - p.out.off[d];
      if (xv < 0 || xv >= p.range[v]) alive = false;
      x[v] = xv;
    }
  }
  for (int j = 0; j < p.n_loop; ++j) {
    if (p.range[p.loop_var[j]] <= 0) alive = false;
  }
  for (int s = 0; s < p.n_solve; ++s) {
    if (p.range[p.solve_var[s]] <= 0) alive = false;
  }

  T acc = p.has_init ? narrow<T>(load_as<T>(p.initp, p.init.dtype, init_off), p.out.dtype)
                     : agg_identity<T>(p.agg, p.out.dtype);

  while (alive) {
    bool ok = true;
    for (int s = 0; s < p.n_solve && ok; ++s) {
      const int d = p.solve_dim[s];
      const int v = p.solve_var[s];
      x[v] = 0;
      long long num = oc[d] - p.out.off[d];
      for (int i = 0; i < p.n_idx; ++i) num -= static_cast<long long>(p.out.coef[d][i]) * x[i];
      const long long xv = floor_div_exact(num, p.out.coef[d][v], &ok);
      if (xv < 0 || xv >= p.range[v]) ok = false;
      x[v] = xv;
    }
    if (!p.direct) {
      for (int d = 0; d < p.out.rank && ok; ++d) {
        long long num = p.out.off[d];
        for (int i = 0; i < p.n_idx; ++i) num += static_cast<long long>(p.out.coef[d][i]) * x[i];
        const long long c = floor_div_exact(num, p.out.den[d], &ok);
        if (c != oc[d]) ok = false;
      }
    }
    for (int c = 0; c < p.n_cons && ok; ++c) {
      long long v = p.cons_off[c];
      for (int i = 0; i < p.n_idx; ++i) v += static_cast<long long>(p.cons_coef[c][i]) * x[i];
      if (v < 0 || v >= p.cons_range[c]) ok = false;
    }
    long long soff[3] = {0, 0, 0};
    for (int s = 0; s < p.n_src && ok; ++s) {
      const GAccess& a = p.src[s];
      for (int d = 0; d < a.rank; ++d) {
        long long num = a.off[d];
        for (int i = 0; i < p.n_idx; ++i) num += static_cast<long long>(a.coef[d][i]) * x[i];
        const long long c = floor_div_exact(num, a.den[d], &ok);
        if (c < 0 || c >= a.sizes[d]) ok = false;
        soff[s] += c * a.strides[d];
      }
    }
    if (ok) {
      T v;
      const int odt = p.out.dtype;
      switch (p.combo) {
        case PMLB_COMBO_MUL:
          v = narrow<T>(load_as<T>(p.srcp[0], p.src[0].dtype, soff[0]) *
                            load_as<T>(p.srcp[1], p.src[1].dtype, soff[1]),
                        odt);
          break;
        case PMLB_COMBO_ADD:
          v = narrow<T>(load_as<T>(p.srcp[0], p.src[0].dtype, soff[0]) +
                            load_as<T>(p.srcp[1], p.src[1].dtype, soff[1]),
                        odt);
          break;
        case PMLB_COMBO_EQ: {
          bool eq;
          if (dtype_is_float(p.src[0].dtype) || dtype_is_float(p.src[1].dtype)) {
            eq = load_as<double>(p.srcp[0], p.src[0].dtype, soff[0]) ==
                 load_as<double>(p.srcp[1], p.src[1].dtype, soff[1]);
          } else {
            eq = load_as<long long>(p.srcp[0], p.src[0].dtype, soff[0]) ==
                 load_as<long long>(p.srcp[1], p.src[1].dtype, soff[1]);
          }
          v = eq ? T(1) : T(0);
          break;
        }
        case PMLB_COMBO_COND: {
          bool eq;
          if (dtype_is_float(p.src[0].dtype) || dtype_is_float(p.src[1].dtype)) {
            eq = load_as<double>(p.srcp[0], p.src[0].dtype, soff[0]) ==
                 load_as<double>(p.srcp[1], p.src[1].dtype, soff[1]);
          } else {
            eq = load_as<long long>(p.srcp[0], p.src[0].dtype, soff[0]) ==
                 load_as<long long>(p.srcp[1], p.src[1].dtype, soff[1]);
          }
          v = eq ? narrow<T>(load_as<T>(p.srcp[2], p.src[2].dtype, soff[2]), odt) : T(0);
          break;
        }
        default:
          v = narrow<T>(load_as<T>(p.srcp[0], p.src[0].dtype, soff[0]), odt);
          break;
      }
      switch (p.agg) {
        case PMLB_AGG_SUM: acc = narrow<T>(acc + v, odt); break;
        case PMLB_AGG_PROD: acc = narrow<T>(acc * v, odt); break;
        case PMLB_AGG_MAX: acc = (acc > v) ? acc : v; break;
        case PMLB_AGG_MIN: acc = (acc < v) ? acc : v; break;
        default: acc = v; break;
      }
    }
    int j = p.n_loop - 1;
    while (j >= 0) {
      const int v = p.loop_var[j];
      if (++x[v] < p.range[v]) break;
      x[v] = 0;
      --j;
    }
    if (j < 0) break;
  }
  store_as<T>(p.outp, p.out.dtype, out_off, acc);
}

// ------------------------------------------------------------------ eltwise

template <class T>
__device__ __forceinline__ T ew_apply(int op, T a, T b, T c, bool a_nz) {
  constexpr bool is_float = static_cast<T>(0.5) != T(0);
  switch (op) {
    case kEwIdent: return a;
    case kEwAdd: return a + b;
    case kEwSub: return a - b;
    case kEwMul: return a * b;
    case kEwDiv:
      if constexpr (is_float) return a / b;
      else return b == T(0) ? T(0) : a / b;
    case kEwMod:
      if constexpr (is_float) return static_cast<T>(fmod(static_cast<double>(a), static_cast<double>(b)));
      else return b == T(0) ? T(0) : a % b;
    case kEwMax: return (a > b) ? a : b;
    case kEwMin: return (a < b) ? a : b;
    case kEwNeg: return T(0) - a;
    case kEwAbs: return a < T(0) ? T(0) - a : a;
    case kEwRelu: return a < T(0) ? T(0) : a;
    case kEwSign: return a > T(0) ? T(1) : (a < T(0) ? T(0) - T(1) : T(0));
    case kEwSelect: return a_nz ? b : c;
    case kEwCmpEq: return a == b ? T(1) : T(0);
    case kEwCmpNe: return a != b ? T(1) : T(0);
    case kEwCmpLt: return a < b ? T(1) : T(0);
    case kEwCmpLe: return a <= b ? T(1) : T(0);
    case kEwCmpGt: return a > b ? T(1) : T(0);
    case kEwCmpGe: return a >= b ? T(1) : T(0);
    case kEwLogicalAnd: return (a != T(0) && b != T(0)) ? T(1) : T(0);
    case kEwLogicalOr: return (a != T(0) || b != T(0)) ? T(1) : T(0);
    case kEwLogicalXor: return ((a != T(0)) != (b != T(0))) ? T(1) : T(0);
    case kEwLogicalNot: return a == T(0) ? T(1) : T(0);
    default: break;
  }
  if constexpr (is_float) {
    const double x = static_cast<double>(a);
    const double y = static_cast<double>(b);
    switch (op) {
      case kEwExp: return static_cast<T>(exp(x));
      case kEwLog: return static_cast<T>(log(x));
      case kEwSqrt: return static_cast<T>(sqrt(x));
      case kEwRsqrt: return static_cast<T>(1.0 / sqrt(x));
      case kEwTanh: return static_cast<T>(tanh(x));
      case kEwSigmoid: return static_cast<T>(1.0 / (1.0 + exp(-x)));
      case kEwSin: return static_cast<T>(sin(x));
      case kEwCos: return static_cast<T>(cos(x));
      case kEwTan: return static_cast<T>(tan(x));
      case kEwSinh: return static_cast<T>(sinh(x));
      case kEwCosh: return static_cast<T>(cosh(x));
      case kEwAsin: return static_cast<T>(asin(x));
      case kEwAcos: return static_cast<T>(acos(x));
      case kEwAtan: return static_cast<T>(atan(x));
      case kEwAsinh: return static_cast<T>(asinh(x));
      case kEwAcosh: return static_cast<T>(acosh(x));
      case kEwAtanh: return static_cast<T>(atanh(x));
      case kEwErf: return static_cast<T>(erf(x));
      case kEwPow: return static_cast<T>(pow(x, y));
      case kEwFloor: return static_cast<T>(floor(x));
      case kEwCeil: return static_cast<T>(ceil(x));
      case kEwRound: return static_cast<T>(round(x));
      default: return a;
    }
  } else {
    switch (op) {
      case kEwBitAnd: return a & b;
      case kEwBitOr: return a | b;
      case kEwBitXor: return a ^ b;
      case kEwBitNot: return ~a;
      case kEwBitShl: return (b < T(0) || b >= T(64)) ? T(0) : static_cast<T>(a << b);
      case kEwBitShr: return (b < T(0) || b >= T(64)) ? T(0) : static_cast<T>(a >> b);
      case kEwPow: {
        T r = 1;
        for (T i = 0; i < b; ++i) r *= a;
        return r;
      }
      case kEwFloor:
      case kEwCeil:
      case kEwRound: return a;
      default: return a;
    }
  }
}

// `T` is the class the operation is evaluated in (chosen from the operand types for
// comparisons, from the result type otherwise); `arith_dtype` is the element type results
// are rounded / wrapped to before the final conversion to the output type.
template <class T>
__device__ __forceinline__ void eltwise_one(const EltwiseParams& p, long long e, const long long (&off)[3]) {
  T a = T(0), b = T(0), c = T(0);
  bool a_nz = false;
  if (p.op == kEwSelect) {
    // the condition keeps its own type; the branches are read in the result class
    a_nz = load_as<double>(p.in[0], p.in_dtype[0], off[0]) != 0.0;
    b = narrow<T>(load_as<T>(p.in[1], p.in_dtype[1], off[1]), p.arith_dtype);
    c = narrow<T>(load_as<T>(p.in[2], p.in_dtype[2], off[2]), p.arith_dtype);
  } else {
    a = load_as<T>(p.in[0], p.in_dtype[0], off[0]);
    if (p.n_in > 1) b = load_as<T>(p.in[1], p.in_dtype[1], off[1]);
    if (p.n_in > 2) c = load_as<T>(p.in[2], p.in_dtype[2], off[2]);
    if (p.narrow_inputs) {
      a = narrow<T>(a, p.arith_dtype);
      b = narrow<T>(b, p.arith_dtype);
      c = narrow<T>(c, p.arith_dtype);
    }
  }
  T r = ew_apply<T>(p.op, a, b, c, a_nz);
  if (p.narrow_result) r = narrow<T>(r, p.arith_dtype);
  store_as<T>(p.out, p.out_dtype, e, r);
}

template <class T>
__global__ void __launch_bounds__(256) eltwise_kernel(const __grid_constant__ EltwiseParams p) {
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= p.elems) return;
  long long rem = e;
  long long off[3] = {0, 0, 0};
  for (int d = p.rank - 1; d >= 0; --d) {
    const long long c = rem % p.sizes[d];
    rem /= p.sizes[d];
    off[0] += c * p.in_strides[0][d];
    off[1] += c * p.in_strides[1][d];
    off[2] += c * p.in_strides[2][d];
  }
  eltwise_one<T>(p, e, off);
}

// Every operand as dense as the result or one value for all of it, any element types: no index arithmetic, four
// elements per thread a grid apart (`one_value` has bit k set if operand k is a single value).
template <class T>
__global__ void __launch_bounds__(256) eltwise_dense_kernel(const __grid_constant__ EltwiseParams p, int one_value,
                                                            long long threads) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= threads) return;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const long long e = t + u * threads;
    if (e >= p.elems) return;
    const long long off[3] = {(one_value & 1) ? 0 : e, (one_value & 2) ? 0 : e, (one_value & 4) ? 0 : e};
    eltwise_one<T>(p, e, off);
  }
}

// The common case of the kernel above -- f32 in and out, every operand either as dense as the result or one value
// for all of it -- without the per-element index arithmetic: eight elements per thread as two 16-byte pieces a grid
// apart, all loads before the arithmetic.  The arithmetic is the same function, so the results are the same bits.
struct DenseF32 {
  const float* in[3];
  int scalar[3];   // operand k: 0 dense, 1 one value, 2 repeats every `period` quads (a bias along the trailing dims),
                   // 3 one value per `period` quads (a column along the leading dims)
  long long period[3];
  float* out;
  long long quads;  // elements / 4
  int op, n_in;
};

__global__ void __launch_bounds__(256) eltwise_f32_dense_kernel(const DenseF32 p, long long threads) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= threads) return;
  float4 v[2][3];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    long long q = t + u * threads;
    if (q >= p.quads) q = p.quads - 1;
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      if (k >= p.n_in) {
        v[u][k] = make_float4(0.f, 0.f, 0.f, 0.f);
      } else if (p.scalar[k] == 1) {
        const float s = p.in[k][0];
        v[u][k] = make_float4(s, s, s, s);
      } else if (p.scalar[k] == 2) {
        v[u][k] = reinterpret_cast<const float4*>(p.in[k])[q % p.period[k]];
      } else if (p.scalar[k] == 3) {
        const float s = p.in[k][q / p.period[k]];
        v[u][k] = make_float4(s, s, s, s);
      } else {
        v[u][k] = reinterpret_cast<const float4*>(p.in[k])[q];
      }
    }
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const long long q = t + u * threads;
    if (q >= p.quads) continue;
    float4 r;
    r.x = ew_apply<float>(p.op, v[u][0].x, v[u][1].x, v[u][2].x, false);
    r.y = ew_apply<float>(p.op, v[u][0].y, v[u][1].y, v[u][2].y, false);
    r.z = ew_apply<float>(p.op, v[u][0].z, v[u][1].z, v[u][2].z, false);
    r.w = ew_apply<float>(p.op, v[u][0].w, v[u][1].w, v[u][2].w, false);
    reinterpret_cast<float4*>(p.out)[q] = r;
  }
}

// The dense form for f16 / bf16 in and out: eight elements per 16-byte piece, the operation evaluated in f32 and
// rounded to the 16-bit type as the general kernel does (operands of that type need no rounding).
template <class S>
struct Dense16 {
  const S* in[3];
  int scalar[3];
  S* out;
  long long octets;
  int op, n_in, dtype;
};

__device__ __forceinline__ float widen(__half v) { return __half2float(v); }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
template <class S> __device__ __forceinline__ S shorten(float v);
template <> __device__ __forceinline__ __half shorten<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 shorten<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <class S>
__global__ void __launch_bounds__(256) eltwise_16bit_dense_kernel(const Dense16<S> p) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= p.octets) return;
  struct alignas(16) Vec { S v[8]; };
  Vec a[3];
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    if (k >= p.n_in) {
#pragma unroll
      for (int i = 0; i < 8; ++i) a[k].v[i] = shorten<S>(0.f);
    } else if (p.scalar[k]) {
      const S s = p.in[k][0];
#pragma unroll
      for (int i = 0; i < 8; ++i) a[k].v[i] = s;
    } else {
      a[k] = reinterpret_cast<const Vec*>(p.in[k])[t];
    }
  }
  Vec r;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float x = ew_apply<float>(p.op, widen(a[0].v[i]), widen(a[1].v[i]), widen(a[2].v[i]), false);
    r.v[i] = shorten<S>(narrow<float>(x, p.dtype));
  }
  reinterpret_cast<Vec*>(p.out)[t] = r;
}

// Dense casts between f32 and the two 16-bit float types (round to nearest even, as the general kernel's store does):
// eight elements per thread, 16- and 32-byte accesses.
template <class In, class Out>
__device__ __forceinline__ Out convert_one(In v);
template <> __device__ __forceinline__ float convert_one<__half, float>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float convert_one<__nv_bfloat16, float>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ __half convert_one<float, __half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 convert_one<float, __nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <class In, class Out>
__global__ void __launch_bounds__(256) convert_dense_kernel(const In* __restrict__ in, Out* __restrict__ out, long long octets) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= octets) return;
  struct alignas(sizeof(In) * 8) InVec { In v[8]; };
  struct alignas(sizeof(Out) * 8) OutVec { Out v[8]; };
  const InVec a = reinterpret_cast<const InVec*>(in)[t];
  OutVec r;
#pragma unroll
  for (int i = 0; i < 8; ++i) r.v[i] = convert_one<In, Out>(a.v[i]);
  reinterpret_cast<OutVec*>(out)[t] = r;
}

template <class T>
__global__ void __launch_bounds__(256) fill_kernel(void* out, int dtype, long long n, T value) {
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e < n) store_as<T>(out, dtype, e, value);
}

unsigned grid_for(long long elems) { return static_cast<unsigned>((elems + 255) / 256); }

}  // namespace

int dtype_class(int dtype) {
  switch (dtype) {
    case PMLB_F16:
    case PMLB_BF16:
    case PMLB_F32: return kClassF32;
    case PMLB_F64: return kClassF64;
    case PMLB_BOOL:
    case PMLB_U8:
    case PMLB_U16:
    case PMLB_U32:
    case PMLB_U64: return kClassU64;
    case PMLB_I8:
    case PMLB_I16:
    case PMLB_I32:
    case PMLB_I64: return kClassI64;
    default: return -1;
  }
}

cudaError_t launch_contract(const GenericParams& p, cudaStream_t stream) {
  if (p.out_elems <= 0) return cudaSuccess;
  const unsigned grid = grid_for(p.out_elems);
  switch (dtype_class(p.out.dtype)) {
    case kClassF32: contract_kernel<float><<<grid, 256, 0, stream>>>(p); break;
    case kClassF64: contract_kernel<double><<<grid, 256, 0, stream>>>(p); break;
    case kClassI64: contract_kernel<long long><<<grid, 256, 0, stream>>>(p); break;
    case kClassU64: contract_kernel<unsigned long long><<<grid, 256, 0, stream>>>(p); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

namespace {
// Fills `d` if the operation takes the dense f32 form: f32 throughout, not a select (its condition has a type of its
// own), a multiple of four elements, 16-byte aligned buffers, and operands that are dense like the result or a single
// value.
bool dense_f32_form(const EltwiseParams& p, DenseF32* d) {
  if (p.compute_class != kClassF32 || p.out_dtype != PMLB_F32 || p.arith_dtype != PMLB_F32 || p.op == kEwSelect) return false;
  if (p.elems % 4 != 0 || reinterpret_cast<uintptr_t>(p.out) % 16 != 0) return false;
  long long dense[PMLB_MAX_RANK];
  long long stride = 1;
  for (int dd = p.rank - 1; dd >= 0; --dd) {
    dense[dd] = stride;
    stride *= p.sizes[dd];
  }
  for (int k = 0; k < p.n_in; ++k) {
    if (p.in_dtype[k] != PMLB_F32) return false;
    bool as_result = true, one_value = true;
    for (int dd = 0; dd < p.rank; ++dd) {
      if (p.sizes[dd] == 1) continue;
      if (p.in_strides[k][dd] != dense[dd]) as_result = false;
      if (p.in_strides[k][dd] != 0) one_value = false;
    }
    int mode = as_result ? 0 : (one_value ? 1 : -1);
    long long period = 0;
    if (mode < 0) {
      // dense over the trailing dims and repeated over the leading ones (a bias), or one value per run of the
      // trailing dims (a column)?
      int split = -1;   // first dim of the trailing part
      bool bias = true, column = true;
      for (int dd = 0; dd < p.rank; ++dd) {
        if (p.sizes[dd] == 1) continue;
        if (p.in_strides[k][dd] != 0 && split < 0) split = dd;
      }
      // bias: stride 0 before `split`, dense strides from `split` on
      for (int dd = 0; dd < p.rank && split >= 0; ++dd) {
        if (p.sizes[dd] == 1) continue;
        if (dd < split ? p.in_strides[k][dd] != 0 : p.in_strides[k][dd] != dense[dd]) bias = false;
      }
      if (split >= 0 && bias) {
        period = dense[split] * p.sizes[split];          // elements of the trailing part
        if (period % 4 == 0) mode = 2;
      }
      if (mode < 0) {
        // column: non-zero strides on a leading part only, dense within that part; zero on the trailing part
        int last = -1;
        for (int dd = 0; dd < p.rank; ++dd) {
          if (p.sizes[dd] != 1 && p.in_strides[k][dd] != 0) last = dd;
        }
        long long run = last >= 0 ? dense[last] : 0;     // elements of the trailing part behind `last`
        for (int dd = 0; dd < p.rank && last >= 0; ++dd) {
          if (p.sizes[dd] == 1) continue;
          if (dd <= last ? p.in_strides[k][dd] * run != dense[dd] : p.in_strides[k][dd] != 0) column = false;
        }
        if (last >= 0 && column && run % 4 == 0) {
          period = run;
          mode = 3;
        }
      }
      if (mode < 0) return false;
      period /= 4;
    }
    if ((mode == 0 || mode == 2) && reinterpret_cast<uintptr_t>(p.in[k]) % 16 != 0) return false;
    d->in[k] = static_cast<const float*>(p.in[k]);
    d->scalar[k] = mode;
    d->period[k] = period;
  }
  d->out = static_cast<float*>(p.out);
  d->quads = p.elems / 4;
  d->op = p.op;
  d->n_in = p.n_in;
  return true;
}
}  // namespace

namespace {
// A cast between f32 and f16 / bf16 of a dense operand, eight elements at a time; false if the operation is not one.
bool launch_dense_convert(const EltwiseParams& p, cudaStream_t stream) {
  if (p.op != kEwIdent || p.n_in != 1 || p.elems % 8 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(p.in[0]) | reinterpret_cast<uintptr_t>(p.out)) % 32 != 0) return false;
  long long stride = 1;
  for (int dd = p.rank - 1; dd >= 0; --dd) {
    if (p.sizes[dd] != 1 && p.in_strides[0][dd] != stride) return false;
    stride *= p.sizes[dd];
  }
  const long long octets = p.elems / 8;
  const unsigned grid = grid_for(octets);
  const int from = p.in_dtype[0], to = p.out_dtype;
  if (from == PMLB_F32 && to == PMLB_F16) {
    convert_dense_kernel<float, __half><<<grid, 256, 0, stream>>>(static_cast<const float*>(p.in[0]), static_cast<__half*>(p.out), octets);
  } else if (from == PMLB_F32 && to == PMLB_BF16) {
    convert_dense_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const float*>(p.in[0]),
                                                                         static_cast<__nv_bfloat16*>(p.out), octets);
  } else if (from == PMLB_F16 && to == PMLB_F32) {
    convert_dense_kernel<__half, float><<<grid, 256, 0, stream>>>(static_cast<const __half*>(p.in[0]), static_cast<float*>(p.out), octets);
  } else if (from == PMLB_BF16 && to == PMLB_F32) {
    convert_dense_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(p.in[0]),
                                                                         static_cast<float*>(p.out), octets);
  } else {
    return false;
  }
  return true;
}
}  // namespace

namespace {
template <class S>
bool launch_dense_16bit(const EltwiseParams& p, int dtype, cudaStream_t stream) {
  if (p.compute_class != kClassF32 || p.out_dtype != dtype || p.arith_dtype != dtype || p.op == kEwSelect) return false;
  if (p.elems % 8 != 0 || reinterpret_cast<uintptr_t>(p.out) % 16 != 0) return false;
  long long dense[PMLB_MAX_RANK];
  long long stride = 1;
  for (int dd = p.rank - 1; dd >= 0; --dd) {
    dense[dd] = stride;
    stride *= p.sizes[dd];
  }
  Dense16<S> d{};
  for (int k = 0; k < p.n_in; ++k) {
    if (p.in_dtype[k] != dtype) return false;
    bool as_result = true, one_value = true;
    for (int dd = 0; dd < p.rank; ++dd) {
      if (p.sizes[dd] == 1) continue;
      if (p.in_strides[k][dd] != dense[dd]) as_result = false;
      if (p.in_strides[k][dd] != 0) one_value = false;
    }
    if (!as_result && !one_value) return false;
    if (as_result && reinterpret_cast<uintptr_t>(p.in[k]) % 16 != 0) return false;
    d.in[k] = static_cast<const S*>(p.in[k]);
    d.scalar[k] = as_result ? 0 : 1;
  }
  d.out = static_cast<S*>(p.out);
  d.octets = p.elems / 8;
  d.op = p.op;
  d.n_in = p.n_in;
  d.dtype = dtype;
  eltwise_16bit_dense_kernel<S><<<grid_for(d.octets), 256, 0, stream>>>(d);
  return true;
}
}  // namespace

cudaError_t launch_eltwise(const EltwiseParams& p, cudaStream_t stream) {
  if (p.elems <= 0) return cudaSuccess;
  if (launch_dense_convert(p, stream)) return cudaGetLastError();
  if (launch_dense_16bit<__half>(p, PMLB_F16, stream) || launch_dense_16bit<__nv_bfloat16>(p, PMLB_BF16, stream)) {
    return cudaGetLastError();
  }
  DenseF32 dense{};
  if (dense_f32_form(p, &dense)) {
    const long long threads = (dense.quads + 1) / 2;
    eltwise_f32_dense_kernel<<<grid_for(threads), 256, 0, stream>>>(dense, threads);
    return cudaGetLastError();
  }
  // every operand dense like the result or a single value?
  {
    long long dense_stride[PMLB_MAX_RANK];
    long long stride = 1;
    for (int dd = p.rank - 1; dd >= 0; --dd) {
      dense_stride[dd] = stride;
      stride *= p.sizes[dd];
    }
    int one_value = 0;
    bool all = true;
    for (int k = 0; k < p.n_in && all; ++k) {
      bool as_result = true, single = true;
      for (int dd = 0; dd < p.rank; ++dd) {
        if (p.sizes[dd] == 1) continue;
        if (p.in_strides[k][dd] != dense_stride[dd]) as_result = false;
        if (p.in_strides[k][dd] != 0) single = false;
      }
      if (!as_result && !single) all = false;
      if (!as_result && single) one_value |= 1 << k;
    }
    if (all) {
      const long long threads = (p.elems + 3) / 4;
      const unsigned g4 = grid_for(threads);
      switch (p.compute_class) {
        case kClassF32: eltwise_dense_kernel<float><<<g4, 256, 0, stream>>>(p, one_value, threads); break;
        case kClassF64: eltwise_dense_kernel<double><<<g4, 256, 0, stream>>>(p, one_value, threads); break;
        case kClassI64: eltwise_dense_kernel<long long><<<g4, 256, 0, stream>>>(p, one_value, threads); break;
        case kClassU64: eltwise_dense_kernel<unsigned long long><<<g4, 256, 0, stream>>>(p, one_value, threads); break;
        default: return cudaErrorInvalidValue;
      }
      return cudaGetLastError();
    }
  }
  const unsigned grid = grid_for(p.elems);
  switch (p.compute_class) {
    case kClassF32: eltwise_kernel<float><<<grid, 256, 0, stream>>>(p); break;
    case kClassF64: eltwise_kernel<double><<<grid, 256, 0, stream>>>(p); break;
    case kClassI64: eltwise_kernel<long long><<<grid, 256, 0, stream>>>(p); break;
    case kClassU64: eltwise_kernel<unsigned long long><<<grid, 256, 0, stream>>>(p); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_fill_f32(float* out, long long n, float value, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  fill_kernel<float><<<grid_for(n), 256, 0, stream>>>(out, PMLB_F32, n, value);
  return cudaGetLastError();
}

}  // namespace pmlb
