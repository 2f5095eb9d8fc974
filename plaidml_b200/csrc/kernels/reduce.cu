// Bandwidth-bound aggregation kernels: the max / min / sum contractions that have no
// multiply (row max, pooling windows, global-average sums).  All of them move 16 bytes
// per load where alignment allows, keep several loads in flight per thread and finish
// with warp shuffles; none of them touches the tensor cores.
#include "reduce.h"

#include <type_traits>

#include "tc_gemm.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

namespace pmlb {

namespace {

template <class T> struct AccOf { using type = float; };
template <> struct AccOf<int32_t> { using type = int32_t; };
template <> struct AccOf<int8_t> { using type = int32_t; };

template <class T> __device__ __forceinline__ typename AccOf<T>::type to_acc(T v);
template <> __device__ __forceinline__ float to_acc<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ int32_t to_acc<int32_t>(int32_t v) { return v; }
template <> __device__ __forceinline__ int32_t to_acc<int8_t>(int8_t v) { return v; }

template <class T, class A> __device__ __forceinline__ T from_acc(A v);
template <> __device__ __forceinline__ float from_acc<float, float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_acc<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ int32_t from_acc<int32_t, int32_t>(int32_t v) { return v; }
template <> __device__ __forceinline__ int8_t from_acc<int8_t, int32_t>(int32_t v) { return static_cast<int8_t>(v); }

template <class A> __device__ __forceinline__ A identity_of(int agg);
template <> __device__ __forceinline__ float identity_of<float>(int agg) {
  return agg == PMLB_AGG_MAX ? -INFINITY : (agg == PMLB_AGG_MIN ? INFINITY : 0.f);
}
template <> __device__ __forceinline__ int32_t identity_of<int32_t>(int agg) {
  return agg == PMLB_AGG_MAX ? (-2147483647 - 1) : (agg == PMLB_AGG_MIN ? 2147483647 : 0);
}

// acc = agg(acc, v); max / min as compare-and-select: (acc > v) ? acc : v.
template <int AGG, class A>
__device__ __forceinline__ A combine(A acc, A v) {
  if constexpr (AGG == PMLB_AGG_MAX) return (acc > v) ? acc : v;
  else if constexpr (AGG == PMLB_AGG_MIN) return (acc < v) ? acc : v;
  else return acc + v;
}

template <class T> struct alignas(16) Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

// ------------------------------------------------------------------ rows
// in [rows][len] -> out [rows]; one warp per row.
template <class T, class TO, int AGG, bool VEC>
__global__ void __launch_bounds__(256)
row_reduce_kernel(const T* __restrict__ in, TO* __restrict__ out, long long rows, long long len,
                  float scale) {
  using A = typename AccOf<T>::type;
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* src = in + row * len;
  A acc = identity_of<A>(AGG);
  if constexpr (VEC) {
    constexpr int N = Vec16<T>::N;
    const long long nvec = len / N;
    const Vec16<T>* vsrc = reinterpret_cast<const Vec16<T>*>(src);
    long long i = lane;
    for (; i + 96 < nvec; i += 128) {
      const Vec16<T> a = vsrc[i];
      const Vec16<T> b = vsrc[i + 32];
      const Vec16<T> c = vsrc[i + 64];
      const Vec16<T> d = vsrc[i + 96];
#pragma unroll
      for (int j = 0; j < N; ++j) acc = combine<AGG, A>(acc, to_acc<T>(a.v[j]));
#pragma unroll
      for (int j = 0; j < N; ++j) acc = combine<AGG, A>(acc, to_acc<T>(b.v[j]));
#pragma unroll
      for (int j = 0; j < N; ++j) acc = combine<AGG, A>(acc, to_acc<T>(c.v[j]));
#pragma unroll
      for (int j = 0; j < N; ++j) acc = combine<AGG, A>(acc, to_acc<T>(d.v[j]));
    }
    for (; i < nvec; i += 32) {
      const Vec16<T> a = vsrc[i];
#pragma unroll
      for (int j = 0; j < N; ++j) acc = combine<AGG, A>(acc, to_acc<T>(a.v[j]));
    }
    for (long long t = nvec * N + lane; t < len; t += 32) acc = combine<AGG, A>(acc, to_acc<T>(src[t]));
  } else {
    for (long long t = lane; t < len; t += 32) acc = combine<AGG, A>(acc, to_acc<T>(src[t]));
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) {
    const A other = __shfl_xor_sync(0xffffffffu, acc, s);
    acc = combine<AGG, A>(acc, other);
  }
  if (lane == 0) {
    if constexpr (AGG == PMLB_AGG_SUM && sizeof(A) == 4 && static_cast<A>(0.5) != A(0)) {
      if (scale != 1.f) acc = scale < 0.f ? acc / -scale : acc * scale;   // (negative: a divisor)
    }
    out[row] = from_acc<TO, A>(acc);
  }
}

// ------------------------------------------------------------------ strided
// in [outer][red][inner] -> out [outer][inner]; one thread per 16 bytes of inner.
template <class T, class TO, int AGG, bool VEC>
__global__ void __launch_bounds__(256)
strided_reduce_kernel(const T* __restrict__ in, TO* __restrict__ out, long long outer, long long red,
                      long long inner, float scale) {
  using A = typename AccOf<T>::type;
  constexpr int N = VEC ? Vec16<T>::N : 1;
  const long long per_outer = inner / N;
  const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (id >= outer * per_outer) return;
  const long long o = id / per_outer;
  const long long iv = id - o * per_outer;
  A acc[N];
#pragma unroll
  for (int j = 0; j < N; ++j) acc[j] = identity_of<A>(AGG);
  const T* src = in + o * red * inner + iv * N;
  for (long long r = 0; r < red; ++r) {
    if constexpr (VEC) {
      const Vec16<T> a = *reinterpret_cast<const Vec16<T>*>(src + r * inner);
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = combine<AGG, A>(acc[j], to_acc<T>(a.v[j]));
    } else {
      acc[0] = combine<AGG, A>(acc[0], to_acc<T>(src[r * inner]));
    }
  }
#pragma unroll
  for (int j = 0; j < N; ++j) {
    A v = acc[j];
    if constexpr (AGG == PMLB_AGG_SUM && sizeof(A) == 4 && static_cast<A>(0.5) != A(0)) {
      if (scale != 1.f) v = scale < 0.f ? v / -scale : v * scale;   // (negative: a divisor)
    }
    out[o * inner + iv * N + j] = from_acc<TO, A>(v);
  }
}

// ------------------------------------------------------------------ NHWC pooling
template <class T, int AGG, bool VEC>
__global__ void __launch_bounds__(256)
pool_kernel(const T* __restrict__ in, T* __restrict__ out, PoolGeom g) {
  using A = typename AccOf<T>::type;
  constexpr int N = VEC ? Vec16<T>::N : 1;
  const int cv = g.c / N;
  const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(g.n) * g.p * g.q * cv;
  if (id >= total) return;
  const int c0 = static_cast<int>(id % cv) * N;
  long long rem = id / cv;
  const int x = static_cast<int>(rem % g.q);
  rem /= g.q;
  const int y = static_cast<int>(rem % g.p);
  const int n = static_cast<int>(rem / g.p);
  A acc[N];
#pragma unroll
  for (int j = 0; j < N; ++j) acc[j] = identity_of<A>(AGG);
  int taps = 0;
  for (int fr = 0; fr < g.r; ++fr) {
    const int iy = y * g.stride_h + fr - g.pad_h;
    if (iy < 0 || iy >= g.h) continue;
    for (int fs = 0; fs < g.s; ++fs) {
      const int ix = x * g.stride_w + fs - g.pad_w;
      if (ix < 0 || ix >= g.w) continue;
      ++taps;
      const T* src = in + ((static_cast<long long>(n) * g.h + iy) * g.w + ix) * g.c + c0;
      if constexpr (VEC) {
        const Vec16<T> a = *reinterpret_cast<const Vec16<T>*>(src);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] = combine<AGG, A>(acc[j], to_acc<T>(a.v[j]));
      } else {
        acc[0] = combine<AGG, A>(acc[0], to_acc<T>(src[0]));
      }
    }
  }
  T* dst = out + ((static_cast<long long>(n) * g.p + y) * g.q + x) * g.c + c0;
  float scale = 1.f;
  if (g.average) scale = 1.f / static_cast<float>(g.include_padding ? g.r * g.s : (taps > 0 ? taps : 1));
  if constexpr (VEC) {
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < N; ++j) {
      A v = acc[j];
      if constexpr (static_cast<A>(0.5) != A(0)) {
        if (g.average) v = v * scale;
      }
      o.v[j] = from_acc<T, A>(v);
    }
    *reinterpret_cast<Vec16<T>*>(dst) = o;
  } else {
    A v = acc[0];
    if constexpr (static_cast<A>(0.5) != A(0)) {
      if (g.average) v = v * scale;
    }
    dst[0] = from_acc<T, A>(v);
  }
}

// Max / min pooling of 16-bit floats on packed pairs: the window's 16-byte groups are combined
// with two-wide max / min instructions in the storage type (no conversion: max and min are
// exact), a quarter of the instructions of the generic kernel, which is bound by instruction
// issue.  One block row (blockIdx.x) per output image row, so that only the position inside
// the row needs a division.  For NaN-free inputs the result equals the compare-and-select
// chain of the definition; a NaN operand is skipped rather than propagated in visiting order.
template <class T2, int AGG>
__device__ __forceinline__ uint32_t combine16x2(uint32_t acc, uint32_t v) {
  const T2 a = *reinterpret_cast<const T2*>(&acc);
  const T2 b = *reinterpret_cast<const T2*>(&v);
  const T2 r = (AGG == PMLB_AGG_MAX) ? __hmax2(a, b) : __hmin2(a, b);
  return *reinterpret_cast<const uint32_t*>(&r);
}

// W = 16-byte groups per thread: 1, or 2 (32-byte loads and stores: 16 channels per thread, half as
// many threads and memory instructions; needs c % 16 == 0 and 32-byte aligned tensors).
template <class T2, int AGG, bool K3X3, int W>
__global__ void __launch_bounds__(256)
pool16_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, PoolGeom g, FastDiv fd_cv,
              FastDiv fd_p, uint32_t identity2) {
  const int cv = g.c / (8 * W);                         // channel groups of one thread's width
  const int pos = blockIdx.y * 256 + threadIdx.x;       // (x, channel group) inside the output row
  if (pos >= g.q * cv) return;
  const int x = fast_div(pos, fd_cv);
  const int cg = pos - x * cv;
  const int row = blockIdx.x;                           // n * p + y
  const int n = fast_div(row, fd_p);
  const int y = row - n * g.p;
  uint32_t acc[4 * W];
#pragma unroll
  for (int j = 0; j < 4 * W; ++j) acc[j] = identity2;
  const int iy0 = y * g.stride_h - g.pad_h, ix0 = x * g.stride_w - g.pad_w;
  const uint4* base = in + ((static_cast<long long>(n) * g.h * g.w) * cv + cg) * W;
  const int r = K3X3 ? 3 : g.r, s = K3X3 ? 3 : g.s;
#pragma unroll
  for (int fr = 0; fr < r; ++fr) {
    const int iy = iy0 + fr;
    if (iy < 0 || iy >= g.h) continue;
#pragma unroll
    for (int fs = 0; fs < s; ++fs) {
      const int ix = ix0 + fs;
      if (ix < 0 || ix >= g.w) continue;
      const uint4* src = base + (static_cast<long long>(iy) * g.w + ix) * cv * W;
      uint32_t v[4 * W];
      if constexpr (W == 2) {
        asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                     : "l"(src));
      } else {
        const uint4 a = __ldg(src);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
      }
#pragma unroll
      for (int j = 0; j < 4 * W; ++j) acc[j] = combine16x2<T2, AGG>(acc[j], v[j]);
    }
  }
  uint4* dst = out + ((static_cast<long long>(row) * g.q + x) * cv + cg) * W;
  if constexpr (W == 2) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 :
                 : "l"(dst), "r"(acc[0]), "r"(acc[1]), "r"(acc[2]), "r"(acc[3]), "r"(acc[4]), "r"(acc[5]), "r"(acc[6]), "r"(acc[7])
                 : "memory");
  } else {
    dst[0] = make_uint4(acc[0], acc[1], acc[2], acc[3]);
  }
}

template <class T2, int W>
cudaError_t launch_pool16_w(const PoolGeom& g, const void* in, void* out, uint32_t neg_inf2,
                            uint32_t pos_inf2, cudaStream_t stream) {
  const int cv = g.c / (8 * W);
  const long long rows = static_cast<long long>(g.n) * g.p;
  const long long per_row = static_cast<long long>(g.q) * cv;
  if (rows > 0x7fffffffLL || (per_row + 255) / 256 > 65535) return cudaErrorInvalidValue;
  dim3 grid(static_cast<unsigned>(rows), static_cast<unsigned>((per_row + 255) / 256));
  const FastDiv fc = make_fastdiv(static_cast<uint32_t>(cv)), fp = make_fastdiv(static_cast<uint32_t>(g.p));
  const uint4* ip = static_cast<const uint4*>(in);
  uint4* op = static_cast<uint4*>(out);
  const bool k3 = g.r == 3 && g.s == 3;
  if (g.agg == PMLB_AGG_MAX) {
    if (k3) pool16_kernel<T2, PMLB_AGG_MAX, true, W><<<grid, 256, 0, stream>>>(ip, op, g, fc, fp, neg_inf2);
    else pool16_kernel<T2, PMLB_AGG_MAX, false, W><<<grid, 256, 0, stream>>>(ip, op, g, fc, fp, neg_inf2);
  } else {
    if (k3) pool16_kernel<T2, PMLB_AGG_MIN, true, W><<<grid, 256, 0, stream>>>(ip, op, g, fc, fp, pos_inf2);
    else pool16_kernel<T2, PMLB_AGG_MIN, false, W><<<grid, 256, 0, stream>>>(ip, op, g, fc, fp, pos_inf2);
  }
  return cudaGetLastError();
}

template <class T2>
cudaError_t launch_pool16(const PoolGeom& g, const void* in, void* out, uint32_t neg_inf2,
                          uint32_t pos_inf2, cudaStream_t stream) {
  const bool wide = g.c % 16 == 0 && (reinterpret_cast<uintptr_t>(in) & 31u) == 0 &&
                    (reinterpret_cast<uintptr_t>(out) & 31u) == 0;
  return wide ? launch_pool16_w<T2, 2>(g, in, out, neg_inf2, pos_inf2, stream)
              : launch_pool16_w<T2, 1>(g, in, out, neg_inf2, pos_inf2, stream);
}

template <class T, class TO, bool VEC>
cudaError_t launch_reduce_t(int agg, const void* in, void* out, long long outer, long long red,
                            long long inner, float scale, cudaStream_t stream) {
  const T* ip = static_cast<const T*>(in);
  TO* op = static_cast<TO*>(out);
  if (inner == 1) {
    const unsigned grid = static_cast<unsigned>((outer + 7) / 8);
    switch (agg) {
      case PMLB_AGG_MAX: row_reduce_kernel<T, TO, PMLB_AGG_MAX, VEC><<<grid, 256, 0, stream>>>(ip, op, outer, red, scale); break;
      case PMLB_AGG_MIN: row_reduce_kernel<T, TO, PMLB_AGG_MIN, VEC><<<grid, 256, 0, stream>>>(ip, op, outer, red, scale); break;
      default: row_reduce_kernel<T, TO, PMLB_AGG_SUM, VEC><<<grid, 256, 0, stream>>>(ip, op, outer, red, scale); break;
    }
  } else {
    constexpr int N = VEC ? Vec16<T>::N : 1;
    const long long threads = outer * (inner / N);
    const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
    switch (agg) {
      case PMLB_AGG_MAX: strided_reduce_kernel<T, TO, PMLB_AGG_MAX, VEC><<<grid, 256, 0, stream>>>(ip, op, outer, red, inner, scale); break;
      case PMLB_AGG_MIN: strided_reduce_kernel<T, TO, PMLB_AGG_MIN, VEC><<<grid, 256, 0, stream>>>(ip, op, outer, red, inner, scale); break;
      default: strided_reduce_kernel<T, TO, PMLB_AGG_SUM, VEC><<<grid, 256, 0, stream>>>(ip, op, outer, red, inner, scale); break;
    }
  }
  return cudaGetLastError();
}

template <class T, class TO>
cudaError_t launch_reduce_v(int agg, const void* in, void* out, long long outer, long long red,
                            long long inner, float scale, cudaStream_t stream) {
  constexpr int N = 16 / sizeof(T);
  const bool aligned = (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
  const bool vec = aligned && (inner == 1 ? (red % N == 0) : (inner % N == 0));
  return vec ? launch_reduce_t<T, TO, true>(agg, in, out, outer, red, inner, scale, stream)
             : launch_reduce_t<T, TO, false>(agg, in, out, outer, red, inner, scale, stream);
}

template <class T, bool VEC>
cudaError_t launch_pool_t(const PoolGeom& g, const void* in, void* out, cudaStream_t stream) {
  constexpr int N = VEC ? static_cast<int>(16 / sizeof(T)) : 1;
  const long long threads = static_cast<long long>(g.n) * g.p * g.q * (g.c / N);
  const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
  const T* ip = static_cast<const T*>(in);
  T* op = static_cast<T*>(out);
  switch (g.agg) {
    case PMLB_AGG_MAX: pool_kernel<T, PMLB_AGG_MAX, VEC><<<grid, 256, 0, stream>>>(ip, op, g); break;
    case PMLB_AGG_MIN: pool_kernel<T, PMLB_AGG_MIN, VEC><<<grid, 256, 0, stream>>>(ip, op, g); break;
    default: pool_kernel<T, PMLB_AGG_SUM, VEC><<<grid, 256, 0, stream>>>(ip, op, g); break;
  }
  return cudaGetLastError();
}

template <class T>
cudaError_t launch_pool_v(const PoolGeom& g, const void* in, void* out, cudaStream_t stream) {
  constexpr int N = 16 / sizeof(T);
  const bool vec = (g.c % N == 0) && (reinterpret_cast<uintptr_t>(in) & 15u) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
  if constexpr (sizeof(T) == 2) {
    // 16-bit floats, max / min: packed-pair kernel (falls through if the grid would not fit)
    if (vec && (g.agg == PMLB_AGG_MAX || g.agg == PMLB_AGG_MIN)) {
      cudaError_t e;
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        e = launch_pool16<__nv_bfloat162>(g, in, out, 0xFF80FF80u, 0x7F807F80u, stream);
      } else {
        e = launch_pool16<__half2>(g, in, out, 0xFC00FC00u, 0x7C007C00u, stream);
      }
      if (e != cudaErrorInvalidValue) return e;
    }
  }
  return vec ? launch_pool_t<T, true>(g, in, out, stream) : launch_pool_t<T, false>(g, in, out, stream);
}

}  // namespace

bool reduce_supported(int agg, int dtype, int out_dtype) {
  if (agg != PMLB_AGG_MAX && agg != PMLB_AGG_MIN && agg != PMLB_AGG_SUM) return false;
  if (dtype == out_dtype) {
    return dtype == PMLB_F32 || dtype == PMLB_BF16 || dtype == PMLB_F16 || dtype == PMLB_I32 ||
           dtype == PMLB_I8;
  }
  return out_dtype == PMLB_F32 && (dtype == PMLB_BF16 || dtype == PMLB_F16);
}

cudaError_t launch_reduce(int agg, int dtype, int out_dtype, const void* in, void* out,
                          long long outer, long long red, long long inner, float scale,
                          cudaStream_t stream) {
  if (outer <= 0 || inner <= 0) return cudaSuccess;
  if (dtype == out_dtype) {
    switch (dtype) {
      case PMLB_F32: return launch_reduce_v<float, float>(agg, in, out, outer, red, inner, scale, stream);
      case PMLB_BF16: return launch_reduce_v<__nv_bfloat16, __nv_bfloat16>(agg, in, out, outer, red, inner, scale, stream);
      case PMLB_F16: return launch_reduce_v<__half, __half>(agg, in, out, outer, red, inner, scale, stream);
      case PMLB_I32: return launch_reduce_v<int32_t, int32_t>(agg, in, out, outer, red, inner, scale, stream);
      case PMLB_I8: return launch_reduce_v<int8_t, int8_t>(agg, in, out, outer, red, inner, scale, stream);
      default: return cudaErrorInvalidValue;
    }
  }
  if (out_dtype == PMLB_F32 && dtype == PMLB_BF16) {
    return launch_reduce_v<__nv_bfloat16, float>(agg, in, out, outer, red, inner, scale, stream);
  }
  if (out_dtype == PMLB_F32 && dtype == PMLB_F16) {
    return launch_reduce_v<__half, float>(agg, in, out, outer, red, inner, scale, stream);
  }
  return cudaErrorInvalidValue;
}

bool pool_supported(int agg, int dtype) {
  if (agg != PMLB_AGG_MAX && agg != PMLB_AGG_MIN && agg != PMLB_AGG_SUM) return false;
  return dtype == PMLB_F32 || dtype == PMLB_BF16 || dtype == PMLB_F16 || dtype == PMLB_I32 ||
         dtype == PMLB_I8;
}

cudaError_t launch_pool(const PoolGeom& g, int dtype, const void* in, void* out,
                        cudaStream_t stream) {
  if (static_cast<long long>(g.n) * g.p * g.q * g.c <= 0) return cudaSuccess;
  switch (dtype) {
    case PMLB_F32: return launch_pool_v<float>(g, in, out, stream);
    case PMLB_BF16: return launch_pool_v<__nv_bfloat16>(g, in, out, stream);
    case PMLB_F16: return launch_pool_v<__half>(g, in, out, stream);
    case PMLB_I32: return launch_pool_v<int32_t>(g, in, out, stream);
    case PMLB_I8: return launch_pool_v<int8_t>(g, in, out, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace pmlb
