// The four tile operations that are not contractions: gather, scatter, argsort, prng.  All of them move bytes and
// indices and wait on memory, so the kernels keep several independent loads per thread in flight and do their position
// arithmetic in 32 bits where the extents allow.
//
// gather    integer positions copy elements -- whole runs of the inner dims as 16-byte pieces, four pieces per thread;
//           float positions interpolate in the tensor's float type with a rounding after every operation, so an
//           f16 / bf16 / f32 / f64 result is what scalar code in that type gives (four results per thread: positions,
//           then all neighbour loads, then the blends).
// scatter   the result starts as a copy of the data (a device copy issued by the launcher side), then every update adds
//           (atomically) or stores; whole rows named by a list of indices go four updates per thread.
// argsort   runs of up to 4096 positions are sorted in shared memory by one block (a bitonic network over (key,
//           position) pairs: a total order, so ties keep their original order; keys of at most 32 bits share a 64-bit
//           word with the position).  Longer lines go on with stable merge passes between two int32 buffers: pass w
//           merges runs of w positions into runs of 2w, every element finding its place by a binary search in the
//           sibling run (elements of the left run go before equal elements of the right run).
// prng      three linear shift-register generators; a thread jumps its generators to its first element by applying
//           precomputed powers of the step matrices over GF(2), then steps through its run, eight numbers per pair of
//           16-byte stores.
#include "special.h"

#include <math.h>

#include "typed_access.cuh"

namespace pmlb {

namespace {

__device__ __forceinline__ void copy_element(void* dst, long long di, const void* src, long long si, int bytes) {
  switch (bytes) {
    case 1: static_cast<uint8_t*>(dst)[di] = static_cast<const uint8_t*>(src)[si]; break;
    case 2: static_cast<uint16_t*>(dst)[di] = static_cast<const uint16_t*>(src)[si]; break;
    case 4: static_cast<uint32_t*>(dst)[di] = static_cast<const uint32_t*>(src)[si]; break;
    case 8: static_cast<unsigned long long*>(dst)[di] = static_cast<const unsigned long long*>(src)[si]; break;
    default: static_cast<uint4*>(dst)[di] = static_cast<const uint4*>(src)[si]; break;  // 16: several elements at once
  }
}

__device__ __forceinline__ long long clamp_ll(long long v, long long lo, long long hi) {
  return v < lo ? lo : (v > hi ? hi : v);
}

// Float -> int32 as the lowering's fptosi (towards zero); where that is undefined the conversion saturates and a
// NaN gives 0.
__device__ __forceinline__ long long to_i32(double v) { return __double2int_rz(v); }
__device__ __forceinline__ long long to_i32(float v) { return __float2int_rz(v); }

// ------------------------------------------------------------------ arithmetic classes of the interpolation

struct ArF32 {
  using T = float;
  enum : int { kDtype = PMLB_F32 };
  static __device__ __forceinline__ T r(T x) { return x; }
  static __device__ __forceinline__ T load(const void* b, long long i) { return static_cast<const float*>(b)[i]; }
  static __device__ __forceinline__ void store(void* b, long long i, T v) { static_cast<float*>(b)[i] = v; }
};
struct ArF16 {
  using T = float;
  enum : int { kDtype = PMLB_F16 };
  static __device__ __forceinline__ T r(T x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ T load(const void* b, long long i) { return __half2float(static_cast<const __half*>(b)[i]); }
  static __device__ __forceinline__ void store(void* b, long long i, T v) { static_cast<__half*>(b)[i] = __float2half_rn(v); }
};
struct ArBF16 {
  using T = float;
  enum : int { kDtype = PMLB_BF16 };
  static __device__ __forceinline__ T r(T x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  static __device__ __forceinline__ T load(const void* b, long long i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(b)[i]);
  }
  static __device__ __forceinline__ void store(void* b, long long i, T v) {
    static_cast<__nv_bfloat16*>(b)[i] = __float2bfloat16_rn(v);
  }
};
struct ArF64 {
  using T = double;
  enum : int { kDtype = PMLB_F64 };
  static __device__ __forceinline__ T r(T x) { return x; }
  static __device__ __forceinline__ T load(const void* b, long long i) { return static_cast<const double*>(b)[i]; }
  static __device__ __forceinline__ void store(void* b, long long i, T v) { static_cast<double*>(b)[i] = v; }
};

__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }

template <class A>
struct Arith {
  using T = typename A::T;
  static __device__ __forceinline__ T mul(T a, T b) { return A::r(mul_rn(a, b)); }
  static __device__ __forceinline__ T add(T a, T b) { return A::r(add_rn(a, b)); }
  static __device__ __forceinline__ T sub(T a, T b) { return A::r(add_rn(a, -b)); }
};

// An interpolated value in two parts, so that a thread can have the loads of several values in flight: the axis
// positions the value reads (1 for nearest, 2 for linear, 4 for cubic; clamped to the axis) ...
template <class A>
__device__ __forceinline__ void neighbours(const GatherParams& p, typename A::T idx, long long pos[4]) {
  using T = typename A::T;
  const long long hi = p.axis_len - 1;
  const T fl = floor(idx);
  if (p.interpolation == 0) {
    long long i;
    const bool half = idx == A::r(add_rn(fl, T(0.5)));
    const long long rounded = to_i32(floor(A::r(add_rn(idx, T(0.5)))));
    switch (p.nearest) {
      case 0: i = half ? to_i32(fl) : rounded; break;
      case 1: i = half ? to_i32(ceil(idx)) : rounded; break;
      case 2: i = to_i32(fl); break;
      case 3: i = to_i32(ceil(idx)); break;
      default: i = to_i32(idx); break;
    }
    pos[0] = clamp_ll(i, 0, hi);
  } else if (p.interpolation == 1) {
    pos[0] = clamp_ll(to_i32(ceil(idx)), 0, hi);
    pos[1] = clamp_ll(to_i32(fl), 0, hi);
  } else {
    const long long fi = to_i32(fl), ci = to_i32(ceil(idx));
    pos[0] = clamp_ll(fi - 1, 0, hi);
    pos[1] = clamp_ll(fi, 0, hi);
    pos[2] = clamp_ll(ci, 0, hi);
    pos[3] = clamp_ll(ci + 1, 0, hi);
  }
}

// ... and the value from the elements at those positions.
template <class A>
__device__ __forceinline__ typename A::T blend(const GatherParams& p, typename A::T idx, const typename A::T g[4]) {
  using T = typename A::T;
  using M = Arith<A>;
  const T fl = floor(idx);
  T result;
  if (p.interpolation == 0) {
    result = g[0];
  } else if (p.interpolation == 1) {
    const T c0 = M::sub(idx, fl);
    const T c1 = M::sub(T(1), c0);
    result = M::add(M::mul(c0, g[0]), M::mul(c1, g[1]));
  } else {
    const T a = A::r(static_cast<T>(p.cube_coeff));
    const T s = M::sub(idx, fl);
    const T s2 = M::mul(s, s);
    const T s3 = M::mul(s2, s);
    const T s_a = M::mul(a, s);
    const T s2_a = M::mul(a, s2);
    const T s3_a = M::mul(a, s3);
    const T s3_a2 = M::mul(M::add(a, T(2)), s3);
    const T s2_a3 = M::mul(M::add(a, T(3)), s2);
    const T s2_2a3 = M::mul(M::add(M::add(a, a), T(3)), s2);
    const T p0 = M::add(M::sub(s3_a, M::mul(s2_a, T(2))), s_a);
    const T p1 = M::add(M::sub(s3_a2, s2_a3), T(1));
    const T p2 = M::sub(M::sub(s2_2a3, s3_a2), s_a);
    const T p3 = M::sub(s2_a, s3_a);
    result = M::add(M::add(M::add(M::mul(p0, g[0]), M::mul(p1, g[1])), M::mul(p2, g[2])), M::mul(p3, g[3]));
  }
  if (p.out_of_bounds == 1 && (idx > static_cast<T>(p.axis_len - 1) || idx < T(0))) result = T(0);
  return result;
}

// Interpolating gather along one axis: four results per thread, a grid apart, computed into registers before any of
// them is stored, so that the four chains position -> neighbours -> value are in flight together.
template <class A, class I>
__global__ void __launch_bounds__(256) gather_interp_kernel(const __grid_constant__ GatherParams p, I threads) {
  using T = typename A::T;
  const I t = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= threads) return;
  const I total = static_cast<I>(p.out_elems);
  const I inner = static_cast<I>(p.inner);
  const I n_idx = static_cast<I>(p.n_idx);
  const bool one_outer = total == inner * n_idx;
  const bool same_type = p.idx_dtype == A::kDtype;
  const int reads = p.interpolation == 0 ? 1 : (p.interpolation == 1 ? 2 : 4);
  T idx[4];
  long long base[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    I e = t + static_cast<I>(u) * threads;
    if (e >= total) e = total - 1;   // (a spare slot repeats the last element; it is not stored)
    const I in = inner == 1 ? 0 : e % inner;
    const I row = inner == 1 ? e : e / inner;
    const I j = one_outer ? row : row % n_idx;
    const I o = one_outer ? 0 : row / n_idx;
    base[u] = static_cast<long long>(o) * p.axis_len * p.inner + in;
    idx[u] = same_type ? A::load(p.indices, j) : A::r(load_as<T>(p.indices, p.idx_dtype, j));
  }
  T g[4][4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    long long pos[4] = {0, 0, 0, 0};
    neighbours<A>(p, idx[u], pos);
#pragma unroll
    for (int k = 0; k < 4; ++k) g[u][k] = k < reads ? A::load(p.tensor, base[u] + pos[k] * p.inner) : T(0);
  }
  T res[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) res[u] = blend<A>(p, idx[u], g[u]);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const I e = t + static_cast<I>(u) * threads;
    if (e < total) A::store(p.out, e, res[u]);
  }
}

// Copying gather along one axis in 16-byte pieces: four pieces per thread, a grid apart, all four positions read
// before any piece is loaded and all four pieces loaded before any is stored (the kernel waits on memory, not on
// arithmetic: one piece per thread left DRAM at half its rate).
template <class I>
__global__ void __launch_bounds__(256) gather_pieces_kernel(const __grid_constant__ GatherParams p, I threads) {
  const I t = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= threads) return;
  const I total = static_cast<I>(p.out_elems);
  const I inner = static_cast<I>(p.inner);
  const I n_idx = static_cast<I>(p.n_idx);
  const bool one_outer = total == inner * n_idx;
  const bool float_idx = dtype_is_float(p.idx_dtype);
  long long src[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    I e = t + static_cast<I>(u) * threads;
    if (e >= total) e = total - 1;   // (a spare slot repeats the last piece; it is not stored)
    const I in = inner == 1 ? 0 : e % inner;
    const I row = inner == 1 ? e : e / inner;
    const I j = one_outer ? row : row % n_idx;
    const I o = one_outer ? 0 : row / n_idx;
    const long long at = float_idx ? to_i32(load_as<double>(p.indices, p.idx_dtype, j))
                                   : load_as<long long>(p.indices, p.idx_dtype, j);
    src[u] = (static_cast<long long>(o) * p.axis_len + clamp_ll(at, 0, p.axis_len - 1)) * p.inner + in;
  }
  uint4 piece[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) piece[u] = static_cast<const uint4*>(p.tensor)[src[u]];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const I e = t + static_cast<I>(u) * threads;
    if (e < total) static_cast<uint4*>(p.out)[e] = piece[u];
  }
}

// Copying gather (integer positions, nd mode).  `I` is the type of the position arithmetic: 32 bits when every extent
// fits, else 64.
template <class I>
__global__ void __launch_bounds__(256) gather_kernel(const __grid_constant__ GatherParams p) {
  const I e = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= static_cast<I>(p.out_elems)) return;
  const I inner = static_cast<I>(p.inner);
  const I in = inner == 1 ? 0 : e % inner;
  const I row = inner == 1 ? e : e / inner;
  if (p.nd) {
    const I per_batch = static_cast<I>(p.rows_per_batch);
    long long off = per_batch == 1 ? row : row / per_batch;
    for (int k = 0; k < p.k; ++k) {
      const long long i = clamp_ll(load_as<long long>(p.indices, p.idx_dtype, static_cast<long long>(row) * p.k + k), 0,
                                   p.dims[k] - 1);
      off = off * p.dims[k] + i;
    }
    copy_element(p.out, e, p.tensor, off * p.inner + in, p.elem_bytes);
    return;
  }
  const I n_idx = static_cast<I>(p.n_idx);
  const bool one_outer = static_cast<I>(p.out_elems) == inner * n_idx;
  const I j = one_outer ? row : row % n_idx;
  const I o = one_outer ? 0 : row / n_idx;
  const long long src_base = static_cast<long long>(o) * p.axis_len * p.inner + in;
  // integer positions select; float positions into an integer tensor are truncated
  const long long at = dtype_is_float(p.idx_dtype) ? to_i32(load_as<double>(p.indices, p.idx_dtype, j))
                                                   : load_as<long long>(p.indices, p.idx_dtype, j);
  copy_element(p.out, e, p.tensor, src_base + clamp_ll(at, 0, p.axis_len - 1) * p.inner, p.elem_bytes);
}

// ------------------------------------------------------------------ scatter

// out[i] += updates[u] for 8- and 16-bit element types: compare-and-swap on the aligned word that holds the element.
__device__ __forceinline__ void atomic_add_narrow(void* base, int dtype, long long i, const void* upd, long long u,
                                                  int bytes) {
  const uintptr_t addr = reinterpret_cast<uintptr_t>(base) + static_cast<uintptr_t>(i) * bytes;
  unsigned* word = reinterpret_cast<unsigned*>(addr & ~static_cast<uintptr_t>(3));
  const unsigned shift = static_cast<unsigned>(addr & 3) * 8;
  const unsigned mask = (bytes == 1 ? 0xFFu : 0xFFFFu) << shift;
  unsigned add_bits;
  if (bytes == 1) add_bits = static_cast<const uint8_t*>(upd)[u];
  else add_bits = static_cast<const uint16_t*>(upd)[u];
  unsigned old = *word, assumed;
  do {
    assumed = old;
    const unsigned cur = (assumed & mask) >> shift;
    unsigned next;
    if (dtype == PMLB_F16) {
      const float s = __half2float(__ushort_as_half(static_cast<unsigned short>(cur))) +
                      __half2float(__ushort_as_half(static_cast<unsigned short>(add_bits)));
      next = __half_as_ushort(__float2half_rn(s));
    } else if (dtype == PMLB_BF16) {
      const float s = __bfloat162float(__ushort_as_bfloat16(static_cast<unsigned short>(cur))) +
                      __bfloat162float(__ushort_as_bfloat16(static_cast<unsigned short>(add_bits)));
      next = __bfloat16_as_ushort(__float2bfloat16_rn(s));
    } else if (dtype == PMLB_BOOL) {
      next = (cur + add_bits) != 0 ? 1u : 0u;
    } else {
      next = cur + add_bits;  // integers wrap
    }
    next = (next << shift) & mask;
    old = atomicCAS(word, assumed, (assumed & ~mask) | next);
  } while (old != assumed);
}

__device__ __forceinline__ void atomic_add_element(void* out, int dtype, long long i, const void* upd, long long u,
                                                   int bytes) {
  switch (dtype) {
    case PMLB_F32: atomicAdd(static_cast<float*>(out) + i, static_cast<const float*>(upd)[u]); break;
    case PMLB_F64: atomicAdd(static_cast<double*>(out) + i, static_cast<const double*>(upd)[u]); break;
    case PMLB_I32:
    case PMLB_U32: atomicAdd(static_cast<unsigned*>(out) + i, static_cast<const unsigned*>(upd)[u]); break;
    case PMLB_I64:
    case PMLB_U64:
      atomicAdd(static_cast<unsigned long long*>(out) + i, static_cast<const unsigned long long*>(upd)[u]);
      break;
    default: atomic_add_narrow(out, dtype, i, upd, u, bytes); break;
  }
}

// The common form -- whole rows of the data named by a list of indices (axis 0, updates [n][row...]) -- with four
// updates per thread, a grid apart: the four index and update loads are in flight together, and the additions leave
// as fire-and-forget reductions.
__global__ void __launch_bounds__(256) scatter_rows_kernel(const __grid_constant__ ScatterParams p, long long inner,
                                                           long long threads) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= threads) return;
  long long row[4], dst[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    long long e = t + u * threads;
    if (e >= p.upd_elems) e = p.upd_elems - 1;
    row[u] = inner == 1 ? e : e / inner;
    dst[u] = e - row[u] * inner;
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) row[u] = load_as<long long>(p.indices, p.idx_dtype, row[u]);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const long long e = t + u * threads;
    if (e >= p.upd_elems || row[u] < 0 || row[u] >= p.sizes[0]) continue;   // spare slot, or lands outside the data
    const long long off = row[u] * inner + dst[u];
    if (p.mode == 0) atomic_add_element(p.out, p.dtype, off, p.updates, e, p.elem_bytes);
    else copy_element(p.out, off, p.updates, e, p.elem_bytes);
  }
}

__global__ void __launch_bounds__(256) scatter_kernel(const __grid_constant__ ScatterParams p) {
  const long long u = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (u >= p.upd_elems) return;
  long long c[PMLB_MAX_RANK];
  long long rem = u;
  for (int d = p.upd_rank - 1; d >= 0; --d) {
    c[d] = rem % p.upd_sizes[d];
    rem /= p.upd_sizes[d];
  }
  long long dst[PMLB_MAX_RANK];
  int nd = 0;
  if (p.mode == 3) {
    // the first idx_rank - 1 coordinates pick a row of indices; its K entries lead the destination
    const int k = static_cast<int>(p.idx_sizes[p.idx_rank - 1]);
    long long row = 0;
    for (int d = 0; d < p.idx_rank - 1; ++d) row = row * p.idx_sizes[d] + c[d];
    for (int i = 0; i < k; ++i) dst[nd++] = load_as<long long>(p.indices, p.idx_dtype, row * k + i);
    for (int d = p.idx_rank - 1; d < p.upd_rank; ++d) dst[nd++] = c[d];
  } else {
    const int first = p.mode == 1 ? p.axis : 0;                       // coordinates that address the indices
    const int tail = p.mode == 1 ? p.axis + p.idx_rank - 1 : p.axis;  // the axis coordinate and what follows it
    long long at = 0;
    for (int d = 0; d < p.idx_rank; ++d) at = at * p.idx_sizes[d] + c[first + d];
    for (int d = 0; d < p.axis; ++d) dst[nd++] = c[d];
    for (int d = tail; d < p.upd_rank; ++d) dst[nd++] = c[d];
    dst[p.axis] = load_as<long long>(p.indices, p.idx_dtype, at);
  }
  long long off = 0;
  for (int d = 0; d < p.rank; ++d) {
    if (dst[d] < 0 || dst[d] >= p.sizes[d]) return;  // lands outside the data: dropped
    off = off * p.sizes[d] + dst[d];
  }
  if (p.mode == 0) atomic_add_element(p.out, p.dtype, off, p.updates, u, p.elem_bytes);
  else copy_element(p.out, off, p.updates, u, p.elem_bytes);
}

// ------------------------------------------------------------------ argsort

// One merge pass over lines longer than a block sorts: `src` holds positions in sorted runs of `w`, `dst` receives
// them in sorted runs of 2 w.
template <class V>
__global__ void __launch_bounds__(256) argsort_pass_kernel(const __grid_constant__ ArgsortParams p,
                                                           const int32_t* __restrict__ src, int32_t* __restrict__ dst,
                                                           long long w, long long total) {
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const long long in = e % p.inner;
  const long long j = (e / p.inner) % p.n;
  const long long line = (e / (p.inner * p.n)) * p.n * p.inner + in;  // element q of the line is at line + q * inner
  auto pos_at = [&](long long q) -> long long { return src[line + q * p.inner]; };
  auto key_at = [&](long long q) -> V { return load_as<V>(p.tensor, p.dtype, line + pos_at(q) * p.inner); };
  auto before = [&](V a, V b) -> bool { return p.descending ? a > b : a < b; };
  const long long base = (j / (2 * w)) * 2 * w;
  const long long mid = base + w < p.n ? base + w : p.n;
  const long long end = base + 2 * w < p.n ? base + 2 * w : p.n;
  const V key = key_at(j);
  long long lo, hi, dest;
  if (j < mid) {
    // elements of the right run that go strictly before this one
    lo = mid;
    hi = end;
    while (lo < hi) {
      const long long m = (lo + hi) >> 1;
      if (before(key_at(m), key)) lo = m + 1; else hi = m;
    }
    dest = j + (lo - mid);
  } else {
    // elements of the left run that do not go after this one
    lo = base;
    hi = mid;
    while (lo < hi) {
      const long long m = (lo + hi) >> 1;
      if (before(key, key_at(m))) hi = m; else lo = m + 1;
    }
    dest = (lo - base) + (j - mid) + base;
  }
  dst[line + dest * p.inner] = static_cast<int32_t>(pos_at(j));
}

// Sorts segments of up to kSortSlots positions in shared memory (a bitonic network over (key, position) pairs, so the
// order is total and ties keep their original order): whole lines when they fit -- several short lines per block --
// or 4096-position runs of longer lines, which the merge passes above then combine.
enum : int { kSortSlots = 4096, kSortThreads = 512 };

template <class V>
__global__ void __launch_bounds__(kSortThreads) argsort_block_kernel(const __grid_constant__ ArgsortParams p,
                                                                     int32_t* __restrict__ dst, int seg_len,
                                                                     long long segs_per_line, long long segments) {
  __shared__ V keys[kSortSlots];
  __shared__ int32_t pos[kSortSlots];
  const int segs_per_block = kSortSlots / seg_len;
  const long long first_seg = static_cast<long long>(blockIdx.x) * segs_per_block;
  auto line_base = [&](long long line) { return (line / p.inner) * p.n * p.inner + line % p.inner; };
  for (int s = threadIdx.x; s < kSortSlots; s += kSortThreads) {
    const long long seg = first_seg + s / seg_len;
    const long long q = (seg % segs_per_line) * seg_len + s % seg_len;
    const bool valid = seg < segments && q < p.n;
    pos[s] = valid ? static_cast<int32_t>(q) : 0x7FFFFFFF;   // (an empty slot sorts behind every element)
    keys[s] = valid ? load_as<V>(p.tensor, p.dtype, line_base(seg / segs_per_line) + q * p.inner) : V(0);
  }
  __syncthreads();
  auto goes_first = [&](int a, int b) -> bool {   // slot a's element before slot b's
    if (pos[a] == 0x7FFFFFFF) return false;
    if (pos[b] == 0x7FFFFFFF) return true;
    const V ka = keys[a], kb = keys[b];
    if (p.descending ? ka > kb : ka < kb) return true;
    if (p.descending ? kb > ka : kb < ka) return false;
    return pos[a] < pos[b];
  };
  for (int size = 2; size <= seg_len; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < kSortSlots / 2; t += kSortThreads) {
        const int a = 2 * t - (t & (stride - 1));
        const int b = a + stride;
        const bool up = (a & (seg_len - 1) & size) == 0;   // this pair's run is being ordered forwards (the last
                                                           // stage orders every segment forwards)
        if (goes_first(b, a) == up) {
          const V k = keys[a];
          keys[a] = keys[b];
          keys[b] = k;
          const int32_t q = pos[a];
          pos[a] = pos[b];
          pos[b] = q;
        }
      }
      __syncthreads();
    }
  }
  for (int s = threadIdx.x; s < kSortSlots; s += kSortThreads) {
    const long long seg = first_seg + s / seg_len;
    const long long q = (seg % segs_per_line) * seg_len + s % seg_len;
    if (seg < segments && q < p.n) dst[line_base(seg / segs_per_line) + q * p.inner] = pos[s];
  }
}

// The same network for element types of at most 32 bits: key and position share one 64-bit word -- an order-preserving
// 32-bit image of the element (inverted for a descending sort) above the position -- so that one integer comparison
// orders a pair, ties by position included.  -0.0 is ordered as +0.0 (they compare equal); NaNs go to the ends.
__device__ __forceinline__ uint32_t sortable_bits(const void* base, int dtype, long long i) {
  switch (dtype) {
    case PMLB_F32:
    case PMLB_F16:
    case PMLB_BF16: {
      float f = load_as<float>(base, dtype, i);
      if (f == 0.0f) f = 0.0f;
      const uint32_t u = __float_as_uint(f);
      return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    }
    case PMLB_U32:
    case PMLB_U16:
    case PMLB_U8:
    case PMLB_BOOL: return static_cast<uint32_t>(load_as<long long>(base, dtype, i));
    default: return static_cast<uint32_t>(load_as<long long>(base, dtype, i)) ^ 0x80000000u;   // signed integers
  }
}

__global__ void __launch_bounds__(kSortThreads) argsort_block32_kernel(const __grid_constant__ ArgsortParams p,
                                                                       int32_t* __restrict__ dst, int seg_len,
                                                                       long long segs_per_line, long long segments) {
  __shared__ unsigned long long slot[kSortSlots];
  const int segs_per_block = kSortSlots / seg_len;
  const long long first_seg = static_cast<long long>(blockIdx.x) * segs_per_block;
  auto line_base = [&](long long line) { return (line / p.inner) * p.n * p.inner + line % p.inner; };
  for (int s = threadIdx.x; s < kSortSlots; s += kSortThreads) {
    const long long seg = first_seg + s / seg_len;
    const long long q = (seg % segs_per_line) * seg_len + s % seg_len;
    unsigned long long v = ~0ull;   // an empty slot sorts behind every element
    if (seg < segments && q < p.n) {
      uint32_t key = sortable_bits(p.tensor, p.dtype, line_base(seg / segs_per_line) + q * p.inner);
      if (p.descending) key = ~key;
      v = (static_cast<unsigned long long>(key) << 32) | static_cast<uint32_t>(q);
    }
    slot[s] = v;
  }
  __syncthreads();
  for (int size = 2; size <= seg_len; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < kSortSlots / 2; t += kSortThreads) {
        const int a = 2 * t - (t & (stride - 1));
        const int b = a + stride;
        const bool up = (a & (seg_len - 1) & size) == 0;
        const unsigned long long va = slot[a], vb = slot[b];
        if ((vb < va) == up) {
          slot[a] = vb;
          slot[b] = va;
        }
      }
      __syncthreads();
    }
  }
  for (int s = threadIdx.x; s < kSortSlots; s += kSortThreads) {
    const long long seg = first_seg + s / seg_len;
    const long long q = (seg % segs_per_line) * seg_len + s % seg_len;
    if (seg < segments && q < p.n) dst[line_base(seg / segs_per_line) + q * p.inner] = static_cast<int32_t>(slot[s]);
  }
}

// ------------------------------------------------------------------ prng

__host__ __device__ __forceinline__ uint32_t prng_step(int c, uint32_t s) {
  switch (c) {
    case 0: return ((s & 4294967294u) << 12) ^ (((s << 13) ^ s) >> 19);
    case 1: return ((s & 4294967288u) << 4) ^ (((s << 2) ^ s) >> 25);
    default: return ((s & 4294967280u) << 17) ^ (((s << 3) ^ s) >> 11);
  }
}

__host__ __device__ __forceinline__ uint32_t gf2_apply(const uint32_t* cols, uint32_t x) {
  uint32_t y = 0;
  for (int b = 0; b < 32; ++b) {
    if ((x >> b) & 1u) y ^= cols[b];
  }
  return y;
}

// The same product from the matrix stored as eight 16-entry tables, one per 4-bit group of x.
__host__ __device__ __forceinline__ uint32_t gf2_apply_groups(const uint32_t* groups, uint32_t x) {
  uint32_t y = 0;
#pragma unroll
  for (int n = 0; n < 8; ++n) y ^= groups[n * 16 + ((x >> (4 * n)) & 15u)];
  return y;
}

__device__ __forceinline__ uint32_t prng_jump(const uint32_t* table, int c, uint32_t s, unsigned long long steps) {
  for (int level = 0; level < kPrngLevels && steps != 0; ++level, steps >>= 1) {
    if (steps & 1ull) s = gf2_apply_groups(table + (c * kPrngLevels + level) * kPrngNibbleWords, s);
  }
  return s;
}

// Every thread produces `chunk` consecutive numbers (a multiple of 8), eight at a time so that each 32-byte sector of
// the result is written whole by one thread.
__global__ void __launch_bounds__(128) prng_kernel(const uint32_t* __restrict__ state, long long state_elems,
                                                   float* __restrict__ out, long long count,
                                                   uint32_t* __restrict__ new_state,
                                                   const uint32_t* __restrict__ table, long long threads, int chunk) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= threads) return;
  // without a place for the numbers only the state after them is wanted: one thread jumps there
  const long long first = out ? t * chunk : count;
  uint32_t s0 = prng_jump(table, 0, state[0], static_cast<unsigned long long>(first));
  uint32_t s1 = prng_jump(table, 1, state[1], static_cast<unsigned long long>(first));
  uint32_t s2 = prng_jump(table, 2, state[2], static_cast<unsigned long long>(first));
  const long long last = first + chunk < count ? first + chunk : count;
  auto next = [&]() -> float {
    const float v = static_cast<float>(static_cast<double>(s0 ^ s1 ^ s2) / 4294967296.0);
    s0 = prng_step(0, s0);
    s1 = prng_step(1, s1);
    s2 = prng_step(2, s2);
    return v;
  };
  long long i = first;
  if (reinterpret_cast<uintptr_t>(out) % 32 == 0) {
    for (; i + 8 <= last; i += 8) {
      float4 lo, hi;
      lo.x = next(); lo.y = next(); lo.z = next(); lo.w = next();
      hi.x = next(); hi.y = next(); hi.z = next(); hi.w = next();
      __stcs(reinterpret_cast<float4*>(out + i), lo);
      __stcs(reinterpret_cast<float4*>(out + i) + 1, hi);
    }
  }
  for (; i < last; ++i) out[i] = next();
  if (last == count && new_state) {  // the thread that holds the last element (thread 0 when there are none)
    new_state[0] = s0;
    new_state[1] = s1;
    new_state[2] = s2;
    for (long long w = 3; w < state_elems; ++w) new_state[w] = state[w];
  }
}

unsigned blocks_for(long long n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }

}  // namespace

cudaError_t launch_gather(const GatherParams& given, cudaStream_t stream) {
  if (given.out_elems <= 0) return cudaSuccess;
  GatherParams p = given;
  const bool float_idx = p.idx_dtype == PMLB_F16 || p.idx_dtype == PMLB_BF16 || p.idx_dtype == PMLB_F32 || p.idx_dtype == PMLB_F64;
  const bool float_data = p.dtype == PMLB_F16 || p.dtype == PMLB_BF16 || p.dtype == PMLB_F32 || p.dtype == PMLB_F64;
  p.copies = p.nd || !float_idx || !float_data;
  // whole runs of the inner dims move as 16-byte pieces when they and the buffers allow it
  const long long run_bytes = p.inner * p.elem_bytes;
  const bool aligned = (reinterpret_cast<uintptr_t>(p.tensor) | reinterpret_cast<uintptr_t>(p.out)) % 16 == 0;
  if (p.copies && p.elem_bytes < 16 && run_bytes % 16 == 0 && aligned) {
    p.out_elems = p.out_elems / p.inner * (run_bytes / 16);
    p.inner = run_bytes / 16;
    p.elem_bytes = 16;
  }
  long long source = p.inner;
  if (p.nd) {
    for (int k = 0; k < p.k; ++k) source *= p.dims[k];
    source *= (p.out_elems / p.inner + p.rows_per_batch - 1) / p.rows_per_batch;
  } else {
    source *= p.axis_len * ((p.out_elems / p.inner + p.n_idx - 1) / p.n_idx);
  }
  const long long limit = 1LL << 31;
  const bool narrow = p.out_elems < limit && source < limit && p.out_elems / p.inner * (p.nd ? p.k : 1) < limit;
  if (p.copies && !p.nd && p.elem_bytes == 16) {
    const long long quarter = (p.out_elems + 3) / 4;
    if (narrow) gather_pieces_kernel<unsigned><<<blocks_for(quarter, 256), 256, 0, stream>>>(p, static_cast<unsigned>(quarter));
    else gather_pieces_kernel<unsigned long long><<<blocks_for(quarter, 256), 256, 0, stream>>>(p, static_cast<unsigned long long>(quarter));
    return cudaGetLastError();
  }
  if (p.copies) {
    if (narrow) gather_kernel<unsigned><<<blocks_for(p.out_elems, 256), 256, 0, stream>>>(p);
    else gather_kernel<unsigned long long><<<blocks_for(p.out_elems, 256), 256, 0, stream>>>(p);
    return cudaGetLastError();
  }
  const long long threads = (p.out_elems + 3) / 4;
  const unsigned blocks = blocks_for(threads, 256);
#define PMLB_INTERP(A)                                                                                              \
  if (narrow) gather_interp_kernel<A, unsigned><<<blocks, 256, 0, stream>>>(p, static_cast<unsigned>(threads));     \
  else gather_interp_kernel<A, unsigned long long><<<blocks, 256, 0, stream>>>(p, static_cast<unsigned long long>(threads))
  switch (p.dtype) {
    case PMLB_F16: PMLB_INTERP(ArF16); break;
    case PMLB_BF16: PMLB_INTERP(ArBF16); break;
    case PMLB_F64: PMLB_INTERP(ArF64); break;
    default: PMLB_INTERP(ArF32); break;
  }
#undef PMLB_INTERP
  return cudaGetLastError();
}

cudaError_t launch_scatter(const ScatterParams& p, cudaStream_t stream) {
  if (p.upd_elems <= 0) return cudaSuccess;
  bool rows = p.mode != 3 && p.axis == 0 && p.idx_rank == 1 && p.upd_rank == p.rank;
  long long inner = 1;
  for (int d = 1; d < p.rank && rows; ++d) {
    rows = p.upd_sizes[d] == p.sizes[d];
    inner *= p.sizes[d];
  }
  if (rows) {
    const long long quarter = (p.upd_elems + 3) / 4;
    scatter_rows_kernel<<<blocks_for(quarter, 256), 256, 0, stream>>>(p, inner, quarter);
    return cudaGetLastError();
  }
  scatter_kernel<<<blocks_for(p.upd_elems, 256), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

namespace {

template <class V>
cudaError_t argsort_passes(const ArgsortParams& p, int32_t* out, int32_t* scratch, cudaStream_t stream) {
  const long long total = p.outer * p.n * p.inner;
  const unsigned blocks = blocks_for(total, 256);
  int passes = 0;
  while ((1LL << passes) < p.n) ++passes;
  // runs of up to 4096 positions are sorted in shared memory; longer lines go on with merge passes from there
  int seg_bits = passes < 12 ? passes : 12;
  if (seg_bits < 1) seg_bits = 1;
  const int seg_len = 1 << seg_bits;
  const long long segs_per_line = (p.n + seg_len - 1) / seg_len;
  const long long segments = p.outer * p.inner * segs_per_line;
  const int merges = passes > seg_bits ? passes - seg_bits : 0;
  int32_t* first = (merges % 2 == 0) ? out : scratch;
  const long long sort_blocks = (segments + kSortSlots / seg_len - 1) / (kSortSlots / seg_len);
  const bool narrow = p.dtype != PMLB_F64 && p.dtype != PMLB_I64 && p.dtype != PMLB_U64;
  if (narrow) {
    argsort_block32_kernel<<<static_cast<unsigned>(sort_blocks), kSortThreads, 0, stream>>>(p, first, seg_len,
                                                                                           segs_per_line, segments);
  } else {
    argsort_block_kernel<V><<<static_cast<unsigned>(sort_blocks), kSortThreads, 0, stream>>>(p, first, seg_len,
                                                                                            segs_per_line, segments);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int32_t* src = first;
  for (int k = 0; k < merges; ++k) {
    int32_t* dst = src == out ? scratch : out;
    argsort_pass_kernel<V><<<blocks, 256, 0, stream>>>(p, src, dst, static_cast<long long>(seg_len) << k, total);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    src = dst;
  }
  return cudaSuccess;
}

}  // namespace

cudaError_t launch_argsort(const ArgsortParams& p, int32_t* out, int32_t* scratch, cudaStream_t stream) {
  if (p.outer * p.n * p.inner <= 0) return cudaSuccess;
  switch (p.dtype) {
    case PMLB_F16:
    case PMLB_BF16:
    case PMLB_F32:
    case PMLB_F64: return argsort_passes<double>(p, out, scratch, stream);
    case PMLB_U64: return argsort_passes<unsigned long long>(p, out, scratch, stream);
    default: return argsort_passes<long long>(p, out, scratch, stream);
  }
}

cudaError_t launch_prng(const uint32_t* state, long long state_elems, float* out, long long count, uint32_t* new_state,
                        const uint32_t* table, cudaStream_t stream) {
  // longer runs per thread amortise the jump to the run's first element (it costs as much as ~200 numbers); short
  // ones keep small results parallel
  int chunk = kPrngChunk;
  while (chunk < 512 && count / chunk > 256LL * 1024) chunk *= 2;   // (measured: ~256 K threads, runs of at most 512)
  long long threads = out ? (count + chunk - 1) / chunk : 1;
  if (threads < 1) threads = 1;
  prng_kernel<<<blocks_for(threads, 128), 128, 0, stream>>>(state, state_elems, out, count, new_state, table, threads,
                                                           chunk);
  return cudaGetLastError();
}

void prng_jump_table(uint32_t* table) {
  for (int c = 0; c < 3; ++c) {
    uint32_t cols[32], next[32];
    for (int b = 0; b < 32; ++b) cols[b] = prng_step(c, 1u << b);      // columns of the one-step matrix
    for (int level = 0; level < kPrngLevels; ++level) {
      uint32_t* groups = table + (c * kPrngLevels + level) * kPrngNibbleWords;
      for (int n = 0; n < 8; ++n) {
        for (uint32_t v = 0; v < 16; ++v) {
          uint32_t y = 0;
          for (int b = 0; b < 4; ++b) {
            if ((v >> b) & 1u) y ^= cols[4 * n + b];
          }
          groups[n * 16 + v] = y;
        }
      }
      for (int b = 0; b < 32; ++b) next[b] = gf2_apply(cols, cols[b]);  // the matrix squared
      for (int b = 0; b < 32; ++b) cols[b] = next[b];
    }
  }
}

}  // namespace pmlb
