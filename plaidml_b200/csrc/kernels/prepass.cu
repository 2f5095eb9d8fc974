#include "prepass.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "pmlb_kernels.h"

namespace pmlb {

namespace {

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// 32x32 tiles through shared memory so that both the read and the (possibly transposed)
// write are row-contiguous.
__device__ __forceinline__ void split_tf32_tile(float (&tile)[32][33], int b, int bx, int by,
                                                const float* __restrict__ in, long long ld,
                                                long long in_batch, float* __restrict__ hi,
                                                float* __restrict__ lo, long long out_ld,
                                                long long out_batch, int rows, int cols, bool transpose);

__global__ void __launch_bounds__(256)
split_tf32_kernel(const float* __restrict__ in, long long ld, long long in_batch,
                  float* __restrict__ hi, float* __restrict__ lo, long long out_ld,
                  long long out_batch, int rows, int cols, bool transpose) {
  __shared__ float tile[32][33];
  split_tf32_tile(tile, blockIdx.z, blockIdx.x, blockIdx.y, in, ld, in_batch, hi, lo, out_ld, out_batch, rows,
                  cols, transpose);
}

// blockIdx.z < a.batch: a tile of operand a, else of operand b; tiles outside an operand's
// (padded) extent return at once.
__global__ void __launch_bounds__(256)
split_tf32_pair_kernel(SplitTf32Args a, SplitTf32Args b, int a_gx, int a_gy, int b_gx, int b_gy) {
  __shared__ float tile[32][33];
  const bool first = static_cast<int>(blockIdx.z) < a.batch;
  const SplitTf32Args& s = first ? a : b;
  if (static_cast<int>(blockIdx.x) >= (first ? a_gx : b_gx) || static_cast<int>(blockIdx.y) >= (first ? a_gy : b_gy)) return;
  split_tf32_tile(tile, first ? blockIdx.z : blockIdx.z - a.batch, blockIdx.x, blockIdx.y, s.in, s.ld, s.in_batch,
                  s.hi, s.lo, s.out_ld, s.out_batch, s.rows, s.cols, s.transpose);
}

__device__ __forceinline__ void split4(const float4& v, float4* h, float4* l) {
  h->x = tf32_round(v.x);
  h->y = tf32_round(v.y);
  h->z = tf32_round(v.z);
  h->w = tf32_round(v.w);
  l->x = tf32_round(v.x - h->x);
  l->y = tf32_round(v.y - h->y);
  l->z = tf32_round(v.z - h->z);
  l->w = tf32_round(v.w - h->w);
}

// The same split on 64 x 64 tiles with 16-byte loads and stores, for operands whose rows, leading dimensions and
// addresses are multiples of four floats (the launcher checks): a plain operand needs no shared memory at all, a
// transposed one is read in rows of the input and written in rows of the output.
__global__ void __launch_bounds__(256)
split_tf32_pair64_kernel(SplitTf32Args a, SplitTf32Args b, int a_gx, int a_gy, int b_gx, int b_gy) {
  __shared__ float tile[64][65];
  const bool first = static_cast<int>(blockIdx.z) < a.batch;
  const SplitTf32Args& s = first ? a : b;
  if (static_cast<int>(blockIdx.x) >= (first ? a_gx : b_gx) || static_cast<int>(blockIdx.y) >= (first ? a_gy : b_gy)) return;
  const long long bz = first ? blockIdx.z : blockIdx.z - a.batch;
  const float* __restrict__ src = s.in + bz * s.in_batch;
  float* __restrict__ dhi = s.hi + bz * s.out_batch;
  float* __restrict__ dlo = s.lo + bz * s.out_batch;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tq = threadIdx.x & 15, tr = threadIdx.x >> 4;   // 16 quads per tile row, 16 tile rows per step
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!s.transpose) {
    for (int i = tr; i < 64; i += 16) {
      const int r = r0 + i, c = c0 + tq * 4;
      if (r < s.rows && c < s.out_ld) {
        const float4 v = c < s.cols ? *reinterpret_cast<const float4*>(src + static_cast<long long>(r) * s.ld + c) : zero;
        float4 h, l;
        split4(v, &h, &l);
        *reinterpret_cast<float4*>(dhi + static_cast<long long>(r) * s.out_ld + c) = h;
        *reinterpret_cast<float4*>(dlo + static_cast<long long>(r) * s.out_ld + c) = l;
      }
    }
    return;
  }
  for (int i = tr; i < 64; i += 16) {
    const int r = r0 + i, c = c0 + tq * 4;
    const float4 v = (r < s.rows && c < s.cols) ? *reinterpret_cast<const float4*>(src + static_cast<long long>(r) * s.ld + c)
                                                : zero;
    tile[i][tq * 4 + 0] = v.x;
    tile[i][tq * 4 + 1] = v.y;
    tile[i][tq * 4 + 2] = v.z;
    tile[i][tq * 4 + 3] = v.w;
  }
  __syncthreads();
  for (int i = tr; i < 64; i += 16) {
    // output row = input column c0 + i; four output columns = input rows r0 + 4 tq .. + 3 (zeros past the input's rows)
    const int oc = c0 + i, orow = r0 + tq * 4;
    if (oc < s.cols && orow < s.out_ld) {
      const float4 v = make_float4(tile[tq * 4 + 0][i], tile[tq * 4 + 1][i], tile[tq * 4 + 2][i], tile[tq * 4 + 3][i]);
      float4 h, l;
      split4(v, &h, &l);
      *reinterpret_cast<float4*>(dhi + static_cast<long long>(oc) * s.out_ld + orow) = h;
      *reinterpret_cast<float4*>(dlo + static_cast<long long>(oc) * s.out_ld + orow) = l;
    }
  }
}

__device__ __forceinline__ void split_tf32_tile(float (&tile)[32][33], int b, int bx, int by,
                                                const float* __restrict__ in, long long ld,
                                                long long in_batch, float* __restrict__ hi,
                                                float* __restrict__ lo, long long out_ld,
                                                long long out_batch, int rows, int cols, bool transpose) {
  const float* src = in + static_cast<long long>(b) * in_batch;
  float* dhi = hi + static_cast<long long>(b) * out_batch;
  float* dlo = lo + static_cast<long long>(b) * out_batch;
  const int r0 = by * 32, c0 = bx * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int i = ty; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + tx;
    tile[i][tx] = (r < rows && c < cols) ? src[static_cast<long long>(r) * ld + c] : 0.f;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    float x;
    long long o;
    bool inside;
    if (transpose) {
      // output row = input column c0 + i, output column = input row r0 + tx
      x = tile[tx][i];
      inside = (c0 + i) < cols && (r0 + tx) < out_ld;
      o = static_cast<long long>(c0 + i) * out_ld + (r0 + tx);
    } else {
      x = tile[i][tx];
      inside = (r0 + i) < rows && (c0 + tx) < out_ld;
      o = static_cast<long long>(r0 + i) * out_ld + (c0 + tx);
    }
    if (inside) {
      const float h = tf32_round(x);
      dhi[o] = h;
      dlo[o] = tf32_round(x - h);
    }
  }
}

template <class T>
__global__ void __launch_bounds__(256)
transpose_kernel(const T* __restrict__ in, long long ld, long long in_batch, T* __restrict__ out,
                 long long out_ld, long long out_batch, int rows, int cols) {
  __shared__ T tile[32][33];
  const int b = blockIdx.z;
  const T* src = in + static_cast<long long>(b) * in_batch;
  T* dst = out + static_cast<long long>(b) * out_batch;
  const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + tx;
    if (r < rows && c < cols) tile[i][tx] = src[static_cast<long long>(r) * ld + c];
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int oc = c0 + i, orow = r0 + tx;
    if (oc < cols && orow < rows) dst[static_cast<long long>(oc) * out_ld + orow] = tile[tx][i];
  }
}

__device__ __forceinline__ float load_filter(const void* p, int dtype, long long i) {
  if (dtype == PMLB_F32) return static_cast<const float*>(p)[i];
  if (dtype == PMLB_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

__global__ void __launch_bounds__(256)
filter_relayout_kernel(const void* __restrict__ in, int in_dtype, void* __restrict__ out,
                       int out_dtype, int taps, int c, int k) {
  const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(taps) * c * k;
  if (id >= total) return;
  // id walks the output [k][taps][c]
  const int ci = static_cast<int>(id % c);
  const long long rem = id / c;
  const int t = static_cast<int>(rem % taps);
  const int ko = static_cast<int>(rem / taps);
  const float v = load_filter(in, in_dtype, (static_cast<long long>(t) * c + ci) * k + ko);
  if (out_dtype == PMLB_BF16) {
    static_cast<__nv_bfloat16*>(out)[id] = __float2bfloat16_rn(v);
  } else {
    static_cast<__half*>(out)[id] = __float2half_rn(v);
  }
}

// fp32 convolutions: filter [taps][c][k] -> high and low TF32 parts, each [k][taps][cp] (cp >= c, zeros in the pad)
__global__ void __launch_bounds__(256)
filter_relayout_split_kernel(const void* __restrict__ in, int in_dtype, float* __restrict__ hi, float* __restrict__ lo,
                             int taps, int c, int cp, int k) {
  const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(taps) * cp * k;
  if (id >= total) return;
  const int ci = static_cast<int>(id % cp);
  const long long rem = id / cp;
  const int t = static_cast<int>(rem % taps);
  const int ko = static_cast<int>(rem / taps);
  const float v = ci < c ? load_filter(in, in_dtype, (static_cast<long long>(t) * c + ci) * k + ko) : 0.f;
  const float h = tf32_round(v);
  hi[id] = h;
  lo[id] = tf32_round(v - h);
}

// One thread per group of 8 output channels of one output pixel (16 bytes).
__global__ void __launch_bounds__(256)
pack_rows_kernel(const uint16_t* __restrict__ in, uint4* __restrict__ out, long long rows, int w,
                 int c, int wp, int cp8, int pad_w) {
  const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = rows * wp * cp8;
  if (id >= total) return;
  const int g = static_cast<int>(id % cp8);
  const long long pix = id / cp8;
  const int x = static_cast<int>(pix % wp);
  const long long row = pix / wp;     // n * h + hh
  const int src_w = x - pad_w;
  uint32_t words[4] = {0u, 0u, 0u, 0u};
  if (src_w >= 0 && src_w < w) {
    const uint16_t* src = in + (row * w + src_w) * c;
    const int c0 = g * 8;
    if (c0 + 8 <= c && (c % 8) == 0 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + c0));
      words[0] = v.x; words[1] = v.y; words[2] = v.z; words[3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t e = (c0 + j < c) ? static_cast<uint32_t>(__ldg(src + c0 + j)) : 0u;
        words[j >> 1] |= e << ((j & 1) * 16);
      }
    }
  }
  out[id] = make_uint4(words[0], words[1], words[2], words[3]);
}

__global__ void __launch_bounds__(256)
filter_pack_rows_kernel(const void* __restrict__ in, int in_dtype, void* __restrict__ out,
                        int out_dtype, int r, int s, int c, int cp, int k) {
  const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(k) * r * 64;
  if (id >= total) return;
  // id walks the output [k][r][64]
  const int e = static_cast<int>(id % 64);
  const long long rem = id / 64;
  const int fr = static_cast<int>(rem % r);
  const int ko = static_cast<int>(rem / r);
  const int fs = e / cp;
  const int ci = e - fs * cp;
  float v = 0.f;
  if (fs < s && ci < c) {
    v = load_filter(in, in_dtype, ((static_cast<long long>(fr) * s + fs) * c + ci) * k + ko);
  }
  if (out_dtype == PMLB_BF16) {
    static_cast<__nv_bfloat16*>(out)[id] = __float2bfloat16_rn(v);
  } else {
    static_cast<__half*>(out)[id] = __float2half_rn(v);
  }
}

template <int C>
__global__ void __launch_bounds__(256)
s2d_pack_kernel(const uint16_t* __restrict__ in, uint4* __restrict__ out, long long total_px, int h,
                int w, int h2, int wp, int pe_h, int pe_w) {
  const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (id >= total_px) return;
  const int x2 = static_cast<int>(id % wp);
  const long long rem = id / wp;
  const int y2 = static_cast<int>(rem % h2);
  const long long img = rem / h2;
  uint32_t words[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
  for (int py = 0; py < 2; ++py) {
    const int y = 2 * y2 + py - pe_h;
#pragma unroll
    for (int px = 0; px < 2; ++px) {
      const int x = 2 * x2 + px - pe_w;
      if (y >= 0 && y < h && x >= 0 && x < w) {
        const uint16_t* src = in + ((img * h + y) * w + x) * C;
#pragma unroll
        for (int ci = 0; ci < C; ++ci) {
          const int ch = (py * 2 + px) * C + ci;
          words[ch >> 1] |= static_cast<uint32_t>(__ldg(src + ci)) << ((ch & 1) * 16);
        }
      }
    }
  }
  // 128-byte swizzle over rows of four pixels: 16-byte chunk c of row number `row` goes to
  // chunk c ^ (row & 7) (wp is a multiple of 32, so images start on whole 8-row groups)
  const long long row = id >> 2;
  const int c0 = static_cast<int>(id & 3) * 2;
  const int x = static_cast<int>(row & 7);
  // (c0 is even, so the pixel's two chunks stay one 32-byte sector, in swapped order when the row
  // number is odd: one 32-byte store)
  const uint4 first = make_uint4(words[0], words[1], words[2], words[3]);
  const uint4 second = make_uint4(words[4], words[5], words[6], words[7]);
  uint4* sector = out + row * 8 + ((c0 ^ x) & ~1);
  const bool swapped = (x & 1) != 0;
  const uint4& a = swapped ? second : first;
  const uint4& b = swapped ? first : second;
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               :
               : "l"(sector), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}

__global__ void __launch_bounds__(256)
filter_s2d_kernel(const void* __restrict__ in, int in_dtype, void* __restrict__ out, int out_dtype,
                  int r, int s, int c, int k, int r2, int s2, int dh, int dw) {
  const int id = blockIdx.x * blockDim.x + threadIdx.x;
  const int sg = (s2 + 3) / 4;                 // groups of four tap columns
  const int total = r2 * sg * 64 * 64;
  if (id >= total) return;
  // id walks the logical output [tr][tap-column group][ko][4 tap columns x 16 channels]
  const int e = id & 63;
  const int ko = (id >> 6) & 63;
  const int blk = id >> 12;
  const int tr = blk / sg, ts = (blk - tr * sg) * 4 + (e >> 4);
  const int ch = e & 15;
  float v = 0.f;
  if (ch < 4 * c && ko < k && ts < s2) {
    const int phase = ch / c, ci = ch - phase * c;
    const int fr = 2 * tr + (phase >> 1) - dh, fs = 2 * ts + (phase & 1) - dw;
    if (fr >= 0 && fr < r && fs >= 0 && fs < s) {
      v = load_filter(in, in_dtype, ((static_cast<long long>(fr) * s + fs) * c + ci) * k + ko);
    }
  }
  // 128-byte swizzle: 16-byte chunk number (e >> 3) exchanged with chunk ^ (row & 7)
  const int o = (id & ~63) | ((((e >> 3) ^ (ko & 7)) << 3) | (e & 7));
  if (out_dtype == PMLB_BF16) {
    static_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
  } else {
    static_cast<__half*>(out)[o] = __float2half_rn(v);
  }
}

// The same weights for the kernel that merges tap columns into the N dimension of its MMAs: logical
// output [3 - tap column][ko][tap row][16 channels] (four blocks of 64 rows of 128 bytes), 128-byte swizzle.
__global__ void __launch_bounds__(256)
filter_s2d_merged_kernel(const void* __restrict__ in, int in_dtype, void* __restrict__ out, int out_dtype,
                         int r, int s, int c, int k, int r2, int s2, int dh, int dw) {
  const int id = blockIdx.x * blockDim.x + threadIdx.x;
  if (id >= 4 * 64 * 64) return;
  const int e = id & 63;
  const int ko = (id >> 6) & 63;
  const int ts = 3 - (id >> 12);
  const int tr = e >> 4;
  const int ch = e & 15;
  float v = 0.f;
  if (ch < 4 * c && ko < k && ts < s2 && tr < r2) {
    const int phase = ch / c, ci = ch - phase * c;
    const int fr = 2 * tr + (phase >> 1) - dh, fs = 2 * ts + (phase & 1) - dw;
    if (fr >= 0 && fr < r && fs >= 0 && fs < s) {
      v = load_filter(in, in_dtype, ((static_cast<long long>(fr) * s + fs) * c + ci) * k + ko);
    }
  }
  const int o = (id & ~63) | ((((e >> 3) ^ (ko & 7)) << 3) | (e & 7));
  if (out_dtype == PMLB_BF16) {
    static_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
  } else {
    static_cast<__half*>(out)[o] = __float2half_rn(v);
  }
}

}  // namespace

cudaError_t launch_filter_s2d_merged(const void* in, int in_dtype, void* out, int out_dtype, int r, int s,
                                     int c, int k, int r2, int s2, int dh, int dw, cudaStream_t stream) {
  filter_s2d_merged_kernel<<<64, 256, 0, stream>>>(in, in_dtype, out, out_dtype, r, s, c, k, r2, s2, dh, dw);
  return cudaGetLastError();
}

cudaError_t launch_s2d_pack(const void* in, void* out, int n, int h, int w, int c, int h2, int wp,
                            int pe_h, int pe_w, cudaStream_t stream) {
  const long long total = static_cast<long long>(n) * h2 * wp;
  if (total <= 0) return cudaSuccess;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  const uint16_t* src = static_cast<const uint16_t*>(in);
  uint4* dst = static_cast<uint4*>(out);
  switch (c) {
    case 1: s2d_pack_kernel<1><<<blocks, 256, 0, stream>>>(src, dst, total, h, w, h2, wp, pe_h, pe_w); break;
    case 2: s2d_pack_kernel<2><<<blocks, 256, 0, stream>>>(src, dst, total, h, w, h2, wp, pe_h, pe_w); break;
    case 3: s2d_pack_kernel<3><<<blocks, 256, 0, stream>>>(src, dst, total, h, w, h2, wp, pe_h, pe_w); break;
    case 4: s2d_pack_kernel<4><<<blocks, 256, 0, stream>>>(src, dst, total, h, w, h2, wp, pe_h, pe_w); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_filter_s2d(const void* in, int in_dtype, void* out, int out_dtype, int r, int s,
                              int c, int k, int r2, int s2, int dh, int dw, cudaStream_t stream) {
  const int total = r2 * ((s2 + 3) / 4) * 64 * 64;
  if (total <= 0) return cudaSuccess;
  filter_s2d_kernel<<<(total + 255) / 256, 256, 0, stream>>>(in, in_dtype, out, out_dtype, r, s, c, k,
                                                             r2, s2, dh, dw);
  return cudaGetLastError();
}

cudaError_t launch_pack_rows(const void* in, void* out, int n, int h, int w, int c, int wp, int cp,
                             int pad_w, cudaStream_t stream) {
  const long long rows = static_cast<long long>(n) * h;
  const long long total = rows * wp * (cp / 8);
  if (total <= 0) return cudaSuccess;
  pack_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint16_t*>(in), static_cast<uint4*>(out), rows, w, c, wp, cp / 8, pad_w);
  return cudaGetLastError();
}

cudaError_t launch_filter_pack_rows(const void* in, int in_dtype, void* out, int out_dtype, int r,
                                    int s, int c, int cp, int k, cudaStream_t stream) {
  const long long total = static_cast<long long>(k) * r * 64;
  if (total <= 0) return cudaSuccess;
  filter_pack_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      in, in_dtype, out, out_dtype, r, s, c, cp, k);
  return cudaGetLastError();
}

cudaError_t launch_split_tf32(const float* in, long long ld, long long in_batch, float* hi,
                              float* lo, long long out_ld, long long out_batch, int rows, int cols,
                              int batch, bool transpose, cudaStream_t stream) {
  // cover the padded output extent so that the pad is written (as zeros)
  const int out_rows = transpose ? cols : rows;
  const int out_cols = static_cast<int>(out_ld);
  const int cover_rows = transpose ? out_cols : out_rows;  // in input-row units
  const int cover_cols = transpose ? out_rows : out_cols;  // in input-col units
  dim3 grid((cover_cols + 31) / 32, (cover_rows + 31) / 32, batch);
  split_tf32_kernel<<<grid, 256, 0, stream>>>(in, ld, in_batch, hi, lo, out_ld, out_batch, rows,
                                              cols, transpose);
  return cudaGetLastError();
}

namespace {
void split_grid(const SplitTf32Args& s, int* gx, int* gy) {
  // cover the padded output extent so that the pad is written (as zeros)
  const int out_rows = s.transpose ? s.cols : s.rows;
  const int out_cols = static_cast<int>(s.out_ld);
  const int cover_rows = s.transpose ? out_cols : out_rows;  // in input-row units
  const int cover_cols = s.transpose ? out_rows : out_cols;  // in input-col units
  *gx = (cover_cols + 31) / 32;
  *gy = (cover_rows + 31) / 32;
}
}  // namespace

namespace {
bool quads_ok(const SplitTf32Args& s) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(s.in) | reinterpret_cast<uintptr_t>(s.hi) | reinterpret_cast<uintptr_t>(s.lo);
  return bits % 16 == 0 && s.ld % 4 == 0 && s.in_batch % 4 == 0 && s.out_ld % 4 == 0 && s.out_batch % 4 == 0 && s.cols % 4 == 0;
}
}  // namespace

cudaError_t launch_split_tf32_pair(const SplitTf32Args& a, const SplitTf32Args& b, cudaStream_t stream) {
  int agx, agy, bgx, bgy;
  split_grid(a, &agx, &agy);
  split_grid(b, &bgx, &bgy);
  if (quads_ok(a) && quads_ok(b)) {
    const int ax = (agx + 1) / 2, ay = (agy + 1) / 2, bx = (bgx + 1) / 2, by = (bgy + 1) / 2;   // 64-wide tiles
    dim3 grid64(ax > bx ? ax : bx, ay > by ? ay : by, a.batch + b.batch);
    if (grid64.y <= 65535u && grid64.z <= 65535u) {
      split_tf32_pair64_kernel<<<grid64, 256, 0, stream>>>(a, b, ax, ay, bx, by);
      return cudaGetLastError();
    }
  }
  dim3 grid(agx > bgx ? agx : bgx, agy > bgy ? agy : bgy, a.batch + b.batch);
  if (grid.y > 65535u || grid.z > 65535u) {
    cudaError_t e = launch_split_tf32(a.in, a.ld, a.in_batch, a.hi, a.lo, a.out_ld, a.out_batch, a.rows, a.cols,
                                      a.batch, a.transpose, stream);
    if (e != cudaSuccess) return e;
    return launch_split_tf32(b.in, b.ld, b.in_batch, b.hi, b.lo, b.out_ld, b.out_batch, b.rows, b.cols, b.batch,
                             b.transpose, stream);
  }
  split_tf32_pair_kernel<<<grid, 256, 0, stream>>>(a, b, agx, agy, bgx, bgy);
  return cudaGetLastError();
}

cudaError_t launch_transpose(const void* in, long long ld, long long in_batch, void* out,
                             long long out_ld, long long out_batch, int rows, int cols, int batch,
                             int elem_bytes, cudaStream_t stream) {
  dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch);
  switch (elem_bytes) {
    case 1:
      transpose_kernel<uint8_t><<<grid, 256, 0, stream>>>(
          static_cast<const uint8_t*>(in), ld, in_batch, static_cast<uint8_t*>(out), out_ld,
          out_batch, rows, cols);
      break;
    case 2:
      transpose_kernel<uint16_t><<<grid, 256, 0, stream>>>(
          static_cast<const uint16_t*>(in), ld, in_batch, static_cast<uint16_t*>(out), out_ld,
          out_batch, rows, cols);
      break;
    case 4:
      transpose_kernel<uint32_t><<<grid, 256, 0, stream>>>(
          static_cast<const uint32_t*>(in), ld, in_batch, static_cast<uint32_t*>(out), out_ld,
          out_batch, rows, cols);
      break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_filter_relayout(const void* in, int in_dtype, void* out, int out_dtype, int taps,
                                   int c, int k, cudaStream_t stream) {
  const long long total = static_cast<long long>(taps) * c * k;
  if (total <= 0) return cudaSuccess;
  filter_relayout_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      in, in_dtype, out, out_dtype, taps, c, k);
  return cudaGetLastError();
}

cudaError_t launch_filter_relayout_split(const void* in, int in_dtype, float* hi, float* lo, int taps, int c, int cp,
                                         int k, cudaStream_t stream) {
  const long long total = static_cast<long long>(taps) * cp * k;
  if (total <= 0) return cudaSuccess;
  filter_relayout_split_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(in, in_dtype, hi, lo, taps,
                                                                                                c, cp, k);
  return cudaGetLastError();
}

namespace {

// One thread per four consecutive output columns (n % 4 == 0) or per column.
template <bool IS_INT, int V>
__global__ void __launch_bounds__(256)
splitk_combine_kernel(const void* __restrict__ partials, int parts, int m, int n, void* __restrict__ out, int out_dtype,
                      long long ldc, int epi_flags, const void* __restrict__ bias, const void* __restrict__ residual,
                      long long ldr) {
  const long long per_row = n / V;
  const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (id >= static_cast<long long>(m) * per_row) return;
  const long long row = id / per_row;
  const int col = static_cast<int>(id - row * per_row) * V;
  const long long plane = static_cast<long long>(m) * n;
  const long long off = row * n + col;
  if constexpr (IS_INT) {
    int acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0;
    const int* src = static_cast<const int*>(partials) + off;
    for (int s = 0; s < parts; ++s) {
      if constexpr (V == 4) {
        const int4 v = *reinterpret_cast<const int4*>(src + s * plane);
        acc[0] += v.x, acc[1] += v.y, acc[2] += v.z, acc[3] += v.w;
      } else {
        acc[0] += src[s * plane];
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      int x = acc[j];
      if (epi_flags & PMLB_EPI_BIAS) x += static_cast<const int*>(bias)[col + j];
      if (epi_flags & PMLB_EPI_RESIDUAL) {
        x += out_dtype == PMLB_I32 ? static_cast<const int*>(residual)[row * ldr + col + j]
                                   : static_cast<const int8_t*>(residual)[row * ldr + col + j];
      }
      if (out_dtype != PMLB_I32) x = static_cast<int8_t>(x);   // wrap first: the ReLU acts on the int8 value
      if (epi_flags & PMLB_EPI_RELU) x = x < 0 ? 0 : x;
      if (out_dtype == PMLB_I32) {
        static_cast<int*>(out)[row * ldc + col + j] = x;
      } else {
        static_cast<int8_t*>(out)[row * ldc + col + j] = static_cast<int8_t>(x);
      }
    }
  } else {
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    const float* src = static_cast<const float*>(partials) + off;
    for (int s = 0; s < parts; ++s) {
      if constexpr (V == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src + s * plane);
        acc[0] += v.x, acc[1] += v.y, acc[2] += v.z, acc[3] += v.w;
      } else {
        acc[0] += src[s * plane];
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float x = acc[j];
      if (epi_flags & PMLB_EPI_BIAS) x += static_cast<const float*>(bias)[col + j];
      if (epi_flags & PMLB_EPI_RESIDUAL) {
        const long long r = row * ldr + col + j;
        if (out_dtype == PMLB_F32) {
          x += static_cast<const float*>(residual)[r];
        } else if (out_dtype == PMLB_BF16) {
          x += __bfloat162float(static_cast<const __nv_bfloat16*>(residual)[r]);
        } else {
          x += __half2float(static_cast<const __half*>(residual)[r]);
        }
      }
      if (epi_flags & PMLB_EPI_RELU) x = x < 0.f ? 0.f : x;   // (ordered compare: NaN passes through)
      const long long o = row * ldc + col + j;
      if (out_dtype == PMLB_F32) {
        static_cast<float*>(out)[o] = x;
      } else if (out_dtype == PMLB_BF16) {
        static_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(x);
      } else {
        static_cast<__half*>(out)[o] = __float2half_rn(x);
      }
    }
  }
}

}  // namespace

cudaError_t launch_splitk_combine(const void* partials, bool is_int, int parts, int m, int n, void* out, int out_dtype,
                                  long long ldc, int epi_flags, const void* bias, const void* residual, long long ldr,
                                  cudaStream_t stream) {
  const bool vec = n % 4 == 0 && (reinterpret_cast<uintptr_t>(partials) & 15u) == 0;
  const long long threads = static_cast<long long>(m) * (vec ? n / 4 : n);
  const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
  if (is_int) {
    if (vec) {
      splitk_combine_kernel<true, 4><<<grid, 256, 0, stream>>>(partials, parts, m, n, out, out_dtype, ldc, epi_flags, bias, residual, ldr);
    } else {
      splitk_combine_kernel<true, 1><<<grid, 256, 0, stream>>>(partials, parts, m, n, out, out_dtype, ldc, epi_flags, bias, residual, ldr);
    }
  } else {
    if (vec) {
      splitk_combine_kernel<false, 4><<<grid, 256, 0, stream>>>(partials, parts, m, n, out, out_dtype, ldc, epi_flags, bias, residual, ldr);
    } else {
      splitk_combine_kernel<false, 1><<<grid, 256, 0, stream>>>(partials, parts, m, n, out, out_dtype, ldc, epi_flags, bias, residual, ldr);
    }
  }
  return cudaGetLastError();
}

}  // namespace pmlb
