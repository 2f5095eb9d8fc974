// Operand preparation kernels that run before a tensor-core contraction.
#pragma once

#include <cuda_runtime.h>

namespace pmlb {

// fp32 [rows][cols] (row stride `ld`) -> TF32 hi and lo parts with hi + lo == x up to
// 2^-22 relative.  transpose == false writes [rows][cols_pad], true writes [cols][rows_pad];
// the padded tail of every output row is zero-filled.  `batch` matrices, `in_batch` /
// `out_batch` elements apart.
cudaError_t launch_split_tf32(const float* in, long long ld, long long in_batch, float* hi,
                              float* lo, long long out_ld, long long out_batch, int rows, int cols,
                              int batch, bool transpose, cudaStream_t stream);

// The same for two operands in one launch (the A and the B of an fp32 GEMM): the launch gap between two
// small kernels is of the order of their run time.
struct SplitTf32Args {
  const float* in;
  long long ld, in_batch;
  float* hi;
  float* lo;
  long long out_ld, out_batch;
  int rows, cols, batch;
  bool transpose;
};
cudaError_t launch_split_tf32_pair(const SplitTf32Args& a, const SplitTf32Args& b, cudaStream_t stream);

// Generic 2-D transpose of `elem_bytes`-sized elements: in [rows][cols] -> out [cols][out_ld].
cudaError_t launch_transpose(const void* in, long long ld, long long in_batch, void* out,
                             long long out_ld, long long out_batch, int rows, int cols, int batch,
                             int elem_bytes, cudaStream_t stream);

// Filter [taps][c][k] (element type `in_dtype`: f32, bf16 or f16) -> [k][taps][c] in the
// 16-bit `out_dtype`.
cudaError_t launch_filter_relayout(const void* in, int in_dtype, void* out, int out_dtype, int taps,
                                   int c, int k, cudaStream_t stream);

// The same for fp32 convolutions (three TF32 products per term): the high and the low TF32 part of the filter,
// each [k][taps][cp] in f32 storage, channels zero-padded from c to cp.
cudaError_t launch_filter_relayout_split(const void* in, int in_dtype, float* hi, float* lo, int taps, int c, int cp,
                                         int k, cudaStream_t stream);

// Packed-row convolution operands (16-bit elements).
// Activation [n][h][w][c] -> [n][h][wp][cp]: `pad_w` zero pixels before every row, zeros after
// it up to `wp` pixels, channels zero-padded from c to cp (a multiple of 8).
cudaError_t launch_pack_rows(const void* in, void* out, int n, int h, int w, int c, int wp, int cp,
                             int pad_w, cudaStream_t stream);
// Filter [r][s][c][k] (f32, bf16 or f16) -> [k][r][64] in the 16-bit `out_dtype`, element
// s * cp + ci of each 64-element row holding tap (r, s) of channel ci, zeros elsewhere.
cudaError_t launch_filter_pack_rows(const void* in, int in_dtype, void* out, int out_dtype, int r,
                                    int s, int c, int cp, int k, cudaStream_t stream);

// Space-to-depth operands (16-bit elements) of the stride-2 route for thin inputs (c <= 4).
// Activation [n][h][w][c] -> [n][h2][wp][16]: channel (py * 2 + px) * c + ci of pixel (y2, x2)
// is input pixel (2 * y2 + py - pe_h, 2 * x2 + px - pe_w), zero outside the image and in the
// unused channels.  wp is a multiple of 32; the result is stored in the 128-byte shared-memory
// swizzle (rows of four pixels, 16-byte chunk c of row number j at chunk c ^ (j & 7)), so that an
// untiled copy that starts at a multiple of 32 pixels lands in operand layout.
cudaError_t launch_s2d_pack(const void* in, void* out, int n, int h, int w, int c, int h2, int wp,
                            int pe_h, int pe_w, cudaStream_t stream);
// Filter [r][s][c][k] (f32, bf16 or f16) -> [r2][ceil(s2 / 4)][64][4][16] in the 16-bit
// `out_dtype`: row ko of block (tr, group) holds, for tap column ts = 4 * group + j at channel
// (py * 2 + px) * c + ci, the weight of filter tap (2 * tr + py - dh, 2 * ts + px - dw) (zero
// outside the filter, in the unused channels and in rows ko >= k); every 64 x 128-byte block is
// stored in the 128-byte shared-memory swizzle.
cudaError_t launch_filter_s2d(const void* in, int in_dtype, void* out, int out_dtype, int r, int s,
                              int c, int k, int r2, int s2, int dh, int dw, cudaStream_t stream);

// The same weights as [3 - tap column][64][tap row][16] (four blocks of 64 rows of 128 bytes, 32 KB):
// the layout of the kernel that fuses the layer with the max pool behind it (s2 = 4, r2 <= 4).
cudaError_t launch_filter_s2d_merged(const void* in, int in_dtype, void* out, int out_dtype, int r, int s,
                                     int c, int k, int r2, int s2, int dh, int dw, cudaStream_t stream);

// Second pass of a GEMM whose K range was split over `parts` CTAs per output tile: sums the partial
// products (f32 or i32, [parts][m][n] dense) in part order and applies the epilogue the single-pass kernel
// would have applied -- bias[n], residual[m][n] (element type of the output, row stride ldr), ReLU, cast
// to out_dtype (row stride ldc).  Integer partials: out_dtype I32 or I8 (wrap, then ReLU).
cudaError_t launch_splitk_combine(const void* partials, bool is_int, int parts, int m, int n, void* out, int out_dtype,
                                  long long ldc, int epi_flags, const void* bias, const void* residual, long long ldr,
                                  cudaStream_t stream);

}  // namespace pmlb
