// Host-side description of one launch of the tensor-core contraction kernel.
#pragma once

#include <cuda_runtime.h>

#include <string>

namespace pmlb {

// NHWC activation [n, h, w, c] convolved with r x s taps into [n, p, q, k_out].
struct ConvGeom {
  int n, h, w, c;
  int r, s;
  int p, q;
  int stride_h, stride_w;
  int pad_h, pad_w;  // zero padding before the first row / column
  int dil_h, dil_w;
};

// Packed-row convolution: the activation has been copied to [n][h][wp][cp] with pad_w zero
// pixels before every row (so output column q reads padded pixels q * stride_w ... + s - 1,
// which are s * cp consecutive elements), the weights to [k_out][r][64].
struct WinGeom {
  int n, h, wp, cp;
  int r, s;
  int p, q;
  int stride_h, stride_w;
  int pad_h;
};

// Halo convolution: a stride-1, undilated ConvGeom whose weights ([k_out][r*s][c], k_out = 64)
// stay in shared memory; a0 is the activation, b0 the weights.
struct HaloGeom {
  ConvGeom conv;
};

// Space-to-depth convolution (stride 2, thin input): a0 is the packed activation [n][h2][wp][16]
// (followed by at least stage_px * 32 readable bytes), b0 the packed weights [r2][ceil(s2 / 4)][64][64],
// both already in the 128-byte swizzle; the output is [n][p][q][k_out], q a multiple of 4.
struct S2dGeom {
  int n, p, q;
  int r2, s2;     // taps of the stride-1 form
  int h2, wp;     // rows per packed image, pixels per row (a multiple of 32)
  int stage_px;   // pixels a 512-position tile reads (a multiple of 32)
};

struct TcLaunch {
  int elem_bytes = 2;   // 1 (int8), 2 (bf16 / f16), 4 (fp32 pre-split into TF32 hi / lo)
  bool is_f16 = false;  // 2-byte operands are IEEE half instead of bfloat16
  int nsplit = 1;       // 2: a0/b0 hold the hi parts, a1/b1 the lo parts
  bool b_mn = false;    // false: B stored [n][k]; true: B stored [k][n]
  int m = 0, n = 0, k = 0, batch = 1;

  const void* a0 = nullptr;
  const void* a1 = nullptr;
  long long lda = 0;             // elements between rows of A
  int k_first = 0;               // > 0 (plain 8/16-bit GEMMs, nsplit == 1, batch 1): A is two tensors side by side
                                 // along K -- columns [0, k_first) from a0, [k_first, k) from a1 (rows lda_second
                                 // apart, its own column 0 first); k_first a multiple of the k-block (128 bytes)
  long long lda_second = 0;
  const ConvGeom* a_second_pixels = nullptr;  // non-null: the second part is an NHWC activation [n][h][w][k - k_first]
                                              // read as a 1x1 convolution with this stride (no padding): row i of the
                                              // product is output pixel i, m = n * p * q
  long long a_batch_stride = 0;  // elements between batch entries, 0 = shared
  const void* b0 = nullptr;
  const void* b1 = nullptr;
  long long ldb = 0;
  long long b_batch_stride = 0;

  const ConvGeom* conv = nullptr;  // non-null: A is an NHWC activation fetched by im2col TMA,
                                   // B holds the weights as [k_out][r*s][c]

  const HaloGeom* halo = nullptr;   // non-null: halo convolution; m, n, batch = n*p*q, k_out, 1
  const S2dGeom* s2d = nullptr;     // non-null: space-to-depth convolution; m, n, batch = n*p*q, k_out, 1
  const WinGeom* window = nullptr;  // non-null: packed-row convolution (a0 / b0 as described there);
                                    // m, n, batch = q, k_out, n * p

  void* out = nullptr;
  long long ldc = 0;
  long long out_batch_stride = 0;
  int out_dtype = 14;
  int epi_flags = 0;
  const void* bias = nullptr;
  const void* residual = nullptr;
  long long ldr = 0;
  long long res_batch_stride = 0;
  float* rowmax = nullptr;

  long long* trace = nullptr;  // debugging: device buffer of 4 * 2048 * 3 int64 for CTA 0's timeline
  int* status = nullptr;  // device word that receives a non-zero code if a wait times out
  int wait_limit_us = 0;  // limit of every device-side wait in microseconds; 0 = two seconds
  bool test_drop_load = false;  // testing: CTA 0's producer skips its first load, so that a wait runs out

  bool force_slow_epilogue = false;  // testing: take the transpose-and-store epilogue
  bool residual_from_global = false;  // testing: staged epilogue reads the residual with plain loads
  int bn_override = 0;    // 0 = choose; else 64, 128 or 256
  int epi_groups_override = 0;  // 0 = choose; else 1 or 2
  int grid_override = 0;  // 0 = one CTA per SM
  int split_tail = -1;    // -1 / 1 = halve the tiles of a short last wave; 0 = never
  int pair_override = -1; // -1 = choose; 0 = never pair CTAs on one tile; 1 = whenever the shape allows
  int halo_merge_columns = 1;  // halo route, 3 filter columns on 64 channels: 1 = one 128 x 192 MMA per filter row
                               // (columns merged into N, shifted adds in the epilogue); 0 = one MMA per tap
};

// Returns 0 on success; otherwise 1 (invalid argument), 2 (CUDA error) or
// 3 (unsupported) with a message in *err.
int tc_launch(const TcLaunch& launch, cudaStream_t stream, std::string* err);

bool tc_supported(std::string* why);

}  // namespace pmlb
