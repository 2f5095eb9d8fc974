// Device-side parameter block shared by the tensor-core contraction kernel and
// the host code that plans it.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace pmlb {

// Element types seen by the epilogue (values follow the public pmlb_dtype enum).
enum : int {
  kDtF32 = 14,
  kDtF16 = 13,
  kDtBF16 = 16,
  kDtI8 = 5,
  kDtI32 = 9,
};

enum : int {
  kEpiBias = 1,      // add bias[col] (f32 for float accumulators, i32 for integer ones)
  kEpiResidual = 2,  // add residual[row, col] (same element type as the output)
  kEpiRelu = 4,      // x < 0 ? 0 : x (ordered compare: NaN passes through)
  kEpiRowMax = 8,    // do not store the tile; fold it into rowmax[row] with atomic max
};

// Division by a launch-time constant as a multiplication: n / d for 0 <= n < 2^31.  (A runtime
// integer division is a chain of some thirty dependent instructions; the roles of the kernel run
// as single warps whose dependent instructions issue several cycles apart.)
struct FastDiv {
  uint32_t mul, shift;
};

inline FastDiv make_fastdiv(uint32_t d) {
  uint32_t s = 0;
  while ((1ull << s) < d) ++s;
  FastDiv f;
  f.shift = 31 + s;
  f.mul = static_cast<uint32_t>(((1ull << f.shift) + d - 1) / d);
  return f;
}

#ifdef __CUDACC__
__device__ __forceinline__ int fast_div(int n, FastDiv f) {
  return static_cast<int>((static_cast<unsigned long long>(static_cast<uint32_t>(n)) * f.mul) >> f.shift);
}
#endif

struct TcParams {
  // Problem (per batch entry): C[m, n] = sum_k A[m, k] * B[n, k]
  int m, n, k, batch;
  int tiles_m, tiles_n;  // tiles per batch entry
  int tiles_full;        // tiles walked whole; the rest (the tail of the last wave) as two half-width tiles each
  int num_kb;            // k-blocks (of 128 bytes of K) per tile
  int group_m;           // m-tiles per rasterisation group (L2 reuse of B panels)
  // divisors of the tile-number arithmetic: tiles per batch entry, tiles per rasterisation group,
  // m-tiles of a full group and of the last (shorter) one, output pixels per image, output
  // columns, halo / space-to-depth tiles per image and positions per padded image row
  FastDiv fd_per_batch, fd_group, fd_gm_full, fd_gm_tail, fd_per_img, fd_q, fd_tiles_per_img, fd_wp;
  int a_bz, b_bz;        // 1: operand has a batch dimension, 0: one matrix shared by all entries

  // Implicit-GEMM convolution (A fetched by im2col TMA); unused for plain GEMM.
  int conv_p, conv_q;          // output rows / columns per image
  int conv_s;                  // filter taps along W
  int conv_cblocks;            // channel blocks per filter tap
  int conv_stride_h, conv_stride_w;
  int conv_lower_h, conv_lower_w;  // bounding-box lower corner (= -pad)
  int conv_dil_h, conv_dil_w;
  // Packed-row convolution (A fetched as whole input rows into a ring of row slots).
  int win_r;                   // filter rows = k-blocks per output row
  int win_slots;               // row slots in the ring (> win_r, at most 16)
  int win_slot_bytes;          // bytes per slot (rows of 128 bytes, a multiple of 1024)

  // Halo convolution (stride 1: the padded pixels of a few image rows fetched once per tile,
  // every filter tap read as a row-shifted window of that buffer, weights resident).
  int halo_wp;                 // padded row width in pixels = output positions per image row
  int halo_th;                 // output image rows per tile (halo_th * halo_wp <= 128)
  int halo_rows;               // image rows fetched per tile = halo_th + r - 1
  int halo_stage_bytes;        // bytes per fetched buffer (a multiple of 1024)
  int halo_stages;             // buffers in the ring
  int halo_tiles_per_img;      // ceil(p / halo_th)
  int conv_r;                  // filter taps along H
  // Space-to-depth convolution (stride 2, thin input): as the halo convolution, on a packed
  // activation of 32-byte pixels whose tiles are 128 consecutive pixel positions; conv_r / conv_s
  // count the taps of the stride-1 form, halo_wp / halo_stage_bytes / halo_stages /
  // halo_tiles_per_img keep their meaning.
  const void* s2d_px;          // packed activation [n][h2][wp][16], pre-swizzled
  const void* s2d_wts;         // packed weights [taps][64][16], pre-swizzled
  int s2d_img_px;              // pixels per packed image = h2 * wp
  int s2d_stage_load;          // bytes copied per tile
  int s2d_box_rows;            // accumulator rows per output store box: 8, 16 or 32 (4 * box rows divides wp)

  // Epilogue
  void* out;
  long long ldc;         // elements between output rows
  long long out_batch;   // elements between batch entries
  int out_dtype;
  int epi_flags;
  const void* bias;
  const void* residual;
  long long ldr;
  long long res_batch;
  float* rowmax;         // kEpiRowMax target, [batch * m]

  int fast_epi;          // 1: staged TMA-store epilogue (needs 16-byte aligned output rows)
  int res_tma;           // 1: the staged epilogue fetches residual rows by TMA into its staging buffers

  uint32_t idesc;        // tcgen05 instruction descriptor
  uint32_t idesc_half;   // the same for a half-width tile
  int wait_limit_us;     // wall-clock limit of every barrier wait of this launch in microseconds; 0 = two seconds
  int test_drop_load;    // testing the time-out path: CTA 0's producer never issues its first operand load
  int a_split_kb;        // > 0: A's k-blocks from this one on come from the second tensor (map a1, its k from 0)
  int a2_pixels;         // 1: that second tensor is an NHWC activation sampled at a stride (im2col map a1): row i of
                         // the product is its pixel (i / (a2_p * a2_q), stride * (i / a2_q % a2_p), stride * (i % a2_q))
  int a2_p, a2_q, a2_stride;
  FastDiv a2_fd_per_img, a2_fd_q;
  int* status;           // device word: 0 = ok, otherwise the first error code seen
  long long* trace;      // debugging: CTA 0 logs (role, tile, event, clock64) records here, or null
};

// The tensor maps of one launch: A (hi / lo parts), B (hi / lo parts), output and residual tiles.
struct TcMaps {
  CUtensorMap a0, a1, b0, b1, c, r;
};

}  // namespace pmlb
