// The tensor-core contraction kernel for sm_100a.
//
// One persistent CTA per SM walks output tiles of 128 x BN.  Three roles:
//   warp 0 (one lane)  TMA producer: fills a ring of shared-memory stages with
//                      128-byte-swizzled operand tiles (A by tiled or im2col TMA).
//   warp 1 (one lane)  MMA issuer: tcgen05.mma from shared memory into one of two
//                      TMEM accumulators, tcgen05.commit to hand stages back.
//   warps 2..5         epilogue: tcgen05.ld the finished accumulator, transpose
//                      through shared memory so that global stores are row-
//                      contiguous, apply bias / residual / ReLU / cast, store.
// The second accumulator lets the epilogue of tile i overlap the main loop of
// tile i+1.
//
// Operand layouts in shared memory: every tile is rows of 128 bytes with the
// 128-byte TMA swizzle.  "K-major" tiles hold one M (or N) index per row and 128
// bytes of K; the MN-major B tile (B stored [k][n]) holds one K index per row and
// 128 bytes of N, split in chunks of 128 bytes of N.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"
#include "tc_gemm.cuh"

namespace pmlb {

template <int EB, int BN_, int NSPLIT_, bool A_IM2COL_, bool B_MN_>
struct TcCfg {
  static constexpr int BM = 128;
  static constexpr int BN = BN_;
  static constexpr int NSPLIT = NSPLIT_;
  static constexpr bool A_IM2COL = A_IM2COL_;
  static constexpr bool B_MN = B_MN_;
  static constexpr int BK = 128 / EB;       // elements of K per stage
  static constexpr int UMMA_K = 32 / EB;    // elements of K per tcgen05.mma
  static constexpr int A_TILE = BM * 128;   // bytes
  static constexpr int B_TILE = BN * 128;   // bytes
  static constexpr int STAGE = NSPLIT * (A_TILE + B_TILE);
  static constexpr int RING_BUDGET = 196 * 1024;
  static constexpr int STAGES_RAW = RING_BUDGET / STAGE;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int STG_BYTES = 4 * 32 * 33 * 4;  // per-warp 32x33 f32 transpose pads
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE + STG_BYTES + BAR_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;            // 128, 256 or 512
  static constexpr int KIND = EB == 2 ? kMmaF16 : (EB == 4 ? kMmaTf32 : kMmaI8);
  static constexpr int B_CHUNKS = BN / BK;            // MN-major: chunks of 128 bytes of N
  static_assert(STAGES >= 2, "ring too small");
  static_assert(!B_MN || (BN % BK == 0), "MN-major B needs BN to be whole chunks");
};

__device__ __forceinline__ float atomic_max_float(float* addr, float v) {
  // Ordered for all non-NaN values, including -inf as the initial content.
  if (v >= 0.f) {
    return __int_as_float(atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v)));
  }
  return __uint_as_float(atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v)));
}

template <bool IS_INT>
__device__ __forceinline__ void epilogue_store(const TcParams& p, long long out_off,
                                               long long res_off, int col, uint32_t raw) {
  if constexpr (IS_INT) {
    int x = static_cast<int>(raw);
    if (p.epi_flags & kEpiBias) x += static_cast<const int*>(p.bias)[col];
    if (p.epi_flags & kEpiResidual) {
      if (p.out_dtype == kDtI32) {
        x += static_cast<const int*>(p.residual)[res_off];
      } else {
        x += static_cast<const int8_t*>(p.residual)[res_off];
      }
    }
    if (p.epi_flags & kEpiRelu) x = x < 0 ? 0 : x;
    if (p.out_dtype == kDtI32) {
      static_cast<int*>(p.out)[out_off] = x;
    } else {
      static_cast<int8_t*>(p.out)[out_off] = static_cast<int8_t>(x);  // two's-complement wrap
    }
  } else {
    float x = __uint_as_float(raw);
    if (p.epi_flags & kEpiBias) x += static_cast<const float*>(p.bias)[col];
    if (p.epi_flags & kEpiResidual) {
      if (p.out_dtype == kDtF32) {
        x += static_cast<const float*>(p.residual)[res_off];
      } else if (p.out_dtype == kDtBF16) {
        x += __bfloat162float(static_cast<const __nv_bfloat16*>(p.residual)[res_off]);
      } else {
        x += __half2float(static_cast<const __half*>(p.residual)[res_off]);
      }
    }
    if (p.epi_flags & kEpiRelu) x = x < 0.f ? 0.f : x;
    if (p.out_dtype == kDtF32) {
      static_cast<float*>(p.out)[out_off] = x;
    } else if (p.out_dtype == kDtBF16) {
      static_cast<__nv_bfloat16*>(p.out)[out_off] = __float2bfloat16_rn(x);
    } else {
      static_cast<__half*>(p.out)[out_off] = __float2half_rn(x);
    }
  }
}

struct TileCoord {
  int b, tm, tn;
};

__device__ __forceinline__ TileCoord tile_coord(const TcParams& p, int t) {
  const int per_batch = p.tiles_m * p.tiles_n;
  TileCoord c;
  c.b = t / per_batch;
  const int r = t - c.b * per_batch;
  const int group = p.group_m * p.tiles_n;
  const int g = r / group;
  const int first_m = g * p.group_m;
  const int gm = min(p.group_m, p.tiles_m - first_m);
  const int rr = r - g * group;
  c.tm = first_m + rr % gm;
  c.tn = rr / gm;
  return c;
}

template <class Cfg>
__global__ void __launch_bounds__(192, 1)
tc_contract_kernel(const __grid_constant__ CUtensorMap tm_a0,
                   const __grid_constant__ CUtensorMap tm_a1,
                   const __grid_constant__ CUtensorMap tm_b0,
                   const __grid_constant__ CUtensorMap tm_b1,
                   const __grid_constant__ TcParams p) {
  constexpr int BN = Cfg::BN;
  constexpr int BK = Cfg::BK;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NSPLIT = Cfg::NSPLIT;
  constexpr bool IS_INT = (Cfg::KIND == kMmaI8);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t ring = (raw_addr + 1023u) & ~1023u;           // shared-space address
  uint8_t* ring_ptr = smem_raw + (ring - raw_addr);            // generic pointer
  float* stg_all = reinterpret_cast<float*>(ring_ptr + STAGES * Cfg::STAGE);
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring_ptr + STAGES * Cfg::STAGE + Cfg::STG_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  // barrier index helpers (8 bytes each)
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* abort_code = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    *abort_flag = 0;
    *abort_code = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_a0);
    tma_prefetch_desc(&tm_b0);
    if (NSPLIT == 2) {
      tma_prefetch_desc(&tm_a1);
      tma_prefetch_desc(&tm_b1);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.batch * p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const TileCoord tc = tile_coord(p, t);
        int pix_w = 0, pix_h = 0, pix_n = 0;
        if constexpr (Cfg::A_IM2COL) {
          const int m0 = tc.tm * 128;
          const int per_img = p.conv_p * p.conv_q;
          pix_n = m0 / per_img;
          const int rem = m0 - pix_n * per_img;
          const int op = rem / p.conv_q;
          const int oq = rem - op * p.conv_q;
          pix_w = p.conv_lower_w + oq * p.conv_stride_w;
          pix_h = p.conv_lower_h + op * p.conv_stride_h;
        }
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            if (*abort_code == 0) *abort_code = 1;
            ok = false;
            break;
          }
          const uint32_t fb = full_bar(stage);
          mbar_arrive_expect_tx(fb, Cfg::STAGE);
          const uint32_t s_a = ring + stage * Cfg::STAGE;
          const uint32_t s_b = s_a + NSPLIT * Cfg::A_TILE;
          if constexpr (Cfg::A_IM2COL) {
            const int tap = kb / p.conv_cblocks;
            const int cb = kb - tap * p.conv_cblocks;
            const int fr = tap / p.conv_s;
            const int fs = tap - fr * p.conv_s;
            tma_load_im2col_4d(s_a, &tm_a0, fb, cb * BK, pix_w, pix_h, pix_n,
                               static_cast<uint16_t>(fs * p.conv_dil_w),
                               static_cast<uint16_t>(fr * p.conv_dil_h));
            // weights laid out [k_out][tap][c_in]: map dims (c_in, tap, k_out)
            tma_load_3d(s_b, &tm_b0, fb, cb * BK, tap, tc.tn * BN);
          } else {
            tma_load_3d(s_a, &tm_a0, fb, kb * BK, tc.tm * 128, tc.b * p.a_bz);
            if constexpr (NSPLIT == 2) {
              tma_load_3d(s_a + Cfg::A_TILE, &tm_a1, fb, kb * BK, tc.tm * 128, tc.b * p.a_bz);
            }
            if constexpr (Cfg::B_MN) {
#pragma unroll
              for (int ch = 0; ch < Cfg::B_CHUNKS; ++ch) {
                tma_load_3d(s_b + ch * (BK * 128), &tm_b0, fb, tc.tn * BN + ch * BK, kb * BK,
                            tc.b * p.b_bz);
              }
            } else {
              tma_load_3d(s_b, &tm_b0, fb, kb * BK, tc.tn * BN, tc.b * p.b_bz);
              if constexpr (NSPLIT == 2) {
                tma_load_3d(s_b + Cfg::B_TILE, &tm_b1, fb, kb * BK, tc.tn * BN, tc.b * p.b_bz);
              }
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
          if (*abort_code == 0) *abort_code = 2;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            if (*abort_code == 0) *abort_code = 3;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t s_a = ring + stage * Cfg::STAGE;
          const uint32_t s_b = s_a + NSPLIT * Cfg::A_TILE;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t accum = (kb > 0 || j > 0) ? 1u : 0u;
            const uint64_t a_hi = make_smem_desc_sw128(s_a + j * 32, 16, 1024);
            uint64_t b_hi;
            if constexpr (Cfg::B_MN) {
              b_hi = make_smem_desc_sw128(s_b + j * (Cfg::UMMA_K * 128), BK * 128, 1024);
            } else {
              b_hi = make_smem_desc_sw128(s_b + j * 32, 16, 1024);
            }
            if constexpr (NSPLIT == 2) {
              // fp32 as three TF32 products; the two cross terms first.
              const uint64_t a_lo = make_smem_desc_sw128(s_a + Cfg::A_TILE + j * 32, 16, 1024);
              const uint64_t b_lo = make_smem_desc_sw128(s_b + Cfg::B_TILE + j * 32, 16, 1024);
              tc_mma<Cfg::KIND>(d_tmem, a_lo, b_hi, p.idesc, accum);
              tc_mma<Cfg::KIND>(d_tmem, a_hi, b_lo, p.idesc, 1u);
              tc_mma<Cfg::KIND>(d_tmem, a_hi, b_hi, p.idesc, 1u);
            } else {
              tc_mma<Cfg::KIND>(d_tmem, a_hi, b_hi, p.idesc, accum);
            }
          }
          tc_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(tfull_bar(acc));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;                     // TMEM lane quarter this warp may read
    float* stg = stg_all + q * (32 * 33);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const TileCoord tc = tile_coord(p, t);
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
        if (*abort_code == 0) *abort_code = 4;
        break;
      }
      tc_fence_after_sync();
      const int row0 = tc.tm * 128 + q * 32;     // first row of this warp
      const int col_base = tc.tn * BN;
      const uint32_t t_acc =
          tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(q * 32) << 16);
      const long long out_b = static_cast<long long>(tc.b) * p.out_batch;
      const long long res_b = static_cast<long long>(tc.b) * p.res_batch;
      float row_best = -INFINITY;

#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        const int col0 = col_base + ch * 32;
        uint32_t v[32];
        tmem_ld_32x32(t_acc + ch * 32, v);
        tmem_ld_wait();
        if (ch == BN / 32 - 1) {
          // accumulator fully read: hand it back before finishing the stores
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
        if (col0 >= p.n) continue;   // warp-uniform
        if (p.epi_flags & kEpiRowMax) {
          if constexpr (!IS_INT) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float x = __uint_as_float(v[j]);
              if (col0 + j < p.n && x > row_best) row_best = x;
            }
          }
          if (p.out == nullptr) continue;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = __uint_as_float(v[j]);
        __syncwarp();
        const int col = col0 + lane;
        if (col < p.n) {
          const int rows = min(32, p.m - row0);
          for (int r = 0; r < rows; ++r) {
            const long long row = row0 + r;
            epilogue_store<IS_INT>(p, out_b + row * p.ldc + col, res_b + row * p.ldr + col, col,
                                   __float_as_uint(stg[r * 33 + lane]));
          }
        }
        __syncwarp();
      }
      if (p.epi_flags & kEpiRowMax) {
        const int row = row0 + lane;
        if (row < p.m) {
          atomic_max_float(p.rowmax + static_cast<long long>(tc.b) * p.m + row, row_best);
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    // A wait gave up.  Report, then give copies and MMAs still in flight a bounded
    // time to land before TMEM and shared memory are released.
    if (threadIdx.x == 0) {
      const int code = *abort_code != 0 ? *abort_code : 9;
      atomicCAS(p.status, 0, code);
    }
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) {
      __nanosleep(2000);
    }
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace pmlb
