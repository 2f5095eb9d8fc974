// The tensor-core contraction kernel for sm_100a.
//
// One persistent CTA per SM walks output tiles of 128 x BN.  Three roles:
//   warp 0 (one lane)  TMA producer: fills a ring of shared-memory stages with
//                      128-byte-swizzled operand tiles (A by tiled or im2col TMA).
//   warp 1 (one lane)  MMA issuer: tcgen05.mma from shared memory into one of two
//                      TMEM accumulators, tcgen05.commit to hand stages back.
//   warps 2..5         epilogue: tcgen05.ld the finished accumulator, apply bias /
//                      residual / ReLU / cast in registers, stage 32 rows x 128
//                      bytes in swizzled shared memory and hand them to a TMA
//                      store (outputs whose rows are not 16-byte aligned take a
//                      slower path through a shared-memory transpose).
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

#include <cstdlib>
#include <type_traits>

#include "ptx.cuh"
#include "tc_gemm.cuh"

namespace pmlb {

// How the A operand reaches shared memory.
enum : int {
  kATiled = 0,   // a [m][k] matrix, tiled TMA
  kAIm2col = 1,  // an NHWC activation, im2col TMA: one k-block per filter tap and channel block
  kAWindow = 2,  // a packed-row activation: one k-block per filter row, each input row fetched
                 // once into a ring of row slots and reused by the output rows that overlap it
  kAHalo = 3,    // an NHWC activation, stride-1 convolution: the zero-padded pixels of a few
                 // image rows are fetched once per tile (tiled TMA, padding = out-of-bounds
                 // fill) and every filter tap is read as a row-shifted window of that buffer;
                 // output positions in the padding columns are computed and discarded
  kAS2d = 4,     // a thin NHWC activation, stride-2 convolution, repacked by a pre-pass to 32-byte
                 // pixels holding the 2 x 2 phases as channels, four pixels to a 128-byte row
                 // and already in the 128-byte swizzle.  A tile is 512 consecutive pixel
                 // positions, fetched with the pixels its taps reach by one untiled bulk copy,
                 // and has four accumulators: row i of accumulator a is position 4 * i + a, so
                 // that the operand of a tap is the buffer read from byte 32 * (a + tap shift)
                 // on, one 32-byte k-step of every 128-byte row (operand rows in any other
                 // layout than 128-byte rows in the 128-byte swizzle were measured to feed the
                 // tensor core at well under half the rate)
};

template <int EB, int BN_, int NSPLIT_, int A_MODE_, bool B_MN_, int OUT_BYTES_ = 4,
          int EPI_GROUPS_ = 1, int CTAS_ = 1>
struct TcCfg {
  // 2: two CTAs (a cluster of two, on neighbouring SMs) work on one 256 x BN tile with
  // cta_group::2 MMAs: each CTA holds 128 rows of A and of the accumulator and half of B's
  // N rows, so that a B tile crosses from L2 to shared memory once per 256 output rows.
  static constexpr int CTAS = CTAS_;
  // 1: four epilogue warps drain both TMEM accumulators in turn (TMEM loads software-
  //    pipelined); 2: eight warps, one group of four per accumulator, for shapes whose main
  //    loop per tile is shorter than the epilogue (small K).
  static constexpr int EPI_GROUPS = EPI_GROUPS_;
  static constexpr int OUT_BYTES = OUT_BYTES_;  // element size the staged epilogue packs to
  static constexpr int CW = 128 / OUT_BYTES_;   // output columns per 128-byte staged row
  static constexpr int BM = 128;
  static constexpr int BN = BN_;
  static constexpr int NSPLIT = NSPLIT_;
  static constexpr int A_MODE = A_MODE_;
  static constexpr bool A_IM2COL = A_MODE_ == kAIm2col;
  static constexpr bool A_WINDOW = A_MODE_ == kAWindow;
  static constexpr bool A_HALO = A_MODE_ == kAHalo;
  static constexpr bool A_S2D = A_MODE_ == kAS2d;
  static constexpr bool B_MN = B_MN_;
  static constexpr int BK = 128 / EB;       // elements of K per stage
  static constexpr int UMMA_K = 32 / EB;    // elements of K per tcgen05.mma
  static constexpr int A_TILE = BM * 128;   // bytes
  static constexpr int B_TILE = (BN / CTAS_) * 128;   // bytes held by one CTA
  static constexpr int STAGE = NSPLIT * (A_TILE + B_TILE);
  static constexpr int STG_BYTES = EPI_GROUPS_ * 4 * 2 * 4096;  // per epilogue warp: two 32-row x 128-byte buffers
  static constexpr int BAR_BYTES = 1024;
  static constexpr int SMEM_LIMIT = 232448;                     // 227 KB per CTA
  static constexpr int RING_BUDGET = SMEM_LIMIT - 1024 - STG_BYTES - BAR_BYTES;
  static constexpr int STAGES_RAW = RING_BUDGET / STAGE;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE + STG_BYTES + BAR_BYTES;
  // MMA-issuing warps.  The tensor pipe queues only three or four MMAs; a 64- or 128-wide MMA
  // lasts 48 / 64 cycles, so the issuing thread's per-tile bookkeeping (barrier waits, commits:
  // several hundred cycles) leaves the pipe idle.  Narrow tiles therefore get two issuers that
  // take alternate tiles, each with its own pair of accumulators.
  static constexpr int ISSUERS = (BN_ <= 64 && CTAS_ == 1 && NSPLIT_ == 1 && A_MODE_ != kAWindow) ? 2 : 1;
  static constexpr int NACC = 2 * ISSUERS;            // TMEM accumulators
  static constexpr int FIRST_EPI_WARP = 1 + ISSUERS;
  static constexpr int THREADS = 32 * FIRST_EPI_WARP + 128 * EPI_GROUPS_;
  static constexpr int TMEM_COLS = NACC * BN;         // 128, 256 or 512
  static constexpr int KIND = EB == 2 ? kMmaF16 : (EB == 4 ? kMmaTf32 : kMmaI8);
  static constexpr int B_CHUNKS = (BN / CTAS_) / BK;  // MN-major: chunks of 128 bytes of N per CTA
  static_assert(STAGES >= 2, "ring too small");
  static_assert(!B_MN || ((BN / CTAS_) % BK == 0), "MN-major B needs whole chunks per CTA");
  static_assert(CTAS_ == 1 || (CTAS_ == 2 && (A_MODE_ == kATiled || A_MODE_ == kAIm2col) && NSPLIT_ == 1),
                "CTA pairs serve plain 8/16-bit GEMMs and im2col convolutions");
};

__device__ __forceinline__ float atomic_max_float(float* addr, float v) {
  // Ordered for all non-NaN values, including -inf as the initial content.  The branch is on the sign
  // bit, not on v >= 0: -0.0 has the bit pattern of the most negative integer and belongs with the
  // negative values (where, as the smallest unsigned pattern of them, it wins as it should).
  if (__float_as_int(v) >= 0) {
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
    // An int8 result is the sum wrapped to 8 bits (two's complement) and the ReLU acts on that value:
    // narrowing comes first, as when every step of the chain is computed in the result type.
    if (p.out_dtype != kDtI32) x = static_cast<int8_t>(x);
    if (p.epi_flags & kEpiRelu) x = x < 0 ? 0 : x;
    if (p.out_dtype == kDtI32) {
      static_cast<int*>(p.out)[out_off] = x;
    } else {
      static_cast<int8_t*>(p.out)[out_off] = static_cast<int8_t>(x);
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

// Pipeline timeline for debugging: CTA 0 appends {tile, event, clock64} triples to one of four
// lanes of the trace buffer (0 producer, 1 MMA issuer, 2 and 3 the first warp of each epilogue
// group).  A null trace pointer (the normal case) costs one predictable branch per event.
constexpr int kTraceRecords = 2048;
__device__ __forceinline__ void trace_event(const TcParams& p, int role, int& n, int tile, int ev) {
  if (p.trace != nullptr && blockIdx.x == 0 && n < kTraceRecords) {
    long long* r = p.trace + (static_cast<long long>(role) * kTraceRecords + n) * 3;
    r[0] = tile;
    r[1] = ev;
    r[2] = clock64();
    ++n;
  }
}

// The timeline records cost the roles several per cent even when no buffer is given (each is a
// divergent branch): they are compiled in only with -DPMLB_TC_TRACE.
#ifdef PMLB_TC_TRACE
#define PMLB_TRACE_EVENT(...) trace_event(__VA_ARGS__)
#else
#define PMLB_TRACE_EVENT(...) ((void)0)
#endif

struct TileCoord {
  int b, tm, tn;
  int n0, bn;   // first output column and width of the tile (set by tile_coord_cta)
};

__device__ __forceinline__ TileCoord tile_coord(const TcParams& p, int t) {
  const int per_batch = p.tiles_m * p.tiles_n;
  TileCoord c;
  c.b = fast_div(t, p.fd_per_batch);
  const int r = t - c.b * per_batch;
  const int group = p.group_m * p.tiles_n;
  const int g = fast_div(r, p.fd_group);
  const int first_m = g * p.group_m;
  const int rr = r - g * group;
  // a full group has group_m m-tiles, the last one of a batch entry the remainder
  const bool full = first_m + p.group_m <= p.tiles_m;
  const int gm = full ? p.group_m : p.tiles_m - first_m;
  c.tn = fast_div(rr, full ? p.fd_gm_full : p.fd_gm_tail);
  c.tm = first_m + rr - c.tn * gm;
  return c;
}

// Packed-row convolution: tile t is output row `op` of strip (image `img`, segment `tm` of 128
// output columns); tiles of a strip are consecutive so that a CTA walking a contiguous range
// of tiles slides its window of input rows down the image.  As a batched problem the tile is
// batch entry img * P + op.
struct WinCoord {
  int strip, img, op, tm;
};

__device__ __forceinline__ WinCoord win_coord(const TcParams& p, int t) {
  WinCoord c;
  c.strip = t / p.conv_p;
  c.op = t - c.strip * p.conv_p;
  c.img = c.strip / p.tiles_m;
  c.tm = c.strip - c.img * p.tiles_m;
  return c;
}

template <class Cfg>
__device__ __forceinline__ TileCoord tile_coord_for(const TcParams& p, int t) {
  if constexpr (Cfg::A_WINDOW) {
    const WinCoord w = win_coord(p, t);
    TileCoord c;
    c.b = w.img * p.conv_p + w.op;
    c.tm = w.tm;
    c.tn = 0;
    return c;
  } else {
    return tile_coord(p, t);
  }
}

// Tile number t as the roles walk it -> coordinates for this CTA.  Tiles below p.tiles_full
// are whole BN-wide tiles; above it every remaining tile appears twice, as its left and its
// right half (the tail of the last wave, cut in two so that it takes half as long).  CTA pairs:
// tm becomes this CTA's 128-row tile number.
template <class Cfg>
__device__ __forceinline__ TileCoord tile_coord_cta(const TcParams& p, int t, uint32_t cta_rank) {
  int idx = t, half = -1;
  if (t >= p.tiles_full) {
    const int u = t - p.tiles_full;
    idx = p.tiles_full + (u >> 1);
    half = u & 1;
  }
  TileCoord c = tile_coord_for<Cfg>(p, idx);
  c.bn = half < 0 ? Cfg::BN : Cfg::BN / 2;
  c.n0 = c.tn * Cfg::BN + (half > 0 ? Cfg::BN / 2 : 0);
  if constexpr (Cfg::CTAS == 2) c.tm = 2 * c.tm + static_cast<int>(cta_rank);
  return c;
}

// Epilogue arithmetic on one staged chunk: CW accumulator columns of this thread's row.
// FULL: the chunk lies wholly inside the matrix, so no per-column guards are needed and
// bias / residual come in 16-byte loads.  The guarded variant serves the last chunk of
// a ragged N.
template <bool FULL, bool IS_INT, int OB, int CW>
__device__ __forceinline__ float epi_apply(const TcParams& p, uint32_t (&v)[CW], int col0, int row,
                                           long long res_row, bool out_bf16, uint32_t res_smem,
                                           int lane, bool relu_later) {
  // res_smem != 0: this warp's 32 x 128-byte residual rows lie in shared memory (swizzled like
  // the staged output; rows and columns outside the matrix hold zeros), else they are read
  // from global memory.
  const int nvalid = FULL ? CW : (p.n - col0);
  const bool want_res = (p.epi_flags & kEpiResidual) && (row < p.m || res_smem != 0);
  const uint32_t res_line = res_smem + static_cast<uint32_t>(lane) * 128u;
  const uint32_t res_xor = static_cast<uint32_t>(lane & 7);
  float chunk_best = -INFINITY;
  if constexpr (IS_INT) {
    // 32-bit integer results (OB == 4)
    if (p.epi_flags & kEpiBias) {
      const int* bp = static_cast<const int*>(p.bias) + col0;
      if constexpr (FULL) {
#pragma unroll
        for (int i = 0; i < CW / 4; ++i) {
          const int4 b4 = __ldg(reinterpret_cast<const int4*>(bp) + i);
          v[4 * i + 0] += static_cast<uint32_t>(b4.x);
          v[4 * i + 1] += static_cast<uint32_t>(b4.y);
          v[4 * i + 2] += static_cast<uint32_t>(b4.z);
          v[4 * i + 3] += static_cast<uint32_t>(b4.w);
        }
      } else {
#pragma unroll
        for (int j = 0; j < CW; ++j) {
          if (j < nvalid) v[j] += static_cast<uint32_t>(__ldg(bp + j));
        }
      }
    }
    if (want_res) {
      const int* rp = static_cast<const int*>(p.residual) + res_row + col0;
      if (FULL || res_smem != 0) {
#pragma unroll
        for (int i = 0; i < CW / 4; ++i) {
          uint4 r4;
          if (res_smem != 0) {
            r4 = ld_shared_v4(res_line + ((static_cast<uint32_t>(i) ^ res_xor) << 4));
          } else {
            r4 = __ldg(reinterpret_cast<const uint4*>(rp) + i);
          }
          v[4 * i + 0] += static_cast<uint32_t>(r4.x);
          v[4 * i + 1] += static_cast<uint32_t>(r4.y);
          v[4 * i + 2] += static_cast<uint32_t>(r4.z);
          v[4 * i + 3] += static_cast<uint32_t>(r4.w);
        }
      } else {
#pragma unroll
        for (int j = 0; j < CW; ++j) {
          if (j < nvalid) v[j] += static_cast<uint32_t>(rp[j]);
        }
      }
    }
    if (p.epi_flags & kEpiRelu) {
#pragma unroll
      for (int j = 0; j < CW; ++j) v[j] = static_cast<uint32_t>(max(static_cast<int>(v[j]), 0));
    }
  } else {
    if (p.epi_flags & kEpiBias) {
      const float* bp = static_cast<const float*>(p.bias) + col0;
      if constexpr (FULL) {
#pragma unroll
        for (int i = 0; i < CW / 4; ++i) {
          const float4 b4 = __ldg(reinterpret_cast<const float4*>(bp) + i);
          v[4 * i + 0] = __float_as_uint(__uint_as_float(v[4 * i + 0]) + b4.x);
          v[4 * i + 1] = __float_as_uint(__uint_as_float(v[4 * i + 1]) + b4.y);
          v[4 * i + 2] = __float_as_uint(__uint_as_float(v[4 * i + 2]) + b4.z);
          v[4 * i + 3] = __float_as_uint(__uint_as_float(v[4 * i + 3]) + b4.w);
        }
      } else {
#pragma unroll
        for (int j = 0; j < CW; ++j) {
          if (j < nvalid) v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldg(bp + j));
        }
      }
    }
    if (want_res) {
      if (FULL || res_smem != 0) {
        const uint4* rp = reinterpret_cast<const uint4*>(
            static_cast<const char*>(p.residual) + (res_row + col0) * OB);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint4 r4;
          if (res_smem != 0) {
            r4 = ld_shared_v4(res_line + ((static_cast<uint32_t>(i) ^ res_xor) << 4));
          } else {
            r4 = __ldg(rp + i);
          }
          const uint32_t w[4] = {r4.x, r4.y, r4.z, r4.w};
          if constexpr (OB == 4) {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              v[4 * i + h] = __float_as_uint(__uint_as_float(v[4 * i + h]) + __uint_as_float(w[h]));
            }
          } else {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              float r0, r1;
              if (out_bf16) {
                r0 = __uint_as_float(w[h] << 16);
                r1 = __uint_as_float(w[h] & 0xffff0000u);
              } else {
                const __half2 hh = *reinterpret_cast<const __half2*>(&w[h]);
                r0 = __low2float(hh);
                r1 = __high2float(hh);
              }
              const int j = 8 * i + 2 * h;
              v[j] = __float_as_uint(__uint_as_float(v[j]) + r0);
              v[j + 1] = __float_as_uint(__uint_as_float(v[j + 1]) + r1);
            }
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < CW; ++j) {
          if (j < nvalid) {
            float r;
            if constexpr (OB == 4) {
              r = static_cast<const float*>(p.residual)[res_row + col0 + j];
            } else if (out_bf16) {
              r = __bfloat162float(static_cast<const __nv_bfloat16*>(p.residual)[res_row + col0 + j]);
            } else {
              r = __half2float(static_cast<const __half*>(p.residual)[res_row + col0 + j]);
            }
            v[j] = __float_as_uint(__uint_as_float(v[j]) + r);
          }
        }
      }
    }
    // (16-bit outputs without a row maximum get their ReLU from the packing conversion)
    if ((p.epi_flags & kEpiRelu) && !relu_later) {
#pragma unroll
      for (int j = 0; j < CW; ++j) v[j] = __float_as_uint(relu_keep_nan(__uint_as_float(v[j])));
    }
    if (p.epi_flags & kEpiRowMax) {
      // Balanced tree of hardware max operations.  For non-NaN values this equals the
      // compare-and-select chain of the definition; with NaNs the definition itself
      // depends on the visiting order.
      float mx[CW];
#pragma unroll
      for (int j = 0; j < CW; ++j) {
        mx[j] = (FULL || j < nvalid) ? __uint_as_float(v[j]) : -INFINITY;
      }
#pragma unroll
      for (int w = CW / 2; w > 0; w >>= 1) {
#pragma unroll
        for (int j = 0; j < w; ++j) mx[j] = fmaxf(mx[j], mx[j + w]);
      }
      chunk_best = mx[0];
    }
  }
  return chunk_best;
}

// PMLB_TC_DEPENDENT_LAUNCH=1 in the environment launches the tensor-core kernels with the programmatic
// stream-serialization attribute (see grid_dependency_wait).  Off by default: measured on ResNet-50 it moved
// a pass by -2 % to +1 %, i.e. within the run-to-run spread (one CTA per SM at 227 KB of shared memory leaves
// nothing for the next kernel's CTAs to overlap with until an SM is vacated).
inline bool dependent_launch_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("PMLB_TC_DEPENDENT_LAUNCH");
    return v && v[0] == '1';
  }();
  return on;
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
tc_contract_kernel(const __grid_constant__ TcMaps tm, const __grid_constant__ TcParams p) {
  constexpr int BN = Cfg::BN;
  constexpr int BK = Cfg::BK;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NSPLIT = Cfg::NSPLIT;
  constexpr bool IS_INT = (Cfg::KIND == kMmaI8);

  // (the next kernel of the stream may be scheduled onto SMs as this one leaves them; it waits for this
  // kernel's completion before it touches memory)
  grid_launch_dependents();
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
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };             // up to 4
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 4 + a); };
  // two residual-arrival barriers per epilogue warp (at most 8 warps)
  auto res_bar = [&](int ew, uint32_t i) { return bar0 + 8u * (2 * STAGES + 8 + 2 * ew + i); };
  // packed-row mode: arrival / release barriers of up to 16 row slots, one for the weights
  auto wfull_bar = [&](uint32_t i) { return bar0 + 8u * (2 * STAGES + 24 + i); };
  auto wempty_bar = [&](uint32_t i) { return bar0 + 8u * (2 * STAGES + 40 + i); };
  const uint32_t wts_bar = bar0 + 8u * (2 * STAGES + 56);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 57);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* abort_code = reinterpret_cast<volatile int*>(tmem_slot + 2);

  // warp number through a shuffle: tells the compiler it is the same in all lanes
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  constexpr int CTAS = Cfg::CTAS;
  // CTA pair: rank 0 issues the pair's MMAs and owns the barriers both producers and both
  // epilogues report to (`full` and `tempty`); `empty` and `tfull` exist in both CTAs and are
  // reached by multicast commits.
  const uint32_t cta_rank = CTAS == 2 ? cluster_ctarank() : 0u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      // Every MMA-issuing warp reports on a stage before it is refilled: the tile's owner when its MMAs
      // have read it (a commit), the other issuer when it has seen the stage arrive (a plain arrive).
      // A parity wait cannot tell a phase from the one two later, so a warp that only watched the
      // stages go by could, if it fell one ring revolution behind, wait for ever.
      mbar_init(empty_bar(s), Cfg::ISSUERS);
    }
    for (int a = 0; a < Cfg::NACC; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4 * CTAS);
    }
    for (int w = 0; w < 8; ++w) {
      mbar_init(res_bar(w, 0), 1);
      mbar_init(res_bar(w, 1), 1);
    }
    if constexpr (Cfg::A_WINDOW) {
      for (uint32_t i = 0; i < 16; ++i) {
        mbar_init(wfull_bar(i), 1);
        mbar_init(wempty_bar(i), 1);
      }
      mbar_init(wts_bar, 1);
    }
    if constexpr (Cfg::A_HALO || Cfg::A_S2D) mbar_init(wts_bar, 1);
    *abort_flag = 0;
    *abort_code = 0;
    abort_flag[2] = p.wait_limit_us;
    fence_mbar_init();
    tma_prefetch_desc(&tm.a0);
    tma_prefetch_desc(&tm.b0);
    if (NSPLIT == 2 || p.a_split_kb > 0) {
      tma_prefetch_desc(&tm.a1);
    }
    if (NSPLIT == 2) {
      tma_prefetch_desc(&tm.b1);
    }
    if (p.fast_epi && p.out != nullptr) tma_prefetch_desc(&tm.c);
    if (p.res_tma) tma_prefetch_desc(&tm.r);
  }
  if (warp == 1) {
    if constexpr (CTAS == 2) {
      tmem_alloc_pair(smem_u32(tmem_slot), Cfg::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (CTAS == 2) {
    cluster_sync_all();   // the other CTA's barriers must exist before anything is sent to them
  } else {
    __syncthreads();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // set-up done: from here on the kernel reads and writes tensors, so the kernel before it must be complete
  grid_dependency_wait();

  // (pairs: p.tiles_m counts 256-row pair tiles; CTA `rank` takes rows 128 * rank .. of each)
  const int total_tiles = 2 * p.batch * p.tiles_m * p.tiles_n - p.tiles_full;   // halves count twice
  // Tiles this CTA walks: every gridDim.x-th one (pairs: every cluster-count-th one), or
  // (packed-row mode) a contiguous range.
  int t_begin = blockIdx.x / CTAS, t_end = total_tiles, t_step = gridDim.x / CTAS;
  if constexpr (Cfg::A_WINDOW) {
    t_begin = static_cast<int>(static_cast<long long>(total_tiles) * blockIdx.x / gridDim.x);
    t_end = static_cast<int>(static_cast<long long>(total_tiles) * (blockIdx.x + 1) / gridDim.x);
    t_step = 1;
  }
  // packed-row mode: the weights of all filter rows stay in shared memory ahead of the row slots
  const uint32_t win_wts = ring;
  const uint32_t win_slots = ring + static_cast<uint32_t>(p.win_r) * Cfg::B_TILE;

  // halo mode: the weights of every (tap, channel block) stay in shared memory ahead of the ring
  // of fetched pixel buffers; halo_nb = k-blocks (taps x channel blocks) per tile
  const int halo_taps = p.conv_r * p.conv_s;
  const uint32_t halo_ring =
      ring + (Cfg::A_S2D ? static_cast<uint32_t>(p.conv_r * ((p.conv_s + 3) / 4)) * 8192u
                         : static_cast<uint32_t>(halo_taps * p.conv_cblocks) * Cfg::B_TILE);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // The whole warp walks the loops (so that addresses and coordinates stay on the uniform
    // datapath); one elected lane issues the copies.
    const bool leader = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int ntrace = 0;
    if constexpr (Cfg::A_S2D) {
      // Weights of every tap, once: a 64-row block of 128-byte rows per four tap columns.
      const uint32_t wts_bytes = static_cast<uint32_t>(p.conv_r * ((p.conv_s + 3) / 4)) * 8192u;
      if (leader) {
        mbar_arrive_expect_tx(wts_bar, wts_bytes);
        bulk_load_1d(ring, p.s2d_wts, wts_bytes, wts_bar);
      }
      // One buffer per tile: the tile's 512 pixel positions and the pixels its taps reach are
      // consecutive in the packed activation.
      const uint32_t nst = static_cast<uint32_t>(p.halo_stages);
      uint32_t hs = 0, hphase = 0;
      for (int t = t_begin; t < t_end && ok; t += t_step) {
        const int img = fast_div(t, p.fd_tiles_per_img);
        const int tt = t - img * p.halo_tiles_per_img;
        if (!mbar_wait_warp(empty_bar(hs), hphase ^ 1u, abort_flag)) {
          if (leader && *abort_code == 0) *abort_code = 1;
          ok = false;
          break;
        }
        if (leader) {
          PMLB_TRACE_EVENT(p, 0, ntrace, t, 0);
          const char* src = static_cast<const char*>(p.s2d_px) +
                            (static_cast<long long>(img) * p.s2d_img_px + tt * 512) * 32;
          mbar_arrive_expect_tx(full_bar(hs), static_cast<uint32_t>(p.s2d_stage_load));
          bulk_load_1d(halo_ring + hs * static_cast<uint32_t>(p.halo_stage_bytes), src,
                       static_cast<uint32_t>(p.s2d_stage_load), full_bar(hs));
        }
        if (++hs == nst) {
          hs = 0;
          hphase ^= 1u;
        }
      }
    } else if constexpr (Cfg::A_HALO) {
      // Weights of every tap and channel block, once: block (tap, cb) at wts + (tap * cblocks + cb).
      if (leader) {
        mbar_arrive_expect_tx(wts_bar, static_cast<uint32_t>(halo_taps * p.conv_cblocks) * Cfg::B_TILE);
        for (int tap = 0; tap < halo_taps; ++tap) {
          for (int cb = 0; cb < p.conv_cblocks; ++cb) {
            tma_load_3d(ring + static_cast<uint32_t>(tap * p.conv_cblocks + cb) * Cfg::B_TILE, &tm.b0,
                        wts_bar, cb * BK, tap, 0);
          }
        }
      }
      // One buffer per tile and channel block: image rows p0 - pad .. of the padded width.
      const uint32_t nst = static_cast<uint32_t>(p.halo_stages);
      uint32_t hs = 0, hphase = 0;
      for (int t = t_begin; t < t_end && ok; t += t_step) {
        const int img = fast_div(t, p.fd_tiles_per_img);
        const int p0 = (t - img * p.halo_tiles_per_img) * p.halo_th;
        for (int cb = 0; cb < p.conv_cblocks; ++cb) {
          if (!mbar_wait_warp(empty_bar(hs), hphase ^ 1u, abort_flag)) {
            if (leader && *abort_code == 0) *abort_code = 1;
            ok = false;
            break;
          }
          if (leader) {
            PMLB_TRACE_EVENT(p, 0, ntrace, t, cb);
            mbar_arrive_expect_tx(full_bar(hs), static_cast<uint32_t>(p.halo_wp * p.halo_rows) * 128u);
            tma_load_4d(halo_ring + hs * static_cast<uint32_t>(p.halo_stage_bytes), &tm.a0, full_bar(hs),
                        cb * BK, p.conv_lower_w, p0 + p.conv_lower_h, img);
          }
          if (++hs == nst) {
            hs = 0;
            hphase ^= 1u;
          }
        }
      }
    } else if constexpr (Cfg::A_WINDOW) {
      // Weights of every filter row, once.
      if (leader) {
        mbar_arrive_expect_tx(wts_bar, static_cast<uint32_t>(p.win_r) * Cfg::B_TILE);
        for (int r = 0; r < p.win_r; ++r) {
          tma_load_3d(win_wts + r * Cfg::B_TILE, &tm.b0, wts_bar, 0, r, 0);
        }
      }
      // Input rows in the order the output rows need them; `cnt` numbers them, row number
      // cnt goes to slot cnt % slots.
      uint32_t cnt = 0;
      int cur_strip = -1, next_h = 0;
      const uint32_t nslots = static_cast<uint32_t>(p.win_slots);
      uint32_t slot = 0, use = 0;   // cnt % nslots, cnt / nslots
      for (int t = t_begin; t < t_end && ok; ++t) {
        const WinCoord wc = win_coord(p, t);
        const int lo = wc.op * p.conv_stride_h + p.conv_lower_h;
        if (wc.strip != cur_strip) {
          cur_strip = wc.strip;
          next_h = lo;
        }
        for (int h = next_h; h < lo + p.win_r; ++h) {
          if (use > 0 && !mbar_wait_warp(wempty_bar(slot), (use - 1u) & 1u, abort_flag)) {
            if (leader && *abort_code == 0) *abort_code = 1;
            ok = false;
            break;
          }
          if (leader) {
            PMLB_TRACE_EVENT(p, 0, ntrace, t, h);
            mbar_arrive_expect_tx(wfull_bar(slot), static_cast<uint32_t>(p.win_slot_bytes));
            tma_load_4d(win_slots + slot * static_cast<uint32_t>(p.win_slot_bytes), &tm.a0,
                        wfull_bar(slot), 0, wc.tm * 128, h, wc.img);
          }
          ++cnt;
          if (++slot == nslots) {
            slot = 0;
            ++use;
          }
        }
        next_h = lo + p.win_r;
      }
    } else {
      for (int t = t_begin; t < t_end && ok; t += t_step) {
        const TileCoord tc = tile_coord_cta<Cfg>(p, t, cta_rank);
        int pix_w = 0, pix_h = 0, pix_n = 0;
        if constexpr (Cfg::A_IM2COL) {
          const int m0 = tc.tm * 128;
          const int per_img = p.conv_p * p.conv_q;
          pix_n = fast_div(m0, p.fd_per_img);
          const int rem = m0 - pix_n * per_img;
          const int op = fast_div(rem, p.fd_q);
          const int oq = rem - op * p.conv_q;
          pix_w = p.conv_lower_w + oq * p.conv_stride_w;
          pix_h = p.conv_lower_h + op * p.conv_stride_h;
        }
        // second part of A as pixels: the tile's first row is pixel (a2_n, a2_h, a2_w) of that activation
        int a2_w = 0, a2_h = 0, a2_n = 0;
        if constexpr (!Cfg::A_IM2COL && NSPLIT == 1) {
          if (p.a2_pixels) {
            const int m0 = tc.tm * 128;
            a2_n = fast_div(m0, p.a2_fd_per_img);
            const int rem = m0 - a2_n * (p.a2_p * p.a2_q);
            const int op = fast_div(rem, p.a2_fd_q);
            a2_w = (rem - op * p.a2_q) * p.a2_stride;
            a2_h = op * p.a2_stride;
          }
        }
        int tap = 0, cb = 0, fr = 0, fs = 0;   // im2col: k-block = (filter tap, channel block)
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait_warp(empty_bar(stage), phase ^ 1u, abort_flag)) {
            if (leader && *abort_code == 0) *abort_code = 1;
            ok = false;
            break;
          }
          const uint32_t fb = full_bar(stage);
          const uint32_t s_a = ring + stage * Cfg::STAGE;
          const uint32_t s_b = s_a + NSPLIT * Cfg::A_TILE;
          // (test of the time-out path: this stage is never filled, so the issuer's wait for it runs out)
          const bool dropped = p.test_drop_load != 0 && blockIdx.x == 0 && t == t_begin && kb == 0;
          if (leader && !dropped) {
            PMLB_TRACE_EVENT(p, 0, ntrace, t, kb);
            if (CTAS == 1 || cta_rank == 0) mbar_arrive_expect_tx(fb, CTAS * Cfg::STAGE);
            if constexpr (Cfg::A_IM2COL && CTAS == 2) {
              // this CTA's 128 pixels and its half of the tile's output channels
              const uint32_t fb0 = mapa_rank(fb, 0);
              tma_load_im2col_4d_pair(s_a, &tm.a0, fb0, cb * BK, pix_w, pix_h, pix_n,
                                      static_cast<uint16_t>(fs * p.conv_dil_w),
                                      static_cast<uint16_t>(fr * p.conv_dil_h));
              tma_load_3d_pair(s_b, &tm.b0, fb0, cb * BK, tap,
                               tc.n0 + static_cast<int>(cta_rank) * (tc.bn / 2));
            } else if constexpr (Cfg::A_IM2COL) {
              tma_load_im2col_4d(s_a, &tm.a0, fb, cb * BK, pix_w, pix_h, pix_n,
                                 static_cast<uint16_t>(fs * p.conv_dil_w),
                                 static_cast<uint16_t>(fr * p.conv_dil_h));
              // weights laid out [k_out][tap][c_in]: map dims (c_in, tap, k_out)
              tma_load_3d(s_b, &tm.b0, fb, cb * BK, tap, tc.n0);
              if constexpr (NSPLIT == 2) {
                // fp32 as three TF32 products: the low parts of the pixels and of the weights
                tma_load_im2col_4d(s_a + Cfg::A_TILE, &tm.a1, fb, cb * BK, pix_w, pix_h, pix_n,
                                   static_cast<uint16_t>(fs * p.conv_dil_w),
                                   static_cast<uint16_t>(fr * p.conv_dil_h));
                tma_load_3d(s_b + Cfg::B_TILE, &tm.b1, fb, cb * BK, tap, tc.n0);
              }
            } else if constexpr (CTAS == 2) {
              // both CTAs count their bytes on the first CTA's barrier, which expects both
              const uint32_t fb0 = mapa_rank(fb, 0);
              const int n0 = tc.n0 + static_cast<int>(cta_rank) * (tc.bn / 2);
              if constexpr (NSPLIT == 1) {
                // (A may be two tensors side by side along K: k-blocks from a_split_kb on come from the second,
                // a matrix or the pixels of an activation sampled at a stride)
                const bool second = p.a_split_kb > 0 && kb >= p.a_split_kb;
                if (second && p.a2_pixels) {
                  tma_load_im2col_4d_pair(s_a, &tm.a1, fb0, (kb - p.a_split_kb) * BK, a2_w, a2_h, a2_n, 0, 0);
                } else {
                  tma_load_3d_pair(s_a, second ? &tm.a1 : &tm.a0, fb0, (second ? kb - p.a_split_kb : kb) * BK,
                                   tc.tm * 128, tc.b * p.a_bz);
                }
              } else {
                tma_load_3d_pair(s_a, &tm.a0, fb0, kb * BK, tc.tm * 128, tc.b * p.a_bz);
              }
              if constexpr (Cfg::B_MN) {
#pragma unroll
                for (int ch = 0; ch < Cfg::B_CHUNKS; ++ch) {
                  tma_load_3d_pair(s_b + ch * (BK * 128), &tm.b0, fb0, n0 + ch * BK, kb * BK,
                                   tc.b * p.b_bz);
                }
              } else {
                tma_load_3d_pair(s_b, &tm.b0, fb0, kb * BK, n0, tc.b * p.b_bz);
              }
            } else {
              if constexpr (NSPLIT == 1) {
                const bool second = p.a_split_kb > 0 && kb >= p.a_split_kb;
                if (second && p.a2_pixels) {
                  tma_load_im2col_4d(s_a, &tm.a1, fb, (kb - p.a_split_kb) * BK, a2_w, a2_h, a2_n, 0, 0);
                } else {
                  tma_load_3d(s_a, second ? &tm.a1 : &tm.a0, fb, (second ? kb - p.a_split_kb : kb) * BK, tc.tm * 128,
                              tc.b * p.a_bz);
                }
              } else {
                tma_load_3d(s_a, &tm.a0, fb, kb * BK, tc.tm * 128, tc.b * p.a_bz);
              }
              if constexpr (NSPLIT == 2) {
                tma_load_3d(s_a + Cfg::A_TILE, &tm.a1, fb, kb * BK, tc.tm * 128, tc.b * p.a_bz);
              }
              if constexpr (Cfg::B_MN) {
#pragma unroll
                for (int ch = 0; ch < Cfg::B_CHUNKS; ++ch) {
                  tma_load_3d(s_b + ch * (BK * 128), &tm.b0, fb, tc.n0 + ch * BK, kb * BK,
                              tc.b * p.b_bz);
                }
              } else {
                tma_load_3d(s_b, &tm.b0, fb, kb * BK, tc.n0, tc.b * p.b_bz);
                if constexpr (NSPLIT == 2) {
                  tma_load_3d(s_b + Cfg::B_TILE, &tm.b1, fb, kb * BK, tc.n0, tc.b * p.b_bz);
                }
              }
            }
          }
          if constexpr (Cfg::A_IM2COL) {
            if (++cb == p.conv_cblocks) {
              cb = 0;
              ++tap;
              if (++fs == p.conv_s) {
                fs = 0;
                ++fr;
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
  } else if (warp < Cfg::FIRST_EPI_WARP) {
    // ------------------------------------------------------------ MMA issuer(s)
    // With two issuers, issuer iw takes the tiles whose local number is iw modulo 2; local tile
    // number `it` uses accumulator it % NACC in barrier phase (it / NACC) & 1, and the ring
    // stages go to tiles in order, so an issuer also walks the stages of the other's tiles.
    const int iw = warp - 1;
    // Same shape: the warp walks the loops and waits, one elected lane issues the MMAs and
    // the commits (a commit covers the MMAs issued by the thread that executes it).
    const bool leader = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    int ntrace = 0;
    // operand descriptors differ from tile to tile only in the start-address field
    const uint64_t desc_k = make_smem_desc_sw128(0, 16, 1024);           // K-major tile
    const uint64_t desc_mn = make_smem_desc_sw128(0, BK * 128, 1024);    // MN-major B tile
    auto desc_at = [](uint64_t base, uint32_t saddr) {
      return base | static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    };
    // the same split into words: low word = leading-offset field | start address >> 4
    const uint32_t dk_lo = static_cast<uint32_t>(desc_k), dk_hi = static_cast<uint32_t>(desc_k >> 32);
    const uint32_t dmn_lo = static_cast<uint32_t>(desc_mn), dmn_hi = static_cast<uint32_t>(desc_mn >> 32);
    auto lo_at = [](uint32_t base_lo, uint32_t saddr) { return base_lo | ((saddr & 0x3FFFFu) >> 4); };
    if constexpr (Cfg::A_S2D) {
      const uint32_t nst = static_cast<uint32_t>(p.halo_stages);
      uint32_t hs = 0, hphase = 0;
      if (t_begin < t_end && !mbar_wait_warp(wts_bar, 0u, abort_flag)) {
        if (leader && *abort_code == 0) *abort_code = 3;
        ok = false;
      }
      // Every issuer walks all tiles and issues the accumulators a = iw, iw + ISSUERS, ... of each:
      // sub-tile number it = 4 * (tiles so far) + a uses accumulator a.  One MMA (K = 16 elements
      // = one pixel's channels) per tap; the weights are ordinary K-major blocks, tap column ts
      // being k-step ts % 4 of block ts / 4 of its tap row.
      int itile = 0;
      for (int t = t_begin; t < t_end && ok; t += t_step, ++itile) {
        if (!mbar_wait_warp(full_bar(hs), hphase, abort_flag)) {
          if (leader && *abort_code == 0) *abort_code = 3;
          ok = false;
          break;
        }
        const uint32_t buf = halo_ring + hs * static_cast<uint32_t>(p.halo_stage_bytes);
        const uint32_t a_row_step = static_cast<uint32_t>(p.halo_wp) * 2u;
        for (int a = iw; a < 4 && ok; a += Cfg::ISSUERS) {
          acc_phase = static_cast<uint32_t>(itile) & 1u;
          if (leader && iw == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 0);
          if (!mbar_wait_warp(tempty_bar(a), acc_phase ^ 1u, abort_flag)) {
            if (leader && *abort_code == 0) *abort_code = 2;
            ok = false;
            break;
          }
          if (leader && iw == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 1);
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(a * BN);
          // position 4 * i + a reads packed pixel 4 * i + a + tr * wp + ts: descriptor low words
          // (16-byte units) start 2 * a into the buffer and advance by 2 per tap column, wp * 2
          // per tap row
          uint32_t a_row = lo_at(dk_lo, buf) + 2u * static_cast<uint32_t>(a);
          uint32_t b_blk = lo_at(dk_lo, ring);
          uint32_t first = 0u;
          for (int tr = 0; tr < p.conv_r; ++tr) {
            uint32_t a_lo = a_row;
            int ts = 0;
            for (; ts + 4 <= p.conv_s; ts += 4) {
              if (leader) tc_mma_x4<Cfg::KIND, 1>(d_tmem, a_lo, b_blk, dk_hi, dk_hi, p.idesc, first, 2u, 2u);
              first = 1u;
              a_lo += 8u;
              b_blk += 512u;
            }
            if (ts < p.conv_s) {
              uint32_t b_lo = b_blk;
              for (; ts < p.conv_s; ++ts) {
                if (leader) {
                  tc_mma<Cfg::KIND>(d_tmem, (static_cast<uint64_t>(dk_hi) << 32) | a_lo,
                                    (static_cast<uint64_t>(dk_hi) << 32) | b_lo, p.idesc, first);
                }
                first = 1u;
                a_lo += 2u;
                b_lo += 2u;
              }
              b_blk += 512u;
            }
            a_row += a_row_step;
          }
          if (leader) {
            tc_commit(tfull_bar(a));
            if (iw == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 3);
          }
        }
        if (!ok) break;
        if (leader) tc_commit(empty_bar(hs));
        if (++hs == nst) {
          hs = 0;
          hphase ^= 1u;
        }
      }
    } else if constexpr (Cfg::A_HALO) {
      const uint32_t nst = static_cast<uint32_t>(p.halo_stages);
      uint32_t hs = 0, hphase = 0;
      if (t_begin < t_end && !mbar_wait_warp(wts_bar, 0u, abort_flag)) {
        if (leader && *abort_code == 0) *abort_code = 3;
        ok = false;
      }
      // A window that starts a whole number of 128-byte rows into a fetched buffer takes the
      // plain descriptor of its start address: TMA and the tensor core both derive the swizzle
      // phase of a row from its shared-memory address (measured: with the row phase also put
      // into the descriptor's base-offset field the results are wrong).
      auto win_desc = [&](uint32_t saddr) { return desc_at(desc_k, saddr); };
      int hsi = 0;
      int it = 0;
      for (int t = t_begin; t < t_end && ok; t += t_step, ++it) {
        if (it % Cfg::ISSUERS != iw) {
          // The other issuer's tile: walk its buffers too, waiting for each to arrive and reporting
          // it seen (the producer refills a buffer only after both issuers have reported on it).
          for (int cb = 0; cb < p.conv_cblocks && ok; ++cb) {
            if (!mbar_wait_warp(full_bar(static_cast<uint32_t>(hsi)), hphase, abort_flag)) {
              if (leader && *abort_code == 0) *abort_code = 3;
              ok = false;
            } else if (leader) {
              mbar_arrive(empty_bar(static_cast<uint32_t>(hsi)));
            }
            if (++hsi == static_cast<int>(nst)) {
              hsi = 0;
              hphase ^= 1u;
            }
          }
          continue;
        }
        hs = static_cast<uint32_t>(hsi);
        acc = it % Cfg::NACC;
        acc_phase = static_cast<uint32_t>(it / Cfg::NACC) & 1u;
        if (leader && iw == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 0);
        if (!mbar_wait_warp(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
          if (leader && *abort_code == 0) *abort_code = 2;
          break;
        }
        if (leader && iw == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 1);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int cb = 0; cb < p.conv_cblocks && ok; ++cb) {
          if (!mbar_wait_warp(full_bar(hs), hphase, abort_flag)) {
            if (leader && *abort_code == 0) *abort_code = 3;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t buf = halo_ring + hs * static_cast<uint32_t>(p.halo_stage_bytes);
          // output position j reads padded pixel j + fr * wp + fs of the buffer: descriptor low
          // words advance by 8 (one 128-byte row) per filter column, wp * 8 per filter row, and
          // the weights' by one B tile per tap (all in 16-byte units)
          uint32_t a_row = lo_at(dk_lo, buf);
          uint32_t b_lo = lo_at(dk_lo, ring + static_cast<uint32_t>(cb) * Cfg::B_TILE);
          const uint32_t b_step = static_cast<uint32_t>(p.conv_cblocks) * (Cfg::B_TILE >> 4);
          const uint32_t a_row_step = static_cast<uint32_t>(p.halo_wp) * 8u;
          uint32_t first = cb > 0 ? 1u : 0u;
          if (leader && iw == 0 && cb == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 2);
          for (int fr = 0; fr < p.conv_r; ++fr) {
            uint32_t a_lo = a_row;
            for (int fs = 0; fs < p.conv_s; ++fs) {
              if (leader) tc_mma_x4<Cfg::KIND, 1>(d_tmem, a_lo, b_lo, dk_hi, dk_hi, p.idesc, first, 2u, 2u);
              first = 1u;
              a_lo += 8u;
              b_lo += b_step;
            }
            a_row += a_row_step;
          }
          if (leader) tc_commit(empty_bar(hs));
          if (++hs == nst) {
            hs = 0;
            hphase ^= 1u;
          }
        }
        hsi = static_cast<int>(hs);
        if (!ok) break;
        if (leader) {
          tc_commit(tfull_bar(acc));
          if (iw == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 3);
        }
      }
    } else if constexpr (Cfg::A_WINDOW) {
      const uint32_t nslots = static_cast<uint32_t>(p.win_slots);
      // Row h of the current strip has number h + delta; `cnt_end` rows have been numbered
      // so far and the rows below number `waited` are known to have arrived.
      uint32_t cnt_end = 0, waited = 0;
      int cur_strip = -1, delta = 0;
      if (t_begin < t_end && !mbar_wait_warp(wts_bar, 0u, abort_flag)) {
        if (leader && *abort_code == 0) *abort_code = 3;
        ok = false;
      }
      for (int t = t_begin; t < t_end && ok; ++t) {
        if (!mbar_wait_warp(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
          if (leader && *abort_code == 0) *abort_code = 2;
          break;
        }
        const WinCoord wc = win_coord(p, t);
        const int lo = wc.op * p.conv_stride_h + p.conv_lower_h;
        if (wc.strip != cur_strip) {
          cur_strip = wc.strip;
          delta = static_cast<int>(cnt_end) - lo;
        }
        const uint32_t c0 = static_cast<uint32_t>(lo + delta);
        for (uint32_t c = (waited > c0 ? waited : c0); c < c0 + p.win_r && ok; ++c) {
          if (!mbar_wait_warp(wfull_bar(c % nslots), (c / nslots) & 1u, abort_flag)) {
            if (leader && *abort_code == 0) *abort_code = 3;
            ok = false;
          }
        }
        if (!ok) break;
        waited = c0 + p.win_r;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        // Rows the next output row of this CTA does not read go back to the producer.
        const bool slides = (t + 1 < t_end) && ((t + 1) / p.conv_p == wc.strip);
        const int nrel = slides ? p.conv_stride_h : p.win_r;
        uint32_t slot = c0 % nslots;
        for (int r = 0; r < p.win_r; ++r) {
          const uint32_t a_lo = lo_at(dk_lo, win_slots + slot * static_cast<uint32_t>(p.win_slot_bytes));
          const uint32_t b_lo = lo_at(dk_lo, win_wts + r * Cfg::B_TILE);
          if (leader) {
            if (r == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 2);
            tc_mma_x4<Cfg::KIND, 1>(d_tmem, a_lo, b_lo, dk_hi, dk_hi, p.idesc, r > 0 ? 1u : 0u, 2u, 2u);
          }
          if (++slot == nslots) slot = 0;
        }
        if (leader) {
          uint32_t rs = c0 % nslots;
          for (int r = 0; r < nrel; ++r) {
            tc_commit(wempty_bar(rs));
            if (++rs == nslots) rs = 0;
          }
          tc_commit(tfull_bar(acc));
          PMLB_TRACE_EVENT(p, 1, ntrace, t, 3);
        }
        cnt_end = c0 + p.win_r;
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    } else if (CTAS == 1 || cta_rank == 0) {
      int it = 0;
      for (int t = t_begin; t < t_end && ok; t += t_step, ++it) {
        if (it % Cfg::ISSUERS != iw) {
          // the other issuer's tile: walk its stages too, waiting for each to arrive and saying so
          for (int kb = 0; kb < p.num_kb && ok; ++kb) {
            if (!mbar_wait_warp(full_bar(stage), phase, abort_flag)) {
              if (leader && *abort_code == 0) *abort_code = 3;
              ok = false;
            } else if (leader) {
              mbar_arrive(empty_bar(stage));
            }
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
          continue;
        }
        acc = it % Cfg::NACC;
        acc_phase = static_cast<uint32_t>(it / Cfg::NACC) & 1u;
        if (leader && iw == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 0);
        if (!mbar_wait_warp(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
          if (leader && *abort_code == 0) *abort_code = 2;
          break;
        }
        if (leader && iw == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 1);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        const uint32_t idesc = t >= p.tiles_full ? p.idesc_half : p.idesc;   // half-width tail tiles
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait_warp(full_bar(stage), phase, abort_flag)) {
            if (leader && *abort_code == 0) *abort_code = 3;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t s_a = ring + stage * Cfg::STAGE;
          const uint32_t s_b = s_a + NSPLIT * Cfg::A_TILE;
          const uint64_t a_hi = desc_at(desc_k, s_a);
          const uint64_t b_hi = desc_at(Cfg::B_MN ? desc_mn : desc_k, s_b);
          // descriptor step per 32 bytes of K: 32 bytes along a K-major row, UMMA_K rows of
          // 128 bytes in an MN-major tile (address field counts 16-byte units)
          constexpr uint32_t kStepA = 2u;
          constexpr uint32_t kStepB = Cfg::B_MN ? (Cfg::UMMA_K * 128u) >> 4 : 2u;
          if (leader) {
            if (kb == 0 && iw == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 2);
            if constexpr (NSPLIT == 2) {
              // fp32 as three TF32 products; the two cross terms first.
              const uint64_t a_lo = desc_at(desc_k, s_a + Cfg::A_TILE);
              const uint64_t b_lo = desc_at(desc_k, s_b + Cfg::B_TILE);
              tc_mma<Cfg::KIND>(d_tmem, a_lo, b_hi, idesc, kb > 0 ? 1u : 0u);
              tc_mma<Cfg::KIND>(d_tmem, a_hi, b_lo, idesc, 1u);
              tc_mma<Cfg::KIND>(d_tmem, a_hi, b_hi, idesc, 1u);
#pragma unroll
              for (int j = 1; j < 4; ++j) {
                tc_mma<Cfg::KIND>(d_tmem, a_lo + kStepA * j, b_hi + kStepB * j, idesc, 1u);
                tc_mma<Cfg::KIND>(d_tmem, a_hi + kStepA * j, b_lo + kStepB * j, idesc, 1u);
                tc_mma<Cfg::KIND>(d_tmem, a_hi + kStepA * j, b_hi + kStepB * j, idesc, 1u);
              }
            } else {
              tc_mma_x4<Cfg::KIND, CTAS>(d_tmem, lo_at(dk_lo, s_a), lo_at(Cfg::B_MN ? dmn_lo : dk_lo, s_b), dk_hi,
                                         Cfg::B_MN ? dmn_hi : dk_hi, idesc, kb > 0 ? 1u : 0u, kStepA, kStepB);
            }
            if constexpr (CTAS == 2) {
              tc_commit_pair(empty_bar(stage), 3);   // the stage is free in both CTAs
            } else {
              tc_commit(empty_bar(stage));
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (leader) {
          if constexpr (CTAS == 2) {
            tc_commit_pair(tfull_bar(acc), 3);       // both CTAs' epilogues may read their half
          } else {
            tc_commit(tfull_bar(acc));
          }
          if (iw == 0) PMLB_TRACE_EVENT(p, 1, ntrace, t, 3);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;                     // TMEM lane quarter this warp may read
    const int ew = warp - Cfg::FIRST_EPI_WARP;  // epilogue warp number
    const int grp = ew >> 2;                    // epilogue group (accumulator owner when two)
    constexpr int G = Cfg::EPI_GROUPS;
    // Local tile number `it` selects the accumulator (it % NACC) and its barrier phase
    // ((it / NACC) & 1); with two groups, group g takes the tiles with (it & 1) == g.
    if (p.fast_epi) {
      constexpr int CW = Cfg::CW;
      constexpr int OB = Cfg::OUT_BYTES;
      const uint32_t stage_buf = smem_u32(stg_all) + static_cast<uint32_t>(ew) * 8192u;
      uint32_t nbuf = 0;
      // Residual rows fetched by TMA land in the staging buffer their chunk is later stored
      // from: chunk number k of this warp (counted over all tiles) uses buffer k & 1 and
      // arrival barrier k & 1 in phase (k >> 1) & 1.  `nreq` counts the chunks requested.
      const bool res_tma = p.res_tma != 0;
      uint32_t nreq = 0;
      // The requests run ahead of the processing across tile boundaries: a cursor walks this
      // group's tiles and their chunks in processing order, and before a chunk is processed the
      // one after it (the next tile's first chunk after a tile's last) is requested, so that
      // every chunk's rows have about one chunk's processing time to arrive.
      int rq_t = t_begin + (G == 2 ? grp : 0) * t_step, rq_ch = 0;
      bool rq_valid = res_tma && rq_t < t_end;
      TileCoord rq_tc;
      if (rq_valid) rq_tc = tile_coord_cta<Cfg>(p, rq_t, cta_rank);
      auto request_ahead = [&](uint32_t upto) {       // until `upto` chunks have been requested
        while (nreq < upto && rq_valid) {
          const int c0 = rq_tc.n0 + rq_ch * CW;
          if (c0 < p.n) {                            // warp-uniform
            if (lane == 0) {
              const uint32_t b = nreq & 1u;
              mbar_arrive_expect_tx(res_bar(ew, b), 4096u);
              tma_load_3d(stage_buf + b * 4096u, &tm.r, res_bar(ew, b), c0, rq_tc.tm * 128 + q * 32, rq_tc.b);
            }
            ++nreq;
          }
          if (++rq_ch >= rq_tc.bn / CW || c0 + CW >= p.n) {
            rq_ch = 0;
            rq_t += G * t_step;
            rq_valid = rq_t < t_end;
            if (rq_valid) rq_tc = tile_coord_cta<Cfg>(p, rq_t, cta_rank);
          }
        }
      };
      bool alive = true;
      const bool out_bf16 = p.out_dtype == kDtBF16;
      const bool relu_in_cvt = OB == 2 && !IS_INT && (p.epi_flags & kEpiRelu) && !(p.epi_flags & kEpiRowMax);
      int it = 0;
      int ntrace = 0;
      const bool tracer = (ew & 3) == 0 && lane == 0;   // first warp of each group
      // (space-to-depth tiles have four accumulators each: `it` then counts those)
      constexpr int SUBS = Cfg::A_S2D ? 4 : 1;
      for (;; ++it) {
        const int t = t_begin + (it / SUBS) * t_step;
        if (t >= t_end || !alive) break;
        if (G == 2 && (it & 1) != grp) continue;
        const int acc = it % Cfg::NACC;
        const uint32_t acc_phase = static_cast<uint32_t>(it / Cfg::NACC) & 1u;
        TileCoord tc;
        if constexpr (Cfg::A_S2D || Cfg::A_HALO) {
          tc.b = t;
          tc.tm = tc.tn = tc.n0 = 0;
          tc.bn = BN;
        } else {
          tc = tile_coord_cta<Cfg>(p, t, cta_rank);
        }
        int row0 = tc.tm * 128 + q * 32;
        int row = row0 + lane;
        // space-to-depth: image row / column of this warp's first position, first output row of the image
        int s2d_op0 = 0, s2d_oq0 = 0, s2d_row0 = 0;
        if constexpr (Cfg::A_S2D) {
          row0 = 0;   // (no per-row epilogue inputs in this mode; the store maps rows itself)
          row = 0;
          const int img = fast_div(t, p.fd_tiles_per_img);
          const int g0 = (t - img * p.halo_tiles_per_img) * 512 + q * 128;
          s2d_op0 = fast_div(g0, p.fd_wp);
          s2d_oq0 = g0 - s2d_op0 * p.halo_wp;
          s2d_row0 = img * p.conv_p;
        }
        if constexpr (Cfg::A_HALO) {
          // accumulator row j = output position j of the tile: image row j / wp, column j % wp;
          // columns past q (the padding columns) and rows past the image are not outputs
          const int img = fast_div(t, p.fd_tiles_per_img);
          const int p0 = (t - img * p.halo_tiles_per_img) * p.halo_th;
          const int j = q * 32 + lane;
          const int pr = fast_div(j, p.fd_wp);
          const int qq = j - pr * p.halo_wp;
          const bool valid = pr < p.halo_th && qq < p.conv_q && p0 + pr < p.conv_p;
          row0 = 0;
          row = valid ? (img * p.conv_p + p0 + pr) * p.conv_q + qq : p.m;
        }
        const int col_base = tc.n0;
        const int nch = tc.bn / CW;                 // chunks of this tile
        if (res_tma && nreq < nbuf + 2 && rq_valid) {
          // Both buffers are free once the stores of the previous tile have read them; the
          // first two chunks' residual rows then arrive while the main loop still runs (in
          // the steady state the first was requested during the previous tile's last chunk).
          if (lane == 0) bulk_wait_group_read<0>();
          request_ahead(nbuf + 2);
        }
        if (tracer) PMLB_TRACE_EVENT(p, 2 + grp, ntrace, t, 0);
        if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
          if (*abort_code == 0) *abort_code = 4;
          break;
        }
        if (tracer) PMLB_TRACE_EVENT(p, 2 + grp, ntrace, t, 1);
        tc_fence_after_sync();
        const uint32_t t_acc =
            tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(q * 32) << 16);
        const long long res_row =
            static_cast<long long>(tc.b) * p.res_batch + static_cast<long long>(row) * p.ldr;
        float row_best = -INFINITY;

        auto issue_load = [&](uint32_t(&v)[CW], int ch) {
          uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&v[0]);
          tmem_ld_32x32(t_acc + ch * CW, lo);
          if constexpr (CW == 64) {
            uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&v[32]);
            tmem_ld_32x32(t_acc + ch * CW + 32, hi);
          }
        };
        // Pins the registers of a finished TMEM load behind the wait: the empty volatile asm
        // statements cannot be moved above `tcgen05.wait::ld`, so neither can their users.
        auto pin = [&](uint32_t(&v)[CW]) {
#pragma unroll
          for (int j = 0; j < CW; ++j) asm volatile("" : "+r"(v[j]));
        };
        auto release_acc = [&]() {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (CTAS == 2) {
              mbar_arrive_cluster(mapa_rank(tempty_bar(acc), 0));
            } else {
              mbar_arrive(tempty_bar(acc));
            }
          }
        };
        auto process = [&](uint32_t(&v)[CW], int ch) {
          const int col0 = col_base + ch * CW;
          if (col0 >= p.n || !alive) return;          // warp-uniform
          uint32_t res_smem = 0;
          if (res_tma) {
            // The chunk after this one takes the buffer the chunk before this one was stored from.
            if (nreq < nbuf + 2 && rq_valid) {
              if (lane == 0) bulk_wait_group_read<0>();
              request_ahead(nbuf + 2);
            }
            if (!mbar_wait(res_bar(ew, nbuf & 1u), (nbuf >> 1) & 1u, abort_flag)) {
              if (*abort_code == 0) *abort_code = 5;
              alive = false;
              return;
            }
            res_smem = stage_buf + (nbuf & 1u) * 4096u;
          }
          const float chunk_best =
              (col0 + CW <= p.n)
                  ? epi_apply<true, IS_INT, OB, CW>(p, v, col0, row, res_row, out_bf16, res_smem, lane, relu_in_cvt)
                  : epi_apply<false, IS_INT, OB, CW>(p, v, col0, row, res_row, out_bf16, res_smem, lane, relu_in_cvt);
          if (p.epi_flags & kEpiRowMax) row_best = fmaxf(row_best, chunk_best);
          if (tracer) PMLB_TRACE_EVENT(p, 2 + grp, ntrace, t, 40);
          // (with TMA-fetched residuals every chunk is stored, rows past M being clipped by
          // the store, so that buffers and barriers stay in step with the requests)
          if (!res_tma && (p.out == nullptr || row0 >= p.m)) return;   // warp-uniform

          uint4 o[8];
          if constexpr (OB == 4) {
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          } else {
#pragma unroll
            auto pack_all = [&](auto bf16, auto relu) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                uint32_t w[4];
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                  w[h] = cvt_pack16<decltype(bf16)::value, decltype(relu)::value>(
                      __uint_as_float(v[8 * i + 2 * h]), __uint_as_float(v[8 * i + 2 * h + 1]));
                }
                o[i] = make_uint4(w[0], w[1], w[2], w[3]);
              }
            };
            using T = std::true_type;
            using F = std::false_type;
            if (out_bf16) {
              if (relu_in_cvt) pack_all(T{}, T{}); else pack_all(T{}, F{});
            } else {
              if (relu_in_cvt) pack_all(F{}, T{}); else pack_all(F{}, F{});
            }
          }
          if constexpr (Cfg::A_HALO) {
            // output pixels of a tile are not a box of the output tensor: each lane writes its
            // own pixel's 128 bytes
            // (32-byte stores: whole sectors; output rows of this mode are 128 or 256 bytes on a
            // 16-byte aligned base, so the 32-byte form needs the base checked once)
            if (row < p.m) {
              char* dst = static_cast<char*>(p.out) + (static_cast<long long>(row) * p.ldc + col0) * OB;
              if ((reinterpret_cast<uintptr_t>(dst) & 31u) == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) st_global_v8(dst + 32 * i, o[2 * i], o[2 * i + 1]);
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) reinterpret_cast<uint4*>(dst)[i] = o[i];
              }
            }
            return;
          }
          // the buffer used two chunks ago must have been read by its TMA store (already
          // true when its residual rows were requested)
          if (tracer) PMLB_TRACE_EVENT(p, 2 + grp, ntrace, t, 41);
          if (!res_tma && lane == 0) bulk_wait_group_read<1>();
          __syncwarp();
          if (tracer) PMLB_TRACE_EVENT(p, 2 + grp, ntrace, t, 42);
          const uint32_t buf = stage_buf + (nbuf & 1u) * 4096u;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            st_shared_v4(buf + lane * 128 + ((i ^ (lane & 7)) << 4), o[i]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (tracer) PMLB_TRACE_EVENT(p, 2 + grp, ntrace, t, 43);
          if (lane == 0) {
            if constexpr (Cfg::A_S2D) {
              // Row i of accumulator a is position 512 * tile + 4 * i + a of the image's padded
              // position grid (wp a multiple of 32 per image row).  The output map is
              // (channels, 4, q / 4, n * p) with output column 4 * c2 + c1 at (c1, c2): every
              // run of p.s2d_box_rows of the warp's rows (32 when an image row holds the whole
              // warp) is one box at c1 = a, c2 = column / 4 of one image row; boxes in the
              // padding columns or below the image are skipped, the map clips the rest.
              const int a = it & 3;
              int op = s2d_op0, oq = s2d_oq0;
              const int box = p.s2d_box_rows;
              for (int r = 0; r < 32; r += box) {
                if (op < p.conv_p && oq < p.conv_q) {
                  tma_store_4d(&tm.c, buf + static_cast<uint32_t>(r) * 128u, col0, a, oq >> 2, s2d_row0 + op);
                }
                oq += 4 * box;
                if (oq >= p.halo_wp) {
                  oq -= p.halo_wp;
                  ++op;
                }
              }
            } else {
              tma_store_3d(&tm.c, buf, col0, row0, tc.b);
            }
            bulk_commit_group();
          }
          ++nbuf;
        };
        // Two register sets: the TMEM load of chunk ch + 1 is in flight while chunk ch is
        // converted, staged and stored.
        if constexpr (G == 1) {
          uint32_t va[CW], vb[CW];
          issue_load(va, 0);
#pragma unroll 1
          for (int ch = 0; ch < nch; ch += 2) {
            tmem_ld_wait();
            pin(va);
            if (ch + 1 < nch) issue_load(vb, ch + 1);
            if (ch == nch - 1) release_acc();
            process(va, ch);
            if (ch + 1 < nch) {
              tmem_ld_wait();
              pin(vb);
              if (ch + 2 < nch) issue_load(va, ch + 2);
              if (ch + 1 == nch - 1) release_acc();
              process(vb, ch + 1);
            }
          }
        } else if (p.out == nullptr && p.epi_flags == kEpiRowMax && !IS_INT) {
          // Row maxima only (nothing stored, no other epilogue term): a lean loop, since this
          // launch is nothing but its epilogue.  Each chunk is reduced by a balanced tree of
          // hardware max operations, as in the general path.
          uint32_t va[CW];
          const int span = p.n - col_base;                         // valid columns from the tile's first on
          const int chunks = span >= nch * CW ? nch : (span + CW - 1) / CW;
#pragma unroll 1
          for (int ch = 0; ch < chunks; ++ch) {
            issue_load(va, ch);
            tmem_ld_wait();
            pin(va);
            if (ch == chunks - 1) release_acc();
            const int nvalid = span - ch * CW;                     // >= 1
            float mx[CW];
            if (nvalid >= CW) {
#pragma unroll
              for (int j = 0; j < CW; ++j) mx[j] = __uint_as_float(va[j]);
            } else {
#pragma unroll
              for (int j = 0; j < CW; ++j) mx[j] = j < nvalid ? __uint_as_float(va[j]) : -INFINITY;
            }
#pragma unroll
            for (int w = CW / 2; w > 0; w >>= 1) {
#pragma unroll
              for (int j = 0; j < w; ++j) mx[j] = fmaxf(mx[j], mx[j + w]);
            }
            row_best = fmaxf(row_best, mx[0]);
          }
        } else {
          // two warps per scheduler hide each other's latencies; one register set suffices
          uint32_t va[CW];
#pragma unroll 1
          for (int ch = 0; ch < nch; ++ch) {
            issue_load(va, ch);
            tmem_ld_wait();
            pin(va);
            if (tracer) PMLB_TRACE_EVENT(p, 2 + grp, ntrace, t, 10 + ch);
            if (ch == nch - 1) release_acc();
            process(va, ch);
            if (tracer) PMLB_TRACE_EVENT(p, 2 + grp, ntrace, t, 30 + ch);
          }
        }
        if (p.epi_flags & kEpiRowMax) {
          if (row < p.m) {
            atomic_max_float(p.rowmax + static_cast<long long>(tc.b) * p.m + row, row_best);
          }
        }
      }
      // staged rows must be read out (and the writes done) before shared memory goes away
      if (lane == 0) bulk_wait_group<0>();
      __syncwarp();
    } else {
      float* stg = stg_all + ew * 2048;          // this warp's 8 KB, used as a 32 x 33 pad
      int it = 0;
      for (int t = t_begin; t < t_end; t += t_step, ++it) {
        if (G == 2 && (it & 1) != grp) continue;
        const int acc = it % Cfg::NACC;
        const uint32_t acc_phase = static_cast<uint32_t>(it / Cfg::NACC) & 1u;
        const TileCoord tc = tile_coord_cta<Cfg>(p, t, cta_rank);
        if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
          if (*abort_code == 0) *abort_code = 4;
          break;
        }
        tc_fence_after_sync();
        const int row0 = tc.tm * 128 + q * 32;     // first row of this warp
        const int col_base = tc.n0;
        const int nch32 = tc.bn / 32;
        const uint32_t t_acc =
            tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(q * 32) << 16);
        const long long out_b = static_cast<long long>(tc.b) * p.out_batch;
        const long long res_b = static_cast<long long>(tc.b) * p.res_batch;
        float row_best = -INFINITY;

#pragma unroll 1
        for (int ch = 0; ch < nch32; ++ch) {
          const int col0 = col_base + ch * 32;
          uint32_t v[32];
          tmem_ld_32x32(t_acc + ch * 32, v);
          tmem_ld_wait();
          if (ch == nch32 - 1) {
            // accumulator fully read: hand it back before finishing the stores
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
            if constexpr (CTAS == 2) {
              mbar_arrive_cluster(mapa_rank(tempty_bar(acc), 0));
            } else {
              mbar_arrive(tempty_bar(acc));
            }
          }
          }
          if (col0 >= p.n) continue;   // warp-uniform
          if ((p.epi_flags & kEpiRowMax) && p.out == nullptr) {
            if constexpr (!IS_INT) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float x = __uint_as_float(v[j]);
                if (col0 + j < p.n && x > row_best) row_best = x;
              }
            }
            continue;
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
          if (p.epi_flags & kEpiRowMax) {
            // row max of what was stored: reread this warp's rows of the chunk
            if constexpr (!IS_INT) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float x = __uint_as_float(v[j]);
                if (col0 + j < p.n && x > row_best) row_best = x;
              }
            }
          }
        }
        if (p.epi_flags & kEpiRowMax) {
          const int row = row0 + lane;
          if (row < p.m) {
            atomic_max_float(p.rowmax + static_cast<long long>(tc.b) * p.m + row, row_best);
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  if constexpr (CTAS == 2) {
    cluster_sync_all();   // neither CTA's shared memory or barriers are touched by the other from here on
  } else {
    __syncthreads();
  }
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
  if constexpr (CTAS == 2) cluster_sync_all();   // (a CTA that reported a time-out has waited above)
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    if constexpr (CTAS == 2) {
      tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    } else {
      tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
  }
}

template <class Cfg>
cudaError_t launch_cfg(const TcMaps& maps, const TcParams& p, int grid, cudaStream_t stream) {
  // The attribute is per device, so it is set on every call (a cheap host-side update).
  const cudaError_t attr_err = cudaFuncSetAttribute(
      tc_contract_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  if (attr_err != cudaSuccess) return attr_err;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if constexpr (Cfg::CTAS == 2) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 2;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (dependent_launch_enabled()) {
    // the kernel's set-up may overlap the tail of the kernel before it (see grid_dependency_wait)
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, tc_contract_kernel<Cfg>, maps, p);
}

// Clusters of two that the device can keep resident at once (0 if the query fails).
template <class Cfg>
int max_resident_pairs() {
  if (cudaFuncSetAttribute(tc_contract_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           Cfg::SMEM_BYTES) != cudaSuccess) {
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, tc_contract_kernel<Cfg>, &cfg) != cudaSuccess) return 0;
  return n;
}

}  // namespace pmlb
