// First layer of an image network and the max pool behind it, as one kernel: a stride-2 convolution with a
// 7-wide filter on at most 4 channels into 64 (space-to-depth form: a stride-1 convolution with 4 x 4 taps
// over 32-byte pixels of 2 x 2 x c values), bias, ReLU, and a 3 x 3 / 2 max pool with one pixel of padding.
// The convolution's output (four times the pooled tensor) never reaches memory.
//
// Tiles.  A tile is 512 consecutive positions of the packed activation's position grid, whose rows are
// exactly 128 positions wide here: four rows of the convolution's output.  Position 4 i + a of the tile is
// row i of accumulator a (four pixels share a 128-byte operand row), so warp q of an epilogue group sees
// output row 4 T + q of the image, its lane l the columns 4 l .. 4 l + 3 in the four accumulators.
//
// MMAs.  Accumulator a's operand for tap (tr, ts) is the pixel buffer read from byte 32 (a + ts + tr * 128)
// on: the seven windows w = a + ts of a tap row serve up to four (accumulator, tap column) pairs each.  With
// the accumulators side by side in TMEM (64 columns each) and the weights stored as
// [tap column, descending][output channel][tap row][16 values], window w times the weight rows of its pairs
// is ONE MMA of N = 64, 128, 192 or 256 columns: 28 MMAs per tile instead of 64, 240 KB of shared-memory
// operand reads instead of 384 KB (the 128 B/clk port, not the tensor pipe, bounds the one-MMA-per-tap form).
// The first MMA of a tile is the full-width window of tap row 0, which initialises all four accumulators.
//
// Pooling.  Each thread reduces its row's columns in registers (one warp shuffle per channel for column
// 4 l - 1), adds the bias, applies ReLU in the conversion to 16 bits (all monotonic, so the maximum may be
// taken first), and holds two pooled columns of 64 channels.  Rows: pooled row 2 T = max of output rows
// 4 T - 1, 4 T, 4 T + 1 and pooled row 2 T + 1 = max of rows 4 T + 1 .. 4 T + 3.  Warps 1 and 3 publish their
// rows in shared memory (swizzled 16-byte units), warps 0 and 2 combine and store 32 bytes per lane and
// chunk.  Row 4 T - 1 is the previous tile's last row: a CTA therefore walks a contiguous run of tiles and
// keeps three tiles' published rows; where its run starts inside an image it first computes the tile before
// the run without storing anything (one tile in ~49).
//
// Roles: warp 0 producer (weights once, one bulk copy per tile), warp 1 MMA issuer (tile with local number it
// into accumulator set it mod 2; a second issuer taking every other tile was measured slower: 137 against
// 121 us for the layer pair at 256 images), warps 2..9 two epilogue groups of four warps (group g = set g).
// Every wait is bounded, as in the general kernel.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"
#include "s2d_pool.h"

namespace pmlb {

constexpr int kSpThreads = 64 + 256;
constexpr int kSpMaxStages = 6;
constexpr int kSpWeightBytes = 4 * 64 * 128;          // [4 tap columns][64 channels] rows of 128 bytes
constexpr int kSpRowBytes = 64 * 128;                 // one published row: 64 pooled columns x 64 channels x 2 bytes
constexpr int kSpHbufBytes = 3 * 2 * kSpRowBytes;     // three tiles x (row 1, row 3)
constexpr int kSpTailBytes = 256 + 512;               // bias, barriers
constexpr int kSpSmemLimit = 232448;

__device__ __forceinline__ void sp_tmem_ld_x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// elementwise maximum of two packed 16-bit pairs (a NaN operand loses)
template <bool BF16>
__device__ __forceinline__ uint32_t sp_max2(uint32_t a, uint32_t b) {
  uint32_t d;
  if constexpr (BF16) {
    asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  } else {
    asm("max.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  }
  return d;
}

template <bool BF16>
__device__ __forceinline__ uint4 sp_max2x4(const uint4& a, const uint4& b) {
  return make_uint4(sp_max2<BF16>(a.x, b.x), sp_max2<BF16>(a.y, b.y), sp_max2<BF16>(a.z, b.z), sp_max2<BF16>(a.w, b.w));
}

template <bool BF16>
__global__ void __launch_bounds__(kSpThreads, 1)
conv_s2d_pool_kernel(const __grid_constant__ S2dPoolParams p) {
  grid_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t ring = (raw_addr + 1023u) & ~1023u;
  uint8_t* ring_ptr = smem_raw + (ring - raw_addr);
  const int nst = p.stages;
  const uint32_t hbuf0 = ring + kSpWeightBytes;
  const uint32_t stages0 = hbuf0 + kSpHbufBytes;
  const uint32_t tail_off = kSpWeightBytes + kSpHbufBytes + static_cast<uint32_t>(nst) * static_cast<uint32_t>(p.stage_bytes);
  float* bias_s = reinterpret_cast<float*>(ring_ptr + tail_off);
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring_ptr + tail_off + 256);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](uint32_t s) { return bar0 + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar0 + 8u * (kSpMaxStages + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kSpMaxStages + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kSpMaxStages + 2 + a); };
  const uint32_t wts_bar = bar0 + 8u * (2 * kSpMaxStages + 4);
  // published rows of tile it live in buffer it % 3: written (2 warps) / read (3 warps: 0 and 2 of the tile,
  // warp 0 of the next tile)
  auto hready_bar = [&](int b) { return bar0 + 8u * (2 * kSpMaxStages + 5 + b); };
  auto hfree_bar = [&](int b) { return bar0 + 8u * (2 * kSpMaxStages + 8 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kSpMaxStages + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* abort_code = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSpMaxStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    for (int b = 0; b < 3; ++b) {
      mbar_init(hready_bar(b), 2);
      mbar_init(hfree_bar(b), 3);
    }
    mbar_init(wts_bar, 1);
    *abort_flag = 0;
    *abort_code = 0;
    abort_flag[2] = p.wait_limit_us;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();
  if (warp >= 2 && warp < 4) {
    const int ch = (warp - 2) * 32 + lane;
    bias_s[ch] = p.bias != nullptr ? __ldg(p.bias + ch) : 0.f;
  }
  __syncthreads();

  // This CTA's run of tiles: [lo, hi) of the image-major tile list, preceded by the tile before it when the
  // run starts inside an image (computed for its last row only).
  const long long total = p.total_tiles;
  const int lo = static_cast<int>(total * blockIdx.x / gridDim.x);
  const int hi = static_cast<int>(total * (blockIdx.x + 1) / gridDim.x);
  const bool lead_in = hi > lo && lo % p.tiles_per_img != 0;
  const int first = lo - (lead_in ? 1 : 0);
  const int count = hi - first;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    const bool leader = elect_one();
    if (leader && count > 0) {
      mbar_arrive_expect_tx(wts_bar, kSpWeightBytes);
      bulk_load_1d(ring, p.wts, kSpWeightBytes, wts_bar);
    }
    uint32_t hs = 0, hphase = 0;
    for (int it = 0; it < count; ++it) {
      const int t = first + it;
      const int img = t / p.tiles_per_img;
      const int tt = t - img * p.tiles_per_img;
      if (!mbar_wait_warp(empty_bar(hs), hphase ^ 1u, abort_flag)) {
        if (leader && *abort_code == 0) *abort_code = 1;
        break;
      }
      if (leader) {
        const char* src = static_cast<const char*>(p.px) + (static_cast<long long>(img) * p.img_px + tt * 512) * 32;
        mbar_arrive_expect_tx(full_bar(hs), static_cast<uint32_t>(p.stage_load));
        bulk_load_1d(stages0 + hs * static_cast<uint32_t>(p.stage_bytes), src, static_cast<uint32_t>(p.stage_load),
                     full_bar(hs));
      }
      if (++hs == static_cast<uint32_t>(nst)) {
        hs = 0;
        hphase ^= 1u;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    const bool leader = elect_one();
    const uint64_t desc_k = make_smem_desc_sw128(0, 16, 1024);
    const uint32_t dk_lo = static_cast<uint32_t>(desc_k);
    const uint64_t dk_hi = static_cast<uint64_t>(static_cast<uint32_t>(desc_k >> 32)) << 32;
    auto lo_at = [](uint32_t base_lo, uint32_t saddr) { return base_lo | ((saddr & 0x3FFFFu) >> 4); };
    bool ok = true;
    if (count > 0 && !mbar_wait_warp(wts_bar, 0u, abort_flag)) {
      if (leader && *abort_code == 0) *abort_code = 3;
      ok = false;
    }
    const uint32_t b_base = lo_at(dk_lo, ring);
    uint32_t hs = 0, hphase = 0;
    for (int it = 0; it < count && ok; ++it) {
      const int set = it & 1;
      const uint32_t d_set = tmem_base + static_cast<uint32_t>(set * 256);
      const uint32_t acc_phase = static_cast<uint32_t>(it >> 1) & 1u;
      if (!mbar_test_wait_warp(tempty_bar(set), acc_phase ^ 1u) && !mbar_wait_warp(tempty_bar(set), acc_phase ^ 1u, abort_flag)) {
        if (leader && *abort_code == 0) *abort_code = 2;
        break;
      }
      if (!mbar_test_wait_warp(full_bar(hs), hphase) && !mbar_wait_warp(full_bar(hs), hphase, abort_flag)) {
        if (leader && *abort_code == 0) *abort_code = 3;
        break;
      }
      tc_fence_after_sync();
      if (leader) {
        // window w of tap row tr: pixels from byte 32 (w + 128 tr) of the buffer on; its pairs are the
        // accumulators a = max(0, w - 3) .. min(3, w) with tap column w - a, i.e. weight blocks
        // 3 - w + a (64 rows of 128 bytes each) from the first on, tap row tr being the row's k-step tr
        uint32_t a_row = lo_at(dk_lo, stages0 + hs * static_cast<uint32_t>(p.stage_bytes));
        for (int tr = 0; tr < p.r2; ++tr) {
          const uint32_t b_row = b_base + 2u * static_cast<uint32_t>(tr);
          // the full-width window first: on tap row 0 it overwrites all four accumulators
          tc_mma<kMmaF16>(d_set, dk_hi | (a_row + 6u), dk_hi | b_row, p.idesc[3], tr > 0 ? 1u : 0u);
#pragma unroll
          for (int w = 0; w < 3; ++w) {
            // accumulators 0 .. w, weight blocks 3 - w ..
            tc_mma<kMmaF16>(d_set, dk_hi | (a_row + 2u * w), dk_hi | (b_row + static_cast<uint32_t>(3 - w) * 512u),
                            p.idesc[w], 1u);
          }
#pragma unroll
          for (int w = 4; w < 7; ++w) {
            // accumulators w - 3 .. 3, weight blocks 0 ..
            tc_mma<kMmaF16>(d_set + static_cast<uint32_t>(w - 3) * 64u, dk_hi | (a_row + 2u * w), dk_hi | b_row,
                            p.idesc[6 - w], 1u);
          }
          a_row += 256u;   // one 128-position row of 32-byte pixels, in 16-byte units
        }
        tc_commit(empty_bar(hs));
        tc_commit(tfull_bar(set));
      }
      __syncwarp();
      if (++hs == static_cast<uint32_t>(nst)) {
        hs = 0;
        hphase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;             // TMEM lane quarter = output row of the tile
    const int grp = (warp - 2) >> 2;    // group g takes the tiles with local number = g mod 2 (accumulator set g)
    const bool relu = p.relu != 0;
    const bool lane_valid = 4 * lane < p.conv_q;
    const uint32_t t_acc = tmem_base + static_cast<uint32_t>(grp * 256) + (static_cast<uint32_t>(q * 32) << 16);
    // this lane's two pooled columns in a published row: unit u (16 bytes) of column col at
    // col * 128 + ((u ^ (lane & 7)) << 4): lanes 0..7 of a store hit eight different bank groups
    const uint32_t lane_off = static_cast<uint32_t>(lane) * 256u;
    const uint32_t key = static_cast<uint32_t>(lane & 7);
    for (int it = grp; it < count; it += 2) {
      const int t = first + it;
      const int img = t / p.tiles_per_img;
      const int tt = t - img * p.tiles_per_img;
      const bool store = !(lead_in && it == 0);
      const uint32_t acc_phase = static_cast<uint32_t>(it >> 1) & 1u;
      const int hb = it % 3;
      const uint32_t hphase = static_cast<uint32_t>(it / 3) & 1u;
      if (!mbar_wait_warp(tfull_bar(grp), acc_phase, abort_flag)) {
        if (lane == 0 && *abort_code == 0) *abort_code = 4;
        break;
      }
      tc_fence_after_sync();
      // 64 channels x two pooled columns of this thread's output row, packed to 16 bits:
      // h[c][0..7] = column 2 l, h[c][8..15] = column 2 l + 1 (16 channels of chunk c each)
      uint32_t h[4][16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v0[16], v1[16], v2[16], v3[16];
        sp_tmem_ld_x16(t_acc + c * 16, v0);
        sp_tmem_ld_x16(t_acc + 64 + c * 16, v1);
        sp_tmem_ld_x16(t_acc + 128 + c * 16, v2);
        sp_tmem_ld_x16(t_acc + 192 + c * 16, v3);
        float bs[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 bb = reinterpret_cast<const float4*>(bias_s + c * 16)[i];
          bs[4 * i] = bb.x, bs[4 * i + 1] = bb.y, bs[4 * i + 2] = bb.z, bs[4 * i + 3] = bb.w;
        }
        tmem_ld_wait();
        if (c == 3) {
          // accumulators fully read: hand the set back to its issuer
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(grp));
        }
        float m0[16], m1[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float x0 = __uint_as_float(v0[i]), x1 = __uint_as_float(v1[i]);
          const float x2 = __uint_as_float(v2[i]), x3 = __uint_as_float(v3[i]);
          // column 4 l - 1 is the previous lane's last column; the image's first column has no such neighbour
          float up = __shfl_up_sync(0xffffffffu, x3, 1);
          up = lane == 0 ? x0 : up;
          m0[i] = fmaxf(fmaxf(up, x0), x1) + bs[i];
          m1[i] = fmaxf(fmaxf(x1, x2), x3) + bs[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          h[c][i] = relu ? cvt_pack16<BF16, true>(m0[2 * i], m0[2 * i + 1]) : cvt_pack16<BF16, false>(m0[2 * i], m0[2 * i + 1]);
          h[c][8 + i] = relu ? cvt_pack16<BF16, true>(m1[2 * i], m1[2 * i + 1]) : cvt_pack16<BF16, false>(m1[2 * i], m1[2 * i + 1]);
        }
      }
      const uint32_t mine = hbuf0 + static_cast<uint32_t>(hb) * (2u * kSpRowBytes);
      if (q & 1) {
        // ---- rows 1 and 3: publish.  The buffer's last use (three tiles ago) must have been read.
        if (it >= 3 && !mbar_wait_warp(hfree_bar(hb), hphase ^ 1u, abort_flag)) {
          if (lane == 0 && *abort_code == 0) *abort_code = 6;
          break;
        }
        const uint32_t row = mine + (q == 3 ? kSpRowBytes : 0u) + lane_off;
        if (lane_valid) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                const uint32_t u = static_cast<uint32_t>(c * 2 + hh);
                st_shared_v4(row + e * 128u + ((u ^ key) << 4),
                             make_uint4(h[c][8 * e + 4 * hh], h[c][8 * e + 4 * hh + 1], h[c][8 * e + 4 * hh + 2],
                                        h[c][8 * e + 4 * hh + 3]));
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(hready_bar(hb));
      } else {
        // ---- rows 0 and 2: combine with the published rows and store one pooled row
        if (!mbar_wait_warp(hready_bar(hb), hphase, abort_flag)) {
          if (lane == 0 && *abort_code == 0) *abort_code = 7;
          break;
        }
        // row 0 pools with row 1 and the previous tile's row 3 (none above the image's first row);
        // row 2 pools with rows 1 and 3
        const bool above = q == 0 && it > 0 && tt > 0;
        const int pb = (it + 2) % 3;   // = (it - 1) % 3
        uint32_t other = mine + kSpRowBytes;
        if (q == 0) {
          other = hbuf0 + static_cast<uint32_t>(pb) * (2u * kSpRowBytes) + kSpRowBytes;
          if (above && !mbar_wait_warp(hready_bar(pb), static_cast<uint32_t>((it - 1) / 3) & 1u, abort_flag)) {
            if (lane == 0 && *abort_code == 0) *abort_code = 8;
            break;
          }
        }
        const bool second = q == 2 || above;
        const int prow = 2 * tt + (q >> 1);
        char* dst = static_cast<char*>(p.out) +
                    ((static_cast<long long>(img) * p.pool_p + prow) * p.pool_q + 2 * lane) * 128;
        if (lane_valid) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              uint4 r[2];
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                const uint32_t u = static_cast<uint32_t>(c * 2 + hh);
                const uint32_t off = lane_off + e * 128u + ((u ^ key) << 4);
                uint4 x = make_uint4(h[c][8 * e + 4 * hh], h[c][8 * e + 4 * hh + 1], h[c][8 * e + 4 * hh + 2],
                                     h[c][8 * e + 4 * hh + 3]);
                x = sp_max2x4<BF16>(x, ld_shared_v4(mine + off));
                if (second) x = sp_max2x4<BF16>(x, ld_shared_v4(other + off));
                r[hh] = x;
              }
              if (store) st_global_v8(dst + e * 128 + c * 32, r[0], r[1]);
            }
          }
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(hfree_bar(hb));
          if (q == 0 && it > 0) mbar_arrive(hfree_bar(pb));
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    if (threadIdx.x == 0) {
      const int code = *abort_code != 0 ? *abort_code : 9;
      atomicCAS(p.status, 0, code);
    }
    // give copies and MMAs still in flight a bounded time to land before TMEM and shared memory go away
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) {
      __nanosleep(2000);
    }
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace pmlb
