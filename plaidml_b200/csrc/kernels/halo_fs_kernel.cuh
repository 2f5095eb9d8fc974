// Stride-1 convolution with three filter columns on 64 input and 64 output channels (the 3x3
// layers of a network's first stage), with two of the three filter columns merged into the N dimension
// of the MMA.
//
// The plain halo route issues one 128 x 64 x 64 product per filter tap and reads the tap's
// 128 x 64 pixel window from shared memory each time: 6 KB of operand reads per 128 x 64 x 16 MMA,
// 48 cycles of the 128 B/clk shared-memory port against 32 cycles of math, with the TMA writes of the
// next pixels competing for the same port (measured: a tile every ~2900 cycles, the loads arriving
// ~6500 cycles after their issue because the operand reads starve them).
//
// Here, per filter row fr and 16-element k-step, two MMAs share one accumulator of 128 columns:
//     D[j,  0.. 63] += pixel[j + fr * wp    ] * W[fr][0]      (one 128 x 128 MMA: columns 0 and 1 of the
//     D[j, 64..127] += pixel[j + fr * wp    ] * W[fr][1]       filter side by side, same pixel window)
//     D[j,  0.. 63] += pixel[j + fr * wp + 2] * W[fr][2]      (one 128 x 64 MMA on the window two pixels on)
// (j = position in the tile's padded position grid, wp = padded row width), so that
//     out[j, ch] = D[j, ch] + D[j + 1, 64 + ch]:
// the product of filter column 1 is computed one position late and the epilogue fetches it from the
// neighbouring TMEM lane with one warp shuffle per channel (lane 31 of a warp takes it from a small
// exchange buffer, the neighbour being the next warp's lane 0 in another quarter of TMEM).  Shared-memory
// reads per k-step and filter row: 8 KB + 6 KB instead of 3 x 6 KB, 112 cycles of the port instead of 144.
// (All three columns in one 128 x 192 MMA need two shuffles per channel and 192-column accumulators, of
// which TMEM holds only two: measured slower, the epilogue of a tile could not overlap enough.)
//
// Roles: warp 0 TMA producer (weights once, then one 4-D tiled load of the tile's padded pixel rows
// per tile into a ring), warp 1 MMA issuer (four TMEM accumulators of 128 columns), warps 2..9 two
// epilogue groups of four warps (group g takes the tiles with local number = g mod 2).
// Every wait is bounded, as in the general kernel.
//
// CTAS = 2: two CTAs (a cluster) work on two neighbouring tiles with one MMA stream: each MMA is 256 rows high
// (cta_group::2; rows 0..127 = the first CTA's tile and accumulator, rows 128..255 the second's), issued by the
// first CTA's issuer, and each CTA holds half of every weight tile's N rows (columns 0 / 1 of the filter for the
// 128-wide MMA, 32 of the 64 output channels of column 2 for the 64-wide one): 36 KB of weights per CTA instead
// of 72 KB, and per filter row and k-step 11 KB of operand reads per CTA (88 cycles of the 128 B/clk port)
// for 96 cycles of math, where a CTA on its own reads 14 KB (112 cycles) for the same math.  Pixel loads are
// per CTA (no multicast) and count on the first CTA's barrier; the second CTA's epilogue hands its accumulator
// back through the first CTA's barrier.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"
#include "tc_gemm.cuh"

namespace pmlb {

constexpr int kFsGroups = 3;                      // epilogue groups of four warps
constexpr int kFsThreads = 64 + 128 * kFsGroups;
constexpr int kFsXbufBytes = kFsGroups * 3 * 256;   // per group: three warp boundaries x 64 floats
constexpr int kFsTailBytes = kFsXbufBytes + 256 + 512;   // exchange buffers, bias, barriers
constexpr int kFsSmemLimit = 232448;
constexpr int kFsMaxStages = 8;

__device__ __forceinline__ void tmem_ld_32x32_x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// OB: bytes per output element (2: bf16 / f16, 4: f32).
template <int OB, int CTAS>
__global__ void __launch_bounds__(kFsThreads, 1)
conv_halo_fs_kernel(const __grid_constant__ TcMaps tm, const __grid_constant__ TcParams p) {
  const uint32_t cta_rank = CTAS == 2 ? cluster_ctarank() : 0u;
  grid_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t ring = (raw_addr + 1023u) & ~1023u;
  uint8_t* ring_ptr = smem_raw + (ring - raw_addr);
  const int nst = p.halo_stages;
  // weights per filter row: 3 x 8 KB, or (pairs) this CTA's 8 KB + 4 KB halves
  const uint32_t wts_row_bytes = CTAS == 2 ? 12288u : 24576u;
  const uint32_t wts_bytes = static_cast<uint32_t>(p.conv_r) * wts_row_bytes;
  const uint32_t stages0 = ring + wts_bytes;
  const uint32_t tail_off = wts_bytes + static_cast<uint32_t>(nst) * static_cast<uint32_t>(p.halo_stage_bytes);
  float* xbuf_all = reinterpret_cast<float*>(ring_ptr + tail_off);
  float* bias_s = reinterpret_cast<float*>(ring_ptr + tail_off + kFsXbufBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring_ptr + tail_off + kFsXbufBytes + 256);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](uint32_t s) { return bar0 + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar0 + 8u * (kFsMaxStages + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * kFsMaxStages + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * kFsMaxStages + 4 + a); };
  const uint32_t wts_bar = bar0 + 8u * (2 * kFsMaxStages + 8);
  // exchange-buffer hand-over inside an epilogue group: published (4 warps) / read (4 warps)
  auto xready_bar = [&](int g) { return bar0 + 8u * (2 * kFsMaxStages + 9 + g); };
  auto xdone_bar = [&](int g) { return bar0 + 8u * (2 * kFsMaxStages + 9 + kFsGroups + g); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kFsMaxStages + 9 + 2 * kFsGroups);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* abort_code = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kFsMaxStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 4; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4 * CTAS);
    }
    for (int g = 0; g < kFsGroups; ++g) {
      mbar_init(xready_bar(g), 4);
      mbar_init(xdone_bar(g), 4);
    }
    mbar_init(wts_bar, 1);
    *abort_flag = 0;
    *abort_code = 0;
    abort_flag[2] = p.wait_limit_us;
    fence_mbar_init();
    tma_prefetch_desc(&tm.a0);
    tma_prefetch_desc(&tm.b0);
  }
  if (warp == 1) {
    if constexpr (CTAS == 2) {
      tmem_alloc_pair(smem_u32(tmem_slot), 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), 512);
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
  if (warp >= 2 && warp < 4) {
    const int ch = (warp - 2) * 32 + lane;
    bias_s[ch] = (p.epi_flags & kEpiBias) ? __ldg(static_cast<const float*>(p.bias) + ch) : 0.f;
  }
  __syncthreads();   // (the staged bias, for the epilogue warps)

  const int total_tiles = p.batch;   // tiles of one 128-position block each
  // Work units: tiles, or (pairs) two neighbouring tiles, one per CTA; a unit's second tile may lie past the
  // end (its loads then bring zeros and nothing of it is stored).
  const int total_units = (total_tiles + CTAS - 1) / CTAS;
  const int u_begin = static_cast<int>(blockIdx.x) / CTAS, u_step = static_cast<int>(gridDim.x) / CTAS;
  auto tile_of = [&](int u) { return u * CTAS + static_cast<int>(cta_rank); };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    const bool leader = elect_one();
    if (leader && u_begin < total_units) {
      if constexpr (CTAS == 2) {
        // this CTA's halves: filter column `rank` (64 rows) for the 128-wide MMA, output channels
        // 32 * rank .. of column 2 for the 64-wide one; all bytes are counted on the first CTA's barrier
        const uint32_t wb0 = mapa_rank(wts_bar, 0);
        if (cta_rank == 0) mbar_arrive_expect_tx(wts_bar, 2u * wts_bytes);
        for (int fr = 0; fr < p.conv_r; ++fr) {
          const uint32_t dst = ring + static_cast<uint32_t>(fr) * wts_row_bytes;
          tma_load_3d_pair(dst, &tm.b0, wb0, 0, fr * 3 + static_cast<int>(cta_rank), 0);
          tma_load_3d_pair(dst + 8192u, &tm.b1, wb0, 0, fr * 3 + 2, 32 * static_cast<int>(cta_rank));
        }
      } else {
        mbar_arrive_expect_tx(wts_bar, wts_bytes);
        for (int tap = 0; tap < p.conv_r * 3; ++tap) {
          tma_load_3d(ring + static_cast<uint32_t>(tap) * 8192u, &tm.b0, wts_bar, 0, tap, 0);
        }
      }
    }
    uint32_t hs = 0, hphase = 0;
    for (int u = u_begin; u < total_units; u += u_step) {
      const int t = tile_of(u);
      // (a tile past the end: image number = batch size, every pixel out of range, i.e. zeros)
      const int img = fast_div(t, p.fd_tiles_per_img);
      const int p0 = (t - img * p.halo_tiles_per_img) * p.halo_th;
      if (!mbar_wait_warp(empty_bar(hs), hphase ^ 1u, abort_flag)) {
        if (leader && *abort_code == 0) *abort_code = 1;
        break;
      }
      if (leader) {
        const uint32_t bytes = static_cast<uint32_t>(p.halo_wp * p.halo_rows) * 128u;
        if constexpr (CTAS == 2) {
          if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(hs), 2u * bytes);
          tma_load_4d_pair(stages0 + hs * static_cast<uint32_t>(p.halo_stage_bytes), &tm.a0, mapa_rank(full_bar(hs), 0), 0,
                           p.conv_lower_w, p0 + p.conv_lower_h, img);
        } else {
          mbar_arrive_expect_tx(full_bar(hs), bytes);
          tma_load_4d(stages0 + hs * static_cast<uint32_t>(p.halo_stage_bytes), &tm.a0, full_bar(hs), 0,
                      p.conv_lower_w, p0 + p.conv_lower_h, img);
        }
      }
      if (++hs == static_cast<uint32_t>(nst)) {
        hs = 0;
        hphase ^= 1u;
      }
    }
  } else if (warp == 1 && cta_rank == 0) {
    // ------------------------------------------------------------ MMA issuer (pairs: the first CTA's)
    const bool leader = elect_one();
    const uint64_t desc_k = make_smem_desc_sw128(0, 16, 1024);
    const uint32_t dk_lo = static_cast<uint32_t>(desc_k), dk_hi = static_cast<uint32_t>(desc_k >> 32);
    auto lo_at = [](uint32_t base_lo, uint32_t saddr) { return base_lo | ((saddr & 0x3FFFFu) >> 4); };
    bool ok = true;
    if (u_begin < total_units && !mbar_wait_warp(wts_bar, 0u, abort_flag)) {
      if (leader && *abort_code == 0) *abort_code = 3;
      ok = false;
    }
    uint32_t hs = 0, hphase = 0;
    int it = 0;
    for (int u = u_begin; u < total_units && ok; u += u_step, ++it) {
      const int acc = it & 3;
      const uint32_t acc_phase = static_cast<uint32_t>(it >> 2) & 1u;
      // (in the steady state both barriers are long complete: probe first, without the suspension a
      // try_wait may take and without the warp vote, and wait properly only when the probe fails)
      if (!mbar_test_wait_warp(tempty_bar(acc), acc_phase ^ 1u) && !mbar_wait_warp(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
        if (leader && *abort_code == 0) *abort_code = 2;
        break;
      }
      if (!mbar_test_wait_warp(full_bar(hs), hphase) && !mbar_wait_warp(full_bar(hs), hphase, abort_flag)) {
        if (leader && *abort_code == 0) *abort_code = 3;
        break;
      }
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * 128);
      // filter row fr: the window that starts fr padded image rows into the buffer times the 128-row
      // weight tile of the row's first two taps (8 KB each, contiguous), then the window two pixels
      // (two 128-byte rows) further on times the third tap's 64 rows, into the first 64 columns
      uint32_t a_lo = lo_at(dk_lo, stages0 + hs * static_cast<uint32_t>(p.halo_stage_bytes));
      uint32_t b_lo = lo_at(dk_lo, ring);
      const uint32_t a_step = static_cast<uint32_t>(p.halo_wp) * 8u;   // 16-byte units per padded image row
      for (int fr = 0; fr < p.conv_r; ++fr) {
        if (leader) {
          // (pairs: the weight halves of a filter row lie 8 KB apart, else the third tap two tiles on)
          tc_mma_x4<kMmaF16, CTAS>(d_tmem, a_lo, b_lo, dk_hi, dk_hi, p.idesc, fr > 0 ? 1u : 0u, 2u, 2u);
          tc_mma_x4<kMmaF16, CTAS>(d_tmem, a_lo + 16u, b_lo + (CTAS == 2 ? 512u : 2u * 512u), dk_hi, dk_hi, p.idesc_half, 1u,
                                   2u, 2u);
        }
        a_lo += a_step;
        b_lo += wts_row_bytes >> 4;
      }
      if (leader) {
        if constexpr (CTAS == 2) {
          tc_commit_pair(empty_bar(hs), 3);    // the pixel buffer is free in both CTAs
          tc_commit_pair(tfull_bar(acc), 3);   // both CTAs' epilogues may read their rows
        } else {
          tc_commit(empty_bar(hs));
          tc_commit(tfull_bar(acc));
        }
      }
      if (++hs == static_cast<uint32_t>(nst)) {
        hs = 0;
        hphase ^= 1u;
      }
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;             // TMEM lane quarter this warp may read
    const int grp = (warp - 2) >> 2;    // group g takes the tiles with local number = g mod 2
    const bool out_bf16 = p.out_dtype == kDtBF16;
    const bool relu = (p.epi_flags & kEpiRelu) != 0;
    // this group's exchange buffer: for warp boundary b = 1..3 the warp of quarter b publishes its lane 0's
    // 64 values of the second block (position j + 1 of the previous warp's lane 31)
    float* xbuf = xbuf_all + grp * (3 * 64);
    float* xmine = xbuf + (q >= 1 ? q - 1 : 0) * 64;
    // what the warp of the next quarter published; the last quarter reads its own slot (and ignores it)
    const float* xnext = xbuf + (q <= 2 ? q : 2) * 64;
    const bool take = q <= 2 && lane == 31;
    // this thread's position in a tile never changes: row pr, column qq of the tile's padded position grid
    const int j = q * 32 + lane;
    const int pr = fast_div(j, p.fd_wp);
    const int qq = j - pr * p.halo_wp;
    const bool in_tile = pr < p.halo_th && qq < p.conv_q;
    uint32_t xphase = 0;
    for (int it = grp; ; it += kFsGroups, xphase ^= 1u) {
      const int u = u_begin + it * u_step;
      if (u >= total_units) break;
      const int t = tile_of(u);
      const int acc = it & 3;
      const uint32_t acc_phase = static_cast<uint32_t>(it >> 2) & 1u;
      const int img = fast_div(t, p.fd_tiles_per_img);
      const int p0 = (t - img * p.halo_tiles_per_img) * p.halo_th;
      const bool valid = in_tile && p0 + pr < p.conv_p && t < total_tiles;
      const long long row = (static_cast<long long>(img) * p.conv_p + p0 + pr) * p.conv_q + qq;
      char* dst = static_cast<char*>(p.out) + row * p.ldc * OB;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
        if (*abort_code == 0) *abort_code = 4;
        break;
      }
      tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + static_cast<uint32_t>(acc * 128) + (static_cast<uint32_t>(q * 32) << 16);
      // the group's previous tile: every warp has read what it needed from the exchange buffer
      if (!mbar_wait(xdone_bar(grp), xphase ^ 1u, abort_flag)) {
        if (*abort_code == 0) *abort_code = 6;
        break;
      }
      if (q >= 1) {
        // lane 0 of this quarter is position j + 1 of the previous warp's last lane
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          uint32_t b1[32];
          tmem_ld_32x32(t_acc + 64 + h * 32, b1);
          tmem_ld_wait();
          if (lane == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              reinterpret_cast<uint4*>(xmine + h * 32)[i] = make_uint4(b1[4 * i], b1[4 * i + 1], b1[4 * i + 2], b1[4 * i + 3]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(xready_bar(grp));
      if (!mbar_wait(xready_bar(grp), xphase, abort_flag)) {
        if (*abort_code == 0) *abort_code = 7;
        break;
      }
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t b0[16], b1[16];
        tmem_ld_32x32_x16(t_acc + c * 16, b0);
        tmem_ld_32x32_x16(t_acc + 64 + c * 16, b1);
        // (every lane loads the neighbour's values and the bias: the same addresses across the warp, i.e.
        // broadcasts; only lane 31 uses the former)
        float x1[16], bs[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 u = reinterpret_cast<const float4*>(xnext + c * 16)[i];
          const float4 bb = reinterpret_cast<const float4*>(bias_s + c * 16)[i];
          x1[4 * i] = u.x, x1[4 * i + 1] = u.y, x1[4 * i + 2] = u.z, x1[4 * i + 3] = u.w;
          bs[4 * i] = bb.x, bs[4 * i + 1] = bb.y, bs[4 * i + 2] = bb.z, bs[4 * i + 3] = bb.w;
        }
        tmem_ld_wait();
        if (c == 3) {
          // accumulator fully read: hand it back to the issuer
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
        float o[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float t1 = __shfl_down_sync(0xffffffffu, __uint_as_float(b1[i]), 1);
          t1 = take ? x1[i] : t1;
          o[i] = (__uint_as_float(b0[i]) + t1) + bs[i];
        }
        if (valid) {
          if constexpr (OB == 2) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (out_bf16) {
                w[i] = relu ? cvt_pack16<true, true>(o[2 * i], o[2 * i + 1]) : cvt_pack16<true, false>(o[2 * i], o[2 * i + 1]);
              } else {
                w[i] = relu ? cvt_pack16<false, true>(o[2 * i], o[2 * i + 1]) : cvt_pack16<false, false>(o[2 * i], o[2 * i + 1]);
              }
            }
            st_global_v8(dst + c * 32, make_uint4(w[0], w[1], w[2], w[3]), make_uint4(w[4], w[5], w[6], w[7]));
          } else {
            if (relu) {
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = relu_keep_nan(o[i]);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              st_global_v8(dst + c * 64 + h * 32,
                           make_uint4(__float_as_uint(o[8 * h]), __float_as_uint(o[8 * h + 1]), __float_as_uint(o[8 * h + 2]),
                                      __float_as_uint(o[8 * h + 3])),
                           make_uint4(__float_as_uint(o[8 * h + 4]), __float_as_uint(o[8 * h + 5]), __float_as_uint(o[8 * h + 6]),
                                      __float_as_uint(o[8 * h + 7])));
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(xdone_bar(grp));
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
  if constexpr (CTAS == 2) cluster_sync_all();   // (a CTA that reported a time-out has waited above)
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    if constexpr (CTAS == 2) {
      tmem_dealloc_pair(tmem_base, 512);
    } else {
      tmem_dealloc(tmem_base, 512);
    }
  }
}

}  // namespace pmlb
