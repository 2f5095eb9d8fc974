// Host side of the tensor-core contraction kernel: tensor-map encoding, tile-shape
// choice and launch.  No allocation happens here; callers own every buffer.
#include "tc_launch.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "tc_gemm_kernel.cuh"
#include "conv_route.h"
#include "halo_fs.h"
#include "tc_instances.h"

namespace pmlb {

// every instance is compiled in one of the tc_inst_*.cu files
#define PMLB_TC_EXTERN(EB, BN, NS, IM, MN, OB, G)                                              \
  extern template cudaError_t launch_cfg<TcCfg<EB, BN, NS, IM, MN, OB, G>>(                     \
      const TcMaps&, const TcParams&, int, cudaStream_t);
PMLB_TC_LIST_H16(PMLB_TC_EXTERN, 1)
PMLB_TC_LIST_H16(PMLB_TC_EXTERN, 2)
PMLB_TC_LIST_MISC(PMLB_TC_EXTERN)
#undef PMLB_TC_EXTERN
#define PMLB_TC_EXTERN(EB, BN, NS, IM, MN, OB, G)                                              \
  extern template cudaError_t launch_cfg<TcCfg<EB, BN, NS, IM, MN, OB, G, 2>>(                  \
      const TcMaps&, const TcParams&, int, cudaStream_t);
PMLB_TC_LIST_PAIR(PMLB_TC_EXTERN)
#undef PMLB_TC_EXTERN
extern template int max_resident_pairs<TcCfg<2, 256, 1, 0, false, 2, 1, 2>>();

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
using EncodeIm2colFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                    cuuint32_t, cuuint32_t, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode_tiled = nullptr;
EncodeIm2colFn g_encode_im2col = nullptr;
std::once_flag g_driver_once;

void load_driver_entry_points() {
  std::call_once(g_driver_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    }
    fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
    }
  });
}

CUtensorMapDataType map_dtype(int eb, bool is_f16) {
  if (eb == 4) return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  if (eb == 2) return is_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  return CU_TENSOR_MAP_DATA_TYPE_UINT8;
}

// 3-D tiled map, 128-byte swizzle, zero fill outside the tensor.
bool encode3d(CUtensorMap* map, CUtensorMapDataType dt, int eb, const void* base, uint64_t d0,
              uint64_t d1, uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes,
              uint32_t b0, uint32_t b1, uint32_t b2, std::string* err) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (stride1_bytes & 15u) != 0 ||
      (stride2_bytes & 15u) != 0) {
    *err = "operand base address and row strides must be multiples of 16 bytes";
    return false;
  }
  if (b0 * static_cast<uint32_t>(eb) != 128u || b1 > 256u || b2 > 256u) {
    *err = "internal: bad TMA box";
    return false;
  }
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode_tiled(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    *err = "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r));
    return false;
  }
  return true;
}

uint32_t make_idesc(int eb, bool is_f16, bool b_mn, int bn, int bm = 128) {
  // bits: [4,6) D format, [7,10) A format, [10,13) B format, 15 A major, 16 B major,
  //       [17,23) N >> 3, [24,29) M >> 4
  uint32_t cfmt, abfmt;
  if (eb == 1) {
    cfmt = 2;   // s32
    abfmt = 1;  // signed 8 bit
  } else if (eb == 4) {
    cfmt = 1;   // f32
    abfmt = 2;  // tf32
  } else {
    cfmt = 1;
    abfmt = is_f16 ? 0u : 1u;
  }
  uint32_t d = 0;
  d |= cfmt << 4;
  d |= abfmt << 7;
  d |= abfmt << 10;
  d |= (b_mn ? 1u : 0u) << 16;
  d |= static_cast<uint32_t>(bn >> 3) << 17;
  d |= static_cast<uint32_t>(bm >> 4) << 24;
  return d;
}

int out_bytes_of(int dtype) {
  switch (dtype) {
    case kDtF32:
    case kDtI32: return 4;
    case kDtBF16:
    case kDtF16: return 2;
    default: return 1;
  }
}

CUtensorMapDataType out_map_dtype(int dtype) {
  switch (dtype) {
    case kDtF32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case kDtI32: return CU_TENSOR_MAP_DATA_TYPE_INT32;
    case kDtF16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int pick_bn(const TcLaunch& L, int num_sms) {
  if (L.bn_override == 64 || L.bn_override == 128 || L.bn_override == 256) return L.bn_override;
  const int max_bn = (L.nsplit == 2) ? 128 : 256;
  if (L.n <= 64) return 64;
  if (L.n <= 128) return 128;
  if (max_bn == 128) {
    // fp32 (three TF32 products per k-step, all tensor-bound): 64-wide tiles when the 128-wide ones
    // would leave SMs without a tile
    const long long tiles128 =
        static_cast<long long>(L.batch) * ((L.m + 127) / 128) * ((L.n + 127) / 128);
    return tiles128 < num_sms ? 64 : 128;
  }
  // 256-wide tiles halve the A re-reads; use them once they still fill the machine.
  const long long tiles256 =
      static_cast<long long>(L.batch) * ((L.m + 127) / 128) * ((L.n + 255) / 256);
  if (L.n % 256 == 0 || L.n > 512) {
    if (tiles256 >= num_sms) return 256;
  }
  // small problems (few rows): 64-wide tiles put a tile on more SMs, and a tile's serial walk over
  // K is shorter per k-block (a 64-wide MMA lasts 48 cycles, a 128-wide one 64)
  const long long tiles128 =
      static_cast<long long>(L.batch) * ((L.m + 127) / 128) * ((L.n + 127) / 128);
  if (tiles128 * 2 <= num_sms) return 64;
  return 128;
}

}  // namespace

bool tc_supported(std::string* why) {
  load_driver_entry_points();
  if (!g_encode_tiled || !g_encode_im2col) {
    if (why) *why = "CUDA driver does not export cuTensorMapEncodeTiled/Im2col";
    return false;
  }
  return true;
}

int tc_launch(const TcLaunch& L, cudaStream_t stream, std::string* err) {
  load_driver_entry_points();
  if (!g_encode_tiled || !g_encode_im2col) {
    *err = "CUDA driver does not export the tensor-map encoders";
    return 3;
  }
  if (L.m <= 0 || L.n <= 0 || L.k <= 0 || L.batch <= 0) {
    *err = "empty problem";
    return 1;
  }
  const int eb = L.elem_bytes;
  if (!(eb == 1 || eb == 2 || eb == 4) || (eb == 4) != (L.nsplit == 2) ||
      (L.nsplit != 1 && L.nsplit != 2)) {
    *err = "unsupported element size / split combination";
    return 1;
  }
  int dev = 0, num_sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);

  int bn = pick_bn(L, num_sms);
  bool prefer_pair = false;   // set where the operand-traffic estimate below prefers CTA pairs
  const int bk = 128 / eb;
  if (L.b_mn && bn < bk) bn = bk;           // MN-major B tiles are whole 128-byte chunks of N
  if (L.b_mn && L.nsplit == 2) {
    *err = "fp32 operands reach this kernel pre-split and K-major";
    return 1;
  }
  if (L.conv && (L.b_mn || !((eb == 2 && L.nsplit == 1) || (eb == 4 && L.nsplit == 2)))) {
    *err = "im2col path takes 16-bit K-major operands, or fp32 ones split into TF32 parts";
    return 1;
  }
  if (L.conv && eb == 4 && bn > 128) bn = 128;   // (the split-operand instances are 64 and 128 wide)

  const int num_kb_plain = (L.k + bk - 1) / bk;
  // Few-tile GEMMs with a long K: 128-wide tiles were chosen above because 256-wide ones would not fill the
  // device.  Such launches run at the pace operands reach an SM, not at the tensor cores': measured on
  // 4096-deep int8 and bf16 GEMMs, a CTA ingests ~48 B/clk with 128 x 128 tiles (32 KB per k-block: ~680
  // cycles where the MMAs need 256) and ~34 B/clk as half of a CTA pair on a 256 x 256 tile (32 KB per
  // k-block too, ~960 cycles for twice the work), whatever the number of CTAs.  So a wave of pair tiles does a
  // quarter more per cycle but is coarser: estimate both (waves x cycles per k-block) and take pairs when
  // they win (1024 x 4096 x 4096: two waves of 128-wide tiles 25.4 us, one wave of pairs 22.7 us; 512 rows:
  // one wave either way, 17.3 against 22.6 us, pairs lose).
  if (bn == 128 && L.bn_override == 0 && L.pair_override != 0 && !L.conv && !L.window && !L.halo && !L.s2d &&
      L.nsplit == 1 && num_kb_plain >= 16 && L.m >= 256 && L.n >= 256) {
    const long long tiles128 = static_cast<long long>(L.batch) * ((L.m + 127) / 128) * ((L.n + 127) / 128);
    const long long pairs256 = static_cast<long long>(L.batch) * ((L.m + 255) / 256) * ((L.n + 255) / 256);
    const long long waves128 = (tiles128 + num_sms - 1) / num_sms;
    const long long waves_pair = (pairs256 + num_sms / 2 - 1) / (num_sms / 2);
    const double t128 = static_cast<double>(waves128) * std::max(256.0, 32768.0 / 48.0);
    const double tpair = static_cast<double>(waves_pair) * std::max(512.0, 32768.0 / 34.0);
    if (tpair < 0.95 * t128) {
      bn = 256;
      prefer_pair = true;
    }
  }
  // Two epilogue groups when the main loop of a tile is short next to its epilogue.
  int groups = (L.conv ? 0 : num_kb_plain) <= 24 ? 2 : 1;
  // CTA pairs: plain GEMMs whose 256-wide tiles have long main loops and fill the machine.
  bool pair = false;
  const bool pair_possible = !L.window && !L.halo && !L.s2d && L.nsplit == 1 && !(L.conv && L.b_mn) &&
                             (bn == 256 || (L.conv && bn == 128 && eb == 2));
  if (pair_possible && !L.conv && num_kb_plain >= 16 && L.m >= 256) {
    const long long pair_tiles =
        static_cast<long long>(L.batch) * ((L.m + 255) / 256) * ((L.n + 255) / 256);
    pair = pair_tiles * 2 >= num_sms || prefer_pair;
  }
  // Convolutions with several taps are bound by the operand traffic from L2 to shared memory
  // (A and B tiles of every tap and channel block): a pair fetches each weight tile once per
  // 256 pixels.  Their main loops are long enough for the single epilogue group of a pair.
  if (pair_possible && L.conv && L.conv->r * L.conv->s > 1 && num_kb_plain >= 9 && L.m >= 256) {
    const long long pair_tiles = static_cast<long long>((L.m + 255) / 256) * ((L.n + bn - 1) / bn);
    pair = pair_tiles * 2 >= num_sms;
  }
  if (L.pair_override == 0) pair = false;
  if (L.pair_override == 1) pair = pair_possible;
  if (const char* env = std::getenv("PMLB_TC_PAIR")) {
    if (env[0] == '0') pair = false;
  }
  static int resident_pairs[64] = {0};
  if (pair) {
    if (dev >= 0 && dev < 64 && resident_pairs[dev] == 0) {
      const int n = max_resident_pairs<TcCfg<2, 256, 1, 0, false, 2, 1, 2>>();
      resident_pairs[dev] = n > 0 ? n : -1;
    }
    if (dev < 0 || dev >= 64 || resident_pairs[dev] <= 0) pair = false;
  }

  TcParams p;
  std::memset(&p, 0, sizeof(p));
  p.m = L.m;
  p.n = L.n;
  p.k = L.k;
  p.batch = L.batch;
  p.tiles_m = pair ? (L.m + 255) / 256 : (L.m + 127) / 128;
  p.tiles_n = (L.n + bn - 1) / bn;
  p.group_m = 16;
  p.a_bz = L.a_batch_stride != 0 ? 1 : 0;
  p.b_bz = L.b_batch_stride != 0 ? 1 : 0;
  p.out = L.out;
  p.ldc = L.ldc;
  p.out_batch = L.out_batch_stride;
  p.out_dtype = L.out_dtype;
  p.epi_flags = L.epi_flags;
  p.bias = L.bias;
  p.residual = L.residual;
  p.ldr = L.ldr;
  p.res_batch = L.res_batch_stride;
  p.rowmax = L.rowmax;
  p.status = L.status;
  p.wait_limit_us = L.wait_limit_us;
  p.test_drop_load = L.test_drop_load ? 1 : 0;
  p.trace = L.trace;
  p.idesc = make_idesc(eb, L.is_f16, L.b_mn, bn, pair ? 256 : 128);

  const CUtensorMapDataType dt = map_dtype(eb, L.is_f16);
  TcMaps maps;
  std::memset(&maps, 0, sizeof(maps));
  CUtensorMap& ta0 = maps.a0;
  CUtensorMap& ta1 = maps.a1;
  CUtensorMap& tb0 = maps.b0;
  CUtensorMap& tb1 = maps.b1;
  CUtensorMap& tc_map = maps.c;

  if (L.s2d) {
    const S2dGeom& g = *L.s2d;
    using S2dCfg = TcCfg<2, 64, 1, kAS2d, false, 2, 2>;
    static_assert(S2dCfg::STAGES * S2dCfg::STAGE == kS2dSmemBytes, "space-to-depth budget");
    const int taps = g.r2 * g.s2;
    const int wts_bytes = g.r2 * ((g.s2 + 3) / 4) * 8192;
    const int stage_bytes = g.stage_px * 32;
    // (the kernel has one pair of barriers per operand-ring stage of its instance)
    const int stages = stage_bytes > 0 ? std::min(S2dCfg::STAGES, (kS2dSmemBytes - wts_bytes) / stage_bytes) : 0;
    if (eb != 2 || L.nsplit != 1 || L.b_mn || L.n > 64 || L.n % 8 != 0 || g.wp % 32 != 0 || g.stage_px % 32 != 0 ||
        g.stage_px < 512 + (g.r2 - 1) * g.wp + g.s2 - 1 || g.wp < g.q + g.s2 - 1 || g.h2 < g.p + g.r2 - 1 ||
        g.q % 4 != 0 || stages < 2 || L.m != g.n * g.p * g.q || L.batch != 1 ||
        (L.epi_flags & (kEpiResidual | kEpiRowMax)) != 0) {
      *err = "space-to-depth convolution: geometry outside what the kernel takes";
      return 3;
    }
    if ((reinterpret_cast<uintptr_t>(L.a0) & 15u) != 0 || (reinterpret_cast<uintptr_t>(L.b0) & 15u) != 0) {
      *err = "space-to-depth convolution: packed operands must be 16-byte aligned";
      return 1;
    }
    bn = 64;
    p.conv_p = g.p;
    p.conv_q = g.q;
    p.conv_r = g.r2;
    p.conv_s = g.s2;
    p.conv_cblocks = 1;
    p.halo_wp = g.wp;
    p.halo_stage_bytes = stage_bytes;
    p.halo_stages = stages;
    p.halo_tiles_per_img = (g.p * g.wp + 511) / 512;
    p.s2d_px = L.a0;
    p.s2d_wts = L.b0;
    p.s2d_img_px = g.h2 * g.wp;
    p.s2d_stage_load = g.stage_px * 32;
    p.s2d_box_rows = g.wp % 128 == 0 ? 32 : (g.wp % 64 == 0 ? 16 : 8);
    p.num_kb = taps;
    p.batch = g.n * p.halo_tiles_per_img;     // tiles of 512 positions
    p.tiles_m = 1;
    p.tiles_n = 1;
    p.idesc = make_idesc(eb, L.is_f16, false, bn);
  } else if (L.halo) {
    const ConvGeom& g = L.halo->conv;
    const int wp = g.w + 2 * g.pad_w;                     // = q + s - 1 for stride 1
    const int th = wp > 0 ? std::min(128 / wp, g.p) : 0;
    const int rows = th + g.r - 1;
    const int cblocks = (g.c + bk - 1) / bk;
    // operand ring plus the staging area this mode's epilogue does not use
    using HaloCfg = TcCfg<2, 64, 1, kAHalo, false, 2, 2>;
    static_assert(HaloCfg::STAGES * HaloCfg::STAGE + HaloCfg::STG_BYTES == kHaloSmemBytes, "halo budget");
    const int ring_bytes = kHaloSmemBytes;
    const int wts_bytes = g.r * g.s * cblocks * 64 * 128;
    const int stage_bytes = (wp * rows * 128 + 1023) / 1024 * 1024;
    // the last tap's window reaches (r - 1) * wp + s - 1 rows past the 128 it needs
    const int overread = std::max(0, ((g.r - 1) * wp + g.s - 1 + 128) * 128 - stage_bytes);
    // (the kernel has one pair of barriers per operand-ring stage of its instance)
    const int stages =
        stage_bytes > 0 ? std::min(HaloCfg::STAGES, (ring_bytes - wts_bytes - overread) / stage_bytes) : 0;
    if (eb != 2 || L.nsplit != 1 || L.b_mn || L.n != 64 || g.c % 64 != 0 || g.stride_h != 1 || g.stride_w != 1 ||
        g.dil_h != 1 || g.dil_w != 1 || th < 1 || wp > 256 || rows > 256 || stages < 2 ||
        g.q != wp - g.s + 1 || g.p != g.h + 2 * g.pad_h - g.r + 1 || L.m != g.n * g.p * g.q || L.batch != 1) {
      *err = "halo convolution: geometry outside what the kernel takes";
      return 3;
    }
    bn = 64;
    p.conv_p = g.p;
    p.conv_q = g.q;
    p.conv_r = g.r;
    p.conv_s = g.s;
    p.conv_cblocks = cblocks;
    p.conv_lower_h = -g.pad_h;
    p.conv_lower_w = -g.pad_w;
    p.halo_wp = wp;
    p.halo_th = th;
    p.halo_rows = rows;
    p.halo_stage_bytes = stage_bytes;
    p.halo_stages = stages;
    p.halo_tiles_per_img = (g.p + th - 1) / th;
    p.num_kb = g.r * g.s * cblocks;
    p.batch = g.n * p.halo_tiles_per_img;     // tiles, one 128-position tile each
    p.tiles_m = 1;
    p.tiles_n = 1;
    p.idesc = make_idesc(eb, L.is_f16, false, bn);
    if ((reinterpret_cast<uintptr_t>(L.a0) & 15u) != 0) {
      *err = "activation base address must be 16-byte aligned";
      return 1;
    }
    // activation (C, W, H, N), box = 64 channels x padded width x fetched rows
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(g.c), static_cast<cuuint64_t>(g.w),
                          static_cast<cuuint64_t>(g.h), static_cast<cuuint64_t>(g.n)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(g.c) * eb, static_cast<cuuint64_t>(g.c) * g.w * eb,
                             static_cast<cuuint64_t>(g.c) * g.w * g.h * eb};
    cuuint32_t box[4] = {64, static_cast<cuuint32_t>(wp), static_cast<cuuint32_t>(rows), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = g_encode_tiled(&ta0, dt, 4, const_cast<void*>(L.a0), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      *err = "cuTensorMapEncodeTiled (halo rows) failed with code " + std::to_string(static_cast<int>(r));
      return 2;
    }
    ta1 = ta0;
    const int taps = g.r * g.s;
    if (!encode3d(&tb0, dt, eb, L.b0, g.c, taps, L.n, static_cast<uint64_t>(g.c) * eb,
                  static_cast<uint64_t>(g.c) * taps * eb, bk, 1, bn, err)) {
      return 1;
    }
    tb1 = tb0;
    // Three filter columns on one channel block, no residual: the filter columns merge into the MMA's N
    // dimension (one 128 x 192 product per filter row; halo_fs_kernel.cuh) and the launch happens here.
    const int ob_out = out_bytes_of(L.out_dtype);
    // CTA pairs (two tiles per MMA, each CTA half of every weight tile) unless asked not to or the device cannot
    // hold a cluster; PMLB_CONV_NO_CTA_PAIRS keeps single CTAs
    const bool fs_pair = L.pair_override != 0 && num_sms >= 2;
    const int fs_stages = halo_fs_stages(fs_pair ? wts_bytes / 2 : wts_bytes, stage_bytes);
    const int fs_overread = std::max(0, ((g.r - 1) * wp + 2 + 128) * 128 - stage_bytes);   // last row's window, two pixels on
    if (L.halo_merge_columns != 0 && g.s == 3 && cblocks == 1 && g.c == 64 && (ob_out == 2 || ob_out == 4) &&
        (L.epi_flags & (kEpiResidual | kEpiRowMax)) == 0 && L.out != nullptr && L.ldc == 64 &&
        (reinterpret_cast<uintptr_t>(L.out) & 31u) == 0 && (!(L.epi_flags & kEpiBias) || L.bias != nullptr) &&
        fs_stages >= 2 && fs_overread <= halo_fs_tail_bytes()) {
      p.halo_stages = fs_stages;
      p.idesc = make_idesc(eb, L.is_f16, false, 128, fs_pair ? 256 : 128);        // filter columns 0 and 1 side by side
      p.idesc_half = make_idesc(eb, L.is_f16, false, 64, fs_pair ? 256 : 128);    // filter column 2
      if (fs_pair && !encode3d(&tb1, dt, eb, L.b0, g.c, taps, L.n, static_cast<uint64_t>(g.c) * eb,
                               static_cast<uint64_t>(g.c) * taps * eb, bk, 1, 32, err)) {
        return 1;
      }
      p.fd_tiles_per_img = make_fastdiv(static_cast<uint32_t>(std::max(1, p.halo_tiles_per_img)));
      p.fd_wp = make_fastdiv(static_cast<uint32_t>(std::max(1, p.halo_wp)));
      int fs_grid = std::min(p.batch, L.grid_override > 0 ? L.grid_override : num_sms);
      if (fs_pair) fs_grid = 2 * std::max(1, std::min((p.batch + 1) / 2, (L.grid_override > 0 ? L.grid_override : num_sms) / 2));
      const cudaError_t fe = launch_halo_fs(maps, p, fs_grid, ob_out, fs_pair, dependent_launch_enabled(), stream);
      if (fe != cudaSuccess) {
        *err = std::string("kernel launch failed: ") + cudaGetErrorString(fe);
        return 2;
      }
      return 0;
    }
  } else if (L.window) {
    const WinGeom& g = *L.window;
    const int row_elems = g.s * g.cp;
    if (eb != 2 || L.nsplit != 1 || L.b_mn || g.cp % 8 != 0 || row_elems > 64 || L.n > 64 ||
        g.stride_h > g.r || g.r > 12 || L.m != g.q || L.batch != g.n * g.p) {
      *err = "packed-row convolution: geometry outside what the kernel takes";
      return 3;
    }
    bn = 64;
    p.tiles_n = 1;
    p.idesc = make_idesc(eb, L.is_f16, false, bn);
    const int slot_rows = std::min(128, (g.q + 7) / 8 * 8);
    p.win_r = g.r;
    p.win_slot_bytes = slot_rows * 128;
    // ring bytes of the 64-wide 16-bit instance with one epilogue group
    const int ring_bytes = TcCfg<2, 64, 1, kAWindow, false, 2, 1>::STAGES *
                           TcCfg<2, 64, 1, kAWindow, false, 2, 1>::STAGE;
    p.win_slots = std::min(16, (ring_bytes - g.r * 64 * 128 - (128 - slot_rows) * 128) /
                                   p.win_slot_bytes);
    if (p.win_slots <= g.r) {
      *err = "packed-row convolution: filter too tall for the row ring";
      return 3;
    }
    p.conv_p = g.p;
    p.conv_stride_h = g.stride_h;
    p.conv_lower_h = -g.pad_h;
    p.num_kb = g.r;
    if ((reinterpret_cast<uintptr_t>(L.a0) & 15u) != 0 || (reinterpret_cast<uintptr_t>(L.b0) & 15u) != 0) {
      *err = "operand base addresses must be 16-byte aligned";
      return 1;
    }
    // activation seen as (row window of s * cp elements, q, h, n): windows of neighbouring
    // output columns overlap, so the q stride is smaller than the window
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(row_elems), static_cast<cuuint64_t>(g.q),
                          static_cast<cuuint64_t>(g.h), static_cast<cuuint64_t>(g.n)};
    const cuuint64_t pitch = static_cast<cuuint64_t>(g.wp) * g.cp * eb;
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(g.stride_w) * g.cp * eb, pitch, pitch * g.h};
    cuuint32_t box[4] = {64, static_cast<cuuint32_t>(slot_rows), 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = g_encode_tiled(&ta0, dt, 4, const_cast<void*>(L.a0), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      *err = "cuTensorMapEncodeTiled (row windows) failed with code " +
             std::to_string(static_cast<int>(r));
      return 2;
    }
    ta1 = ta0;
    // weights [k_out][r][64]
    if (!encode3d(&tb0, dt, eb, L.b0, 64, g.r, L.n, 64ull * eb, 64ull * g.r * eb, bk, 1, bn, err)) {
      return 1;
    }
    tb1 = tb0;
  } else if (L.conv) {
    const ConvGeom& g = *L.conv;
    if ((g.c * eb) % 16 != 0) {
      *err = "im2col path needs whole 16-byte groups of channels per pixel";
      return 3;
    }
    p.conv_p = g.p;
    p.conv_q = g.q;
    p.conv_s = g.s;
    p.conv_cblocks = (g.c + bk - 1) / bk;
    p.conv_stride_h = g.stride_h;
    p.conv_stride_w = g.stride_w;
    p.conv_lower_h = -g.pad_h;
    p.conv_lower_w = -g.pad_w;
    p.conv_dil_h = g.dil_h;
    p.conv_dil_w = g.dil_w;
    p.num_kb = g.r * g.s * p.conv_cblocks;
    // activation (C, W, H, N), bounding box chosen so that exactly p x q base pixels exist
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(g.c), static_cast<cuuint64_t>(g.w),
                          static_cast<cuuint64_t>(g.h), static_cast<cuuint64_t>(g.n)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(g.c) * eb,
                             static_cast<cuuint64_t>(g.c) * g.w * eb,
                             static_cast<cuuint64_t>(g.c) * g.w * g.h * eb};
    // upper corner such that (extent + upper - lower - 1) / stride + 1 == outputs
    int lower[2] = {-g.pad_w, -g.pad_h};
    int upper[2] = {(g.q - 1) * g.stride_w + 1 - g.pad_w - g.w,
                    (g.p - 1) * g.stride_h + 1 - g.pad_h - g.h};
    cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(g.stride_w),
                          static_cast<cuuint32_t>(g.stride_h), 1};
    if ((reinterpret_cast<uintptr_t>(L.a0) & 15u) != 0) {
      *err = "activation base address must be 16-byte aligned";
      return 1;
    }
    CUresult r = g_encode_im2col(&ta0, dt, 4, const_cast<void*>(L.a0), dims, strides, lower, upper,
                                 static_cast<cuuint32_t>(bk), 128u, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      *err = "cuTensorMapEncodeIm2col failed with code " + std::to_string(static_cast<int>(r));
      return 2;
    }
    {
      // Drivers up to CUDA 13.1 encode im2col maps of tensors below 128 KiB with a
      // flag that makes the copy misbehave; CUTLASS clears it the same way.
      int driver_version = 0;
      cudaDriverGetVersion(&driver_version);
      const unsigned long long bytes =
          static_cast<unsigned long long>(g.c) * g.w * g.h * g.n * eb;
      if (driver_version <= 13010 && bytes < 131072ull) {
        reinterpret_cast<uint64_t*>(&ta0)[1] &= ~(1ull << 21);
      }
    }
    ta1 = ta0;
    if (L.nsplit == 2) {
      // the low TF32 parts: the same geometry over the second tensor
      if (L.a1 == nullptr || L.b1 == nullptr || (reinterpret_cast<uintptr_t>(L.a1) & 15u) != 0) {
        *err = "fp32 convolution: the low parts of the operands are missing";
        return 1;
      }
      r = g_encode_im2col(&ta1, dt, 4, const_cast<void*>(L.a1), dims, strides, lower, upper, static_cast<cuuint32_t>(bk), 128u,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) {
        *err = "cuTensorMapEncodeIm2col (low parts) failed with code " + std::to_string(static_cast<int>(r));
        return 2;
      }
      int driver_version = 0;
      cudaDriverGetVersion(&driver_version);
      const unsigned long long bytes = static_cast<unsigned long long>(g.c) * g.w * g.h * g.n * eb;
      if (driver_version <= 13010 && bytes < 131072ull) reinterpret_cast<uint64_t*>(&ta1)[1] &= ~(1ull << 21);
    }
    // weights [k_out][taps][c]
    const int taps = g.r * g.s;
    if (!encode3d(&tb0, dt, eb, L.b0, g.c, taps, L.n, static_cast<uint64_t>(g.c) * eb,
                  static_cast<uint64_t>(g.c) * taps * eb, bk, 1, pair ? bn / 2 : bn, err)) {
      return 1;
    }
    tb1 = tb0;
    if (L.nsplit == 2 && !encode3d(&tb1, dt, eb, L.b1, g.c, taps, L.n, static_cast<uint64_t>(g.c) * eb,
                                   static_cast<uint64_t>(g.c) * taps * eb, bk, 1, bn, err)) {
      return 1;
    }
  } else {
    p.num_kb = (L.k + bk - 1) / bk;
    const uint64_t a_bs = p.a_bz ? static_cast<uint64_t>(L.a_batch_stride) * eb
                                 : static_cast<uint64_t>(L.lda) * eb * L.m;
    // A of two tensors side by side along K: each gets a map of its own columns (reads past a tensor's last
    // column arrive as zeros, so only the first tensor's width must be whole k-blocks)
    const bool two_a = L.k_first > 0;
    if (two_a && (L.nsplit != 1 || L.batch != 1 || L.k_first >= L.k || L.k_first % bk != 0 || L.a1 == nullptr ||
                  (!L.a_second_pixels && L.lda_second < L.k - L.k_first))) {
      *err = "GEMM with A in two parts: needs 8/16-bit operands, one matrix, a first part of whole k-blocks";
      return 3;
    }
    p.a_split_kb = two_a ? L.k_first / bk : 0;
    if (!encode3d(&ta0, dt, eb, L.a0, two_a ? L.k_first : L.k, L.m, p.a_bz ? L.batch : 1,
                  static_cast<uint64_t>(L.lda) * eb, a_bs, bk, 128, 1, err)) {
      return 1;
    }
    ta1 = ta0;
    if (two_a && L.a_second_pixels) {
      const ConvGeom& g2 = *L.a_second_pixels;
      const int c2 = L.k - L.k_first;
      if (g2.r != 1 || g2.s != 1 || g2.pad_h != 0 || g2.pad_w != 0 || g2.stride_h != g2.stride_w || g2.c != c2 || c2 % 8 != 0 ||
          static_cast<long long>(g2.n) * g2.p * g2.q != L.m || (g2.p - 1) * g2.stride_h >= g2.h || (g2.q - 1) * g2.stride_w >= g2.w ||
          (reinterpret_cast<uintptr_t>(L.a1) & 15u) != 0) {
        *err = "GEMM with A's second part as pixels: a 1x1 unpadded sampling of whole 8-channel groups over m = n * p * q rows";
        return 3;
      }
      cuuint64_t dims[4] = {static_cast<cuuint64_t>(g2.c), static_cast<cuuint64_t>(g2.w), static_cast<cuuint64_t>(g2.h),
                            static_cast<cuuint64_t>(g2.n)};
      cuuint64_t strides[3] = {static_cast<cuuint64_t>(g2.c) * eb, static_cast<cuuint64_t>(g2.c) * g2.w * eb,
                               static_cast<cuuint64_t>(g2.c) * g2.w * g2.h * eb};
      int lower[2] = {0, 0};
      int upper[2] = {(g2.q - 1) * g2.stride_w + 1 - g2.w, (g2.p - 1) * g2.stride_h + 1 - g2.h};
      cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(g2.stride_w), static_cast<cuuint32_t>(g2.stride_h), 1};
      CUresult r = g_encode_im2col(&ta1, dt, 4, const_cast<void*>(L.a1), dims, strides, lower, upper, static_cast<cuuint32_t>(bk),
                                   128u, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) {
        *err = "cuTensorMapEncodeIm2col (second part of A) failed with code " + std::to_string(static_cast<int>(r));
        return 2;
      }
      {
        // (the same driver quirk as for the convolution's own map below)
        int driver_version = 0;
        cudaDriverGetVersion(&driver_version);
        const unsigned long long bytes = static_cast<unsigned long long>(g2.c) * g2.w * g2.h * g2.n * eb;
        if (driver_version <= 13010 && bytes < 131072ull) reinterpret_cast<uint64_t*>(&ta1)[1] &= ~(1ull << 21);
      }
      p.a2_pixels = 1;
      p.a2_p = g2.p;
      p.a2_q = g2.q;
      p.a2_stride = g2.stride_w;
      p.a2_fd_per_img = make_fastdiv(static_cast<uint32_t>(g2.p * g2.q));
      p.a2_fd_q = make_fastdiv(static_cast<uint32_t>(g2.q));
    } else if (two_a && !encode3d(&ta1, dt, eb, L.a1, L.k - L.k_first, L.m, 1, static_cast<uint64_t>(L.lda_second) * eb,
                                  static_cast<uint64_t>(L.lda_second) * eb * L.m, bk, 128, 1, err)) {
      return 1;
    }
    if (L.nsplit == 2 &&
        !encode3d(&ta1, dt, eb, L.a1, L.k, L.m, p.a_bz ? L.batch : 1,
                  static_cast<uint64_t>(L.lda) * eb, a_bs, bk, 128, 1, err)) {
      return 1;
    }
    if (L.b_mn) {
      const uint64_t b_bs = p.b_bz ? static_cast<uint64_t>(L.b_batch_stride) * eb
                                   : static_cast<uint64_t>(L.ldb) * eb * L.k;
      if (!encode3d(&tb0, dt, eb, L.b0, L.n, L.k, p.b_bz ? L.batch : 1,
                    static_cast<uint64_t>(L.ldb) * eb, b_bs, bk, bk, 1, err)) {
        return 1;
      }
      tb1 = tb0;
    } else {
      const uint64_t b_bs = p.b_bz ? static_cast<uint64_t>(L.b_batch_stride) * eb
                                   : static_cast<uint64_t>(L.ldb) * eb * L.n;
      if (!encode3d(&tb0, dt, eb, L.b0, L.k, L.n, p.b_bz ? L.batch : 1,
                    static_cast<uint64_t>(L.ldb) * eb, b_bs, bk, pair ? bn / 2 : bn, 1, err)) {
        return 1;
      }
      tb1 = tb0;
      if (L.nsplit == 2 &&
          !encode3d(&tb1, dt, eb, L.b1, L.k, L.n, p.b_bz ? L.batch : 1,
                    static_cast<uint64_t>(L.ldb) * eb, b_bs, bk, bn, 1, err)) {
        return 1;
      }
    }
  }

  // Staged TMA-store epilogue when every output (and residual) row starts on a 16-byte
  // boundary; otherwise the kernel's transpose-and-store path.
  const int ob = out_bytes_of(L.out_dtype);
  // A launch that stores nothing (row maxima only) takes the 16-bit-output instance whatever the
  // declared output type: its chunks are 64 accumulator columns instead of 32, i.e. half as many
  // TMEM round trips per tile, and nothing of it depends on the output element size.
  const bool no_store = L.out == nullptr && !(L.epi_flags & kEpiResidual);
  const int ob_tmpl = (eb == 2 && (ob == 2 || no_store)) ? 2 : 4;
  {
    bool fast = (ob == 2 || ob == 4) && (ob == ob_tmpl || no_store);
    if (L.out != nullptr) {
      fast = fast && aligned16(L.out) && (L.ldc * ob) % 16 == 0 &&
             (L.batch == 1 || (L.out_batch_stride * ob) % 16 == 0);
    }
    if (L.epi_flags & kEpiResidual) {
      fast = fast && aligned16(L.residual) && (L.ldr * ob) % 16 == 0 &&
             (L.batch == 1 || (L.res_batch_stride * ob) % 16 == 0);
    }
    if (L.epi_flags & kEpiBias) fast = fast && aligned16(L.bias);
    if (L.force_slow_epilogue) fast = false;
    if (fast && L.out != nullptr) {
      const uint64_t c_bs = L.batch > 1 ? static_cast<uint64_t>(L.out_batch_stride) * ob
                                        : static_cast<uint64_t>(L.ldc) * ob * L.m;
      if (L.s2d) {
        // (channels, column % 4, column / 4, n * p); boxes of 8 columns that are 4 apart
        const S2dGeom& g = *L.s2d;
        const cuuint64_t pix = static_cast<cuuint64_t>(L.ldc) * ob;
        cuuint64_t dims[4] = {static_cast<cuuint64_t>(L.n), 4, static_cast<cuuint64_t>(g.q / 4),
                              static_cast<cuuint64_t>(g.n) * g.p};
        cuuint64_t strides[3] = {pix, 4 * pix, pix * g.q};
        cuuint32_t box[4] = {static_cast<cuuint32_t>(128 / ob), 1, static_cast<cuuint32_t>(p.s2d_box_rows), 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        CUresult r = g_encode_tiled(&tc_map, out_map_dtype(L.out_dtype), 4, L.out, dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
          *err = "cuTensorMapEncodeTiled (strided output columns) failed with code " +
                 std::to_string(static_cast<int>(r));
          return 2;
        }
      } else if (!encode3d(&tc_map, out_map_dtype(L.out_dtype), ob, L.out, L.n, L.m, L.batch,
                           static_cast<uint64_t>(L.ldc) * ob, c_bs, 128 / ob, 32, 1, err)) {
        return 1;
      }
    }
    p.fast_epi = fast ? 1 : 0;
    // Residual rows ride the same staging buffers: fetched by TMA ahead of their chunk.
    if ((L.halo || L.s2d) && (!fast || L.out == nullptr)) {
      *err = "halo / space-to-depth convolution: output rows must be 16-byte aligned";
      return 3;
    }
    if (fast && L.out != nullptr && (L.epi_flags & kEpiResidual) && !L.residual_from_global && !L.halo) {
      const uint64_t r_bs = L.batch > 1 ? static_cast<uint64_t>(L.res_batch_stride) * ob
                                        : static_cast<uint64_t>(L.ldr) * ob * L.m;
      if (!encode3d(&maps.r, out_map_dtype(L.out_dtype), ob, L.residual, L.n, L.m, L.batch,
                    static_cast<uint64_t>(L.ldr) * ob, r_bs, 128 / ob, 32, 1, err)) {
        return 1;
      }
      p.res_tma = 1;
    }
  }

  {
    auto fd = [](long long d) { return make_fastdiv(static_cast<uint32_t>(std::max<long long>(1, d))); };
    p.fd_per_batch = fd(static_cast<long long>(p.tiles_m) * p.tiles_n);
    p.fd_group = fd(static_cast<long long>(p.group_m) * p.tiles_n);
    p.fd_gm_full = fd(p.group_m);
    p.fd_gm_tail = fd(p.tiles_m % p.group_m);
    p.fd_per_img = fd(static_cast<long long>(p.conv_p) * p.conv_q);
    p.fd_q = fd(p.conv_q);
    p.fd_tiles_per_img = fd(p.halo_tiles_per_img);
    p.fd_wp = fd(p.halo_wp);
  }
  const long long total = static_cast<long long>(p.batch) * p.tiles_m * p.tiles_n;
  if (total > 0x3fffffffLL) {
    *err = "too many tiles";
    return 1;
  }
  // Tail of the last wave: when the tiles left over after the full waves occupy at most half of
  // the CTAs (pairs), they are walked as two half-width tiles each and take half as long.
  p.tiles_full = static_cast<int>(total);
  p.idesc_half = p.idesc;
  if (bn == 256 && !L.window && !L.halo && !L.s2d && L.split_tail != 0) {
    const long long workers = pair ? resident_pairs[dev] : num_sms;
    const long long rem = total % workers;
    if (total > workers && rem > 0 && 2 * rem <= workers) {
      p.tiles_full = static_cast<int>(total - rem);
      p.idesc_half = make_idesc(eb, L.is_f16, L.b_mn, bn / 2, pair ? 256 : 128);
    }
  }
  const long long walked = 2 * total - p.tiles_full;
  int grid = static_cast<int>(std::min<long long>(walked, num_sms));
  if (L.grid_override > 0) grid = std::min<long long>(walked, L.grid_override);
  if (pair) {
    long long pairs = std::min<long long>(walked, resident_pairs[dev]);
    if (L.grid_override > 0) pairs = std::min<long long>(pairs, std::max(1, L.grid_override / 2));
    grid = static_cast<int>(2 * pairs);
  }

  cudaError_t ce = cudaErrorInvalidValue;
  if (L.conv) groups = p.num_kb <= 24 ? 2 : 1;
  if (L.epi_groups_override == 1 || L.epi_groups_override == 2) groups = L.epi_groups_override;
  if (const char* env = std::getenv("PMLB_TC_EPI_GROUPS")) {
    if (env[0] == '1' || env[0] == '2') groups = env[0] - '0';
  }
  if (L.halo || L.s2d) groups = 2;
  if (L.window || pair) groups = 1;  // (the row ring leaves room for one group's staging buffers only)
  const int a_mode = L.s2d ? kAS2d : (L.halo ? kAHalo : (L.window ? kAWindow : (L.conv ? kAIm2col : kATiled)));
  bool launched = false;
#define PMLB_TC_CASE(EB, BN, NS, IM, MN, OB, G)                                                 \
  if (!launched && eb == EB && bn == BN && L.nsplit == NS && a_mode == static_cast<int>(IM) &&  \
      L.b_mn == MN && ob_tmpl == OB && groups == G) {                                           \
    ce = launch_cfg<TcCfg<EB, BN, NS, IM, MN, OB, G>>(maps, p, grid, stream);                   \
    launched = true;                                                                            \
  }
#define PMLB_TC_CASE_PAIR(EB, BN, NS, IM, MN, OB, G)                                            \
  if (!launched && pair && eb == EB && bn == BN && a_mode == static_cast<int>(IM) &&            \
      L.b_mn == MN && ob_tmpl == OB) {                                                          \
    ce = launch_cfg<TcCfg<EB, BN, NS, IM, MN, OB, G, 2>>(maps, p, grid, stream);                \
    launched = true;                                                                            \
  }
  PMLB_TC_LIST_PAIR(PMLB_TC_CASE_PAIR)
#undef PMLB_TC_CASE_PAIR
  if (pair && !launched) {
    *err = "no CTA-pair instance for this configuration";
    return 3;
  }
  for (int attempt = 0; attempt < 2 && !launched; ++attempt) {
    PMLB_TC_LIST_H16(PMLB_TC_CASE, 1)
    PMLB_TC_LIST_H16(PMLB_TC_CASE, 2)
    PMLB_TC_LIST_MISC(PMLB_TC_CASE)
    if (!launched) groups = 1;  // not every shape has a two-group instance
  }
#undef PMLB_TC_CASE
  if (!launched) {
    *err = "no kernel instance for this tile configuration";
    return 3;
  }
  if (ce != cudaSuccess) {
    *err = std::string("kernel launch failed: ") + cudaGetErrorString(ce);
    return 2;
  }
  return 0;
}

}  // namespace pmlb
