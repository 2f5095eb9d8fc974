// Host-side checks of the kernel library's pure decision code: the division constants used for
// tile coordinates, and which convolution descriptors take which route.  Prints one line per
// check ("ok <name>" / "FAIL <name> ...") and exits non-zero on any failure.
#include <cstdint>
#include <cstdio>
#include <random>

#include "conv_route.h"
#include "tc_gemm.cuh"

static int failures = 0;
static void check(bool ok, const char* name) {
  std::printf("%s %s\n", ok ? "ok" : "FAIL", name);
  if (!ok) ++failures;
}

static uint32_t apply(uint32_t n, pmlb::FastDiv f) {
  return static_cast<uint32_t>((static_cast<unsigned long long>(n) * f.mul) >> f.shift);
}

static pmlb_conv_desc conv(int n, int h, int w, int c, int r, int s, int k, int stride, int pad, int epi = 0) {
  pmlb_conv_desc d = {};
  d.in_dtype = PMLB_BF16;
  d.out_dtype = PMLB_BF16;
  d.n = n; d.h = h; d.w = w; d.c = c; d.r = r; d.s = s; d.k = k;
  d.stride_h = d.stride_w = stride;
  d.pad_h = d.pad_w = pad;
  d.dil_h = d.dil_w = 1;
  d.p = (h + 2 * pad - r) / stride + 1;
  d.q = (w + 2 * pad - s) / stride + 1;
  d.epilogue = epi;
  return d;
}

int main() {
  // n / d for every small pair and for random pairs up to 2^31 - 1
  bool ok = true;
  for (uint32_t d = 1; d < 3000 && ok; ++d) {
    const pmlb::FastDiv f = pmlb::make_fastdiv(d);
    for (uint32_t n = 0; n < 12000; ++n) ok = ok && apply(n, f) == n / d;
  }
  check(ok, "fastdiv small");
  std::mt19937_64 g(7);
  ok = true;
  for (int i = 0; i < 4000000 && ok; ++i) {
    uint32_t d = static_cast<uint32_t>(g() & 0x7fffffffu) | 1u;
    if (i & 1) d = d % 100000u + 1u;
    const uint32_t n = static_cast<uint32_t>(g() & 0x7fffffffu);
    ok = apply(n, pmlb::make_fastdiv(d)) == n / d;
  }
  check(ok, "fastdiv random");
  const uint32_t edge[] = {1u, 2u, 3u, 0x40000000u, 0x40000001u, 0x7fffffffu};
  ok = true;
  for (uint32_t d : edge) {
    for (uint32_t n : {0u, 1u, d - 1u, d, d + 1u, 0x7ffffffeu, 0x7fffffffu}) {
      if (n <= 0x7fffffffu) ok = ok && apply(n, pmlb::make_fastdiv(d)) == n / d;
    }
  }
  check(ok, "fastdiv edges");

  // routes of ResNet-50's convolutions
  check(pmlb::conv_takes_s2d(conv(256, 224, 224, 3, 7, 7, 64, 2, 3, PMLB_EPI_BIAS | PMLB_EPI_RELU)), "7x7/2 on 3 channels: space to depth");
  check(!pmlb::conv_takes_s2d(conv(2, 33, 45, 4, 5, 5, 48, 2, 2)), "output width 23: not space to depth");
  check(pmlb::conv_takes_packed_rows(conv(2, 33, 45, 4, 5, 5, 48, 2, 2)), "... but packed rows");
  check(!pmlb::conv_takes_s2d(conv(2, 20, 20, 3, 3, 3, 64, 2, 1, PMLB_EPI_RESIDUAL)), "residual input: not space to depth");
  check(!pmlb::conv_takes_s2d(conv(2, 64, 64, 8, 3, 3, 64, 2, 1)), "8 channels: not space to depth");
  check(!pmlb::conv_takes_s2d(conv(1, 1024, 1024, 3, 7, 7, 64, 2, 3)), "1024-wide rows: tile buffers do not fit");
  check(pmlb::conv_takes_halo(conv(256, 56, 56, 64, 3, 3, 64, 1, 1)), "3x3 64 -> 64 at 56x56: halo rows");
  check(!pmlb::conv_takes_halo(conv(256, 28, 28, 128, 3, 3, 128, 1, 1)), "128 output channels: im2col");
  check(!pmlb::conv_takes_halo(conv(256, 56, 56, 64, 3, 3, 64, 2, 1)), "stride 2: im2col");
  check(!pmlb::conv_takes_halo(conv(4, 7, 7, 64, 3, 3, 64, 1, 1)), "7x7 image: too few real rows per tile");
  // shapes of the space-to-depth form
  {
    const pmlb::S2dShape g = pmlb::conv_s2d_shape(conv(256, 224, 224, 3, 7, 7, 64, 2, 3));
    check(g.pe_h == 4 && g.dh == 1 && g.r2 == 4 && g.s2 == 4 && g.h2 == 115 && g.wp == 128 && g.stage_px == 928,
          "7x7/2 pad 3 -> 4x4 taps, 115 rows of 128 pixels, 928 pixels per tile");
    const pmlb::S2dShape e = pmlb::conv_s2d_shape(conv(2, 20, 22, 2, 4, 2, 16, 2, 1));
    check(e.pe_h == 2 && e.dh == 1 && e.r2 == 3 && e.s2 == 2 && e.wp % 32 == 0 && e.stage_px % 32 == 0, "even filter, odd padding");
  }
  return failures == 0 ? 0 : 1;
}
