"""Parity of the implicit-GEMM (im2col TMA) convolution kernel with the CPU oracle."""

import numpy as np
import pytest

import oracle
from plaidml_b200 import kernels as K
from gpu_util import as_f32, check_close, dev, dev_bf16, empty, ptr, rng

pytestmark = pytest.mark.gpu


def out_size(i, f, s, pad_before, pad_after, d=1):
    return (i + pad_before + pad_after - d * (f - 1) - 1) // s + 1


def run_conv(seed, n, h, w, c, r, s, k, stride=1, pad=None, out_dtype=K.F32, epilogue=0, tile_n=0, dil=1,
             same_upper=False, flags=0):
    g = rng(seed)
    if pad is None:
        pad = (r - 1) // 2
    if same_upper:
        # SAME_UPPER of plaidml/op/lib/ops.cc:347-382: out = ceil(in / stride), the odd pad goes after
        p, q = -(-h // stride), -(-w // stride)
        pad_h = max(0, (p - 1) * stride + r - h) // 2
        pad_w = max(0, (q - 1) * stride + s - w) // 2
    else:
        pad_h = pad_w = pad
        p = out_size(h, r, stride, pad, pad, dil)
        q = out_size(w, s, stride, pad, pad, dil)
    x = dev_bf16(g.uniform(0, 1, size=(n, h, w, c)))
    f32 = (g.standard_normal((r, s, c, k)) * np.sqrt(2.0 / (r * s * c))).astype(np.float32)
    f_bf = oracle.bf16_to_f32(oracle.f32_to_bf16(f32))
    bias = g.standard_normal(k).astype(np.float32) if epilogue & K.EPI_BIAS else None
    res = dev_bf16(g.standard_normal((n, p, q, k))) if epilogue & K.EPI_RESIDUAL and out_dtype == K.BF16 else None
    if epilogue & K.EPI_RESIDUAL and out_dtype == K.F32:
        res = dev(g.standard_normal((n, p, q, k)).astype(np.float32))
    d = K.ConvDesc()
    d.in_dtype, d.out_dtype = K.BF16, out_dtype
    d.n, d.h, d.w, d.c, d.r, d.s, d.k, d.p, d.q = n, h, w, c, r, s, k, p, q
    d.stride_h = d.stride_w = stride
    d.pad_h, d.pad_w = pad_h, pad_w
    d.dil_h = d.dil_w = dil
    d.epilogue, d.tile_n, d.flags = epilogue, tile_n, flags
    plan = K.Plan("conv", d)
    f_dev = dev(f32)
    plan.set_filter(ptr(f_dev), K.F32)
    out = empty((n, p, q, k), out_dtype)
    out.fill_(0)
    bias_dev = dev(bias) if bias is not None else None
    plan.conv(ptr(x), ptr(out), ptr(bias_dev), ptr(res))
    plan.check()
    ref = oracle.conv2d_nhwc_f32(as_f32(x), f_bf, bias, None if res is None else as_f32(res), (stride, stride),
                                 (pad_h, pad_w), (dil, dil), bool(epilogue & K.EPI_RELU), out_hw=(p, q))
    return as_f32(out), ref, plan


def test_conv1x1():
    out, ref, plan = run_conv(1, 2, 16, 16, 64, 1, 1, 64)
    assert plan.kernel == "tc_conv"
    check_close(out, ref, 1e-4)


def test_conv3x3_same_small():
    out, ref, _ = run_conv(2, 2, 16, 16, 64, 3, 3, 64)
    check_close(out, ref, 1e-4)


def test_conv3x3_56x56_reference_layer():
    # the layer of plaidml/edsl/tests/edsl_test.cc:685-712: 1x56x56x64 (*) 3x3x64x64, same padding
    out, ref, _ = run_conv(3, 1, 56, 56, 64, 3, 3, 64)
    check_close(out, ref, 1e-4)


def test_conv3x3_bias_relu_bf16_out():
    out, ref, _ = run_conv(4, 4, 28, 28, 128, 3, 3, 128, out_dtype=K.BF16, epilogue=K.EPI_BIAS | K.EPI_RELU)
    check_close(out, oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)


def test_conv3x3_stride2():
    out, ref, _ = run_conv(5, 2, 28, 28, 64, 3, 3, 128, stride=2)
    check_close(out, ref, 1e-4)


def test_conv3x3_stride2_same_upper():
    out, ref, _ = run_conv(6, 2, 28, 28, 64, 3, 3, 64, stride=2, same_upper=True)
    check_close(out, ref, 1e-4)


def test_conv1x1_stride2_residual_relu():
    out, ref, _ = run_conv(7, 2, 28, 28, 128, 1, 1, 256, stride=2, pad=0, out_dtype=K.BF16,
                           epilogue=K.EPI_BIAS | K.EPI_RESIDUAL | K.EPI_RELU)
    check_close(out, oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)


def test_conv_channels_not_multiple_of_block():
    # 32 and 96 input channels: the last (only) channel block is partly out of range
    out, ref, _ = run_conv(8, 2, 14, 14, 32, 3, 3, 64)
    check_close(out, ref, 1e-4)
    out, ref, _ = run_conv(9, 2, 14, 14, 96, 3, 3, 48)
    check_close(out, ref, 1e-4)


def test_conv7x7_stride2_pad3():
    out, ref, _ = run_conv(10, 2, 32, 32, 8, 7, 7, 64, stride=2, pad=3)
    check_close(out, ref, 1e-4)


def test_conv_small_tensor_below_128k():
    # activation tensor smaller than 128 KiB
    out, ref, _ = run_conv(11, 1, 8, 8, 64, 3, 3, 64)
    check_close(out, ref, 1e-4)


def test_conv_dilated():
    out, ref, _ = run_conv(12, 2, 20, 20, 64, 3, 3, 64, pad=2, dil=2)
    check_close(out, ref, 1e-4)


def test_conv_rejects_odd_channels():
    d = K.ConvDesc()
    d.in_dtype, d.out_dtype = K.BF16, K.F32
    # 36 channels: not whole 16-byte groups, and too many for the packed-row route
    d.n, d.h, d.w, d.c, d.r, d.s, d.k, d.p, d.q = 1, 8, 8, 36, 3, 3, 8, 8, 8
    d.stride_h = d.stride_w = d.dil_h = d.dil_w = 1
    d.pad_h = d.pad_w = 1
    with pytest.raises(K.KernelError) as e:
        K.Plan("conv", d)
    assert e.value.status == K.ERR_UNSUPPORTED


# --- CTA pairs on the im2col route (two CTAs per 256-pixel tile, each fetching half of the weights) ---

@pytest.mark.parametrize("case", [
    dict(n=3, h=20, w=20, c=128, r=3, s=3, k=128),                    # 128-wide tiles; 1200 pixels: ragged last pair
    dict(n=5, h=14, w=14, c=256, r=3, s=3, k=256),                    # 256-wide tiles
    dict(n=2, h=9, w=11, c=64, r=3, s=3, k=512, stride=2),            # two column tiles, stride 2, 60 pixels (one CTA idle)
    dict(n=40, h=14, w=14, c=128, r=3, s=3, k=384),                   # 31 pair tiles x 2 column tiles, last one half-width
], ids=["n128", "n256", "stride2", "ragged_n"])
def test_conv_cta_pairs_match_oracle_and_single_ctas(case):
    pairs, ref, _ = run_conv(95, flags=K.CONV_CTA_PAIRS, **case)
    check_close(pairs, ref, 1e-4)
    single, _, _ = run_conv(95, flags=K.CONV_NO_CTA_PAIRS, **case)
    check_close(pairs, single, 1e-5)


def test_conv_cta_pairs_bf16_epilogue_and_default_choice():
    out, ref, _ = run_conv(96, 7, 7, 7, 512, 3, 3, 512, out_dtype=K.BF16, epilogue=K.EPI_BIAS | K.EPI_RELU,
                           flags=K.CONV_CTA_PAIRS)
    check_close(out, oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)
    # large enough for the library to pair CTAs by itself (74 pair tiles and more)
    out, ref, _ = run_conv(97, 24, 28, 28, 128, 3, 3, 128, out_dtype=K.BF16, epilogue=K.EPI_BIAS | K.EPI_RESIDUAL | K.EPI_RELU)
    check_close(out, oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)


# --- packed-row route (thin inputs: the first layer of image networks) -------------------------

def test_stem_conv7x7_stride2_three_channels():
    # ResNet's first layer at a small size: 3 input channels (no 16-byte channel groups), 7x7 / 2, pad 3
    out, ref, plan = run_conv(30, 3, 40, 40, 3, 7, 7, 64, stride=2, pad=3, out_dtype=K.BF16,
                              epilogue=K.EPI_BIAS | K.EPI_RELU, flags=K.CONV_NO_S2D)
    assert plan.kernel == "tc_conv_rows"
    check_close(out, oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)


def test_stem_conv_matches_im2col_route():
    # 8 channels take either route; more tiles than SMs so that CTAs slide their row windows and wrap the ring
    args = dict(n=5, h=70, w=36, c=8, r=7, s=7, k=64, stride=2, pad=3)
    rows, ref, plan = run_conv(31, **args)
    assert plan.kernel == "tc_conv_rows"
    check_close(rows, ref, 1e-4)
    im2col, _, plan2 = run_conv(31, flags=K.CONV_NO_PACKED_ROWS, **args)
    assert plan2.kernel == "tc_conv"
    check_close(rows, im2col, 1e-5)


@pytest.mark.parametrize("case", [
    dict(n=2, h=19, w=300, c=3, r=3, s=3, k=32, stride=1, pad=1),     # q = 300: three column segments per row
    dict(n=2, h=33, w=45, c=4, r=5, s=5, k=48, stride=2, pad=2),      # q = 23 (not a multiple of 8), k < 64
    dict(n=1, h=9, w=9, c=1, r=3, s=3, k=8, stride=1, pad=0),         # one channel, no padding, tiny
    dict(n=2, h=30, w=30, c=16, r=3, s=4, k=64, stride=3, pad=1),     # 16 channels, stride = filter height
    dict(n=3, h=24, w=24, c=3, r=7, s=7, k=64, stride=2, same_upper=True),
], ids=["wide", "ragged", "tiny", "stride3", "same_upper"])
def test_packed_row_geometries(case):
    out, ref, plan = run_conv(32, flags=K.CONV_NO_S2D, **case)
    assert plan.kernel == "tc_conv_rows"
    check_close(out, ref, 1e-4)


def test_packed_rows_residual_f32_and_bf16():
    out, ref, plan = run_conv(33, 2, 20, 20, 3, 3, 3, 64, epilogue=K.EPI_RESIDUAL | K.EPI_RELU)
    assert plan.kernel == "tc_conv_rows"
    check_close(out, ref, 1e-4)
    out, ref, _ = run_conv(34, 2, 20, 20, 3, 3, 3, 64, out_dtype=K.BF16, epilogue=K.EPI_BIAS | K.EPI_RESIDUAL)
    check_close(out, oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)


# --- space-to-depth route (stride 2, at most 4 input channels: 2 x 2 phases packed as channels) ---

@pytest.mark.parametrize("case", [
    dict(n=3, h=40, w=40, c=3, r=7, s=7, k=64, stride=2, pad=3),      # ResNet's first layer at a small size
    dict(n=2, h=33, w=47, c=4, r=5, s=5, k=48, stride=2, pad=2),      # odd extents, k < 64, even padding
    dict(n=3, h=24, w=24, c=3, r=7, s=7, k=64, stride=2, same_upper=True),   # more padding after than before
    dict(n=2, h=31, w=50, c=1, r=3, s=3, k=8, stride=2, pad=0),       # one channel, no padding
    dict(n=2, h=20, w=22, c=2, r=4, s=2, k=16, stride=2, pad=1),      # even filter extents, odd padding
    dict(n=160, h=64, w=64, c=3, r=7, s=7, k=64, stride=2, pad=3),    # 640 tiles: the ring wraps several times
], ids=["stem", "ragged", "same_upper", "one_channel", "even_filter", "many"])
def test_s2d_route_matches_oracle_and_packed_rows(case):
    out, ref, plan = run_conv(80, **case)
    assert plan.kernel == "tc_conv_s2d"
    check_close(out, ref, 1e-4)
    rows, _, plan2 = run_conv(80, flags=K.CONV_NO_S2D, **case)
    assert plan2.kernel == "tc_conv_rows"
    check_close(out, rows, 1e-5)


def test_s2d_route_bias_relu_bf16_out():
    out, ref, plan = run_conv(81, 3, 40, 40, 3, 7, 7, 64, stride=2, pad=3, out_dtype=K.BF16,
                              epilogue=K.EPI_BIAS | K.EPI_RELU)
    assert plan.kernel == "tc_conv_s2d"
    check_close(out, oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)
    # a residual input, or an output width that is not a multiple of 4, is outside the route: the layer falls
    # through to packed rows
    _, _, plan = run_conv(82, 2, 20, 20, 3, 3, 3, 64, stride=2, epilogue=K.EPI_RESIDUAL)
    assert plan.kernel == "tc_conv_rows"
    out, ref, plan = run_conv(83, 2, 33, 45, 4, 5, 5, 48, stride=2, pad=2)
    assert plan.kernel == "tc_conv_rows"
    check_close(out, ref, 1e-4)


# --- halo route (stride 1, 64 output channels, weights resident) ----------------------------------

@pytest.mark.parametrize("case", [
    dict(n=3, h=56, w=56, c=64, r=3, s=3, k=64),                      # the first-stage layer: 2 image rows per tile
    dict(n=2, h=15, w=20, c=64, r=3, s=3, k=64),                      # 5 rows per tile, 15 rows: exact; 22-wide rows
    dict(n=2, h=17, w=36, c=64, r=3, s=5, k=64, pad=2),               # 3x5 taps, over-padded rows, ragged last tile
    dict(n=70, h=14, w=14, c=64, r=3, s=3, k=64),                     # more tiles than SMs
], ids=["56x56", "15x20", "3x5", "many"])
def test_halo_route_matches_oracle_and_im2col(case):
    halo, ref, plan = run_conv(70, **case)
    assert plan.kernel == "tc_conv_halo"
    check_close(halo, ref, 1e-4)
    im2col, _, plan2 = run_conv(70, flags=K.CONV_NO_HALO, **case)
    assert plan2.kernel == "tc_conv"
    check_close(halo, im2col, 1e-5)


def test_halo_route_epilogues():
    out, ref, plan = run_conv(71, 2, 28, 28, 64, 3, 3, 64, out_dtype=K.BF16, epilogue=K.EPI_BIAS | K.EPI_RESIDUAL | K.EPI_RELU)
    assert plan.kernel == "tc_conv_halo"
    check_close(out, oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)
    out, ref, plan = run_conv(72, 2, 28, 28, 64, 3, 3, 64, epilogue=K.EPI_BIAS | K.EPI_RESIDUAL)
    assert plan.kernel == "tc_conv_halo"
    check_close(out, ref, 1e-4)


@pytest.mark.parametrize("out_dtype", [K.BF16, K.F32], ids=["bf16_out", "f32_out"])
@pytest.mark.parametrize("case", [
    dict(n=5, h=56, w=56, c=64, r=3, s=3, k=64),        # two image rows per tile, more tiles than one per SM for some
    dict(n=2, h=13, w=30, c=64, r=3, s=3, k=64),        # four rows per tile, ragged last tile of an image
    dict(n=3, h=9, w=126, c=64, r=1, s=3, k=64, pad=1), # one filter row; a single image row fills a tile
    dict(n=40, h=28, w=28, c=64, r=5, s=3, k=64, pad=1),# five filter rows (rows shrink: p = 26), many tiles per CTA
], ids=["56x56", "13x30", "1x3", "5x3"])
def test_halo_columns_merged_into_n_matches_one_mma_per_tap(case, out_dtype):
    # three filter columns side by side in one 128 x 192 MMA per filter row, the shifted adds in the epilogue:
    # same numbers as one MMA per tap up to the order of three additions, and both match the oracle
    epi = K.EPI_BIAS | K.EPI_RELU
    merged, ref, plan = run_conv(74, out_dtype=out_dtype, epilogue=epi, **case)
    assert plan.kernel == "tc_conv_halo"
    per_tap, _, plan2 = run_conv(74, out_dtype=out_dtype, epilogue=epi, flags=K.CONV_NO_COLUMN_MERGE, **case)
    assert plan2.kernel == "tc_conv_halo"
    if out_dtype == K.F32:
        check_close(merged, ref, 1e-4)
        check_close(merged, per_tap, 1e-5)
    else:
        check_close(merged, oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)
        # at most one bf16 step apart where the f32 sums straddle a rounding boundary
        assert np.max(np.abs(merged - per_tap)) <= np.max(np.abs(ref)) * 2.0 ** -7


# --- IEEE half operands (PLAIDML_DATA_FLOAT16 programs): every route, f16 output packed with and without ReLU ---

@pytest.mark.parametrize("case", [
    dict(n=2, h=20, w=20, c=64, r=3, s=3, k=64, stride=1, pad=1, route="tc_conv_halo"),
    dict(n=2, h=18, w=18, c=32, r=3, s=3, k=96, stride=1, pad=1, route="tc_conv"),
    dict(n=2, h=40, w=40, c=3, r=7, s=7, k=64, stride=2, pad=3, route="tc_conv_s2d"),
    dict(n=2, h=19, w=30, c=3, r=3, s=3, k=32, stride=1, pad=1, route="tc_conv_rows"),
], ids=["halo", "im2col", "s2d", "rows"])
@pytest.mark.parametrize("relu", [False, True], ids=["linear", "relu"])
def test_conv_f16_operands_and_output(case, relu):
    import torch
    g = rng(60)
    n, h, w, c, r, s, k, stride, pad = (case[x] for x in ("n", "h", "w", "c", "r", "s", "k", "stride", "pad"))
    p, q = out_size(h, r, stride, pad, pad), out_size(w, s, stride, pad, pad)
    x16 = g.uniform(-1, 1, size=(n, h, w, c)).astype(np.float16)
    f16 = (g.standard_normal((r, s, c, k)) * np.sqrt(2.0 / (r * s * c))).astype(np.float16)
    bias = g.standard_normal(k).astype(np.float32)
    d = K.ConvDesc()
    d.in_dtype, d.out_dtype = K.F16, K.F16
    d.n, d.h, d.w, d.c, d.r, d.s, d.k, d.p, d.q = n, h, w, c, r, s, k, p, q
    d.stride_h = d.stride_w = stride
    d.pad_h = d.pad_w = pad
    d.dil_h = d.dil_w = 1
    d.epilogue = K.EPI_BIAS | (K.EPI_RELU if relu else 0)
    plan = K.Plan("conv", d)
    assert plan.kernel == case["route"]
    f_dev = dev(f16)
    plan.set_filter(ptr(f_dev), K.F16)
    x_dev, b_dev = dev(x16), dev(bias)
    out = empty((n, p, q, k), K.F16)
    plan.conv(ptr(x_dev), ptr(out), ptr(b_dev), None)
    plan.check()
    ref = oracle.conv2d_nhwc_f32(x16.astype(np.float32), f16.astype(np.float32), bias, None, (stride, stride), (pad, pad),
                                 (1, 1), relu, out_hw=(p, q))
    got = out.cpu().numpy().astype(np.float32)
    if relu:
        assert (got >= 0).all()
    check_close(got, ref.astype(np.float16).astype(np.float32), 2e-3)


def test_reference_microkernel_convolution_on_the_tensor_core_routes():
    # the reference's only printed convolution result (1x6x5x7 (*) 1x1x7x11, pmlc/target/x86/tests/xsmm_call.mlir):
    # all values are small integers, exact in bf16, so the bf16 kernels must reproduce it exactly -- as a 1x1
    # convolution, and as a 3x3 one whose centre tap is that filter (zero padding and eight zero taps) on the
    # packed-row route (which takes the seven channels as they are) and on the im2col route (whole 16-byte channel
    # groups: a zero eighth channel)
    import json
    from pathlib import Path
    kat = {k["name"]: k for k in json.loads((Path(__file__).parent / "golden" / "reference_xsmm_kats.json").read_text())}["xsmm_conv_1x1"]
    x, f = (np.array(v, dtype=np.float32) for v in kat["inputs"])
    want = np.array(kat["outputs"][0], dtype=np.float32).reshape(1, 6, 5, 11)
    for r, c, flags, route in [(1, 8, 0, "tc_conv"), (3, 7, 0, "tc_conv_rows"), (3, 8, 0, "tc_conv_rows"),
                               (3, 8, K.CONV_NO_PACKED_ROWS, "tc_conv")]:
        xc = np.zeros((1, 6, 5, c), dtype=np.float32)
        xc[..., :7] = x
        fc = np.zeros((r, r, c, 11), dtype=np.float32)
        fc[r // 2, r // 2, :7] = f[0, 0]
        d = K.ConvDesc()
        d.in_dtype, d.out_dtype = K.BF16, K.F32
        d.n, d.h, d.w, d.c, d.r, d.s, d.k, d.p, d.q = 1, 6, 5, c, r, r, 11, 6, 5
        d.stride_h = d.stride_w = d.dil_h = d.dil_w = 1
        d.pad_h = d.pad_w = r // 2
        d.flags = flags
        plan = K.Plan("conv", d)
        assert plan.kernel == route
        f_dev = dev(fc)
        plan.set_filter(ptr(f_dev), K.F32)
        x_dev = dev_bf16(xc)
        out = empty((1, 6, 5, 11), K.F32)
        plan.conv(ptr(x_dev), ptr(out), None, None)
        plan.check()
        np.testing.assert_array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("n,h,w,c,r,pad,epi", [
    (2, 32, 200, 3, 7, 3, K.EPI_BIAS | K.EPI_RELU),         # fewer tiles than SMs: one tile per CTA and lead-in tiles
    (3, 224, 224, 3, 7, 3, K.EPI_BIAS | K.EPI_RELU),        # ResNet's first layer: 84 tiles
    (200, 64, 200, 3, 7, 3, K.EPI_BIAS | K.EPI_RELU),       # 1600 tiles: runs of ~11 tiles that start inside images
    (37, 48, 208, 4, 7, 3, K.EPI_RELU),                     # four channels, no bias, 222 tiles of 104 columns
    (5, 122, 250, 1, 7, 2, K.EPI_BIAS),                     # one channel, pad 2, no ReLU (negative maxima), 124 columns
    (4, 62, 222, 3, 8, 4, K.EPI_BIAS | K.EPI_RELU),         # 8 x 8 filter
    (2, 30, 224, 3, 7, 3, 0),                               # 15 output rows: refused
    (2, 32, 32, 3, 7, 3, 0),                                # rows of 32 packed positions: refused
])
def test_first_layer_fused_with_its_max_pool(n, h, w, c, r, pad, epi):
    # the convolution's output is never written: conv + bias + ReLU + 3x3/2 max pool (pad 1) in one kernel,
    # against the oracle's convolution followed by the oracle's pool, and against the two-kernel route
    g = rng(4100 + n + h)
    s = 7 if r != 8 else 8
    p, q = out_size(h, r, 2, pad, pad, 1), out_size(w, s, 2, pad, pad, 1)
    x = dev_bf16(g.uniform(-1, 1, size=(n, h, w, c)))
    f32 = (g.standard_normal((r, s, c, 64)) * np.sqrt(2.0 / (r * s * c))).astype(np.float32)
    bias = g.standard_normal(64).astype(np.float32) if epi & K.EPI_BIAS else None
    d = K.ConvDesc()
    d.in_dtype, d.out_dtype = K.BF16, K.BF16
    d.n, d.h, d.w, d.c, d.r, d.s, d.k, d.p, d.q = n, h, w, c, r, s, 64, p, q
    d.stride_h = d.stride_w = 2
    d.pad_h = d.pad_w = pad
    d.dil_h = d.dil_w = 1
    d.epilogue, d.flags = epi, K.CONV_MAX_POOL_3X3_S2
    if p % 4 != 0 or not 96 < q + 3 <= 128:
        with pytest.raises(K.KernelError):
            K.Plan("conv", d)
        return
    plan = K.Plan("conv", d)
    assert plan.kernel == "tc_conv_s2d_pool"
    f_dev = dev(f32)
    plan.set_filter(ptr(f_dev), K.F32)
    out = empty((n, p // 2, q // 2, 64), K.BF16)
    out.fill_(float("nan"))
    bias_dev = dev(bias) if bias is not None else None
    for _ in range(2):      # (a second launch: barriers and buffers start clean every time)
        plan.conv(ptr(x), ptr(out), ptr(bias_dev), None)
        plan.check()
    conv_ref = oracle.conv2d_nhwc_f32(as_f32(x), oracle.bf16_to_f32(oracle.f32_to_bf16(f32)), bias, None, (2, 2), (pad, pad),
                                      (1, 1), bool(epi & K.EPI_RELU), out_hw=(p, q))
    conv_ref = oracle.bf16_to_f32(oracle.f32_to_bf16(conv_ref))
    ref = oracle.pool2d_nhwc_f32(conv_ref, "max", (3, 3), (2, 2), (1, 1), (p // 2, q // 2))
    got = as_f32(out)
    assert np.isfinite(got).all()
    check_close(got, ref, 1e-2)
    # the unfused route: the same convolution kernel family, then the pooling kernel; equal up to the
    # summation order of the taps (the fused kernel walks the tap columns in another order)
    d2 = K.ConvDesc()
    for fld in ("in_dtype", "out_dtype", "n", "h", "w", "c", "r", "s", "k", "p", "q", "stride_h", "stride_w", "pad_h",
                "pad_w", "dil_h", "dil_w", "epilogue"):
        setattr(d2, fld, getattr(d, fld))
    plan2 = K.Plan("conv", d2)
    plan2.set_filter(ptr(f_dev), K.F32)
    mid = empty((n, p, q, 64), K.BF16)
    plan2.conv(ptr(x), ptr(mid), ptr(bias_dev), None)
    plan2.check()
    two = oracle.pool2d_nhwc_f32(as_f32(mid), "max", (3, 3), (2, 2), (1, 1), (p // 2, q // 2))
    check_close(got, two, 1e-2)
    assert (got != two).mean() < 0.02


@pytest.mark.parametrize("n,h,w,c,r,k,stride,pad,epi", [
    (2, 14, 14, 64, 3, 64, 1, 1, K.EPI_BIAS | K.EPI_RELU),
    (3, 28, 28, 128, 3, 128, 1, 1, 0),
    (2, 56, 56, 256, 1, 512, 2, 0, K.EPI_BIAS),                 # a strided 1x1 projection
    (2, 64, 64, 3, 7, 64, 2, 3, K.EPI_BIAS | K.EPI_RELU),       # first layer: 3 channels, padded to 4
    (1, 17, 19, 20, 5, 40, 2, 2, K.EPI_RELU),                   # channels that are not a multiple of 32, odd sizes
    (2, 12, 12, 36, 3, 72, 1, 2, K.EPI_BIAS | K.EPI_RESIDUAL | K.EPI_RELU),   # residual, wide padding
    (2, 8, 8, 32, 3, 32, 2, 1, K.EPI_BIAS | K.EPI_RESIDUAL | K.EPI_RELU),     # 32 output pixels in all: one ragged tile
    (2, 8, 8, 32, 3, 32, 2, 1, K.EPI_BIAS | K.EPI_RESIDUAL),
    (2, 8, 8, 32, 3, 32, 2, 1, K.EPI_BIAS),
])
def test_fp32_convolution_on_tensor_cores(n, h, w, c, r, k, stride, pad, epi):
    # fp32 activations and filter: three TF32 products per term on the im2col route (activation and filter split into
    # high and low parts by pre-passes), f32 accumulation; against the oracle's f64-accumulated loop nest to 1e-5
    g = rng(6100 + h + c)
    p, q = out_size(h, r, stride, pad, pad, 1), out_size(w, r, stride, pad, pad, 1)
    x = g.uniform(-1, 1, size=(n, h, w, c)).astype(np.float32)
    f = (g.standard_normal((r, r, c, k)) * np.sqrt(2.0 / (r * r * c))).astype(np.float32)
    bias = g.standard_normal(k).astype(np.float32) if epi & K.EPI_BIAS else None
    res = g.standard_normal((n, p, q, k)).astype(np.float32) if epi & K.EPI_RESIDUAL else None
    d = K.ConvDesc()
    d.in_dtype, d.out_dtype = K.F32, K.F32
    d.n, d.h, d.w, d.c, d.r, d.s, d.k, d.p, d.q = n, h, w, c, r, r, k, p, q
    d.stride_h = d.stride_w = stride
    d.pad_h = d.pad_w = pad
    d.dil_h = d.dil_w = 1
    d.epilogue = epi
    plan = K.Plan("conv", d)
    assert plan.kernel == "tc_conv"
    x_dev, f_dev = dev(x), dev(f)
    plan.set_filter(ptr(f_dev), K.F32)
    out = empty((n, p, q, k), K.F32)
    out.fill_(float("nan"))
    bias_dev = dev(bias) if bias is not None else None
    res_dev = dev(res) if res is not None else None
    for _ in range(2):
        plan.conv(ptr(x_dev), ptr(out), ptr(bias_dev), ptr(res_dev))
        plan.check()
    ref = oracle.conv2d_nhwc_f32(x, f, bias, res, (stride, stride), (pad, pad), (1, 1), bool(epi & K.EPI_RELU), out_hw=(p, q))
    check_close(out.cpu().numpy(), ref, 1e-5)
