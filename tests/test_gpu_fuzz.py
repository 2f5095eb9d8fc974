"""Seeded random shapes through the kernel C ABI against the CPU oracle: GEMMs (all element types,
both B layouts, every epilogue combination, forced tile widths and CTA pairs) and convolutions (every
route the planner can pick, thin and wide inputs, strides, paddings, epilogues).  The shapes are small
enough for the oracle's loop nests; the seeds are fixed, so a failure names a reproducible case."""

import numpy as np
import pytest

import oracle
from plaidml_b200 import kernels as K
from gpu_util import as_f32, bits16, check_close, dev, dev_bf16, empty, ptr, rng

from test_gpu_conv import out_size, run_conv
from test_gpu_gemm import run_gemm

pytestmark = pytest.mark.gpu


def random_gemm_case(g):
    kind = ["bf16", "bf16", "bf16", "i8", "f32"][int(g.integers(0, 5))]
    m = int(g.integers(1, 700))
    n = int(g.integers(1, 90)) * 8            # output rows 16-byte aligned (other widths: the ragged tests)
    k = int(g.integers(1, 60)) * 16
    batch = int(g.choice([1, 1, 1, 3]))
    b_is_nk = bool(g.integers(0, 2))
    tile_n = int(g.choice([0, 0, 64, 128, 256]))
    flags = int(g.choice([0, 0, K.GEMM_CTA_PAIRS, K.GEMM_NO_CTA_PAIRS, K.GEMM_NO_TAIL_SPLIT]))
    epi = int(g.integers(0, 8))               # any subset of bias, residual, relu
    return dict(kind=kind, m=m, n=n, k=k, batch=batch, b_is_nk=b_is_nk, tile_n=tile_n, flags=flags, epi=epi)


@pytest.mark.parametrize("seed", range(100))
def test_random_gemm(seed):
    g = rng(9000 + seed)
    c = random_gemm_case(g)
    m, n, k, batch = c["m"], c["n"], c["k"], c["batch"]
    if c["kind"] == "f32":
        c["tile_n"] = c["tile_n"] if c["tile_n"] in (0, 64, 128) else 0
        c["flags"] = 0
    if c["tile_n"] == 64 and not c["b_is_nk"] and c["kind"] != "f32":
        c["tile_n"] = 0                       # (B stored [k][n] is fetched in whole 128-byte chunks of N)
    bshape = (batch, n, k) if c["b_is_nk"] else (batch, k, n)
    epi = c["epi"]
    if c["kind"] == "i8":
        a = g.integers(-128, 128, size=(batch, m, k), dtype=np.int8)
        b = g.integers(-128, 128, size=bshape, dtype=np.int8)
        bias = g.integers(-1000, 1000, size=n, dtype=np.int32) if epi & K.EPI_BIAS else None
        res = g.integers(-1000, 1000, size=(batch, m, n), dtype=np.int32) if epi & K.EPI_RESIDUAL else None
        out, _, _ = run_gemm(K.I8, K.I32, dev(a), dev(b), m, n, k, batch, c["b_is_nk"], epilogue=epi,
                             bias=None if bias is None else dev(bias), residual=None if res is None else dev(res),
                             tile_n=c["tile_n"], flags=c["flags"])
        ref = np.stack([oracle.gemm_i8_i32(a[i], b[i], c["b_is_nk"]) for i in range(batch)])
        if bias is not None:
            ref = ref + bias[None, None, :]
        if res is not None:
            ref = ref + res
        if epi & K.EPI_RELU:
            ref = np.maximum(ref, 0)
        np.testing.assert_array_equal(out.cpu().numpy(), ref.astype(np.int32), err_msg=str(c))
        return
    if c["kind"] == "f32":
        a = g.uniform(-1, 1, size=(batch, m, k)).astype(np.float32)
        b = g.uniform(-1, 1, size=bshape).astype(np.float32)
        bias = g.standard_normal(n).astype(np.float32) if epi & K.EPI_BIAS else None
        res = g.standard_normal((batch, m, n)).astype(np.float32) if epi & K.EPI_RESIDUAL else None
        out, _, _ = run_gemm(K.F32, K.F32, dev(a), dev(b), m, n, k, batch, c["b_is_nk"], epilogue=epi,
                             bias=None if bias is None else dev(bias), residual=None if res is None else dev(res),
                             tile_n=c["tile_n"], flags=c["flags"])
        ref = np.stack([oracle.gemm_f32_acc64(a[i], b[i], c["b_is_nk"]) for i in range(batch)]).astype(np.float64)
        tol = 1e-5
    else:
        a_t = dev_bf16(g.standard_normal((batch, m, k)))
        b_t = dev_bf16(g.standard_normal(bshape))
        out_dt = K.BF16 if g.integers(0, 2) else K.F32
        bias = g.standard_normal(n).astype(np.float32) if epi & K.EPI_BIAS else None
        res = None
        if epi & K.EPI_RESIDUAL:
            res = dev_bf16(g.standard_normal((batch, m, n))) if out_dt == K.BF16 else dev(
                g.standard_normal((batch, m, n)).astype(np.float32))
        out, _, _ = run_gemm(K.BF16, out_dt, a_t, b_t, m, n, k, batch, c["b_is_nk"], epilogue=epi,
                             bias=None if bias is None else dev(bias), residual=res, tile_n=c["tile_n"], flags=c["flags"])
        ref = oracle.gemm_h16_f32(bits16(a_t), bits16(b_t), False, c["b_is_nk"]).astype(np.float64)
        res = None if res is None else as_f32(res)
        tol = 1e-2 if out_dt == K.BF16 else 1e-4
    if bias is not None:
        ref = ref + bias[None, None, :]
    if res is not None:
        ref = ref + res
    if epi & K.EPI_RELU:
        ref = np.maximum(ref, 0)
    ref = ref.astype(np.float32)
    if c["kind"] == "bf16" and tol == 1e-2:
        ref = oracle.bf16_to_f32(oracle.f32_to_bf16(ref))
    try:
        check_close(as_f32(out), ref, tol)
    except AssertionError as e:
        raise AssertionError(f"{c}: {e}") from None


@pytest.mark.parametrize("seed", range(100))
def test_random_conv(seed):
    g = rng(9500 + seed)
    thin = bool(g.integers(0, 3) == 0)
    c = int(g.choice([1, 2, 3, 4])) if thin else int(g.choice([8, 16, 32, 64, 64, 128]))
    r = int(g.choice([1, 3, 3, 5, 7]))
    s = int(g.choice([3, 5, 7])) if thin else int(g.choice([1, 3, 3, 5]))
    if thin:
        r = max(r, 2)
        while s * 8 > 64:                      # a filter row of a thin input is one 64-element k-block
            s -= 2
    stride = int(g.choice([1, 1, 2]))
    pad = int(g.integers(0, (min(r, s) + 1) // 2 + 1))
    h = int(g.integers(max(r, 6), 30))
    w = int(g.integers(max(s, 6), 34))
    n = int(g.integers(1, 5))
    k = int(g.choice([8, 16, 64, 64, 96, 128])) if not thin else int(g.choice([8, 32, 64]))
    out_dtype = K.BF16 if g.integers(0, 2) else K.F32
    epi = int(g.integers(0, 8))
    flags = int(g.choice([0, 0, 0, K.CONV_NO_HALO, K.CONV_NO_S2D, K.CONV_CTA_PAIRS]))
    case = dict(n=n, h=h, w=w, c=c, r=r, s=s, k=k, stride=stride, pad=pad, out_dtype=out_dtype, epilogue=epi, flags=flags)
    out, ref, plan = run_conv(9500 + seed, **case)
    tol = 1e-4
    if out_dtype == K.BF16:
        ref = oracle.bf16_to_f32(oracle.f32_to_bf16(ref))
        tol = 1e-2
    try:
        check_close(out, ref, tol)
    except AssertionError as e:
        raise AssertionError(f"{case} on {plan.kernel}: {e}") from None


@pytest.mark.parametrize("seed", range(24))
def test_random_gemm_many_tiles_per_cta(seed):
    # several tiles per CTA: ring wrap-around, accumulator hand-over between tiles, residual requests running ahead
    # across tile boundaries, the half-width tail, CTA pairs walking more than one tile
    g = rng(9800 + seed)
    m = int(g.integers(150, 420)) * 128 + int(g.integers(0, 128))
    n = int(g.choice([64, 128, 192, 256, 512, 768, 1024]))
    k = int(g.choice([64, 128, 256, 512, 1024, 1088]))
    b_is_nk = bool(g.integers(0, 2))
    out_dt = K.BF16 if g.integers(0, 3) else K.F32
    epi = int(g.integers(0, 8))
    flags = int(g.choice([0, 0, K.GEMM_CTA_PAIRS, K.GEMM_NO_CTA_PAIRS]))
    # forced widths: 64-wide tiles (two MMA-issuing warps on alternate tiles) with main loops longer than the ring
    tile_n = int(g.choice([0, 0, 64, 64, 128])) if seed >= 12 else 0
    a_t = dev_bf16(g.standard_normal((1, m, k)))
    b_t = dev_bf16(g.standard_normal((1, n, k) if b_is_nk else (1, k, n)))
    bias = g.standard_normal(n).astype(np.float32) if epi & K.EPI_BIAS else None
    res = None
    if epi & K.EPI_RESIDUAL:
        res = dev_bf16(g.standard_normal((1, m, n))) if out_dt == K.BF16 else dev(g.standard_normal((1, m, n)).astype(np.float32))
    out, _, _ = run_gemm(K.BF16, out_dt, a_t, b_t, m, n, k, 1, b_is_nk, epilogue=epi,
                         bias=None if bias is None else dev(bias), residual=res, flags=flags, tile_n=tile_n)
    ref = oracle.gemm_h16_f32(bits16(a_t), bits16(b_t), False, b_is_nk).astype(np.float64)
    if bias is not None:
        ref = ref + bias[None, None, :]
    if res is not None:
        ref = ref + as_f32(res)
    if epi & K.EPI_RELU:
        ref = np.maximum(ref, 0)
    ref = ref.astype(np.float32)
    tol = 1e-4
    if out_dt == K.BF16:
        ref, tol = oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2
    case = dict(m=m, n=n, k=k, b_is_nk=b_is_nk, out=out_dt, epi=epi, flags=flags, tile_n=tile_n)
    try:
        check_close(as_f32(out), ref, tol)
    except AssertionError as e:
        raise AssertionError(f"{case}: {e}") from None


@pytest.mark.parametrize("seed", range(30))
def test_random_gemm_with_k_split_over_ctas(seed):
    # two passes: partial products of 2..8 slices of K as a batch, then the parts summed in order with the epilogue;
    # int8 must stay bit-exact, 16-bit inputs within the one-pass tolerances; forced on arbitrary shapes, and the
    # library's own choice on few-tile shapes
    g = rng(9700 + seed)
    kind = ["i8", "bf16", "bf16"][int(g.integers(0, 3))]
    bk = 128 if kind == "i8" else 64
    m = int(g.integers(1, 600))
    n = int(g.integers(1, 60)) * 8
    k = bk * int(g.choice([2, 3, 4, 6, 8, 12, 16, 24]))
    b_is_nk = bool(g.integers(0, 2))
    epi = int(g.integers(0, 8))
    forced = bool(g.integers(0, 3))
    flags = K.GEMM_SPLIT_K if forced else 0
    bshape = (1, n, k) if b_is_nk else (1, k, n)
    case = dict(kind=kind, m=m, n=n, k=k, b_is_nk=b_is_nk, epi=epi, forced=forced)
    if kind == "i8":
        out_dt = K.I32 if g.integers(0, 3) else K.I8
        a = g.integers(-128, 128, size=(1, m, k), dtype=np.int8)
        b = g.integers(-128, 128, size=bshape, dtype=np.int8)
        if out_dt == K.I8:
            epi &= K.EPI_RELU | K.EPI_RESIDUAL      # (a bias is 32-bit: the result would be, too)
        bias = g.integers(-1000, 1000, size=n, dtype=np.int32) if epi & K.EPI_BIAS else None
        res = None
        if epi & K.EPI_RESIDUAL:
            res = g.integers(-1000, 1000, size=(1, m, n), dtype=np.int32) if out_dt == K.I32 else g.integers(
                -128, 128, size=(1, m, n), dtype=np.int8)
        out, _, plan = run_gemm(K.I8, out_dt, dev(a), dev(b), m, n, k, 1, b_is_nk, epilogue=epi,
                                bias=None if bias is None else dev(bias), residual=None if res is None else dev(res), flags=flags)
        ref = oracle.gemm_i8_i32(a[0], b[0], b_is_nk)[None].astype(np.int64)
        if bias is not None:
            ref = ref + bias[None, None, :]
        if res is not None:
            ref = ref + res
        if out_dt == K.I8:
            ref = ref.astype(np.int8)                # wrap, then the ReLU
        if epi & K.EPI_RELU:
            ref = np.maximum(ref, 0)
        if forced and (b_is_nk or n % 16 == 0):      # (a [k][n] B whose rows are not 16-byte multiples is copied
            assert plan.split_k > 1, case            #  transposed first and keeps the one-pass route)
        np.testing.assert_array_equal(out.cpu().numpy(), ref.astype(np.int32 if out_dt == K.I32 else np.int8), err_msg=str(case))
        return
    a_t = dev_bf16(g.standard_normal((1, m, k)))
    b_t = dev_bf16(g.standard_normal(bshape))
    out_dt = K.BF16 if g.integers(0, 2) else K.F32
    bias = g.standard_normal(n).astype(np.float32) if epi & K.EPI_BIAS else None
    res = None
    if epi & K.EPI_RESIDUAL:
        res = dev_bf16(g.standard_normal((1, m, n))) if out_dt == K.BF16 else dev(g.standard_normal((1, m, n)).astype(np.float32))
    out, _, plan = run_gemm(K.BF16, out_dt, a_t, b_t, m, n, k, 1, b_is_nk, epilogue=epi,
                            bias=None if bias is None else dev(bias), residual=res, flags=flags)
    if forced:
        assert plan.split_k > 1, case
    ref = oracle.gemm_h16_f32(bits16(a_t), bits16(b_t), False, b_is_nk).astype(np.float64)
    if bias is not None:
        ref = ref + bias[None, None, :]
    if res is not None:
        ref = ref + as_f32(res)
    if epi & K.EPI_RELU:
        ref = np.maximum(ref, 0)
    ref = ref.astype(np.float32)
    tol = 1e-4
    if out_dt == K.BF16:
        ref, tol = oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2
    try:
        check_close(as_f32(out), ref, tol)
    except AssertionError as e:
        raise AssertionError(f"{case} split_k={plan.split_k}: {e}") from None


@pytest.mark.parametrize("seed", range(8))
def test_random_few_tile_long_k_gemm(seed):
    # the shapes of a sharded GEMM (a few hundred rows against a wide, deep B): the library picks 128-wide tiles or CTA
    # pairs on 256-wide ones from an operand-traffic estimate; int8 bit-exact either way
    g = rng(9750 + seed)
    m = int(g.choice([256, 384, 512, 640, 1024, 1152]))
    n = int(g.choice([1024, 2048, 4096]))
    k = int(g.choice([2048, 4096]))
    a = g.integers(-128, 128, size=(1, m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(1, k, n), dtype=np.int8)
    out, _, _ = run_gemm(K.I8, K.I32, dev(a), dev(b), m, n, k, 1, False, flags=K.GEMM_NO_SPLIT_K)
    rows = np.sort(g.choice(m, size=24, replace=False))
    np.testing.assert_array_equal(out.cpu().numpy()[0][rows], oracle.gemm_i8_i32(np.ascontiguousarray(a[0][rows]), b[0], False))
    # every row through the row-sum identity
    np.testing.assert_array_equal(out.cpu().numpy()[0].astype(np.int64).sum(axis=1),
                                  a[0].astype(np.int64) @ b[0].astype(np.int64).sum(axis=1))


@pytest.mark.parametrize("seed", range(30))
def test_random_halo_conv_with_merged_filter_columns(seed):
    # three filter columns on 64 channels into 64: two columns side by side in one MMA, the third from a shifted
    # window, the shifted add in the epilogue; image sizes, filter heights and paddings at random (row widths from
    # 6 to 126 padded positions: one to many image rows per tile, ragged last tiles, more tiles than SMs)
    g = rng(9600 + seed)
    r = int(g.choice([1, 3, 3, 3, 5]))
    pad_w = 1
    while True:     # the route wants three quarters of a tile's 128 rows to be outputs
        w = int(g.integers(4, 125))
        h = int(g.integers(max(r, 3), 40))
        pad_h = int(g.integers(0, r // 2 + 1))
        if min(128 // (w + 2), h + 2 * pad_h - r + 1) * w >= 96:
            break
    n = int(g.integers(1, 7)) if w * h < 1500 else int(g.integers(1, 3))
    out_dtype = K.BF16 if g.integers(0, 2) else K.F32
    epi = int(g.choice([0, K.EPI_BIAS, K.EPI_RELU, K.EPI_BIAS | K.EPI_RELU]))
    g2 = rng(9600 + seed)
    p, q = h + 2 * pad_h - r + 1, w + 2 * pad_w - 3 + 1
    x = dev_bf16(g2.uniform(-1, 1, size=(n, h, w, 64)))
    f32 = (g2.standard_normal((r, 3, 64, 64)) * np.sqrt(2.0 / (r * 3 * 64))).astype(np.float32)
    bias = g2.standard_normal(64).astype(np.float32) if epi & K.EPI_BIAS else None
    outs = []
    for flags in (0, K.CONV_NO_COLUMN_MERGE):
        d = K.ConvDesc()
        d.in_dtype, d.out_dtype = K.BF16, out_dtype
        d.n, d.h, d.w, d.c, d.r, d.s, d.k, d.p, d.q = n, h, w, 64, r, 3, 64, p, q
        d.stride_h = d.stride_w = d.dil_h = d.dil_w = 1
        d.pad_h, d.pad_w = pad_h, pad_w
        d.epilogue, d.flags = epi, flags
        plan = K.Plan("conv", d)
        if plan.kernel != "tc_conv_halo":
            pytest.skip(f"shape takes {plan.kernel}")
        f_dev = dev(f32)
        plan.set_filter(ptr(f_dev), K.F32)
        out = empty((n, p, q, 64), out_dtype)
        out.fill_(float("nan"))
        plan.conv(ptr(x), ptr(out), ptr(dev(bias)) if bias is not None else None, None)
        plan.check()
        outs.append(as_f32(out))
    ref = oracle.conv2d_nhwc_f32(as_f32(x), oracle.bf16_to_f32(oracle.f32_to_bf16(f32)), bias, None, (1, 1), (pad_h, pad_w),
                                 (1, 1), bool(epi & K.EPI_RELU), out_hw=(p, q))
    case = dict(n=n, h=h, w=w, r=r, pad_h=pad_h, out=out_dtype, epi=epi)
    try:
        if out_dtype == K.F32:
            check_close(outs[0], ref, 1e-4)
            check_close(outs[0], outs[1], 1e-5)
        else:
            check_close(outs[0], oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)
    except AssertionError as e:
        raise AssertionError(f"{case}: {e}") from None


@pytest.mark.parametrize("seed", range(40))
def test_random_gemm_with_a_in_two_parts(seed):
    # C = [A1 | A2] * B (+ bias, ReLU): A2 a matrix with its own row stride or an NHWC activation sampled at a stride;
    # int8 bit-exact, bf16 against the oracle on the concatenated operand
    g = rng(9800 + seed)
    kind = "i8" if seed % 4 == 0 else "bf16"
    bk = 128 if kind == "i8" else 64
    pixels = seed % 2 == 1
    k1 = bk * int(g.integers(1, 5))
    k2 = 8 * int(g.integers(1, 40)) if kind == "bf16" else 16 * int(g.integers(1, 24))
    n_cols = 8 * int(g.integers(1, 70))
    b_is_nk = bool(g.integers(0, 2))
    epi = int(g.choice([0, K.EPI_BIAS, K.EPI_RELU, K.EPI_BIAS | K.EPI_RELU])) if kind == "bf16" else 0
    d = K.GemmDesc()
    if pixels:
        stride = int(g.integers(1, 4))
        n_img, h, w = int(g.integers(1, 5)), int(g.integers(3, 30)), int(g.integers(3, 30))
        m = n_img * (-(-h // stride)) * (-(-w // stride))
        d.a2_stride, d.a2_n, d.a2_h, d.a2_w = stride, n_img, h, w
    else:
        m = int(g.integers(1, 900))
        d.lda2 = k2 + (16 if kind == "i8" else 8) * int(g.integers(0, 3))
    k = k1 + k2
    d.m, d.n, d.k, d.batch = m, n_cols, k, 1
    d.lda, d.k_first = k1, k1
    d.ldb, d.ldc = (k if b_is_nk else n_cols), n_cols
    d.stride_a, d.stride_b, d.stride_c = m * k1, n_cols * k, m * n_cols
    d.b_is_nk, d.epilogue = int(b_is_nk), epi
    d.ldr, d.stride_r = n_cols, m * n_cols
    d.flags = int(g.choice([0, 0, K.GEMM_CTA_PAIRS, K.GEMM_NO_CTA_PAIRS]))
    d.tile_n = int(g.choice([0, 0, 64, 128]))
    bshape = (n_cols, k) if b_is_nk else (k, n_cols)
    case = dict(kind=kind, m=m, n=n_cols, k1=k1, k2=k2, pixels=pixels, b_is_nk=b_is_nk, epi=epi, flags=d.flags, tile=d.tile_n)
    if kind == "i8":
        d.in_dtype, d.out_dtype = K.I8, K.I32
        a1 = g.integers(-128, 128, size=(m, k1), dtype=np.int8)
        if pixels:
            x = g.integers(-128, 128, size=(n_img, h, w, k2), dtype=np.int8)
            a2_rows, a2_dev = x[:, ::stride, ::stride, :].reshape(m, k2), dev(x)
        else:
            a2 = np.zeros((m, d.lda2), dtype=np.int8)
            a2[:, :k2] = g.integers(-128, 128, size=(m, k2), dtype=np.int8)
            a2_rows, a2_dev = a2[:, :k2], dev(a2)
        b = g.integers(-128, 128, size=bshape, dtype=np.int8)
        if not b_is_nk and n_cols % 16 != 0:
            pytest.skip("int8 B as [k][n] with rows that are not 16-byte multiples takes the transposed copy")
        plan = K.Plan("gemm", d)
        out = empty((1, m, n_cols), K.I32)
        a1d, bd = dev(a1), dev(b)
        plan.gemm_two(ptr(a1d), ptr(a2_dev), ptr(bd), ptr(out))
        plan.check()
        ref = oracle.gemm_i8_i32(np.concatenate([a1, a2_rows], axis=1), b, b_is_nk)
        np.testing.assert_array_equal(out.cpu().numpy()[0], ref, err_msg=str(case))
        return
    d.in_dtype, d.out_dtype = K.BF16, K.F32
    a1 = dev_bf16(g.standard_normal((m, k1)))
    if pixels:
        x = dev_bf16(g.standard_normal((n_img, h, w, k2)))
        a2_rows, a2_dev = bits16(x)[:, ::stride, ::stride, :].reshape(m, k2), x
    else:
        a2_host = np.zeros((m, d.lda2), dtype=np.float32)
        a2_host[:, :k2] = g.standard_normal((m, k2))
        a2_dev = dev_bf16(a2_host)
        a2_rows = bits16(a2_dev)[:, :k2]
    b = dev_bf16(g.standard_normal(bshape))
    bias = g.standard_normal(n_cols).astype(np.float32) if epi & K.EPI_BIAS else None
    plan = K.Plan("gemm", d)
    out = empty((1, m, n_cols), K.F32)
    out.fill_(float("nan"))
    bias_dev = dev(bias) if bias is not None else None
    plan.gemm_two(ptr(a1), ptr(a2_dev), ptr(b), ptr(out), ptr(bias_dev))
    plan.check()
    a_cat = np.concatenate([bits16(a1), a2_rows], axis=1)
    ref = oracle.gemm_h16_f32(a_cat[None], bits16(b)[None], False, b_is_nk)[0].astype(np.float64)
    if bias is not None:
        ref = ref + bias[None, :]
    if epi & K.EPI_RELU:
        ref = np.maximum(ref, 0)
    try:
        check_close(out.cpu().numpy()[0], ref.astype(np.float32), 1e-4)
    except AssertionError as e:
        raise AssertionError(f"{case}: {e}") from None


@pytest.mark.parametrize("seed", range(16))
def test_random_first_layer_with_fused_pool(seed):
    # 7-wide stride-2 convolutions of 1..4 channels into 64 + bias / ReLU + 3x3 / 2 max pool as one kernel: random image
    # counts and heights (runs of tiles that start inside images, fewer tiles than SMs, many tiles per CTA), widths
    # over the accepted range, both paddings; against the oracle's convolution followed by its pool
    g = rng(9900 + seed)
    c = int(g.integers(1, 5))
    pad = int(g.choice([2, 3]))
    q = 4 * int(g.integers(24, 32))                      # 96 .. 124 output columns
    w = 2 * (q - 1) + 7 - 2 * pad + int(g.integers(0, 2))
    p = 4 * int(g.integers(1, 9))
    h = 2 * (p - 1) + 7 - 2 * pad + int(g.integers(0, 2))
    n = int(g.integers(1, 40)) if p <= 12 else int(g.integers(1, 8))
    epi = int(g.choice([0, K.EPI_BIAS, K.EPI_RELU, K.EPI_BIAS | K.EPI_RELU]))
    assert out_size(h, 7, 2, pad, pad, 1) == p and out_size(w, 7, 2, pad, pad, 1) == q
    x = dev_bf16(g.uniform(-1, 1, size=(n, h, w, c)))
    f32 = (g.standard_normal((7, 7, c, 64)) * np.sqrt(2.0 / (49 * c))).astype(np.float32)
    bias = g.standard_normal(64).astype(np.float32) if epi & K.EPI_BIAS else None
    d = K.ConvDesc()
    d.in_dtype, d.out_dtype = K.BF16, K.BF16
    d.n, d.h, d.w, d.c, d.r, d.s, d.k, d.p, d.q = n, h, w, c, 7, 7, 64, p, q
    d.stride_h = d.stride_w = 2
    d.pad_h = d.pad_w = pad
    d.dil_h = d.dil_w = 1
    d.epilogue, d.flags = epi, K.CONV_MAX_POOL_3X3_S2
    plan = K.Plan("conv", d)
    assert plan.kernel == "tc_conv_s2d_pool"
    f_dev = dev(f32)
    plan.set_filter(ptr(f_dev), K.F32)
    out = empty((n, p // 2, q // 2, 64), K.BF16)
    out.fill_(float("nan"))
    bias_dev = dev(bias) if bias is not None else None
    plan.conv(ptr(x), ptr(out), ptr(bias_dev), None)
    plan.check()
    conv_ref = oracle.conv2d_nhwc_f32(as_f32(x), oracle.bf16_to_f32(oracle.f32_to_bf16(f32)), bias, None, (2, 2), (pad, pad),
                                      (1, 1), bool(epi & K.EPI_RELU), out_hw=(p, q))
    conv_ref = oracle.bf16_to_f32(oracle.f32_to_bf16(conv_ref))
    ref = oracle.pool2d_nhwc_f32(conv_ref, "max", (3, 3), (2, 2), (1, 1), (p // 2, q // 2))
    case = dict(n=n, h=h, w=w, c=c, pad=pad, epi=epi)
    try:
        check_close(as_f32(out), ref, 1e-2)
    except AssertionError as e:
        raise AssertionError(f"{case}: {e}") from None


@pytest.mark.parametrize("seed", range(40))
def test_random_pool(seed):
    # NHWC pooling: the packed two-wide max / min kernel for 16-bit floats and the generic kernel (f32, sums,
    # averages, channel counts that are not a multiple of 8), windows, strides and paddings at random
    import torch
    from gpu_util import empty, ptr
    g = rng(9900 + seed)
    dt = [K.BF16, K.BF16, K.F16, K.F32][int(g.integers(0, 4))]
    mode = ["max", "max", "min", "sum", "avg"][int(g.integers(0, 5))]
    c = int(g.choice([8, 16, 24, 64, 5, 12]))
    r, s = int(g.integers(1, 5)), int(g.integers(1, 5))
    stride = int(g.integers(1, 4))
    pad = int(g.integers(0, min(r, s)))
    n, h, w = int(g.integers(1, 4)), int(g.integers(max(r, 4), 20)), int(g.integers(max(s, 4), 24))
    p, q = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - s) // stride + 1
    x = g.standard_normal((n, h, w, c)).astype(np.float32)
    if dt == K.F32:
        xd = dev(x)
    elif dt == K.BF16:
        xd = dev_bf16(x)
    else:
        xd = dev(x.astype(np.float16))
    d = K.PoolDesc()
    d.agg = {"max": K.AGG_MAX, "min": K.AGG_MIN, "sum": K.AGG_SUM, "avg": K.AGG_SUM}[mode]
    d.dtype = dt
    d.n, d.h, d.w, d.c, d.r, d.s, d.p, d.q = n, h, w, c, r, s, p, q
    d.stride_h = d.stride_w = stride
    d.pad_h = d.pad_w = pad
    d.average = int(mode == "avg")
    d.include_padding = int(g.integers(0, 2)) if mode == "avg" else 0
    plan = K.Plan("pool", d)
    out = empty((n, p, q, c), dt)
    plan.pool(ptr(xd), ptr(out))
    torch.cuda.synchronize()
    ref = oracle.pool2d_nhwc_f32(as_f32(xd), "sum" if mode == "avg" else mode, (r, s), (stride, stride), (pad, pad), (p, q),
                                 average=mode == "avg", include_padding=bool(d.include_padding))
    case = dict(dt=dt, mode=mode, n=n, h=h, w=w, c=c, r=r, s=s, stride=stride, pad=pad)
    got = as_f32(out)
    # a window that lies wholly in the padding has no tap: both sides leave the aggregation's identity there
    finite = np.isfinite(ref)
    assert np.array_equal(np.isfinite(got), finite), case
    if mode in ("max", "min"):
        np.testing.assert_array_equal(got[finite], ref[finite], err_msg=str(case))      # exact: no arithmetic
    else:
        tol = 1e-5 if dt == K.F32 else 1e-2
        if dt != K.F32:
            ref = oracle.bf16_to_f32(oracle.f32_to_bf16(ref)) if dt == K.BF16 else ref.astype(np.float16).astype(np.float32)
        try:
            check_close(got, ref, tol)
        except AssertionError as e:
            raise AssertionError(f"{case}: {e}") from None
