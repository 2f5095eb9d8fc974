"""The contraction-built operations of the op library (plaidml/op/lib/ops.cc) run on the GPU and are
compared with numpy restatements of their definitions."""

import numpy as np
import pytest

from plaidml_b200 import op
from plaidml_b200.core import DType, Program
from plaidml_b200.edsl import Placeholder
from plaidml_b200.exec import Runner
from gpu_util import rng

pytestmark = pytest.mark.gpu


def run(build, *arrays, dtype=DType.FLOAT32):
    ins = [Placeholder(dtype, list(a.shape)) for a in arrays]
    out = build(*ins)
    outs = out if isinstance(out, (list, tuple)) else [out]
    res = Runner(Program("op", ins, list(outs)), "cuda.0").run(list(arrays))
    return res if isinstance(out, (list, tuple)) else res[0]


def test_all_any():
    x = (rng(1).integers(0, 3, size=(3, 4, 5)) > 0).astype(np.float32) * rng(2).standard_normal((3, 4, 5)).astype(np.float32)
    x[1, :, 2] = 1.0
    x[2, :, 3] = 0.0
    np.testing.assert_array_equal(run(lambda X: op.all(X, axis=1), x), np.all(x != 0, axis=1).astype(np.uint8))
    np.testing.assert_array_equal(run(lambda X: op.any(X, axis=1, keepdims=True), x),
                                  np.any(x != 0, axis=1, keepdims=True).astype(np.uint8))
    np.testing.assert_array_equal(run(lambda X: op.any(X), x), np.uint8(1))


def test_argmax_takes_the_position_of_the_maximum():
    x = rng(3).standard_normal((4, 7, 5)).astype(np.float32)
    np.testing.assert_array_equal(run(lambda X: op.argmax(X, axis=1), x), np.argmax(x, axis=1).astype(np.uint32))
    np.testing.assert_array_equal(run(lambda X: op.argmax(X), x), np.argmax(x, axis=-1).astype(np.uint32))


def test_binary_crossentropy_and_hard_sigmoid():
    g = rng(4)
    t = g.integers(0, 2, size=(6, 9)).astype(np.float32)
    p = g.uniform(0, 1, size=(6, 9)).astype(np.float32)
    p[0, 0], p[0, 1] = 0.0, 1.0
    eps = 1e-3
    pc = np.clip(p, eps, 1 - eps)
    ref = -t * np.log(pc) - (1 - t) * np.log(1 - pc)
    np.testing.assert_allclose(run(lambda T, P: op.binary_crossentropy(T, P, eps), t, p), ref, rtol=2e-5, atol=1e-6)
    x = g.uniform(-5, 5, size=(50,)).astype(np.float32)
    np.testing.assert_allclose(run(lambda X: op.hard_sigmoid(X, 0.2), x), np.clip(0.2 * x + 0.5, 0, 1), rtol=1e-6, atol=1e-7)


def test_broadcast_concatenate_repeat_tile():
    g = rng(5)
    a = g.standard_normal((3, 1)).astype(np.float32)
    np.testing.assert_array_equal(run(lambda A: op.broadcast(A, [2, 3, 5], [1, 2]), a), np.broadcast_to(a, (2, 3, 5)))
    x = g.standard_normal((2, 3, 4)).astype(np.float32)
    y = g.standard_normal((2, 5, 4)).astype(np.float32)
    np.testing.assert_array_equal(run(lambda X, Y: op.concatenate([X, Y, X], axis=1), x, y), np.concatenate([x, y, x], axis=1))
    np.testing.assert_array_equal(run(lambda X: op.repeat(X, 3, 1), x), np.repeat(x, 3, axis=1))
    np.testing.assert_array_equal(run(lambda X: op.tile(X, [2, 1, 3]), x), np.tile(x, (2, 1, 3)))


def test_cumprod():
    x = rng(6).uniform(0.5, 1.5, size=(3, 6, 2)).astype(np.float32)
    np.testing.assert_allclose(run(lambda X: op.cumprod(X, 1), x), np.cumprod(x, axis=1), rtol=1e-5)


def test_explicit_padding_constant_and_edge():
    x = rng(7).standard_normal((2, 3, 4)).astype(np.float32)
    lo, hi = [0, 1, 2], [1, 0, 3]
    pads = list(zip(lo, hi))
    np.testing.assert_array_equal(run(lambda X: op.explicit_padding(X, lo, hi, op.PadMode.CONSTANT, -1.5), x),
                                  np.pad(x, pads, mode="constant", constant_values=-1.5))
    np.testing.assert_array_equal(run(lambda X: op.explicit_padding(X, lo, hi, op.PadMode.EDGE), x), np.pad(x, pads, mode="edge"))


def test_l2norm_lrn_mvn():
    g = rng(8)
    x = g.standard_normal((2, 6, 5, 4)).astype(np.float32)
    ss = (x * x).sum(axis=(1, 2), keepdims=True)
    np.testing.assert_allclose(run(lambda X: op.l2norm(X, [1, 2], 1e-2, op.EpsMode.ADD), x), np.sqrt(ss + 1e-2), rtol=1e-5)
    np.testing.assert_allclose(run(lambda X: op.l2norm(X, [1, 2], 50.0, op.EpsMode.MAX), x), np.sqrt(np.maximum(ss, 50.0)), rtol=1e-5)
    # local response normalisation over a 3-wide window of the last axis
    sq = np.pad(x * x, [(0, 0), (0, 0), (0, 0), (1, 1)])
    win = sq[..., 0:4] + sq[..., 1:5] + sq[..., 2:6]
    np.testing.assert_allclose(run(lambda X: op.lrn(X, [3], [-1], alpha=0.1, beta=0.75, epsilon=2.0), x),
                               x / (0.1 * win + 2.0) ** 0.75, rtol=2e-5)
    mean = x.mean(axis=(2, 3), keepdims=True)
    std = np.sqrt(((x - mean) ** 2).mean(axis=(2, 3), keepdims=True))
    np.testing.assert_allclose(run(lambda X: op.mvn(X, across_channels=False, layout="NCHW"), x),
                               (x - mean) / np.maximum(std, 1e-9), rtol=1e-4, atol=1e-5)


def test_reorg_yolo_and_its_inverse():
    x = rng(9).standard_normal((2, 4, 6, 6)).astype(np.float32)
    s = 2
    n, c, h, w = x.shape
    ref = np.zeros((n, c * s * s, h // s, w // s), np.float32)
    for yy in range(s):
        for xx in range(s):
            ref[:, (xx + yy * s) * c:(xx + yy * s + 1) * c] = x[:, :, yy::s, xx::s]
    got = run(lambda X: op.reorg_yolo(X, s, False), x)
    np.testing.assert_array_equal(got, ref)
    np.testing.assert_array_equal(run(lambda X: op.reorg_yolo(X, s, True), ref), x)


def test_slice_of():
    x = rng(10).standard_normal((5, 6, 7, 8)).astype(np.float32)
    sl = [slice(None), 1, slice(None, None, -1), slice(1, 7, 2)]
    np.testing.assert_array_equal(run(lambda X: op.slice_of(X, sl), x), x[:, 1, ::-1, 1:7:2])
    sl = [slice(-3, None), -1, slice(5, 1, -2), slice(None, -2)]
    np.testing.assert_array_equal(run(lambda X: op.slice_of(X, sl), x), x[-3:, -1, 5:1:-2, :-2])


def test_scale_gradient_is_the_identity_forward():
    x = rng(11).standard_normal((3, 3)).astype(np.float32)
    np.testing.assert_array_equal(run(lambda X: op.scale_gradient(X, 0.5) + 0.0, x), x)


# ---- convolution variants that run on the general contraction kernel --------------------------------

def conv_ref(x, f, groups=1, stride=1, dil=1, ddil=1, pad=0):
    """x [n,h,w,ci], f [kh,kw,ci/groups,co] with output channel block g = co // (co_total/groups) reading input
    channel block g; data dilation inserts ddil-1 zeros between input elements."""
    n, h, w, ci = x.shape
    if ddil > 1:
        xd = np.zeros((n, (h - 1) * ddil + 1, (w - 1) * ddil + 1, ci), x.dtype)
        xd[:, ::ddil, ::ddil] = x
        x, h, w = xd, xd.shape[1], xd.shape[2]
    kh, kw, cig, co = f.shape
    xp = np.pad(x, [(0, 0), (pad, pad), (pad, pad), (0, 0)])
    p = (h + 2 * pad - dil * (kh - 1) - 1) // stride + 1
    q = (w + 2 * pad - dil * (kw - 1) - 1) // stride + 1
    out = np.zeros((n, p, q, co), np.float64)
    cog = co // groups
    for g in range(groups):
        for r in range(kh):
            for s in range(kw):
                patch = xp[:, r * dil:r * dil + (p - 1) * stride + 1:stride, s * dil:s * dil + (q - 1) * stride + 1:stride,
                           g * cig:(g + 1) * cig]
                out[..., g * cog:(g + 1) * cog] += patch.astype(np.float64) @ f[r, s, :, g * cog:(g + 1) * cog].astype(np.float64)
    return out.astype(np.float32)


def test_grouped_convolution_group_layouts():
    g = rng(20)
    x = g.standard_normal((2, 9, 9, 8)).astype(np.float32)
    groups = 2
    f = g.standard_normal((3, 3, 4, 6)).astype(np.float32)          # [kh, kw, ci/groups, co]: the IN_K layout
    ref = conv_ref(x, f, groups=groups, pad=1)
    got = run(lambda X, F: op.convolution(X, F, groups=groups, autopad_mode=op.AutoPadMode.EXPLICIT, manual_padding=[1, 1],
                                          group_layout=op.GroupLayout.IN_K, autogroup_mode=op.AutoGroupMode.EXPLICIT), x, f)
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)
    # the same filter with an explicit group dimension: [kh, kw, g, ci/g, co/g]
    f_sep = np.stack([f[:, :, :, :3], f[:, :, :, 3:]], axis=2)
    got = run(lambda X, F: op.convolution(X, F, groups=groups, autopad_mode=op.AutoPadMode.EXPLICIT, manual_padding=[1, 1],
                                          filter_layout=op.TensorLayout.XGCK, group_layout=op.GroupLayout.SEPARATE,
                                          autogroup_mode=op.AutoGroupMode.AUTO), x, f_sep)
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)
    # groups folded into the filter's input-channel dimension: [kh, kw, ci, co/g], block g of ci belongs to group g
    f_inc = np.concatenate([f[:, :, :, :3], f[:, :, :, 3:]], axis=2)
    got = run(lambda X, F: op.convolution(X, F, groups=groups, autopad_mode=op.AutoPadMode.EXPLICIT, manual_padding=[1, 1],
                                          group_layout=op.GroupLayout.IN_C, autogroup_mode=op.AutoGroupMode.EXPLICIT), x, f_inc)
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)


def test_depthwise_convolution():
    g = rng(21)
    x = g.standard_normal((2, 10, 10, 6)).astype(np.float32)
    f = g.standard_normal((3, 3, 1, 12)).astype(np.float32)         # channel multiplier 2
    ref = conv_ref(x, f, groups=6, pad=1)
    got = run(lambda X, F: op.convolution(X, F, autopad_mode=op.AutoPadMode.EXPLICIT, manual_padding=[1, 1],
                                          group_layout=op.GroupLayout.IN_K, autogroup_mode=op.AutoGroupMode.DEPTHWISE), x, f)
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)


def test_dilated_strided_and_data_dilated_convolutions():
    g = rng(22)
    x = g.standard_normal((1, 12, 12, 4)).astype(np.float32)
    f = g.standard_normal((3, 3, 4, 5)).astype(np.float32)
    got = run(lambda X, F: op.convolution(X, F, strides=[2, 2], dilations=[2, 2], autopad_mode=op.AutoPadMode.EXPLICIT,
                                          manual_padding=[2, 2]), x, f)
    np.testing.assert_allclose(got, conv_ref(x, f, stride=2, dil=2, pad=2), rtol=1e-4, atol=1e-5)
    # data dilation (the forward form of a transposed convolution): only taps that land on an input element count
    got = run(lambda X, F: op.convolution(X, F, data_dilations=[2, 2], autopad_mode=op.AutoPadMode.EXPLICIT,
                                          manual_padding=[1, 1]), x, f)
    np.testing.assert_allclose(got, conv_ref(x, f, ddil=2, pad=1), rtol=1e-4, atol=1e-5)


def resize_ref(x, fh, fw, h_axis):
    """Bilinear image_resize as the op library defines it (plaidml/op/lib/ops.cc:1873-1912): every input
    pixel spreads a (2 fh - 1) x (2 fw - 1) triangle, centred on output position (fh * y, fw * x), over a zero background."""
    def ramp(f):
        return np.array([min(y + 1, 2 * f - 1 - y) for y in range(2 * f - 1)], np.float64) * np.float64(np.float32(1.0 / f))
    kern = np.float32(ramp(fh))[:, None].astype(np.float64) * np.float32(ramp(fw))[None, :].astype(np.float64)
    kern = kern.astype(np.float32).astype(np.float64)
    x = np.moveaxis(x.astype(np.float64), (h_axis, h_axis + 1), (-2, -1))
    h, w = x.shape[-2:]
    out = np.zeros(x.shape[:-2] + (fh * h, fw * w))
    for y in range(h):
        for xx in range(w):
            for j in range(2 * fh - 1):
                for i in range(2 * fw - 1):
                    oy, ox = fh * y + j - fh + 1, fw * xx + i - fw + 1
                    if 0 <= oy < fh * h and 0 <= ox < fw * w:
                        out[..., oy, ox] += x[..., y, xx] * kern[j, i]
    return np.moveaxis(out, (-2, -1), (h_axis, h_axis + 1)).astype(np.float32)


def test_image_resize_nearest_and_bilinear_in_both_layouts():
    g = rng(31)
    x = g.standard_normal((2, 5, 7, 3)).astype(np.float32)
    got = run(lambda X: op.image_resize(X, [2, 3], op.InterpolationMode.NEAREST, op.TensorLayout.NXC), x)
    np.testing.assert_array_equal(got, np.repeat(np.repeat(x, 2, axis=1), 3, axis=2))
    got = run(lambda X: op.image_resize(X, [3, 2], op.InterpolationMode.NEAREST, op.TensorLayout.NCX), x)
    np.testing.assert_array_equal(got, np.repeat(np.repeat(x, 3, axis=2), 2, axis=3))
    for fh, fw in ((2, 2), (2, 3), (1, 4), (3, 1)):
        got = run(lambda X: op.image_resize(X, [fh, fw], op.InterpolationMode.BILINEAR, op.TensorLayout.NXC), x)
        assert got.shape == (2, 5 * fh, 7 * fw, 3)
        np.testing.assert_allclose(got, resize_ref(x, fh, fw, 1), rtol=1e-5, atol=1e-6)
        got = run(lambda X: op.image_resize(X, [fh, fw], op.InterpolationMode.BILINEAR, op.TensorLayout.NCX), x)
        assert got.shape == (2, 5, 7 * fh, 3 * fw)
        np.testing.assert_allclose(got, resize_ref(x, fh, fw, 2), rtol=1e-5, atol=1e-6)
    # a constant image stays constant away from the zero-padded far edge (the triangles sum to one)
    ones = np.ones((1, 4, 4, 1), np.float32)
    got = run(lambda X: op.image_resize(X, [2, 2], op.InterpolationMode.BILINEAR, op.TensorLayout.NXC), ones)
    np.testing.assert_allclose(got[0, :7, :7, 0], 1.0, rtol=1e-6)
    np.testing.assert_allclose(got[0, 7, :7, 0], 0.5, rtol=1e-6)
