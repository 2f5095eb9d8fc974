"""Pins the CPU oracle against the known-answer vectors of the reference's own tests
(tests/golden/reference_kats.json, extracted by tests/golden/make_reference_kats.py).

Each contraction is written here by hand as an index-box descriptor, independently of this
library's EDSL front-end, and evaluated by the oracle's definition-order walker."""

import json
from pathlib import Path

import numpy as np
import pytest

import oracle
from plaidml_b200 import kernels as K

KATS = {k["name"]: k for k in json.loads((Path(__file__).parent / "golden" / "reference_kats.json").read_text())}
XSMM = {k["name"]: k for k in json.loads((Path(__file__).parent / "golden" / "reference_xsmm_kats.json").read_text())}

NP = {"INT64": (np.int64, K.I64), "UINT64": (np.uint64, K.U64), "INT32": (np.int32, K.I32), "INT8": (np.int8, K.I8),
      "FLOAT32": (np.float32, K.F32)}


def contract(desc, srcs, out_shape, np_dtype, init=None):
    out = np.zeros(out_shape, dtype=np_dtype)
    oracle.contract(desc, [np.ascontiguousarray(s) for s in srcs], init, out)
    return out


@pytest.mark.parametrize("name", ["GEMM_INT64", "GEMM_UINT64", "GEMM_INT32", "GEMM_INT8", "GEMM_FLOAT32"])
def test_gemm_known_answers(name):
    kat = KATS[name]
    npdt, dt = NP[kat["dtype"]]
    a, b, c = (np.array(v, dtype=npdt).reshape(3, 3) for v in kat["inputs"])
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_MUL, 3, 2
    d.range[0] = d.range[1] = d.range[2] = 3
    d.out = K.make_access(dt, [3, 3], [{0: 1}, {1: 1}])
    d.src[0] = K.make_access(dt, [3, 3], [{0: 1}, {2: 1}])
    d.src[1] = K.make_access(dt, [3, 3], [{2: 1}, {1: 1}])
    got = contract(d, [a, b], (3, 3), npdt) + c
    want = np.array(kat["outputs"][0], dtype=npdt).reshape(3, 3)
    if npdt == np.float32:
        # the reference compares its own backend's floats exactly; a different (but valid) order
        # of the three additions may differ in the last bit
        np.testing.assert_allclose(got, want, rtol=2e-7)
    else:
        np.testing.assert_array_equal(got.astype(npdt), want)


def test_row_max_known_answer():
    kat = KATS["Max"]
    a = np.array(kat["inputs"][0], dtype=np.float32).reshape(3, 3)
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_MAX, K.COMBO_NONE, 2, 1
    d.range[0] = d.range[1] = 3
    d.out = K.make_access(K.F32, [3], [{0: 1}])
    d.src[0] = K.make_access(K.F32, [3, 3], [{0: 1}, {1: 1}])
    np.testing.assert_array_equal(contract(d, [a], (3,), np.float32), np.array(kat["outputs"][0], dtype=np.float32))


def test_defract_known_answers():
    # O[i] += I[(i - j + 1) / 2] * K[j]: only integral index values contribute
    kat = KATS["test_defract"]
    i_in, k_in = (np.array(v, dtype=np.float32) for v in kat["inputs"])
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_MUL, 2, 2
    d.range[0], d.range[1] = 5, 3
    d.out = K.make_access(K.F32, [5], [{0: 1}])
    d.src[0] = K.make_access(K.F32, [3], [{0: 1, 1: -1}], offs=[1], dens=[2])
    d.src[1] = K.make_access(K.F32, [3], [{1: 1}])
    np.testing.assert_array_equal(contract(d, [i_in, k_in], (5,), np.float32), np.array(kat["outputs"][0], dtype=np.float32))

    kat = KATS["test_defract_short"]
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_NONE, 1, 1
    d.range[0] = 6
    d.out = K.make_access(K.F32, [6], [{0: 1}])
    d.src[0] = K.make_access(K.F32, [3], [{0: 1}], offs=[-1], dens=[2])
    got = contract(d, [np.array(kat["inputs"][0], dtype=np.float32)], (6,), np.float32)
    np.testing.assert_array_equal(got, np.array(kat["outputs"][0], dtype=np.float32))


def test_defract_long_known_answer():
    # the transposed-convolution shaped case: I[n, (x0+k0-1)/2, (x1+k1-1)/2, ci] * K[2-k0, 2-k1, co, ci]
    kat = KATS["test_defract_long"]
    i_in = np.array(kat["inputs"][0], dtype=np.float32)
    k_in = np.array(kat["inputs"][1], dtype=np.float32)
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_MUL, 7, 2
    # variables: n, x0, x1, co, ci, k0, k1
    for v, r in enumerate([1, 5, 5, 1, 1, 3, 3]):
        d.range[v] = r
    d.out = K.make_access(K.F32, [1, 5, 5, 1], [{0: 1}, {1: 1}, {2: 1}, {3: 1}])
    d.src[0] = K.make_access(K.F32, [1, 3, 3, 1], [{0: 1}, {1: 1, 5: 1}, {2: 1, 6: 1}, {4: 1}], offs=[0, -1, -1, 0],
                             dens=[1, 2, 2, 1])
    # K really has shape [1, 3, 3, 1]: its first index 2 - k0 is in range only for k0 == 2
    d.src[1] = K.make_access(K.F32, [1, 3, 3, 1], [{5: -1}, {6: -1}, {3: 1}, {4: 1}], offs=[2, 2, 0, 0])
    got = contract(d, [i_in, k_in], (1, 5, 5, 1), np.float32)
    np.testing.assert_array_equal(got, np.array(kat["outputs"][0], dtype=np.float32))


def test_oracle_fast_paths_agree_with_walker():
    g = np.random.Generator(np.random.PCG64(7))
    a = g.standard_normal((6, 9)).astype(np.float32)
    b = g.standard_normal((9, 5)).astype(np.float32)
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_MUL, 3, 2
    d.range[0], d.range[1], d.range[2] = 6, 5, 9
    d.out = K.make_access(K.F32, [6, 5], [{0: 1}, {1: 1}])
    d.src[0] = K.make_access(K.F32, [6, 9], [{0: 1}, {2: 1}])
    d.src[1] = K.make_access(K.F32, [9, 5], [{2: 1}, {1: 1}])
    np.testing.assert_array_equal(contract(d, [a, b], (6, 5), np.float32), oracle.gemm_f32(a, b))
    ai = g.integers(-128, 128, size=(4, 7), dtype=np.int8)
    bi = g.integers(-128, 128, size=(7, 3), dtype=np.int8)
    np.testing.assert_array_equal(oracle.gemm_i8_i32(ai, bi), ai.astype(np.int32) @ bi.astype(np.int32))
    x = g.standard_normal((2, 7, 6, 3)).astype(np.float32)
    f = g.standard_normal((3, 3, 3, 4)).astype(np.float32)
    ref = oracle.conv2d_nhwc_f32(x, f, pad=(1, 1))
    xp = np.pad(x, ((0, 0), (1, 1), (1, 1), (0, 0)))
    want = np.zeros((2, 7, 6, 4), dtype=np.float64)
    for r in range(3):
        for s in range(3):
            want += np.einsum("nhwc,ck->nhwk", xp[:, r:r + 7, s:s + 6, :].astype(np.float64), f[r, s].astype(np.float64))
    np.testing.assert_allclose(ref, want, rtol=1e-5, atol=1e-5)
    pooled = oracle.pool2d_nhwc_f32(x, "max", (3, 3), (2, 2), (1, 1), (4, 3))
    xm = np.pad(x, ((0, 0), (1, 1), (1, 1), (0, 0)), constant_values=-np.inf)
    want = np.stack([[xm[:, 2 * y:2 * y + 3, 2 * xx:2 * xx + 3, :].max(axis=(1, 2)) for xx in range(3)] for y in range(4)])
    np.testing.assert_array_equal(pooled, np.transpose(want, (2, 0, 1, 3)))


def test_microkernel_dot_known_answer():
    # the 8 x 8 product printed by the reference's x86 microkernel test (integer-valued: exact in f32)
    kat = XSMM["xsmm_dot_8x8"]
    a, b = (np.array(v, dtype=np.float32) for v in kat["inputs"])
    want = np.array(kat["outputs"][0], dtype=np.float32)
    np.testing.assert_array_equal(oracle.gemm_f32(a, b), want)
    np.testing.assert_array_equal(oracle.gemm_f32_acc64(a, b), want)
    np.testing.assert_array_equal(oracle.gemm_i8_i32(a.astype(np.int8), np.clip(b, -128, 127).astype(np.int8))[:, :5],
                                  (a.astype(np.int32) @ np.clip(b, -128, 127).astype(np.int32))[:, :5])
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_MUL, 3, 2
    d.range[0] = d.range[1] = d.range[2] = 8
    d.out = K.make_access(K.F32, [8, 8], [{0: 1}, {1: 1}])
    d.src[0] = K.make_access(K.F32, [8, 8], [{0: 1}, {2: 1}])
    d.src[1] = K.make_access(K.F32, [8, 8], [{2: 1}, {1: 1}])
    np.testing.assert_array_equal(contract(d, [a, b], (8, 8), np.float32), want)


def test_microkernel_convolution_known_answer():
    # the only convolution numbers the reference's tests hold: 1x6x5x7 (*) 1x1x7x11, printed by the same test.
    # Both the convolution loop nest (which checks every convolution, pooling and ResNet test) and the index-box
    # walker must reproduce them exactly; so must the loop nest when the same filter sits in the centre of a
    # zero 3x3 one (padding 1), which exercises its out-of-range taps.
    kat = XSMM["xsmm_conv_1x1"]
    x, f = (np.array(v, dtype=np.float32) for v in kat["inputs"])
    want = np.array(kat["outputs"][0], dtype=np.float32).reshape(1, 6, 5, 11)
    assert x.shape == (1, 6, 5, 7) and f.shape == (1, 1, 7, 11)
    np.testing.assert_array_equal(oracle.conv2d_nhwc_f32(x, f), want)
    f3 = np.zeros((3, 3, 7, 11), dtype=np.float32)
    f3[1, 1] = f[0, 0]
    np.testing.assert_array_equal(oracle.conv2d_nhwc_f32(x, f3, pad=(1, 1)), want)
    bias = np.arange(11, dtype=np.float32) - 400
    np.testing.assert_array_equal(oracle.conv2d_nhwc_f32(x, f, bias, None, relu=True), np.maximum(want + bias, 0))
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_MUL, 4, 2
    for v, r in enumerate([6, 5, 7, 11]):          # x, y, ci, co
        d.range[v] = r
    d.out = K.make_access(K.F32, [1, 6, 5, 11], [{}, {0: 1}, {1: 1}, {3: 1}])
    d.src[0] = K.make_access(K.F32, [1, 6, 5, 7], [{}, {0: 1}, {1: 1}, {2: 1}])
    d.src[1] = K.make_access(K.F32, [1, 1, 7, 11], [{}, {}, {2: 1}, {3: 1}])
    np.testing.assert_array_equal(contract(d, [x, f], (1, 6, 5, 11), np.float32), want)
