"""The reference's own test cases for gather / scatter / argsort / prng (tests/golden/reference_special_kats.json,
extracted from plaidml/edsl/tests/edsl_test.cc by tests/golden/make_special_kats.py), with what each test builds.

Shared by the CPU test that pins the oracle to them and the GPU tests that run the same cases on the device."""

import json
from pathlib import Path

import numpy as np

from oracle import special as S

KATS = json.loads((Path(__file__).resolve().parent / "golden" / "reference_special_kats.json").read_text())
NP = {"FLOAT16": np.float16, "FLOAT32": np.float32, "FLOAT64": np.float64, "INT32": np.int32, "UINT32": np.uint32}

# name -> (operation, keyword arguments, tolerance or None for exact); the cited line is the one that builds the op
CASES = {
    "Gather": ("gather", dict(axis=1), None),                                                            # :1493
    "InterpolatedGatherNearest": ("gather", dict(axis=1, interpolation=S.NEAREST, nearest=S.ROUND_PREFER_CEIL), None),  # :1513
    "InterpolatedGatherLinear": ("gather", dict(axis=-1, interpolation=S.LINEAR), None),                # :1526
    "InterpolatedGatherLinearOutOfBoundsReturnZero":
        ("gather", dict(axis=-1, interpolation=S.LINEAR, out_of_bounds=S.RETURN_ZERO), None),           # :1538
    "InterpolatedGatherCubic": ("gather", dict(axis=1, interpolation=S.CUBIC, cube_coeff=-0.5), 1e-5),  # :1551
    "InterpolatedGatherCubicOutOfBoundsReturnZero":
        ("gather", dict(axis=1, interpolation=S.CUBIC, cube_coeff=-0.5, out_of_bounds=S.RETURN_ZERO), 1e-5),  # :1564
    "InterpolatedGatherCubicDouble": ("gather", dict(axis=1, interpolation=S.CUBIC, cube_coeff=-0.5), 1e-5),  # :1581
    "InterpolatedGatherCubicHalf": ("gather", dict(axis=1, interpolation=S.CUBIC, cube_coeff=-0.5), 1e-2),    # :1594
    "InterpolatedGatherMultiDIndices": ("gather", dict(axis=1, interpolation=S.NEAREST), None),         # :1620
    "GatherND": ("gather_nd", dict(batch_dims=0), None),                                                # :1665
    "GatherNDWithBatchDims": ("gather_nd", dict(batch_dims=2), None),                                   # :1689
    "Scatter1D": ("scatter", dict(axis=0, mode=S.SCATTER_ADD), None),                                   # :1878
    "Scatter3D": ("scatter", dict(axis=0, mode=S.SCATTER_ADD), None),
    "ScatterDup1D": ("scatter", dict(axis=0, mode=S.SCATTER_ADD), None),
    "ScatterDup3D": ("scatter", dict(axis=0, mode=S.SCATTER_ADD), None),
    "Scatter1DUpdateSlice": ("scatter", dict(axis=0, mode=S.SCATTER_SLICE), None),                      # :1966
    "Scatter3DUpdateSlice": ("scatter", dict(axis=0, mode=S.SCATTER_SLICE), None),
    "ScatterNDUpdateSlice": ("scatter", dict(axis=0, mode=S.SCATTER_ND), None),                         # :2010
    "ScatterNDUpdateSlice2": ("scatter", dict(axis=0, mode=S.SCATTER_ND), None),
    "ScatterNDUpdateSlice3": ("scatter", dict(axis=0, mode=S.SCATTER_ND), None),
    "ScatterElt": ("scatter", dict(axis=1, mode=S.SCATTER_ELT), None),                                  # :2084
    "ArgSort1d": ("argsort", dict(axis=0, descending=False), None),
    "ArgSort1dInt": ("argsort", dict(axis=0, descending=False), None),
    "ArgSort1dDup": ("argsort", dict(axis=0, descending=False), None),
    "ArgSort2dAxis0": ("argsort", dict(axis=0, descending=False), None),
    "ArgSort2dAxis1": ("argsort", dict(axis=1, descending=False), None),
    "ArgSort3dAxis0Asc": ("argsort", dict(axis=0, descending=False), None),
    "ArgSort3dAxis2Desc": ("argsort", dict(axis=2, descending=True), None),
    "ArgSort3dAxisNeg2Asc": ("argsort", dict(axis=-2, descending=False), None),
    "Prng": ("prng", dict(dims=[2, 3]), 1e-5),                                                          # :1141
}

_INPUT_NAMES = {"gather": ("in1", "in2"), "gather_nd": ("in1", "in2"), "scatter": ("data", "indices", "updates"),
                "argsort": ("input",), "prng": ("state",)}
_HOLDERS = {"gather": ("A", "B"), "gather_nd": ("A", "B"), "scatter": ("D", "I", "U"), "argsort": ("I",)}
_EXPECTED = {"gather": "out", "gather_nd": "out", "scatter": "expected", "argsort": "output"}


def inputs(name):
    """The test's input arrays in operand order."""
    kind = CASES[name][0]
    kat = KATS[name]
    if kind == "prng":
        return [np.array(kat["vectors"]["state"], dtype=np.uint32).reshape(1, 3)]
    arrays = []
    for vec, holder in zip(_INPUT_NAMES[kind], _HOLDERS[kind]):
        ph = kat["placeholders"][holder]
        arrays.append(np.array(kat["vectors"][vec], dtype=np.float64).astype(NP[ph["dtype"]]).reshape(ph["shape"]))
    return arrays


def expected(name):
    """The expected outputs the test states, flat (the reference compares buffers element by element)."""
    kind = CASES[name][0]
    v = KATS[name]["vectors"]
    if kind == "prng":
        return [np.array(v["result"], dtype=np.float32), np.array(v["new_state"], dtype=np.uint32)]
    return [np.array(v[_EXPECTED[kind]], dtype=np.float64)]


def run_oracle(name):
    kind, kw, _ = CASES[name]
    ins = inputs(name)
    if kind == "gather":
        return [S.gather(ins[0], ins[1], **kw)]
    if kind == "gather_nd":
        return [S.gather_nd(ins[0], ins[1], **kw)]
    if kind == "scatter":
        return [S.scatter(ins[0], ins[1], ins[2], **kw)]
    if kind == "argsort":
        return [S.argsort(ins[0], **kw)]
    numbers, state = S.prng(ins[0], int(np.prod(kw["dims"])))
    return [numbers.reshape(kw["dims"]), state]


def check(name, got):
    """Applies the test's own comparison: element-wise equality in the result's type, or closeness at its tolerance."""
    tol = CASES[name][2]
    for g, want in zip(got, expected(name)):
        g = np.asarray(g).reshape(-1)
        assert g.shape == want.reshape(-1).shape, (name, g.shape, want.shape)
        if tol is None:
            np.testing.assert_array_equal(g, want.reshape(-1).astype(g.dtype), err_msg=name)
        else:
            np.testing.assert_allclose(g.astype(np.float64), want.reshape(-1).astype(np.float64), rtol=tol, atol=tol,
                                       err_msg=name)
