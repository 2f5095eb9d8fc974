"""EDSL programs shared by the CPU (build-only) and GPU (run) tests.  Each builder restates a
program of the reference's own test-suite with this library's Python EDSL."""

import numpy as np

from plaidml_b200 import core, edsl, op
from plaidml_b200.core import DType, Program
from plaidml_b200.edsl import Contraction, Placeholder, TensorDims, TensorIndexes, cast


def gemm_plus_c(dtype: DType, shape=(3, 3)):
    """plaidml/edsl/examples/gemm.cc: O = sum_k A[i,k] * B[k,j] + C"""
    A = Placeholder(dtype, shape)
    B = Placeholder(dtype, shape)
    C = Placeholder(dtype, shape)
    I, J, Kd = TensorDims(3)
    i, j, k = TensorIndexes(3)
    A.bind_dims(I, Kd)
    B.bind_dims(Kd, J)
    O = Contraction().outShape(I, J).outAccess(i, j).sum(A[i, k] * B[k, j]).build() + C
    return Program("gemm", [A, B, C], [O])


def row_max():
    """plaidml/edsl/tests/edsl_test.cc:576-590"""
    A = Placeholder(DType.FLOAT32, [3, 3])
    I, Kd = TensorDims(2)
    i, j = TensorIndexes(2)
    A.bind_dims(I, Kd)
    R = Contraction().outShape(I).outAccess(i).max(A[i, j]).build()
    return Program("max", [A], [R])


def add(dtype=DType.FLOAT32, shape=(3, 3)):
    A = Placeholder(dtype, shape)
    B = Placeholder(dtype, shape)
    return Program("simple_add", [A, B], [A + B])


def higher_precision_constants_cc():
    """edsl_test.cc:141-157: f32 + ui64 literal stays f32, + f64 literal becomes f64"""
    A = Placeholder(DType.FLOAT32, [3, 3])
    C = A + cast(edsl.Tensor(value=1), DType.UINT64) + cast(edsl.Tensor(value=2.0), DType.FLOAT64)
    return Program("higher_precision_constants", [A], [C])


def higher_precision_constants():
    """edsl_test.py: I + 1 + 2.0 with untyped literals stays float32"""
    I = Placeholder(DType.FLOAT32, [3, 3])
    return Program("higher_precision_constants", [I], [I + 1 + 2.0])


def defract():
    I = Placeholder(DType.FLOAT32, [3], name="I")
    Kt = Placeholder(DType.FLOAT32, [3], name="K")
    i, j = TensorIndexes(2)
    O = Contraction().outShape(5).outAccess(i).sum(I[(i - j + 1) // 2] * Kt[j]).build()
    return Program("defract_test", [I, Kt], [O])


def defract_short():
    I = Placeholder(DType.FLOAT32, [3], name="I")
    i, j = TensorIndexes(2)
    O = Contraction().outShape(6).outAccess(i).sum(I[(i - 1) // 2]).build()
    return Program("defract_short_test", [I], [O])


def defract_long():
    shape = [1, 3, 3, 1]
    I = Placeholder(DType.FLOAT32, shape, name="I")
    Kt = Placeholder(DType.FLOAT32, shape, name="K")
    n, x0, x1, c0, c1, co, ci, k0, k1 = TensorIndexes(9)
    O = Contraction().outShape(1, 5, 5, 1).outAccess(n, x0, x1, co).sum(
        I[n, (x0 + k0 - 1) // 2, (x1 + k1 - 1) // 2, ci] * Kt[2 - k0, 2 - k1, co, ci]).build()
    return Program("defract_long", [I, Kt], [O])


def broadcast_cmp():
    A = Placeholder(DType.INT64, [3, 4])
    B = Placeholder(DType.INT64, [3, 1])
    return Program("broadcast_cmp", [A, B], [cast(A >= B, DType.INT64)])


def eltwise():
    A = Placeholder(DType.FLOAT32, [3])
    B = Placeholder(DType.FLOAT32, [3])
    return Program("eltwise_add", [A, B], [A + B])


GOLDEN_BUILDERS = {
    "GEMM_INT64": lambda: gemm_plus_c(DType.INT64), "GEMM_UINT64": lambda: gemm_plus_c(DType.UINT64),
    "GEMM_INT32": lambda: gemm_plus_c(DType.INT32), "GEMM_INT8": lambda: gemm_plus_c(DType.INT8),
    "GEMM_FLOAT32": lambda: gemm_plus_c(DType.FLOAT32), "Max": row_max, "SimpleAdd": add,
    "HigherPrecisionConstants": higher_precision_constants_cc, "test_defract": defract,
    "test_defract_short": defract_short, "test_defract_long": defract_long, "test_broadcast_cmp": broadcast_cmp,
    "test_eltwise": eltwise, "test_higher_precision_constants": higher_precision_constants,
}


# the benchmark configurations live in the package so that bench.py can use them too
from plaidml_b200.programs import conv_bias_relu, tile_gemm  # noqa: E402,F401
