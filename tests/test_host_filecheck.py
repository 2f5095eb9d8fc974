"""Replays the FileCheck expectations of the reference's C++ EDSL tests (plaidml/edsl/tests/edsl_test.cc,
extracted by tests/golden/make_filecheck_fixtures.py) on the text plaidml_program_repr returns for the same
programs built through this library's EDSL.  No GPU: programs are built and printed, not run."""

import functools
import json
import os

import numpy as np
import pytest

import filecheck
from plaidml_b200.core import DType, Program
from plaidml_b200 import edsl
from plaidml_b200.edsl import (Constant, Contraction, Placeholder, TensorDims, TensorIndexes, cast, exp, layer, reshape,
                               select, shape, sqrt, trace)

with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "edsl_filecheck.json")) as f:
    CHECKS = json.load(f)


def dot(A, B):
    I, J, K = TensorDims(3)
    i, j, k = TensorIndexes(3)
    A.bind_dims(I, K)
    B.bind_dims(K, J)
    return Contraction().outShape(I, J).outAccess(i, j).sum(A[i, k] * B[k, j]).build()


def relu(I):
    return select(I < 0.0, cast(0.0, I.dtype), I)


def softmax(X):
    I, J = TensorDims(2)
    i, j = TensorIndexes(2)
    X.bind_dims(I, J)
    M = Contraction().outShape(I, 1).outAccess(i, 0).max(X[i, j]).build()
    E = exp(X - M)
    N = Contraction().outShape(I, 1).outAccess(i, 0).sum(E[i, j]).build()
    return E / N


def conv_same(I, K):
    # edsl_test.cc:685-698: stride 1, output as large as the input, window centred
    CI, CO, K0, K1, N, X0, X1 = TensorDims(7)
    n, x0, x1, k0, k1, ci, co = TensorIndexes(7)
    I.bind_dims(N, X0, X1, CI)
    K.bind_dims(K0, K1, CI, CO)
    return (Contraction().outShape(N, X0, X1, CO).outAccess(n, x0, x1, co)
            .sum(I[n, x0 + k0 - (K0 // 2), x1 + k1 - (K1 // 2), ci] * K[k0, k1, ci, co]).build())


def max_pool_2x2(I):
    N, X0, X1, C = TensorDims(4)
    n, x0, x1, i, j, c = TensorIndexes(6)
    I.bind_dims(N, X0, X1, C)
    return (Contraction().outShape(N, (X0 + 1) // 2, (X1 + 1) // 2, C).outAccess(n, x0, x1, c)
            .max(I[n, 2 * x0 + i, 2 * x1 + j, c]).add_constraint(i < 2).add_constraint(j < 2).build())


def flatten(X):
    dims = TensorDims(X.rank)
    X.bind_dims(*dims)
    return reshape(X, (1, functools.reduce(lambda a, b: a * b, dims[1:])))


def complex_conv_2d(I, K, s, d):
    # edsl_test.cc:930-964: grouped, strided, dilated convolution with "same-lower" padding
    N, G, GCI, GCO = TensorDims(4)
    X, KX = TensorDims(2), TensorDims(2)
    n, g, gci, gco = TensorIndexes(4)
    x, k = TensorIndexes(2), TensorIndexes(2)
    I.bind_dims(N, X[0], X[1], G, GCI)
    K.bind_dims(KX[0], KX[1], G, GCI, GCO)
    Y = [(X[i] + s[i] - 1) // s[i] for i in range(2)]
    EK = [d[i] * (KX[i] - 1) + 1 for i in range(2)]
    P = [((Y[i] - 1) * s[i] + EK[i] - X[i]) // 2 for i in range(2)]
    return (Contraction().outShape(N, Y[0], Y[1], G, GCO).outAccess(n, x[0], x[1], g, gco)
            .sum(I[n, s[0] * x[0] + d[0] * k[0] - P[0], s[1] * x[1] + d[1] * k[1] - P[1], g, gci] *
                 K[k[0], k[1], g, gci, gco]).build())


def f32(*dims, name=""):
    return Placeholder(DType.FLOAT32, list(dims), name=name) if name else Placeholder(DType.FLOAT32, list(dims))


def build_simple_tensor():
    A = f32(3, 3)
    return Program("simple_tensor", [A], [A])


def build_const_add():
    A = Constant(np.array([4, 3, 2, 1], np.int32), name="A")
    B = Constant(np.array([1, 2, 3, 4], np.int32), name="B")
    return Program("const_add", [], [A + B])


def build_dot():
    A, B = f32(8, 16), f32(16, 32)
    return Program("dot", [A, B], [dot(A, B)])


def build_dot_f16():
    A, B = Placeholder(DType.FLOAT16, [8, 16]), Placeholder(DType.FLOAT16, [16, 32])
    return Program("dot_f16", [A, B], [dot(A, B)])


def build_double_dot():
    A, B, C = f32(10, 20), f32(20, 30), f32(30, 40)
    return Program("double_dot", [A, B, C], [dot(dot(A, B), C)])


def build_eltwise_add():
    A, B = f32(10, 20), f32(10, 20)
    return Program("eltwise_add", [A, B], [A + B])


def build_eltwise_mod():
    A, B = Placeholder(DType.INT32, [3, 3]), Placeholder(DType.INT32, [3, 3])
    return Program("mod", [A, B], [A % B])


def build_relu():
    A = f32(10, 20)
    return Program("relu", [A], [relu(A)])


def build_mnist_mlp():
    x = f32(1, 784)
    k1, b1, k2, b2, k3, b3 = f32(784, 512), f32(512), f32(512, 512), f32(512), f32(512, 10), f32(10)
    d1 = relu(dot(x, k1) + b1)
    d2 = relu(dot(d1, k2) + b2)
    d3 = softmax(dot(d2, k3) + b3)
    return Program("mnist_mlp", [x, k1, b1, k2, b2, k3, b3], [d3])


def build_convolution():
    I, K = f32(1, 56, 56, 64), f32(3, 3, 64, 64)
    return Program("convolution", [I, K], [conv_same(I, K)])


def build_mnist_cnn():
    x = f32(1, 224, 224, 1)
    k1, b1, k2, b2 = f32(3, 3, 1, 32), f32(32), f32(3, 3, 32, 64), f32(64)
    c1 = relu(conv_same(x, k1) + b1)
    c2 = relu(conv_same(c1, k2) + b2)
    flat = flatten(max_pool_2x2(c2))
    assert flat.compute_shape().sizes == [1, 802816]
    k3, b3, k4, b4 = f32(802816, 128), f32(128), f32(128, 100), f32(100)
    d1 = relu(dot(flat, k3) + b3)
    d2 = softmax(dot(d1, k4) + b4)
    return Program("mnist_cnn", [x, k1, b1, k2, b2, k3, b3, k4, b4], [d2])


def build_repeat_elements():
    I = f32(10, 10, 10)
    N0, N1, N2 = TensorDims(3)
    n0, n1, n2, k = TensorIndexes(4)
    I.bind_dims(N0, N1, N2)
    O = Contraction().outShape(N0, 3 * N1, N2).outAccess(n0, 3 * n1 + k, n2).assign(I[n0, n1, n2]).add_constraint(k < 3).build()
    return Program("repeat_elts", [I], [O])


def build_unique_names():
    A, B, C0, C1 = f32(1, name="A"), f32(1, name="B"), f32(1, name="C"), f32(1, name="C")
    return Program("unique_names", [A, B, C0, C1], [A + B + C0 + C1])


def build_global_min():
    I = f32(10, 10, 10, name="I")
    i, j, k = TensorIndexes(3)
    neg = -I
    O = -Contraction().max(neg[i, j, k]).build()
    return Program("global_min", [I], [O])


def build_cumsum():
    I = f32(10, name="I")
    N, = TensorDims(1)
    i, k = TensorIndexes(2)
    I.bind_dims(N)
    O = Contraction().outShape(N).outAccess(i).sum(I[k]).add_constraint(i - k < N).build()
    return Program("cumsum", [I], [O])


def build_complex_conv_2d():
    I, K = f32(1, 224, 224, 3, 3), f32(3, 3, 3, 3, 32)
    return Program("complex_conv_2d", [I, K], [complex_conv_2d(I, K, [2, 2], [3, 3])])


def build_reciprocal():
    A = f32(6, name="A")
    return Program("reciprocal", [A], [1.0 / A])


def build_defract_long():
    I, K = f32(1, 3, 3, 1, name="I"), f32(1, 3, 3, 1, name="K")
    n, x0, x1, k0, k1, co, ci = TensorIndexes(7)
    O = (Contraction().outShape(1, 5, 5, 1).outAccess(n, x0, x1, co)
         .sum(I[n, (x0 + k0 - 1) // 2, (x1 + k1 - 1) // 2, ci] * K[2 - k0, 2 - k1, co, ci]).build())
    return Program("defract_long", [I, K], [O])


def build_dup_out():
    A, B, C = f32(10, 20), f32(20, 30), f32(30, 40)
    R = dot(dot(A, B), C)
    return Program("dup_out", [A, B, C], [R, R, R])


def build_select():
    I = f32(10, 20)
    one, zero = cast(1.0, DType.FLOAT32), cast(0.0, DType.FLOAT32)
    return Program("select", [I], [select(I == 0, zero, one)])


def build_conv_i8():
    I, K = Placeholder(DType.INT8, [1, 224, 224, 3]), Placeholder(DType.INT8, [3, 3, 3, 32])
    return Program("convolution", [I, K], [conv_same(I, K)])


def build_higher_precision_constants():
    A = f32(3, 3)
    return Program("higher_precision_constants", [A], [A + cast(1, DType.UINT64) + cast(2.0, DType.FLOAT64)])


def build_lars_momentum_4d():
    # edsl_test.cc:796-827
    def normalize(X):
        sq = X * X
        idxs = TensorIndexes(X.rank)
        return sqrt(Contraction().sum(sq[tuple(idxs)]).build())

    X, G, V = f32(4, 7, 3, 9), f32(4, 7, 3, 9), f32(4, 7, 3, 9)
    LR = Placeholder(DType.FLOAT32, [])
    coeff, decay, momentum = 1. / 1024., 1. / 2048., 1. / 8.
    xn, gn = normalize(X), normalize(G)
    loc = LR * coeff * xn / (gn + decay * xn)
    nv = momentum * V + loc * (G + decay * X)
    return Program("lars_momentum4d", [X, G, V, LR], [X - nv, nv])


def build_reshape(name, src_dims, dst_dims):
    A = Placeholder(DType.INT32, src_dims, name="A")
    return Program(name, [A], [reshape(A, dst_dims)])


def build_shape():
    I = f32(2, 3)
    return Program("shape", [I], [shape(I)])


def build_trace():
    I = f32(3, 3)
    return Program("trace", [I], [trace(I, "msg")])


def build_layer():
    A = f32(10, 20)
    return Program("relu", [A], [layer("relu", [A], lambda: select(A < 0.0, 0.0, A))])


def build_layer_operand_order():
    A, B = f32(10, 20), f32(10, 20)
    return Program("LayerOperandOrder", [A, B], [layer("sum", [A, B], lambda: A + B)])


def _const_10x20(name):
    data = np.zeros(200, dtype=np.float32)
    data[:4] = [1, 2, 3, 4]
    return Constant(data.reshape(10, 20), name=name)


def build_layer_embedded_const():
    A = f32(10, 20)
    return Program("LayerEmbeddedConst", [A], [layer("sum", [A], lambda: A + _const_10x20("B"))])


def build_layer_unused_operand():
    A = f32(10, 20)
    B = _const_10x20("B")
    return Program("LayerUnusedOperand", [A], [layer("sum", [A, B], lambda: A + _const_10x20("C"))])


def build_layer_multi():
    A = f32(10, 20)
    B = layer("sum", [A], lambda: A + _const_10x20("C"))
    O = layer("sum", [B], lambda: B + _const_10x20("C"))
    return Program("LayerMulti", [A], [O])


def build_layer_exception():
    A = f32(10, 20)

    def failing():
        _const_10x20("C")
        raise RuntimeError("exception")

    with pytest.raises(RuntimeError):
        layer("sum", [A], failing)
    # the failed layer is closed: the next one is built at the function's level again
    return Program("LayerException", [A], [layer("sum", [A], lambda: A + _const_10x20("C"))])


def build_layer_multiple_return_values():
    A = f32(10, 5)

    def body():
        idxs = edsl.argsort(A, 0)
        return [edsl.gather(A, idxs), idxs]

    return Program("LayerMultipleReturnValues", [A], layer("two_output", [A], body))


def build_prng():
    S = Constant(np.array([[5, 6, 7]], dtype=np.uint32), name="S")
    O, NS = edsl.prng(S, [2, 3])
    return Program("prng", [], [O, NS])


def build_argsort(dtype, dims, axis, direction=edsl.SortDirection.ASC):
    I = Placeholder(dtype, dims)
    return Program("argsort", [I], [edsl.argsort(I, axis, direction)])


BUILDERS = {
    "LayerMultipleReturnValues": build_layer_multiple_return_values, "Prng": build_prng,
    "LayerMulti": build_layer_multi, "LayerException": build_layer_exception,
    "ArgSort1d": lambda: build_argsort(DType.FLOAT32, [20], 0),
    "ArgSort1dInt": lambda: build_argsort(DType.INT32, [20], 0),
    "ArgSort1dDup": lambda: build_argsort(DType.FLOAT32, [20], 0),
    "ArgSort2dAxis0": lambda: build_argsort(DType.FLOAT32, [5, 4], 0),
    "ArgSort2dAxis1": lambda: build_argsort(DType.FLOAT32, [5, 4], 1),
    "ArgSort3dAxis0Asc": lambda: build_argsort(DType.FLOAT32, [3, 4, 5], 0),
    "ArgSort3dAxis2Desc": lambda: build_argsort(DType.FLOAT32, [3, 4, 5], 2, edsl.SortDirection.DESC),
    "ArgSort3dAxisNeg2Asc": lambda: build_argsort(DType.FLOAT32, [2, 2, 2], -2),
    "Shape": build_shape, "Trace": build_trace,
    "Layer": build_layer, "LayerOperandOrder": build_layer_operand_order, "LayerEmbeddedConst": build_layer_embedded_const,
    "LayerUnusedOperand": build_layer_unused_operand,
    "HigherPrecisionConstants": build_higher_precision_constants, "LarsMomentum4d": build_lars_momentum_4d,
    "ReshapeFold": lambda: build_reshape("reshape_fold", [3, 3], [3, 3]),
    "ReshapeScalar": lambda: build_reshape("reshape_scalar", [], []),
    "ReshapeIntoScalar": lambda: build_reshape("reshape_into_scalar", [1, 1, 1], []),
    "ReshapeFromScalar": lambda: build_reshape("reshape_from_scalar", [], [1, 1, 1]),
    "SimpleTensor": build_simple_tensor, "ConstAdd": build_const_add, "Dot": build_dot, "DotF16": build_dot_f16,
    "DoubleDot": build_double_dot, "EltwiseAdd": build_eltwise_add, "EltwiseMod": build_eltwise_mod, "Relu": build_relu,
    "MnistMlp": build_mnist_mlp, "Convolution": build_convolution, "MnistCnn": build_mnist_cnn,
    "RepeatElements": build_repeat_elements, "UniqueNames": build_unique_names, "GlobalMin": build_global_min,
    "CumSum": build_cumsum, "ComplexConv2d": build_complex_conv_2d, "Reciprocal": build_reciprocal,
    "DefractLong": build_defract_long, "dup_out": build_dup_out, "Select": build_select, "ConvI8": build_conv_i8,
}


def test_every_extracted_test_has_a_builder():
    assert sorted(CHECKS) == sorted(BUILDERS)


@pytest.mark.parametrize("name", sorted(BUILDERS))
def test_printed_program_satisfies_the_reference_expectations(name):
    text = str(BUILDERS[name]())
    filecheck.run(CHECKS[name], text)


def test_filecheck_itself_rejects_what_it_should():
    text = "module @m {\n  %cst = tile.constant(0.000000e+00 : f64) : tensor<f32>\n  %0 = tile.add %a, %cst : x\n  return %0 : t\n}\n"
    filecheck.run([["CHECK", "%[[c:.*]] = tile.constant(0.000000e+00 : f64)"], ["CHECK", "tile.add %{{.*}},   %[[c]] : x"],
                   ["CHECK-NEXT", "return %0"]], text)
    with pytest.raises(filecheck.CheckFailure):
        filecheck.run([["CHECK", "tile.add"], ["CHECK", "tile.constant"]], text)          # order matters
    with pytest.raises(filecheck.CheckFailure):
        filecheck.run([["CHECK", "module @m"], ["CHECK-NEXT", "tile.add"]], text)         # not on the next line
    with pytest.raises(filecheck.CheckFailure):
        filecheck.run([["CHECK", "tile.add"], ["CHECK-SAME", "return"]], text)            # not on the same line
    with pytest.raises(filecheck.CheckFailure):
        filecheck.run([["CHECK", "tile.add %[[u]]"]], text)                                # undefined variable
    filecheck.run([["CHECK-DAG", "return %0"], ["CHECK-DAG", "tile.constant"], ["CHECK", "}"]], text)


def test_layer_that_reads_a_tensor_it_was_not_given_is_rejected():
    # plaidml/edsl/tests/edsl_test.cc LayerMissingOperand: building the program throws
    A, B = f32(10, 20), f32(10, 20)
    O = layer("sum", [A], lambda: A + B)
    with pytest.raises(Exception, match="not among its operands"):
        Program("LayerMissingOperand", [A, B], [O])


def test_nested_layers_and_several_results_print_as_nested_regions():
    A, B = f32(4, 6), f32(4, 6)

    def outer_body():
        s = layer("inner_sum", [A, B], lambda: A + B, attrs={"axis": 1})
        return [s * A, select(s < 0.0, 0.0, s)]

    P, Q = layer("outer", [A, B], outer_body)
    text = str(Program("nested", [A, B], [P + Q, Q]))
    filecheck.run([
        ["CHECK", "func @main(%[[A:.*]]: tensor<4x6xf32>, %[[B:.*]]: tensor<4x6xf32>) -> (tensor<4x6xf32>, tensor<4x6xf32>)"],
        ["CHECK", "%[[OUT:.*]]:2 = layer.box \"outer\"(%[[A]], %[[B]]) {attrs = {}} : tensor<4x6xf32>, tensor<4x6xf32> -> tensor<4x6xf32>, tensor<4x6xf32>"],
        ["CHECK-NEXT", "^bb0(%[[A1:.*]]: tensor<4x6xf32>, %[[B1:.*]]: tensor<4x6xf32>):"],
        ["CHECK", "%[[IN:.*]] = layer.box \"inner_sum\"(%[[A1]], %[[B1]]) {attrs = {axis = 1 : i64}} : tensor<4x6xf32>, tensor<4x6xf32> -> tensor<4x6xf32>"],
        ["CHECK-NEXT", "^bb0(%[[A2:.*]]: tensor<4x6xf32>, %[[B2:.*]]: tensor<4x6xf32>):"],
        ["CHECK", "%[[S:.*]] = tile.add %[[A2]], %[[B2]]"],
        ["CHECK", "layer.return %[[S]] : tensor<4x6xf32>"],
        ["CHECK", "%[[M:.*]] = tile.mul %[[IN]], %[[A1]]"],
        ["CHECK", "layer.return %[[M]], %{{.*}} : tensor<4x6xf32>, tensor<4x6xf32>"],
        ["CHECK", "%[[T:.*]] = tile.add %[[OUT]]#0, %[[OUT]]#1"],
        ["CHECK", "return %[[T]], %{{.*}} : tensor<4x6xf32>, tensor<4x6xf32>"],
    ], text)
