"""Host-side logic of the EDSL boundary, runnable without a GPU: expression building, shape and type
inference, bounds, the printed program and the error behaviour of the C ABI.  The programs follow the
reference's own Python tests (plaidml/edsl/tests/edsl_test.py) so that a maintainer can read them side by
side; the execution halves of those tests are the `gpu`-marked tests."""

import functools

import numpy as np
import pytest

import plaidml_b200 as plaidml
from plaidml_b200 import core, exec as pexec, op
from plaidml_b200.core import DType, Program, TensorShape
from plaidml_b200.edsl import (Contraction, Constant, Placeholder, TensorDims, TensorIndexes, TensorLens, cast, cond, exp,
                               index, reshape, select, sqrt, trace)
from plaidml_b200.ffi import Error


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


def conv_2d(I, K, I_layout="NHWC", K_layout="HWCK"):
    I_lens = TensorLens(I_layout, "NHWC")
    K_lens = TensorLens(K_layout, "HWCK")
    I = I.use(I_lens)
    K = K.use(K_lens)
    CI, CO, K0, K1, N, X0, X1 = TensorDims(7)
    n, x0, x1, k0, k1, ci, co = TensorIndexes(7)
    I.bind_dims(N, X0, X1, CI)
    K.bind_dims(K0, K1, CI, CO)
    return (Contraction(I_lens).outShape(N, X0 - (K0 - 1), X1 - (K1 - 1), CO).outAccess(n, x0, x1, co)
            .sum(I[n, x0 + k0 - (K0 // 2), x1 + k1 - (K1 // 2), ci] * K[k0, k1, ci, co]).build())


def max_pool_2d(I):
    N, X0, X1, C = TensorDims(4)
    n, x0, x1, i, j, c = TensorIndexes(6)
    I.bind_dims(N, X0, X1, C)
    return (Contraction().outShape(N, (X0 + 1) // 2, (X1 + 1) // 2, C).outAccess(n, x0, x1, c)
            .max(I[n, 2 * x0 + i, 2 * x1 + j, c]).add_constraint(i < 2).add_constraint(j < 2).build())


def flatten(X):
    dims = TensorDims(X.rank)
    X.bind_dims(*dims)
    return reshape(X, (1, functools.reduce(lambda a, b: a * b, dims[1:])))


def bounds_text(prog) -> str:
    """The program after bounds inference (index ranges, rational accesses): the second entry of the passes list."""
    return dict(prog.passes)["bounds"]


def shape_str(t) -> str:
    return str(t.compute_shape())


def test_settings_round_trip():
    core.settings_set("FOO", "bar")
    assert core.settings_get("FOO") == "bar"


def test_targets_name_the_cuda_target_only():
    assert core.list_targets() == ["cuda"]


def test_version_is_a_string():
    assert isinstance(plaidml.__version__, str) and plaidml.__version__


def test_placeholder_shapes_print_like_the_reference():
    # plaidml/edsl/tests/edsl_test.py:534-543
    I = Placeholder(DType.INT32)
    Program("placeholder_noshape", [I], [I])
    assert shape_str(I) == "si32"
    I = Placeholder(DType.INT32, [1, 1])
    assert shape_str(I) == "1x1xsi32"
    I = Placeholder(DType.INT32, [1, 1], name="I")
    assert shape_str(I) == "1x1xsi32"


def test_tensor_shape_strides_and_bytes():
    s = TensorShape(DType.FLOAT32, [2, 3, 4])
    assert s.sizes == [2, 3, 4] and s.strides == [12, 4, 1] and s.rank == 3
    assert s.dtype == DType.FLOAT32
    assert TensorShape(DType.BFLOAT16, [8]).dtype == DType.BFLOAT16


def test_dot_program_text_has_the_bounded_contraction():
    A = Placeholder(DType.FLOAT32, [4, 5])
    B = Placeholder(DType.FLOAT32, [5, 6])
    prog = Program("g", [A, B], [dot(A, B)])
    assert "tile.contract add, mul, %cst, %arg0, %arg1" in str(prog)
    text = bounds_text(prog)
    assert "tile.contract add, mul" in text
    assert "x0 in [0, 4)" in text and "x1 in [0, 6)" in text and "x2 in [0, 5)" in text
    assert [s.sizes for s in prog.inputs] == [[4, 5], [5, 6]]
    assert [s.sizes for s in prog.outputs] == [[4, 6]]


def test_mnist_cnn_shapes():
    # plaidml/edsl/tests/edsl_test.py:322-345: the flattened shape is the checked value there
    I = Placeholder(DType.FLOAT32, [1, 224, 224, 1])
    K1 = Placeholder(DType.FLOAT32, [3, 3, 1, 32])
    B1 = Placeholder(DType.FLOAT32, [32])
    C1 = relu(conv_2d(I, K1) + B1)
    K2 = Placeholder(DType.FLOAT32, [3, 3, 32, 64])
    B2 = Placeholder(DType.FLOAT32, [64])
    C2 = relu(conv_2d(C1, K2) + B2)
    P1 = max_pool_2d(C2)
    F = flatten(P1)
    assert shape_str(F) == "1x774400xf32"
    K3 = Placeholder(DType.FLOAT32, [774400, 128])
    B3 = Placeholder(DType.FLOAT32, [128])
    D1 = relu(dot(F, K3) + B3)
    K4 = Placeholder(DType.FLOAT32, [128, 100])
    B4 = Placeholder(DType.FLOAT32, [100])
    D2 = softmax(dot(D1, K4) + B4)
    prog = Program("mnist_cnn", [I, K1, B1, K2, B2, K3, B3, K4, B4], [D2])
    assert prog.outputs[0].sizes == [1, 100]
    prog.compile("cuda")


def test_arg_max_shape_and_type():
    # plaidml/edsl/tests/edsl_test.py:347-352
    I = Placeholder(DType.FLOAT32, [1, 10, 10])
    X0, X1, X2 = TensorDims(3)
    x0, x1, x2 = TensorIndexes(3)
    I.bind_dims(X0, X1, X2)
    Max = Contraction().outShape(X0, X2).outAccess(x0, x2).max(I[x0, x1, x2]).build()
    IX = index([X1], 0)
    O = Contraction().outShape(X0, X2).outAccess(x0, x2).max(cond(I[x0, x1, x2], Max[x0, x2], IX[x1])).build()
    O = cast(O, DType.UINT32)
    assert shape_str(O) == "1x10xui32"
    Program("arg_max", [I], [O])


def test_lens_reorders_dims_and_indexes():
    # plaidml/edsl/tests/edsl_test.py:578-588: NCHW / CKHW seen through lenses written for NHWC / HWCK
    I = Placeholder(DType.FLOAT32, [1, 224, 224, 3])
    K = Placeholder(DType.FLOAT32, [3, 3, 3, 32])
    O = conv_2d(I, K)
    assert O.compute_shape().sizes == [1, 222, 222, 32]
    I = Placeholder(DType.FLOAT32, [1, 3, 224, 224])
    K = Placeholder(DType.FLOAT32, [3, 32, 7, 7])
    O = conv_2d(I, K, I_layout="NCHW", K_layout="CKHW")
    assert O.compute_shape().sizes == [1, 32, 218, 218]
    with pytest.raises(ValueError):
        TensorLens("NCHW", "NHW")
    with pytest.raises(ValueError):
        TensorLens("NCHW", "NHWX")


def test_unique_names_and_two_outputs_print_identically():
    # plaidml/edsl/tests/edsl_test.py:360-366, 513-532
    A = Placeholder(DType.FLOAT32, name="A")
    B = Placeholder(DType.FLOAT32, name="B")
    C0 = Placeholder(DType.FLOAT32, name="C")
    C1 = Placeholder(DType.FLOAT32, name="C")
    Program("unique_names", [A, B, C0, C1], [A + B + C0 + C1])
    I = Placeholder(DType.FLOAT32, [3], name="I")
    p1 = Program("two_outputs", [I], [I, I])
    O1, O2 = I, I
    p2 = Program("two_outputs", [I], [O1, O2])
    assert str(p1) == str(p2)
    assert len(p1.outputs) == 2


def test_constants_are_not_program_inputs():
    # plaidml/edsl/tests/edsl_test.py:545-561
    A = Constant(np.array([4, 3, 2, 1], np.int32), name="A")
    B = Constant(np.array([1, 2, 3, 4], np.int32), name="B")
    prog = Program("const_add", [], [A + B])
    assert len(prog.inputs) == 0 and len(prog.outputs) == 1
    assert prog.outputs[0].dtype == DType.INT32


def test_collect_passes_starts_with_tile():
    # plaidml/edsl/tests/edsl_test.py:563-571
    A = Placeholder(DType.FLOAT32, [10, 10])
    B = Placeholder(DType.FLOAT32, [10, 10])
    prog = Program("collect_passes", [A, B], [dot(A, B)])
    core.settings_set("PLAIDML_TARGET", "cuda")     # an empty target means "the PLAIDML_TARGET setting"
    prog.compile(debug=True)
    assert prog.passes[0][0] == "tile" and prog.passes[0][1] == str(prog)
    assert prog.passes[1][0] == "bounds" and "x0 in [0, 10)" in prog.passes[1][1]


def test_trace_builds():
    I = Placeholder(DType.FLOAT32, [3, 3])
    Program("trace", [I], [trace(I, "msg")])


def test_type_promotion_follows_the_reference_ranks():
    # pmlc/dialect/tile/ir/util.cc:35-91: float beats int, wider beats narrower, bf16 sits between f16 and f32
    f16 = Placeholder(DType.FLOAT16, [4])
    bf = Placeholder(DType.BFLOAT16, [4])
    f32 = Placeholder(DType.FLOAT32, [4])
    i8 = Placeholder(DType.INT8, [4])
    i32 = Placeholder(DType.INT32, [4])
    assert (f16 + bf).dtype == DType.BFLOAT16
    assert (bf + f32).dtype == DType.FLOAT32
    assert (i8 + i32).dtype == DType.INT32
    assert (i32 + f16).dtype == DType.FLOAT16
    assert (i8 * i8).dtype == DType.INT8
    assert (f32 < 0.0).dtype == DType.BOOLEAN
    assert (f16 + 1.0).dtype == DType.FLOAT16       # literals adopt the tensor's type
    assert (i32 + 1).dtype == DType.INT32


def test_broadcast_rules():
    a = Placeholder(DType.FLOAT32, [3, 1, 5])
    b = Placeholder(DType.FLOAT32, [4, 1])
    assert (a + b).compute_shape().sizes == [3, 4, 5]
    c = Placeholder(DType.FLOAT32, [2, 5])
    with pytest.raises(Error):
        (a + Placeholder(DType.FLOAT32, [3, 2, 4])).compute_shape()
    assert (a + c).compute_shape().sizes == [3, 2, 5]


def test_bounds_of_a_strided_window_and_a_fractional_index():
    # the fractional access of plaidml/edsl/tests/edsl_test.py:408-419 bounds j by K and i by the output
    I = Placeholder(DType.FLOAT32, [3], name="I")
    K = Placeholder(DType.FLOAT32, [3], name="K")
    i, j = TensorIndexes(2)
    O = Contraction().outShape(5).outAccess(i).sum(I[(i - j + 1) // 2] * K[j]).build()
    text = bounds_text(Program("defract", [I, K], [O]))
    assert "x0 in [0, 5)" in text and "x1 in [0, 3)" in text
    # a pooling window: the window index is bounded by its constraint only
    P = Placeholder(DType.FLOAT32, [1, 7, 7, 2])
    text = str(Program("pool", [P], [max_pool_2d(P)]))
    assert "max" in text and "tensor<1x4x4x2xf32>" in text


def test_bounds_of_the_reference_compute_bounds_cases():
    # pmlc/dialect/tile/tests/compute-bounds.mlir:7-25 (@dot: sink (j, k), srcs (j, i) and (i, k) over tensors
    # 1x784 and 784x512): the pass annotates lowerBounds (0, 0, 0) and upperBounds (783, 0, 511) for (i, j, k)
    A = Placeholder(DType.FLOAT32, [1, 784])
    B = Placeholder(DType.FLOAT32, [784, 512])
    i, j, k = TensorIndexes(3)
    O = Contraction().outShape(1, 512).outAccess(j, k).sum(A[j, i] * B[i, k]).build()
    text = bounds_text(Program("dot", [A, B], [O]))
    # indices are numbered in order of first appearance (sink first): x0 = j, x1 = k, x2 = i
    assert "x0 in [0, 1)" in text and "x1 in [0, 512)" in text and "x2 in [0, 784)" in text
    # :29-47 (@no_reduce: sink d0 * 10 + d1 with both indices held to [0, 9] by constraints; an assignment)
    T = Placeholder(DType.FLOAT32, [10, 10])
    a, b = TensorIndexes(2)
    flat = Contraction().outShape(100).outAccess(a * 10 + b).assign(T[a, b]).build()
    text = bounds_text(Program("no_reduce", [T], [flat]))
    assert "x0 in [0, 10)" in text and "x1 in [0, 10)" in text


def test_bounds_of_indices_limited_only_by_sums_and_differences():
    # neither 0 <= i + j < 9 nor 0 <= i - j + 4 < 9 bounds i or j alone; together they do (the reference finds
    # the box with an integer program per index, pmlc/dialect/tile/transforms/contraction.cc:576-655): the
    # hull is i, j in [-2, 6]
    A = Placeholder(DType.FLOAT32, [9, 9])
    i, j = TensorIndexes(2)
    O = Contraction().outShape(9).outAccess(i + j).sum(A[i + j, i - j + 4]).build()
    text = bounds_text(Program("skew", [A], [O]))
    assert "x0 in [-2, 7)" in text and "x1 in [-2, 7)" in text
    # three coupled indices: 0 <= i + j < 4, 0 <= j + k < 4, 0 <= i + k < 4 and 0 <= i - j + 3 < 7
    B = Placeholder(DType.FLOAT32, [4, 4, 4, 7])
    i, j, k = TensorIndexes(3)
    O = Contraction().outShape(4).outAccess(i + j).sum(B[i + j, j + k, i + k, i - j + 3]).build()
    text = bounds_text(Program("skew3", [B], [O]))
    for v in ("x0", "x1", "x2"):
        lo, hi = (int(t) for t in text.split(v + " in [")[1].split(")")[0].split(", "))
        assert -4 <= lo <= 0 and 3 < hi <= 8, text     # finite, and wide enough for every feasible point


def test_bind_dims_mismatch_is_an_error():
    A = Placeholder(DType.FLOAT32, [5, 1])
    B = Placeholder(DType.FLOAT32, [2, 5])
    with pytest.raises(Error):
        dot(A, B)        # K bound to 1 by A, then to 2 by B
    with pytest.raises(Error):
        A.bind_dims(*TensorDims(3))


def test_an_index_no_access_bounds_is_an_error():
    A = Placeholder(DType.FLOAT32, [4])
    i, j = TensorIndexes(2)
    ok = Contraction().outShape(4).outAccess(i).sum(A[i + j]).add_constraint(j < 2).build()
    text = bounds_text(Program("window", [A], [ok]))       # j is held to [0, 2) by the constraint and by A's range
    assert "x1 in [0, 2)" in text
    free = Contraction().outShape(4).outAccess(i).sum(A[i] * A[i + 0 * j]).build()
    with pytest.raises(Error):
        Program("free_index", [A], [free])


def test_op_library_shape_rules():
    I = Placeholder(DType.FLOAT32, [1, 224, 224, 3])
    F = Placeholder(DType.FLOAT32, [7, 7, 3, 64])
    O = op.convolution(I, F, strides=[2, 2], autopad_mode=op.AutoPadMode.EXPLICIT, manual_padding=[3, 3])
    assert O.compute_shape().sizes == [1, 112, 112, 64]
    O = op.convolution(I, F, strides=[2, 2], autopad_mode=op.AutoPadMode.SAME_UPPER)
    assert O.compute_shape().sizes == [1, 112, 112, 64]
    O = op.convolution(I, F, strides=[1, 1], autopad_mode=op.AutoPadMode.VALID)
    assert O.compute_shape().sizes == [1, 218, 218, 64]
    X = Placeholder(DType.FLOAT32, [2, 112, 112, 64])
    P = op.pool(X, op.PoolMode.MAX, [3, 3], [2, 2], op.AutoPadMode.EXPLICIT, [1, 1], op.TensorLayout.NXC)
    assert P.compute_shape().sizes == [2, 56, 56, 64]
    assert op.mean(X, axes=[1, 2]).compute_shape().sizes == [2, 64]
    assert op.sum(X, axes=[3], keepdims=True).compute_shape().sizes == [2, 112, 112, 1]
    assert op.softmax(Placeholder(DType.FLOAT32, [8, 10]), axis=1).compute_shape().sizes == [8, 10]
    assert op.dot(Placeholder(DType.FLOAT32, [8, 10]), Placeholder(DType.FLOAT32, [10, 3])).compute_shape().sizes == [8, 3]
    # rank >= 2: the operands' dims are bound independently (plaidml/op/lib/ops.cc:1534-1543), so contracted
    # extents that differ are accepted and the shorter one bounds the sum; two vectors share their one dim
    assert op.dot(Placeholder(DType.FLOAT32, [8, 10]), Placeholder(DType.FLOAT32, [11, 3])).compute_shape().sizes == [8, 3]
    with pytest.raises(Error):
        op.dot(Placeholder(DType.FLOAT32, [10]), Placeholder(DType.FLOAT32, [11]))
    with pytest.raises(Error):
        op.op("no_such_operation", [X])


def test_jit_needs_a_compiled_program_and_a_cuda_device_id():
    A = Placeholder(DType.FLOAT32, [4, 5])
    B = Placeholder(DType.FLOAT32, [5, 6])
    prog = Program("g", [A, B], [dot(A, B)])
    with pytest.raises(Error, match="compiled"):
        pexec.Executable(prog, "cuda.0")
    with pytest.raises(Error):
        Program("g2", [A, B], [dot(A, B)]).compile("llvm_cpu")
    prog.compile("cuda")
    with pytest.raises(Error):
        pexec.Executable(prog, "llvm_cpu.0")
    with pytest.raises(Error):
        pexec.Executable(prog, "cuda.x")


def test_no_cpu_execution_path():
    """Without an sm_100 device plaidml_jit fails with a message saying so; nothing falls back to host code."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    A = Placeholder(DType.FLOAT32, [4, 5])
    B = Placeholder(DType.FLOAT32, [5, 6])
    prog = Program("g", [A, B], [dot(A, B)]).compile("cuda")
    assert pexec.list_devices() == []
    with pytest.raises(Error, match="(?i)cuda|device"):
        pexec.Executable(prog, "cuda.0")


def test_resnet50_program_builds_with_the_expected_layer_count():
    from plaidml_b200 import programs
    built = programs.resnet50(2, programs.resnet50_weights(seed=1))
    prog = built[0] if isinstance(built, tuple) else built
    text = str(prog)
    assert prog.outputs[0].sizes == [2, 1000]
    assert text.count("tile.contract add, mul") >= 53 + 1     # 53 convolutions and the classifier


def test_more_op_library_shapes_and_errors():
    X = Placeholder(DType.FLOAT32, [2, 3, 4, 5])
    assert shape_str(op.all(X, axis=1)) == "2x4x5xui8"
    assert shape_str(op.argmax(X, axis=-1)) == "2x3x4xui32"
    assert op.concatenate([X, X], axis=2).compute_shape().sizes == [2, 3, 8, 5]
    assert op.explicit_padding(X, [0, 1, 2, 0], [0, 1, 0, 3]).compute_shape().sizes == [2, 5, 6, 8]
    assert op.slice_of(X, [slice(None), 1, slice(None, None, -1), slice(1, 4, 2)]).compute_shape().sizes == [2, 4, 2]
    assert op.tile(X, [2, 1, 3]).compute_shape().sizes == [4, 3, 12, 5]
    assert op.repeat(X, 3, 2).compute_shape().sizes == [2, 3, 12, 5]
    assert op.reorg_yolo(Placeholder(DType.FLOAT32, [1, 4, 6, 6]), 2, False).compute_shape().sizes == [1, 16, 3, 3]
    assert op.broadcast(Placeholder(DType.FLOAT32, [3, 1]), [2, 3, 5], [1, 2]).compute_shape().sizes == [2, 3, 5]
    with pytest.raises(Error, match="0 and 0.5"):
        op.binary_crossentropy(X, X, 0.7)
    with pytest.raises(Error, match="positive slope"):
        op.hard_sigmoid(X, 0.0)
    with pytest.raises(Error, match="step size 0"):
        op.slice_of(X, [slice(None, None, 0), 0, 0, 0])
    with pytest.raises(Error, match="Unimplemented padding mode"):
        op.explicit_padding(X, [0, 0, 0, 0], [0, 0, 0, 0], op.PadMode.REFLECT)
    with pytest.raises(Error, match="tiling factors"):
        op.tile(X, [])


def test_image_resize_shapes_and_argument_errors():
    # plaidml/op/lib/ops.cc:1822-1866: positive factors, two of them, two spatial dimensions, NXC or NCX
    x = Placeholder(DType.FLOAT32, [2, 5, 7, 3])
    near = op.image_resize(x, [2, 3], op.InterpolationMode.NEAREST, op.TensorLayout.NXC)
    assert near.compute_shape().sizes == [2, 10, 21, 3]
    bil = op.image_resize(x, [2, 3], op.InterpolationMode.BILINEAR, op.TensorLayout.NCX)
    assert bil.compute_shape().sizes == [2, 5, 14, 9] and bil.compute_shape().dtype == DType.FLOAT32
    text = str(Program("resize", [x], [bil]))
    assert text.count('name = "image_resize"') == 6 and "tensor<3x5xf32>" in text     # two ramps, their vectors, kernel, resize
    with pytest.raises(Error, match="must be positive"):
        op.image_resize(x, [0, 2], op.InterpolationMode.BILINEAR, op.TensorLayout.NXC)
    with pytest.raises(Error, match="spatial scaling factors"):
        op.image_resize(x, [2], op.InterpolationMode.BILINEAR, op.TensorLayout.NXC)
    with pytest.raises(Error, match="layout"):
        op.image_resize(x, [2, 2], op.InterpolationMode.BILINEAR, op.TensorLayout.KCX)
    with pytest.raises(Error, match="2 spatial dims"):
        op.image_resize(Placeholder(DType.FLOAT32, [2, 5, 3]), [2, 2], op.InterpolationMode.NEAREST, op.TensorLayout.NXC)


def test_nms_builds_and_refuses_the_ssd_decoding():
    from plaidml_b200 import op as oplib
    B = Placeholder(DType.FLOAT32, [2, 10, 4])
    S = Placeholder(DType.FLOAT32, [2, 3, 10])
    I = Placeholder(DType.FLOAT32, [1])
    T = Placeholder(DType.FLOAT32, [1])
    boxes, scores, valid = oplib.nms(B, S, I, T, 4)
    assert boxes.compute_shape().sizes == [24, 3] and boxes.dtype == DType.INT32
    assert scores.compute_shape().sizes == [24, 3] and scores.dtype == DType.FLOAT32
    assert valid.compute_shape().sizes == [1]
    text = str(Program("nms", [B, S, I, T], [boxes, scores, valid]))
    assert "tile.argsort desc" in text and "tile.gather" in text and "tile.scatter" in text
    with pytest.raises(Error):      # BoxesDecodeMode::SSD
        oplib.op("nms", [B, S, I, T, 4, 0.0, False, True, int(DType.INT32), 1, False, False, 0, 0, None, None, False, None, 2,
                         True, True])


def test_gather_family_shape_rules():
    # pmlc/ast/ast_ops.cc:54-72 (argsort), :101-186 (gather), :188-205 (prng), :226-264 (scatter)
    from plaidml_b200 import edsl as E
    from plaidml_b200 import op as oplib
    X = Placeholder(DType.FLOAT16, [3, 5, 7])
    I = Placeholder(DType.INT32, [2, 4])
    assert E.gather(X, I, axis=1).compute_shape().sizes == [3, 2, 4, 7] and E.gather(X, I, axis=1).dtype == DType.FLOAT16
    assert E.gather(X, I, axis=-1).compute_shape().sizes == [3, 5, 2, 4]
    assert E.gather(X, 2, axis=0).compute_shape().sizes == [1, 5, 7]
    nd = Placeholder(DType.INT32, [3, 6, 2])
    assert oplib.gatherND(X, nd, batch_dims=1).compute_shape().sizes == [3, 6]
    assert oplib.gatherND(X, Placeholder(DType.INT32, [9, 2])).compute_shape().sizes == [9, 7]
    with pytest.raises(Error):
        E.gather(X, Placeholder(DType.FLOAT32, [9, 2]), mode=E.GatherMode.ND)      # nd indices must be integers
    with pytest.raises(Error):
        oplib.gatherND(X, Placeholder(DType.INT32, [9, 4]))                          # addresses 4 dims of a rank-3 tensor
    A = E.argsort(X, -2, E.SortDirection.DESC)
    assert A.compute_shape().sizes == [3, 5, 7] and A.dtype == DType.INT32
    assert oplib.sort(X, 1).compute_shape().sizes == [3, 5, 7] and oplib.sort(X, 1).dtype == DType.FLOAT16
    vals, pos = oplib.topk(X, 2, axis=1)
    assert vals.compute_shape().sizes == [3, 2, 7] and pos.compute_shape().sizes == [3, 2, 7] and pos.dtype == DType.INT32
    D = Placeholder(DType.FLOAT32, [8, 4])
    U = Placeholder(DType.FLOAT32, [3, 4])
    S = E.scatter(D, Placeholder(DType.INT32, [3]), U)
    assert S.compute_shape().sizes == [8, 4] and S.dtype == DType.FLOAT32
    with pytest.raises(Error):
        E.scatter(D, Placeholder(DType.INT64, [3]), U)                               # 32-bit indices only
    numbers, state = E.prng(Placeholder(DType.UINT32, [1, 3]), [2, 3])
    assert numbers.compute_shape().sizes == [2, 3] and numbers.dtype == DType.FLOAT32
    assert state.compute_shape().sizes == [1, 3] and state.dtype == DType.UINT32
    text = str(Program("family", [X, I], [E.gather(X, I, axis=1), A]))
    assert "tile.gather" in text and "tile.argsort desc" in text and "[-2]" in text
