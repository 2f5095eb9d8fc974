"""End-to-end parity through the reference-facing API: programs built with the EDSL, compiled
for the `cuda` target and run on `cuda.0`, checked against the reference's known-answer
vectors and against the CPU oracle on seeded inputs."""

import json
from pathlib import Path

import numpy as np
import pytest

import oracle
from plaidml_b200 import core, edsl, op
from plaidml_b200.core import Buffer, DType, Program, bf16_bits_to_f32, f32_to_bf16_bits
from plaidml_b200.edsl import Contraction, Placeholder, TensorDims, TensorIndexes, cast
from plaidml_b200.exec import Executable, Runner, list_devices

import edsl_programs as P
from gpu_util import check_close, max_rel, rng

pytestmark = pytest.mark.gpu

KATS = json.loads((Path(__file__).parent / "golden" / "reference_kats.json").read_text())


def test_devices_and_targets():
    assert core.list_targets() == ["cuda"]
    devs = list_devices()
    assert devs and devs[0] == "cuda.0"


@pytest.mark.parametrize("kat", KATS, ids=[k["name"] for k in KATS])
def test_reference_known_answers(kat):
    program = P.GOLDEN_BUILDERS[kat["name"]]()
    runner = Runner(program, "cuda.0")
    ins = [np.array(v).reshape(s.sizes).astype(s.dtype.into_numpy()) for v, s in zip(kat["inputs"], program.inputs)]
    outs = runner.run(ins)
    for got, want, shape in zip(outs, kat["outputs"], program.outputs):
        want = np.array(want).reshape(shape.sizes)
        if got.dtype.kind == "f":
            # the reference checks floats exactly against its own backend; ours may order the
            # additions differently: one float32 ulp of slack
            np.testing.assert_allclose(got, want.astype(got.dtype), rtol=3e-7)
        else:
            np.testing.assert_array_equal(got, want.astype(got.dtype))


XSMM = {k["name"]: k for k in json.loads((Path(__file__).parent / "golden" / "reference_xsmm_kats.json").read_text())}


def test_reference_microkernel_known_answers():
    # the 8 x 8 dot product and the 1x1 convolution 1x6x5x7 (*) 1x1x7x11 printed by the reference's x86
    # microkernel test, through the EDSL (fp32 products this small run on the general kernel, in plain f32)
    kat = XSMM["xsmm_dot_8x8"]
    a, b = (np.array(v, dtype=np.float32) for v in kat["inputs"])
    A, B, C = P.tile_gemm(DType.FLOAT32, 8, 8, 8)
    runner = Runner(Program("xsmm_dot", [A, B], [C]), "cuda.0")
    assert "generic_contract" in runner.executable.describe()
    np.testing.assert_array_equal(runner.run([a, b])[0], np.array(kat["outputs"][0], dtype=np.float32))
    kat = XSMM["xsmm_conv_1x1"]
    x, f = (np.array(v, dtype=np.float32) for v in kat["inputs"])
    I = Placeholder(DType.FLOAT32, [1, 6, 5, 7])
    F = Placeholder(DType.FLOAT32, [1, 1, 7, 11])
    O = op.convolution(I, F, strides=[1, 1], autopad_mode=op.AutoPadMode.VALID)
    runner = Runner(Program("xsmm_conv", [I, F], [O]), "cuda.0")
    np.testing.assert_array_equal(runner.run([x, f])[0], np.array(kat["outputs"][0], dtype=np.float32).reshape(1, 6, 5, 11))


def test_small_fp32_gemm_is_exact_like_the_reference_expects():
    # plaidml/edsl/examples/gemm.cc GEMM_FLOAT32 is checked with checkExact in the reference: any true f32
    # arithmetic reproduces it bit for bit (three TF32 products per term would not)
    kat = next(k for k in KATS if k["name"] == "GEMM_FLOAT32")
    program = P.GOLDEN_BUILDERS["GEMM_FLOAT32"]()
    ins = [np.array(v, dtype=np.float32).reshape(3, 3) for v in kat["inputs"]]
    got = Runner(program, "cuda.0").run(ins)[0]
    np.testing.assert_array_equal(got, np.array(kat["outputs"][0], dtype=np.float32).reshape(3, 3))


def test_funky_sum_of_the_reference():
    # plaidml/edsl/tests/edsl_test.cc:2709-2719 (CppEdsl.FunkySum), checked exactly there
    I = Placeholder(DType.FLOAT32, [3])
    Kt = Placeholder(DType.FLOAT32, [3])
    i, j = TensorIndexes(2)
    O = Contraction().outShape(5).outAccess(i).sum(I[(i - j + 1) // 2] * Kt[j]).build()
    got = Runner(Program("funky_sum", [I, Kt], [O]), "cuda.0").run([np.array([1, 2, 3], np.float32), np.array([1, 2, 3], np.float32)])[0]
    np.testing.assert_array_equal(got, np.array([2, 5, 4, 9, 6], np.float32))


def test_contraction_whose_indices_only_sums_and_differences_bound():
    # O[i + j] += A[i + j, i - j + 4]: the index box comes from Fourier-Motzkin elimination, a little larger than
    # the set of feasible points; the kernel's per-point range checks make the result the definition's
    g = rng(1261)
    a = g.standard_normal((9, 9)).astype(np.float32)
    A = Placeholder(DType.FLOAT32, [9, 9])
    i, j = TensorIndexes(2)
    O = Contraction().outShape(9).outAccess(i + j).sum(A[i + j, i - j + 4]).build()
    got = Runner(Program("skew", [A], [O]), "cuda.0").run([a])[0]
    want = np.zeros(9, dtype=np.float64)
    for ii in range(-10, 20):
        for jj in range(-10, 20):
            r, c = ii + jj, ii - jj + 4
            if 0 <= r < 9 and 0 <= c < 9:
                want[r] += a[r, c]
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)


def test_run_on_adopted_caller_memory():
    # buffers that borrow the caller's (pageable) numpy memory, as the reference's C++ Buffer(ptr, shape) does:
    # inputs are read from it and outputs land in it
    g = rng(1260)
    a = g.integers(-128, 128, size=(96, 64), dtype=np.int8)
    b = g.integers(-128, 128, size=(64, 80), dtype=np.int8)
    c = np.full((96, 80), -7, dtype=np.int32)
    A, B, C = P.tile_gemm(DType.INT8, 96, 80, 64, acc=DType.INT32)
    program = Program("adopted", [A, B], [C])
    program.compile("cuda")
    exe = Executable(program, "cuda.0")
    ins = [Buffer.adopt(a), Buffer.adopt(b)]
    outs = [Buffer.adopt(c)]
    exe.run(ins, outs)
    np.testing.assert_array_equal(c, oracle.gemm_i8_i32(a, b))
    a[:] = 1                                   # the buffer is the array: a second run sees the new contents
    exe.run(ins, outs)
    np.testing.assert_array_equal(c, np.broadcast_to(b.astype(np.int32).sum(axis=0), (96, 80)))


def test_known_answers_also_on_the_general_kernel(monkeypatch):
    monkeypatch.setenv("PLAIDML_CUDA_GENERIC_ONLY", "1")
    for kat in KATS:
        if not kat["name"].startswith("GEMM"):
            continue
        program = P.GOLDEN_BUILDERS[kat["name"]]()
        runner = Runner(program, "cuda.0")
        assert "generic_contract" in runner.executable.describe()
        ins = [np.array(v).reshape(s.sizes).astype(s.dtype.into_numpy()) for v, s in zip(kat["inputs"], program.inputs)]
        got = runner.run(ins)[0]
        want = np.array(kat["outputs"][0]).reshape(3, 3)
        if got.dtype.kind == "f":
            np.testing.assert_allclose(got, want, rtol=3e-7)
        else:
            np.testing.assert_array_equal(got, want.astype(got.dtype))


def test_fp32_tile_gemm_1024_within_1e5():
    # configuration 1: C[i,j] += A[i,k] * B[k,j], M = N = K = 1024, uniform [-1, 1)
    g = rng(1234)
    a = g.uniform(-1, 1, size=(1024, 1024)).astype(np.float32)
    b = g.uniform(-1, 1, size=(1024, 1024)).astype(np.float32)
    A, B, C = P.tile_gemm(DType.FLOAT32, 1024, 1024, 1024)
    runner = Runner(Program("gemm_f32", [A, B], [C]), "cuda.0")
    assert runner.executable.describe().startswith("tc_gemm")
    got = runner.run([a, b])[0]
    ref64 = oracle.gemm_f32_acc64(a, b)
    assert max_rel(got, ref64) < 1e-5
    check_close(got, oracle.gemm_f32(a, b), 1e-5)


def test_int8_tile_gemm_bit_exact():
    # configuration 2 at a size the CPU oracle finishes quickly; operands cast to int32
    g = rng(1235)
    m = n = k = 512
    a = g.integers(-128, 128, size=(m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(k, n), dtype=np.int8)
    A, B, C = P.tile_gemm(DType.INT8, m, n, k, acc=DType.INT32)
    runner = Runner(Program("gemm_i8", [A, B], [C]), "cuda.0")
    desc = runner.executable.describe()
    assert desc.startswith("tc_gemm") and "in=si8 out=si32" in desc
    np.testing.assert_array_equal(runner.run([a, b])[0], oracle.gemm_i8_i32(a, b))


def test_full_size_int8_gemm_through_the_sliced_run():
    # configuration 2 at full size: plaidml_executable_run moves the rows of A and C in four slices so that
    # upload and download overlap; the result must equal the single-pass run bit for bit, and a checksum of
    # row sums pins both against the operands (sum_j C[i, j] = A[i, :] . rowsum(B))
    g = rng(1240)
    m = n = k = 4096
    a = g.integers(-128, 128, size=(m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(k, n), dtype=np.int8)
    A, B, C = P.tile_gemm(DType.INT8, m, n, k, acc=DType.INT32)
    sliced = Runner(Program("gemm_i8_full", [A, B], [C]), "cuda.0").run([a, b])[0]
    core.settings_set("PLAIDML_CUDA_SLICED_RUN", "0")
    try:
        whole = Runner(Program("gemm_i8_full", [A, B], [C]), "cuda.0").run([a, b])[0]
    finally:
        core.settings_set("PLAIDML_CUDA_SLICED_RUN", "1")
    np.testing.assert_array_equal(sliced, whole)
    np.testing.assert_array_equal(sliced.astype(np.int64).sum(axis=1), a.astype(np.int64) @ b.astype(np.int64).sum(axis=1))
    rows = [0, 1023, 1024, 2047, 3072, 4095]
    np.testing.assert_array_equal(sliced[rows], oracle.gemm_i8_i32(np.ascontiguousarray(a[rows]), b))


@pytest.mark.parametrize("b_transposed", [False, True], ids=["B_kn", "B_nk"])
def test_bf16_gemm_sliced_run_with_column_blocks(b_transposed):
    # B is a host input as well: the first row slice is computed in four column blocks, each after its quarter of B
    # (a pitched rectangle of B[k][n], a run of rows of B[n][k]); results must equal the single-pass run exactly
    g = rng(1241)
    m, n, k = 4096, 4096, 192
    a = f32_to_bf16_bits(g.standard_normal((m, k)))
    b = f32_to_bf16_bits(g.standard_normal((n, k) if b_transposed else (k, n)))
    A, B, C = P.tile_gemm(DType.BFLOAT16, m, n, k, acc=DType.FLOAT32, out_bf16=True, b_transposed=b_transposed)
    sliced = Runner(Program("gemm_bf16_blocks", [A, B], [C]), "cuda.0").run([a, b])[0]
    core.settings_set("PLAIDML_CUDA_SLICED_RUN", "0")
    try:
        whole = Runner(Program("gemm_bf16_blocks", [A, B], [C]), "cuda.0").run([a, b])[0]
    finally:
        core.settings_set("PLAIDML_CUDA_SLICED_RUN", "1")
    np.testing.assert_array_equal(sliced, whole)
    af, bf = oracle.bf16_to_f32(a[:8]), oracle.bf16_to_f32(b)
    ref = af @ (bf.T if b_transposed else bf)
    check_close(oracle.bf16_to_f32(sliced[:8]), oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)


def test_int8_without_casts_wraps_like_the_reference():
    g = rng(1236)
    a = g.integers(-128, 128, size=(64, 48), dtype=np.int8)
    b = g.integers(-128, 128, size=(48, 32), dtype=np.int8)
    A, B, C = P.tile_gemm(DType.INT8, 64, 32, 48)
    got = Runner(Program("gemm_i8_wrap", [A, B], [C]), "cuda.0").run([a, b])[0]
    np.testing.assert_array_equal(got, oracle.gemm_i8_i32(a, b).astype(np.int8))


def test_conv_bias_relu_bf16_fused():
    # configuration 3 at batch 4
    g = rng(1237)
    n, h, w, c, k = 4, 56, 56, 64, 64
    x = f32_to_bf16_bits(g.uniform(0, 1, size=(n, h, w, c)))
    f = f32_to_bf16_bits(g.standard_normal((3, 3, c, k)) * np.sqrt(2.0 / 576))
    bias = (g.standard_normal(k) * 0.1).astype(np.float32)
    program = P.conv_bias_relu(n, h, w, c, k, filt=f, bias=bias)
    runner = Runner(program, "cuda.0")
    desc = runner.executable.describe()
    assert desc.count("\n") == 1 and desc.startswith("tc_conv") and "+bias+relu+cast" in desc, desc
    got = bf16_bits_to_f32(runner.run([x])[0])
    ref = oracle.conv2d_nhwc_f32(bf16_bits_to_f32(x), bf16_bits_to_f32(f), bias, None, pad=(1, 1), relu=True)
    # 1e-2 relative: the stated tolerance for this configuration (bf16 result)
    check_close(got, bf16_bits_to_f32(f32_to_bf16_bits(ref)), 1e-2)


def test_qk_batched_gemm_then_row_max():
    # configuration 5 at batch 8: S[b,i,j] += Q[b,i,k] * K[b,j,k] (bf16 in, f32 acc), R[b,i] >= S[b,i,j]
    g = rng(1238)
    b, m, k = 8, 512, 64
    q = f32_to_bf16_bits(g.standard_normal((b, m, k)))
    kk = f32_to_bf16_bits(g.standard_normal((b, m, k)))
    Q, Kt, S = P.tile_gemm(DType.BFLOAT16, m, m, k, acc=DType.FLOAT32, batch=b, b_transposed=True)
    bb, i, j = TensorIndexes(3)
    R = Contraction(name="rowmax").outShape(b, m).outAccess(bb, i).max(S[bb, i, j]).build()
    runner = Runner(Program("qk_rowmax", [Q, Kt], [S, R]), "cuda.0")
    desc = runner.executable.describe()
    # the row maximum rides in the GEMM's epilogue: one step, no second pass over S
    assert "tc_gemm" in desc and "+rowmax" in desc and "row_reduce" not in desc, desc
    s_out, r_out = runner.run([q, kk])
    ref = oracle.gemm_h16_f32(q, kk, False, True)
    check_close(s_out, ref, 1e-2)
    np.testing.assert_array_equal(r_out, s_out.max(axis=2))   # exact given identical S
    # the same maxima when only R is asked for (S is then never written) ...
    only_r = Runner(Program("qk_rowmax_only", [Q, Kt], [R]), "cuda.0")
    assert "+rowmax" in only_r.executable.describe()
    np.testing.assert_array_equal(only_r.run([q, kk])[0], r_out)
    # ... and from the separate reduction kernel when S comes from somewhere else
    Sin = Placeholder(DType.FLOAT32, [b, m, m])
    R2 = Contraction(name="rowmax").outShape(b, m).outAccess(bb, i).max(Sin[bb, i, j]).build()
    plain = Runner(Program("rowmax_alone", [Sin], [R2]), "cuda.0")
    assert "row_reduce" in plain.executable.describe()
    np.testing.assert_array_equal(plain.run([s_out])[0], r_out)


def test_dense_bias_then_softmax():
    # a GEMM that already carries a bias keeps its softmax's max-reduction as a separate step (the kernel
    # folds row maxima only into a product without other epilogue terms); the program must still plan and
    # its numbers follow the definition
    g = rng(1250)
    m, k, n = 96, 160, 200
    x = g.standard_normal((m, k)).astype(np.float32)
    w = g.standard_normal((k, n)).astype(np.float32) * 0.1
    bias = g.standard_normal(n).astype(np.float32)
    X = Placeholder(DType.FLOAT32, [m, k])
    logits = op.dot(X, edsl.Constant(w, name="w")) + edsl.Constant(bias, name="b")
    sm = op.softmax(logits, axis=1)
    runner = Runner(Program("dense_softmax", [X], [logits, sm]), "cuda.0")
    desc = runner.executable.describe()
    assert "tc_gemm" in desc and "+bias" in desc and "+rowmax" not in desc, desc
    got_logits, got_sm = runner.run([x])
    ref = oracle.gemm_f32_acc64(x, w) + bias
    assert max_rel(got_logits, ref) < 1e-5
    e = np.exp(ref - ref.max(axis=1, keepdims=True))
    np.testing.assert_allclose(got_sm, e / e.sum(axis=1, keepdims=True), rtol=2e-4, atol=1e-7)
    # the same with a ReLU between them and only the softmax asked for
    sm2 = op.softmax(op.relu(logits), axis=1)
    only = Runner(Program("dense_relu_softmax", [X], [sm2]), "cuda.0")
    r = np.maximum(ref, 0)
    e = np.exp(r - r.max(axis=1, keepdims=True))
    np.testing.assert_allclose(only.run([x])[0], e / e.sum(axis=1, keepdims=True), rtol=2e-4, atol=1e-7)


def test_gemm_that_covers_part_of_its_output_leaves_zeros():
    # the index ranges span 48 of the output's 64 rows (and only column block 0..31 of 40): the rest keeps
    # the aggregation's identity, 0, which rules out the tensor-core route (it writes only what it covers)
    g = rng(1251)
    a = g.standard_normal((48, 64)).astype(np.float32)
    b = g.standard_normal((64, 32)).astype(np.float32)
    A = Placeholder(DType.FLOAT32, [48, 64])
    B = Placeholder(DType.FLOAT32, [64, 32])
    i, j, k = TensorIndexes(3)
    C = Contraction().outShape(64, 40).outAccess(i, j).sum(A[i, k] * B[k, j]).build()
    runner = Runner(Program("partial_cover", [A, B], [C]), "cuda.0")
    assert "generic_contract" in runner.executable.describe()
    got = runner.run([a, b])[0]
    want = np.zeros((64, 40), dtype=np.float32)
    want[:48, :32] = oracle.gemm_f32_acc64(a, b)
    assert max_rel(got, want) < 1e-5
    assert not got[48:].any() and not got[:, 32:].any()


def test_int8_gemm_relu_without_casts_wraps_first():
    g = rng(1252)
    m, n, k = 64, 32, 256
    a = g.integers(-128, 128, size=(m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(k, n), dtype=np.int8)
    A, B, C = P.tile_gemm(DType.INT8, m, n, k)
    got = Runner(Program("gemm_i8_relu", [A, B], [op.relu(C)]), "cuda.0").run([a, b])[0]
    np.testing.assert_array_equal(got, np.maximum(oracle.gemm_i8_i32(a, b).astype(np.int8), 0))


def test_maxpool_and_mean_and_softmax():
    g = rng(1239)
    x = g.standard_normal((2, 12, 12, 16)).astype(np.float32)
    I = Placeholder(DType.FLOAT32, x.shape)
    pooled = op.pool(I, op.PoolMode.MAX, [3, 3], [2, 2], op.AutoPadMode.EXPLICIT, [1, 1, 1, 1], op.TensorLayout.NXC)
    avg = op.mean(pooled, axes=[1, 2])
    sm = op.softmax(avg, axis=1)
    runner = Runner(Program("pool_mean_softmax", [I], [pooled, avg, sm]), "cuda.0")
    desc = runner.executable.describe()
    assert "nhwc_pool" in desc and "strided_reduce" in desc, desc
    got_pool, got_avg, got_sm = runner.run([x])
    ref_pool = oracle.pool2d_nhwc_f32(x, "max", (3, 3), (2, 2), (1, 1), (6, 6))
    np.testing.assert_array_equal(got_pool, ref_pool)
    ref_avg = ref_pool.astype(np.float64).mean(axis=(1, 2))
    np.testing.assert_allclose(got_avg, ref_avg, rtol=1e-5, atol=1e-6)
    e = np.exp(ref_avg - ref_avg.max(axis=1, keepdims=True))
    np.testing.assert_allclose(got_sm, e / e.sum(axis=1, keepdims=True), rtol=1e-5, atol=1e-7)


def test_layers_run_like_the_operations_they_enclose():
    # plaidml/edsl/tests/edsl_test.cc Layer, LayerOperandOrder, LayerEmbeddedConst: runProgram after the FileCheck lines
    g = rng(1260)
    a = g.standard_normal((10, 20)).astype(np.float32)
    b = g.standard_normal((10, 20)).astype(np.float32)
    A, B = Placeholder(DType.FLOAT32, [10, 20]), Placeholder(DType.FLOAT32, [10, 20])
    relu_layer = edsl.layer("relu", [A], lambda: edsl.select(A < 0.0, 0.0, A))
    sum_layer = edsl.layer("sum", [A, B], lambda: A + B)
    const_layer = edsl.layer("sum", [A], lambda: A + edsl.Constant(b, name="B"))
    nested = edsl.layer("outer", [A, B], lambda: op.relu(edsl.layer("inner", [A, B], lambda: op.dot(A, op.transpose(B)))))
    runner = Runner(Program("layers", [A, B], [relu_layer, sum_layer, const_layer, nested]), "cuda.0")
    assert "layer.box" in str(runner.program)
    r, s, c, n = runner.run([a, b])
    np.testing.assert_array_equal(r, np.maximum(a, 0))
    np.testing.assert_array_equal(s, a + b)
    np.testing.assert_array_equal(c, a + b)
    np.testing.assert_allclose(n, np.maximum(a.astype(np.float64) @ b.astype(np.float64).T, 0), rtol=1e-5, atol=1e-5)


def test_shortcut_projection_runs_inside_the_blocks_last_layer(monkeypatch):
    # relu(y . W2 + b2 + cast(cast(x . W1 + b1, bf16), f32)): a residual block's last 1x1 layer whose residual is the
    # block's shortcut projection.  One GEMM over [y | x] and the stacked weights; equal to the two-step form up to the
    # one rounding of the projection that the fused form leaves out
    g = rng(1262)
    m, c_mid, c_in, c_out = 4 * 14 * 14, 64, 128, 256
    y = f32_to_bf16_bits(g.standard_normal((m, c_mid)))
    x = f32_to_bf16_bits(g.standard_normal((m, c_in)))
    w2 = f32_to_bf16_bits(g.standard_normal((c_mid, c_out)) * 0.1)
    w1 = f32_to_bf16_bits(g.standard_normal((c_in, c_out)) * 0.1)
    b2 = g.standard_normal(c_out).astype(np.float32)
    b1 = g.standard_normal(c_out).astype(np.float32)

    def build():
        Y, X = Placeholder(DType.BFLOAT16, [m, c_mid]), Placeholder(DType.BFLOAT16, [m, c_in])
        W2 = cast(edsl.Constant(w2, name="w2", dtype=DType.BFLOAT16), DType.FLOAT32)
        W1 = cast(edsl.Constant(w1, name="w1", dtype=DType.BFLOAT16), DType.FLOAT32)
        shortcut = cast(op.dot(cast(X, DType.FLOAT32), W1) + edsl.Constant(b1, name="b1"), DType.BFLOAT16)
        main = op.dot(cast(Y, DType.FLOAT32), W2) + edsl.Constant(b2, name="b2")
        return Program("block_tail", [Y, X], [cast(op.relu(main + cast(shortcut, DType.FLOAT32)), DType.BFLOAT16)])

    fused = Runner(build(), "cuda.0")
    desc = fused.executable.describe()
    assert desc.count("tc_gemm") == 1 and "+shortcut(k128)" in desc and "k192" in desc, desc
    got = bf16_bits_to_f32(fused.run([y, x])[0])
    yf, xf = bf16_bits_to_f32(y).astype(np.float64), bf16_bits_to_f32(x).astype(np.float64)
    exact = np.maximum(yf @ bf16_bits_to_f32(w2) + b2 + xf @ bf16_bits_to_f32(w1) + b1, 0)
    check_close(got, bf16_bits_to_f32(f32_to_bf16_bits(exact.astype(np.float32))), 1e-2)
    monkeypatch.setenv("PLAIDML_CUDA_NO_SHORTCUT_FUSION", "1")
    plain = Runner(build(), "cuda.0")
    assert plain.executable.describe().count("tc_gemm") == 2
    check_close(got, bf16_bits_to_f32(plain.run([y, x])[0]), 1e-2)
    monkeypatch.delenv("PLAIDML_CUDA_NO_SHORTCUT_FUSION")


def test_strided_shortcut_projection_runs_inside_the_blocks_last_layer():
    # a block that halves the resolution: main = conv1x1(y) on 14x14, shortcut = conv1x1 / 2 of x on 28x28; the
    # projection's pixels are the second part of the last layer's A (an im2col load per k-block), its weights stacked
    g = rng(1263)
    n, c_mid, c_in, c_out = 3, 64, 128, 256
    y = f32_to_bf16_bits(g.standard_normal((n, 14, 14, c_mid)))
    x = f32_to_bf16_bits(g.standard_normal((n, 28, 28, c_in)))
    w2 = f32_to_bf16_bits(g.standard_normal((1, 1, c_mid, c_out)) * 0.1)
    w1 = f32_to_bf16_bits(g.standard_normal((1, 1, c_in, c_out)) * 0.1)
    b2 = g.standard_normal(c_out).astype(np.float32)
    b1 = g.standard_normal(c_out).astype(np.float32)
    Y, X = Placeholder(DType.BFLOAT16, list(y.shape)), Placeholder(DType.BFLOAT16, list(x.shape))
    W2 = cast(edsl.Constant(w2, name="w2", dtype=DType.BFLOAT16), DType.FLOAT32)
    W1 = cast(edsl.Constant(w1, name="w1", dtype=DType.BFLOAT16), DType.FLOAT32)
    shortcut = op.convolution(cast(X, DType.FLOAT32), W1, strides=[2, 2], autopad_mode=op.AutoPadMode.VALID, name="proj")
    shortcut = cast(shortcut + edsl.Constant(b1, name="b1"), DType.BFLOAT16)
    main = op.convolution(cast(Y, DType.FLOAT32), W2, name="last") + edsl.Constant(b2, name="b2")
    O = cast(op.relu(main + cast(shortcut, DType.FLOAT32)), DType.BFLOAT16)
    runner = Runner(Program("down_block_tail", [Y, X], [O]), "cuda.0")
    desc = runner.executable.describe()
    assert desc.count("\n") == 1 and "tc_gemm" in desc and "+shortcut(k128/2)" in desc, desc
    got = bf16_bits_to_f32(runner.run([y, x])[0])
    yf, xf = bf16_bits_to_f32(y), bf16_bits_to_f32(x)
    ref = oracle.conv2d_nhwc_f32(yf, bf16_bits_to_f32(w2), b2) + oracle.conv2d_nhwc_f32(xf, bf16_bits_to_f32(w1), b1, None, (2, 2))
    check_close(got, bf16_bits_to_f32(f32_to_bf16_bits(np.maximum(ref, 0))), 1e-2)


def test_fp32_network_layers_run_on_tensor_cores():
    # the reference's own networks are fp32 (networks/oplib/resnet50.cc): its convolutions take the im2col route as three
    # TF32 products per term, 1x1 stride-1 layers the fp32 GEMM; nothing falls to the general kernel; 1e-5 like the fp32 GEMM
    g = rng(1264)
    n = 2
    x = g.uniform(-1, 1, (n, 32, 32, 3)).astype(np.float32)
    w1 = (g.standard_normal((7, 7, 3, 64)) * np.sqrt(2.0 / 147)).astype(np.float32)
    w2 = (g.standard_normal((1, 1, 64, 32)) * np.sqrt(2.0 / 64)).astype(np.float32)
    w3 = (g.standard_normal((3, 3, 32, 32)) * np.sqrt(2.0 / 288)).astype(np.float32)
    w4 = (g.standard_normal((1, 1, 64, 32)) * np.sqrt(2.0 / 64)).astype(np.float32)
    b1 = g.standard_normal(64).astype(np.float32) * 0.1
    b3 = g.standard_normal(32).astype(np.float32) * 0.1
    I = Placeholder(DType.FLOAT32, list(x.shape))
    y = op.relu(op.convolution(I, edsl.Constant(w1, name="w1"), strides=[2, 2], autopad_mode=op.AutoPadMode.EXPLICIT,
                               manual_padding=[3, 3, 3, 3]) + edsl.Constant(b1, name="b1"))
    y = op.pool(y, op.PoolMode.MAX, [3, 3], [2, 2], op.AutoPadMode.EXPLICIT, [1, 1, 1, 1], op.TensorLayout.NXC)
    z = op.relu(op.convolution(y, edsl.Constant(w2, name="w2")))
    z = op.convolution(z, edsl.Constant(w3, name="w3"), strides=[2, 2], autopad_mode=op.AutoPadMode.EXPLICIT,
                       manual_padding=[1, 1, 1, 1]) + edsl.Constant(b3, name="b3")
    sc = op.convolution(y, edsl.Constant(w4, name="w4"), strides=[2, 2], autopad_mode=op.AutoPadMode.VALID)
    O = op.relu(z + sc)
    runner = Runner(Program("fp32_block", [I], [O]), "cuda.0")
    desc = runner.executable.describe()
    assert "generic_contract" not in desc and desc.count("tc_conv") >= 3 and "tc_gemm" in desc, desc
    got = runner.run([x])[0]
    r1 = oracle.conv2d_nhwc_f32(x, w1, b1, None, (2, 2), (3, 3), (1, 1), True)
    r1 = oracle.pool2d_nhwc_f32(r1, "max", (3, 3), (2, 2), (1, 1), (8, 8))
    r2 = oracle.conv2d_nhwc_f32(r1, w2, None, None, (1, 1), (0, 0), (1, 1), True)
    r3 = oracle.conv2d_nhwc_f32(r2, w3, b3, None, (2, 2), (1, 1))
    r4 = oracle.conv2d_nhwc_f32(r1, w4, None, None, (2, 2))
    check_close(got, np.maximum(r3 + r4, 0), 2e-5)


def _stem_program(n, h, with_side_output=False, w_img=224):
    g = rng(1251)
    w = f32_to_bf16_bits(g.standard_normal((7, 7, 3, 64)) * np.sqrt(2.0 / 147))
    b = (g.standard_normal(64) * 0.1).astype(np.float32)
    I = Placeholder(DType.BFLOAT16, [n, h, w_img, 3])
    F = cast(edsl.Constant(w, name="w", dtype=DType.BFLOAT16), DType.FLOAT32)
    y = op.convolution(cast(I, DType.FLOAT32), F, strides=[2, 2], autopad_mode=op.AutoPadMode.EXPLICIT,
                       manual_padding=[3, 3, 3, 3]) + edsl.Constant(b, name="b")
    y = cast(op.relu(y), DType.BFLOAT16)
    pooled = op.pool(y, op.PoolMode.MAX, [3, 3], [2, 2], op.AutoPadMode.EXPLICIT, [1, 1, 1, 1], op.TensorLayout.NXC)
    x = f32_to_bf16_bits(g.uniform(-1, 1, (n, h, w_img, 3)).astype(np.float32))
    return Program("stem", [I], [pooled, y] if with_side_output else [pooled]), x, w, b


def test_first_convolution_and_its_max_pool_run_as_one_kernel(monkeypatch):
    # conv 7x7/2 + bias + ReLU + cast -> max pool 3x3/2 pad 1: one step whose output is the pooled tensor;
    # same values as the two separate steps, and as the oracle's convolution followed by its pool
    prog, x, w, b = _stem_program(5, 96)
    runner = Runner(prog, "cuda.0")
    desc = runner.executable.describe()
    assert "tc_conv_s2d_pool" in desc and "+maxpool3x3/2" in desc and "nhwc_pool" not in desc, desc
    got = bf16_bits_to_f32(runner.run([x])[0])
    conv = oracle.conv2d_nhwc_f32(bf16_bits_to_f32(x), bf16_bits_to_f32(w), b, None, (2, 2), (3, 3), (1, 1), True, out_hw=(48, 112))
    conv = oracle.bf16_to_f32(oracle.f32_to_bf16(conv))
    ref = oracle.pool2d_nhwc_f32(conv, "max", (3, 3), (2, 2), (1, 1), (24, 56))
    check_close(got, ref, 1e-2)
    monkeypatch.setenv("PLAIDML_CUDA_NO_POOL_FUSION", "1")
    two = Runner(_stem_program(5, 96)[0], "cuda.0")
    desc2 = two.executable.describe()
    assert "tc_conv_s2d " in desc2 and "nhwc_pool" in desc2, desc2
    got2 = bf16_bits_to_f32(two.run([x])[0])
    check_close(got, got2, 1e-2)
    assert (got != got2).mean() < 0.02
    monkeypatch.delenv("PLAIDML_CUDA_NO_POOL_FUSION")
    # the convolution's output read by anything else (here: a program output) keeps the two steps
    prog, x, _, _ = _stem_program(2, 64, with_side_output=True)
    both = Runner(prog, "cuda.0")
    assert "nhwc_pool" in both.executable.describe() and "tc_conv_s2d_pool" not in both.executable.describe()
    pooled, y = both.run([x])
    ref = oracle.pool2d_nhwc_f32(bf16_bits_to_f32(y), "max", (3, 3), (2, 2), (1, 1), (16, 56))
    np.testing.assert_array_equal(bf16_bits_to_f32(pooled), ref)
    # rows of the packed activation that are not 128 positions wide (a 96-wide image) keep the two steps, too
    narrow = Runner(_stem_program(2, 64, w_img=96)[0], "cuda.0")
    assert "nhwc_pool" in narrow.executable.describe() and "tc_conv_s2d_pool" not in narrow.executable.describe()


def test_mean_tail_folds_into_the_reduction():
    # sum -> / count -> cast back to bf16 (the global average pool of a bf16 network): one kernel that divides its
    # f32 sum by the count and rounds once; the same values as the three separate steps (general kernels)
    g = rng(1242)
    x = f32_to_bf16_bits(g.standard_normal((3, 7, 7, 32)))
    I = Placeholder(DType.BFLOAT16, x.shape)
    mean = op.mean(cast(I, DType.FLOAT32), axes=[1, 2])
    O = cast(mean, DType.BFLOAT16)
    runner = Runner(Program("gap", [I], [O]), "cuda.0")
    desc = runner.executable.describe()
    assert desc.count("\n") == 1 and "strided_reduce" in desc and "+div+cast" in desc, desc
    got = runner.run([x])[0]
    sums = bf16_bits_to_f32(x).astype(np.float32).sum(axis=(1, 2), dtype=np.float64)
    ref = f32_to_bf16_bits((sums.astype(np.float32) / np.float32(49)).astype(np.float32))
    # (the f32 sum's rounding depends on the summation order: allow one bf16 ulp)
    assert np.abs(got.astype(np.int32) - ref.astype(np.int32)).max() <= 1
    # a mean that stays f32 folds the division only, and a mean that is itself an output is not folded past
    runner = Runner(Program("gap32", [I], [mean]), "cuda.0")
    assert "+div" in runner.executable.describe() and "+cast" not in runner.executable.describe()
    np.testing.assert_allclose(runner.run([x])[0], sums / 49.0, rtol=1e-5, atol=1e-6)


def test_avgpool_counts_only_in_range_taps():
    g = rng(1240)
    x = g.standard_normal((1, 7, 7, 4)).astype(np.float32)
    I = Placeholder(DType.FLOAT32, x.shape)
    O = op.pool(I, op.PoolMode.AVG, [3, 3], [1, 1], op.AutoPadMode.SAME_UPPER, [], op.TensorLayout.NXC)
    got = Runner(Program("avgpool", [I], [O]), "cuda.0").run([x])[0]
    ref = oracle.pool2d_nhwc_f32(x, "sum", (3, 3), (1, 1), (1, 1), (7, 7), average=True)
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-6)


def test_residual_block_fusion_and_order(monkeypatch):
    # relu(conv_c(x) + bias + shortcut(x)) with the shortcut branch lowered after the main one
    g = rng(1241)
    n, h, w, c, k = 2, 14, 14, 64, 128
    x = f32_to_bf16_bits(g.uniform(0, 1, size=(n, h, w, c)))
    f1 = f32_to_bf16_bits(g.standard_normal((1, 1, c, k)) * np.sqrt(2.0 / c))
    f2 = f32_to_bf16_bits(g.standard_normal((1, 1, c, k)) * np.sqrt(2.0 / c))
    b1 = (g.standard_normal(k) * 0.1).astype(np.float32)
    I = Placeholder(DType.BFLOAT16, [n, h, w, c])
    xi = cast(I, DType.FLOAT32)
    F1 = cast(edsl.Constant(f1, dtype=DType.BFLOAT16), DType.FLOAT32)
    F2 = cast(edsl.Constant(f2, dtype=DType.BFLOAT16), DType.FLOAT32)
    main = op.convolution(xi, F1, name="main") + edsl.Constant(b1)
    short = cast(cast(op.convolution(xi, F2, name="shortcut"), DType.BFLOAT16), DType.FLOAT32)
    O = cast(op.relu(main + short), DType.BFLOAT16)
    xf = bf16_bits_to_f32(x)
    sc = bf16_bits_to_f32(f32_to_bf16_bits(oracle.conv2d_nhwc_f32(xf, bf16_bits_to_f32(f2))))
    ref = oracle.conv2d_nhwc_f32(xf, bf16_bits_to_f32(f1), b1, sc, relu=True)
    # the shortcut is a projection of the same rows: it joins the main product in one GEMM over [x | x]
    runner = Runner(Program("block", [I], [O]), "cuda.0")
    desc = runner.executable.describe()
    assert desc.count("tc_gemm") == 1 and "+bias+shortcut(k64)+relu+cast" in desc, desc
    check_close(bf16_bits_to_f32(runner.run([x])[0]), bf16_bits_to_f32(f32_to_bf16_bits(ref)), 1e-2)
    # ... and as the residual of the main product when that fusion is off
    monkeypatch.setenv("PLAIDML_CUDA_NO_SHORTCUT_FUSION", "1")
    runner = Runner(Program("block", [I], [O]), "cuda.0")
    desc = runner.executable.describe()
    assert "+bias+residual+relu+cast" in desc, desc
    got = bf16_bits_to_f32(runner.run([x])[0])
    check_close(got, bf16_bits_to_f32(f32_to_bf16_bits(ref)), 1e-2)


def test_run_argument_checks_and_timing():
    A, B, C = P.tile_gemm(DType.FLOAT32, 16, 16, 16)
    program = Program("chk", [A, B], [C]).compile("cuda")
    exe = Executable(program, "cuda.0")
    a = Buffer(program.inputs[0])
    b = Buffer(program.inputs[1])
    c = Buffer(program.outputs[0])
    ms = exe.run([a, b], [c])
    assert ms > 0
    with pytest.raises(core.Error, match="expects 2 inputs"):
        exe.run([a], [c])
    wrong = Buffer(core.TensorShape(DType.FLOAT32, [16, 8]))
    with pytest.raises(core.Error, match="Shape mismatch"):
        exe.run([a, wrong], [c])
    assert exe.run_resident(3) > 0 and exe.launch_count >= 1


def test_reshaped_outputs_and_constants_on_either_side():
    # an output that is a reshaped view (or a reshape that changes nothing) is copied through tile.ident, and a
    # commutative operation keeps its scalar constant on the right whichever way it was written
    g = rng(77)
    a = g.standard_normal((4, 6)).astype(np.float32)
    A = Placeholder(DType.FLOAT32, [4, 6])
    outs = [edsl.reshape(A, [3, 8]), edsl.reshape(A, [4, 6]), 2.0 * A, A * 2.0, 1.0 - A, edsl.reshape(A + 1.0, [24])]
    prog = Program("views", [A], outs)
    text = str(prog)
    assert text.count("tile.ident") == 3 and text.count("tile.reshape") == 2
    assert text.count("tile.mul %arg0, %cst") == 2
    got = Runner(prog, "cuda.0").run([a])
    np.testing.assert_array_equal(got[0], a.reshape(3, 8))
    np.testing.assert_array_equal(got[1], a)
    np.testing.assert_array_equal(got[2], 2.0 * a)
    np.testing.assert_array_equal(got[3], 2.0 * a)
    np.testing.assert_array_equal(got[4], 1.0 - a)
    np.testing.assert_array_equal(got[5], (a + 1.0).reshape(24))


def test_shape_and_trace_run():
    # tile.shape is known when the program is built (nothing runs for it); tile.pragma runs as a copy of its operand
    g = rng(78)
    a = g.standard_normal((2, 3)).astype(np.float32)
    A = Placeholder(DType.FLOAT32, [2, 3])
    prog = Program("shape_trace", [A], [edsl.shape(A), edsl.trace(A * 2.0, "after doubling"), edsl.trace(A, "input")])
    text = str(prog)
    assert "tile.shape %arg0" in text and text.count("tile.pragma") == 2 and 'msg = "input"' in text
    got = Runner(prog, "cuda.0").run([a])
    np.testing.assert_array_equal(got[0], np.array([2, 3], np.int32))
    np.testing.assert_array_equal(got[1], a * 2.0)
    np.testing.assert_array_equal(got[2], a)


def test_uploads_of_late_inputs_overlap_the_kernels_and_results_follow_the_inputs():
    # x . W1 . W2 ... W6 with every weight a program INPUT (as the reference's network builders pass them): the
    # weights are first needed at increasing depths, so the run uploads them in groups and starts each part of the
    # kernel sequence when its group is there.  Every run gets new contents for every input; a step that started
    # before its weights arrived would multiply by the previous run's.
    from plaidml_b200 import op
    n, depth = 1024, 6
    X = Placeholder(DType.FLOAT32, [256, n])
    Ws = [Placeholder(DType.FLOAT32, [n, n]) for _ in range(depth)]
    y = X
    for W in Ws:
        y = op.dot(y, W)
    r = Runner(Program("chain", [X] + Ws, [y]), "cuda.0")
    g = rng(77)
    for run in range(4):
        x = g.standard_normal((256, n)).astype(np.float32)
        ws = [(g.standard_normal((n, n)) / np.sqrt(n)).astype(np.float32) for _ in range(depth)]
        out, = r.run([x] + ws)
        ref = x.astype(np.float64)
        for w in ws:
            ref = ref @ w.astype(np.float64)
        check_close(out, ref, 1e-4)
        assert r.executable.upload_groups >= 2, r.executable.upload_groups
    assert r.executable.uses_graph


def test_upload_overlap_can_be_turned_off():
    from plaidml_b200 import op
    from plaidml_b200.core import settings_set
    settings_set("PLAIDML_CUDA_UPLOAD_OVERLAP", "0")
    try:
        A = Placeholder(DType.FLOAT32, [256, 1024])
        B = Placeholder(DType.FLOAT32, [1024, 2048])
        C = Placeholder(DType.FLOAT32, [2048, 2048])
        r = Runner(Program("two", [A, B, C], [op.dot(op.dot(A, B), C)]), "cuda.0")
        g = rng(78)
        a, b, c = (g.standard_normal(s).astype(np.float32) for s in ((256, 1024), (1024, 2048), (2048, 2048)))
        out, = r.run([a, b, c])
        check_close(out, (a.astype(np.float64) @ b) @ c, 1e-4)
        assert r.executable.upload_groups == 1
    finally:
        settings_set("PLAIDML_CUDA_UPLOAD_OVERLAP", "1")


def test_an_input_no_operation_reads_is_accepted_and_left_on_the_host():
    # (the reference's ResNet-50 builder lists its 108 weight tensors as inputs although its operations use constants)
    A = Placeholder(DType.FLOAT32, [64, 64])
    unused = Placeholder(DType.FLOAT32, [4096, 4096])
    B = Placeholder(DType.FLOAT32, [64, 64])
    r = Runner(Program("unused", [A, unused, B], [A + B]), "cuda.0")
    g = rng(79)
    a, b = g.standard_normal((64, 64)).astype(np.float32), g.standard_normal((64, 64)).astype(np.float32)
    out, = r.run([a, np.full((4096, 4096), np.nan, dtype=np.float32), b])
    np.testing.assert_array_equal(out, a + b)
