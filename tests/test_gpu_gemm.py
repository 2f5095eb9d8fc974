"""Parity of the tcgen05 GEMM kernels with the CPU oracle, through the kernel C ABI."""

import numpy as np
import pytest
import torch

import oracle
from plaidml_b200 import kernels as K
from gpu_util import as_f32, bits16, check_close, dev, dev_bf16, empty, max_rel, ptr, rng

pytestmark = pytest.mark.gpu


def run_gemm(in_dtype, out_dtype, a_t, b_t, m, n, k, batch=1, b_is_nk=True, epilogue=0, bias=None, residual=None,
             tile_n=0, flags=0, stride_a=None, stride_b=None, want_rowmax=False, store=True):
    d = K.GemmDesc()
    d.in_dtype, d.out_dtype = in_dtype, out_dtype
    d.m, d.n, d.k, d.batch = m, n, k, batch
    d.lda = k
    d.ldb = k if b_is_nk else n
    d.ldc = n
    d.stride_a = m * k if stride_a is None else stride_a
    d.stride_b = n * k if stride_b is None else stride_b
    d.stride_c = m * n
    d.b_is_nk = int(b_is_nk)
    d.epilogue = epilogue
    d.ldr, d.stride_r = n, m * n
    d.tile_n, d.flags = tile_n, flags
    plan = K.Plan("gemm", d)
    c = empty((batch, m, n), out_dtype) if store else None
    if c is not None:
        c.fill_(0)
    rowmax = empty((batch, m), K.F32) if want_rowmax else None
    plan.gemm(ptr(a_t), ptr(b_t), ptr(c), ptr(bias), ptr(residual), ptr(rowmax))
    plan.check()
    return c, rowmax, plan


def bf16_case(seed, m, n, k, batch=1, b_is_nk=True, **kw):
    g = rng(seed)
    a = dev_bf16(g.standard_normal((batch, m, k)))
    bshape = (batch, n, k) if b_is_nk else (batch, k, n)
    b = dev_bf16(g.standard_normal(bshape))
    c, _, plan = run_gemm(K.BF16, K.F32, a, b, m, n, k, batch, b_is_nk, **kw)
    ref = oracle.gemm_h16_f32(bits16(a), bits16(b), False, b_is_nk)
    return c.cpu().numpy(), ref, plan


# --- bf16, both operands K-major (the Q.K^T shape) -------------------------------------

def test_bf16_nt_single_tile():
    c, ref, plan = bf16_case(1, 128, 128, 64)
    assert plan.kernel == "tc_gemm"
    check_close(c, ref, 1e-4)


def test_bf16_nt_multi_kblock():
    c, ref, _ = bf16_case(2, 128, 128, 512)
    check_close(c, ref, 1e-4)


@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_bf16_nt_multi_tile(tile_n):
    c, ref, _ = bf16_case(3, 384, 512, 256, tile_n=tile_n)
    check_close(c, ref, 1e-4)


def test_bf16_nt_ragged():
    # M, N not multiples of the tile; K not a multiple of the 64-element k-block
    c, ref, _ = bf16_case(4, 200, 136, 72)
    check_close(c, ref, 1e-4)


def test_bf16_nt_batched_many_tiles():
    # more tiles than SMs: every CTA walks several tiles and both TMEM accumulators
    c, ref, _ = bf16_case(5, 256, 256, 128, batch=40)
    check_close(c, ref, 1e-4)


def test_bf16_nt_shared_b():
    g = rng(6)
    a = dev_bf16(g.standard_normal((3, 130, 64)))
    b = dev_bf16(g.standard_normal((1, 96, 64)))
    c, _, _ = run_gemm(K.BF16, K.F32, a, b, 130, 96, 64, batch=3, stride_b=0)
    ref = oracle.gemm_h16_f32(bits16(a), bits16(b), False, True)
    check_close(c.cpu().numpy(), ref, 1e-4)


# --- bf16, B stored [k][n] (the Tile GEMM C[i,j] += A[i,k] * B[k,j]) ---------------------

@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_bf16_nn(tile_n):
    c, ref, _ = bf16_case(7, 256, 512, 192, b_is_nk=False, tile_n=tile_n)
    check_close(c, ref, 1e-4)


def test_bf16_nn_ragged():
    c, ref, _ = bf16_case(8, 130, 200, 88, b_is_nk=False)
    check_close(c, ref, 1e-4)


def test_bf16_nn_via_transposed_scratch():
    c, ref, plan = bf16_case(9, 256, 320, 136, b_is_nk=False, flags=K.GEMM_TRANSPOSE_B)
    assert plan.scratch_bytes > 0
    check_close(c, ref, 1e-4)


# --- epilogues -----------------------------------------------------------------------------

def test_bf16_bias_relu_bf16_out():
    g = rng(10)
    m, n, k = 256, 192, 128
    a = dev_bf16(g.standard_normal((1, m, k)))
    b = dev_bf16(g.standard_normal((1, n, k)))
    bias = dev(g.standard_normal(n).astype(np.float32))
    res = dev_bf16(g.standard_normal((1, m, n)))
    c, _, _ = run_gemm(K.BF16, K.BF16, a, b, m, n, k, epilogue=K.EPI_BIAS | K.EPI_RESIDUAL | K.EPI_RELU,
                       bias=bias, residual=res)
    ref = oracle.gemm_h16_f32(bits16(a), bits16(b), False, True)
    ref = ref + bias.cpu().numpy()[None, None, :] + as_f32(res)
    ref = np.where(ref < 0, 0, ref)
    ref_bf16 = oracle.bf16_to_f32(oracle.f32_to_bf16(ref))
    # 1e-2 relative: the stated tolerance for bf16 results (one bf16 ulp is 2^-8)
    check_close(as_f32(c), ref_bf16, 1e-2)


def test_bf16_residual_partial_chunk_and_plain_stores():
    # N = 200 leaves a partial 64-column chunk; the same case through the plain-store epilogue
    g = rng(13)
    m, n, k = 160, 200, 64
    a = dev_bf16(g.standard_normal((2, m, k)))
    b = dev_bf16(g.standard_normal((2, n, k)))
    bias = dev(g.standard_normal(n).astype(np.float32))
    res = dev_bf16(g.standard_normal((2, m, n)))
    ref = oracle.gemm_h16_f32(bits16(a), bits16(b), False, True)
    ref = ref + bias.cpu().numpy()[None, None, :] + as_f32(res)
    ref = oracle.bf16_to_f32(oracle.f32_to_bf16(np.where(ref < 0, 0, ref)))
    outs = []
    for flags in (0, K.GEMM_PLAIN_STORES, K.GEMM_PLAIN_RESIDUAL):
        c, _, _ = run_gemm(K.BF16, K.BF16, a, b, m, n, k, batch=2, flags=flags,
                           epilogue=K.EPI_BIAS | K.EPI_RESIDUAL | K.EPI_RELU, bias=bias, residual=res)
        check_close(as_f32(c), ref, 1e-2)
        outs.append(bits16(c))
    np.testing.assert_array_equal(outs[0], outs[1])   # all three epilogue routes round identically
    np.testing.assert_array_equal(outs[0], outs[2])


@pytest.mark.parametrize("k,tile_n", [(64, 0), (64, 128), (1664, 256), (192, 64)])
def test_bf16_residual_many_tiles_per_sm(k, tile_n):
    # more tiles than SMs (each CTA walks several, so the residual buffers and their barriers wrap many
    # times), ragged M and N; short and long main loops take the two-group and one-group epilogues
    g = rng(40 + k)
    m, n = 128 * 150 + 40, 456
    a = dev_bf16(g.standard_normal((1, m, k)))
    b = dev_bf16(g.standard_normal((1, n, k)) * 0.1)
    res = dev_bf16(g.standard_normal((1, m, n)))
    bias = dev(g.standard_normal(n).astype(np.float32))
    outs = []
    for flags in (0, K.GEMM_PLAIN_RESIDUAL):
        c, _, _ = run_gemm(K.BF16, K.BF16, a, b, m, n, k, flags=flags, tile_n=tile_n,
                           epilogue=K.EPI_BIAS | K.EPI_RESIDUAL | K.EPI_RELU, bias=bias, residual=res)
        outs.append(bits16(c))
    np.testing.assert_array_equal(outs[0], outs[1])
    ref = oracle.gemm_h16_f32(bits16(a), bits16(b), False, True)
    ref = ref + bias.cpu().numpy()[None, None, :] + as_f32(res)
    ref = oracle.bf16_to_f32(oracle.f32_to_bf16(np.where(ref < 0, 0, ref)))
    check_close(oracle.bf16_to_f32(outs[0]), ref, 1e-2)


def test_f32_out_residual_f32():
    g = rng(14)
    m, n, k = 256, 128, 64
    a = dev_bf16(g.standard_normal((1, m, k)))
    b = dev_bf16(g.standard_normal((1, n, k)))
    res = dev(g.standard_normal((1, m, n)).astype(np.float32))
    c, _, _ = run_gemm(K.BF16, K.F32, a, b, m, n, k, epilogue=K.EPI_RESIDUAL, residual=res)
    ref = oracle.gemm_h16_f32(bits16(a), bits16(b), False, True) + res.cpu().numpy()
    check_close(c.cpu().numpy(), ref, 1e-4)


def test_int8_bias_relu_residual_exact():
    g = rng(15)
    m, n, k = 256, 160, 128
    a = g.integers(-128, 128, size=(1, m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(1, n, k), dtype=np.int8)
    bias = g.integers(-1000, 1000, size=n, dtype=np.int32)
    res = g.integers(-100000, 100000, size=(1, m, n), dtype=np.int32)
    c, _, _ = run_gemm(K.I8, K.I32, dev(a), dev(b), m, n, k, bias=dev(bias), residual=dev(res),
                       epilogue=K.EPI_BIAS | K.EPI_RESIDUAL | K.EPI_RELU)
    ref = oracle.gemm_i8_i32(a, b, True) + bias[None, None, :] + res
    np.testing.assert_array_equal(c.cpu().numpy(), np.maximum(ref, 0))


def test_f16_nt():
    g = rng(11)
    m, n, k = 128, 128, 128
    a = dev(g.standard_normal((1, m, k)).astype(np.float16))
    b = dev(g.standard_normal((1, n, k)).astype(np.float16))
    c, _, _ = run_gemm(K.F16, K.F32, a, b, m, n, k)
    ref = oracle.gemm_h16_f32(bits16(a), bits16(b), True, True)
    check_close(c.cpu().numpy(), ref, 1e-4)


def test_bf16_rowmax_epilogue():
    g = rng(12)
    batch, m, n, k = 4, 256, 512, 64
    a = dev_bf16(g.standard_normal((batch, m, k)))
    b = dev_bf16(g.standard_normal((batch, n, k)))
    c, rowmax, _ = run_gemm(K.BF16, K.F32, a, b, m, n, k, batch=batch, epilogue=K.EPI_ROWMAX, want_rowmax=True)
    s = c.cpu().numpy()
    # exact given identical S: the fused max sees the same f32 values that were stored
    np.testing.assert_array_equal(rowmax.cpu().numpy(), s.max(axis=2))
    _, rowmax2, _ = run_gemm(K.BF16, K.F32, a, b, m, n, k, batch=batch, epilogue=K.EPI_ROWMAX, want_rowmax=True,
                             store=False)
    np.testing.assert_array_equal(rowmax2.cpu().numpy(), s.max(axis=2))


# --- int8 -> int32, bit exact ---------------------------------------------------------------

def int8_case(seed, m, n, k, b_is_nk, **kw):
    g = rng(seed)
    a = g.integers(-128, 128, size=(1, m, k), dtype=np.int8)
    bshape = (1, n, k) if b_is_nk else (1, k, n)
    b = g.integers(-128, 128, size=bshape, dtype=np.int8)
    c, _, plan = run_gemm(K.I8, K.I32, dev(a), dev(b), m, n, k, 1, b_is_nk, **kw)
    return c.cpu().numpy(), oracle.gemm_i8_i32(a, b, b_is_nk), plan


def test_int8_nt_exact():
    c, ref, _ = int8_case(20, 256, 256, 512, True)
    np.testing.assert_array_equal(c, ref)


@pytest.mark.parametrize("tile_n", [128, 256])
def test_int8_nn_exact(tile_n):
    c, ref, _ = int8_case(21, 384, 512, 384, False, tile_n=tile_n)
    np.testing.assert_array_equal(c, ref)


def test_int8_nn_ragged_exact():
    c, ref, _ = int8_case(22, 200, 144, 208, False)
    np.testing.assert_array_equal(c, ref)


def test_int8_nn_via_transposed_scratch_exact():
    c, ref, _ = int8_case(23, 256, 256, 256, False, flags=K.GEMM_TRANSPOSE_B)
    np.testing.assert_array_equal(c, ref)


def test_int8_wraps_to_int8():
    # int8 (*) int8 without casts yields int8: the 32-bit sum truncated (GEMM_INT8 of
    # plaidml/edsl/examples/gemm.cc)
    g = rng(24)
    m = n = k = 128
    a = g.integers(-128, 128, size=(1, m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(1, n, k), dtype=np.int8)
    c, _, _ = run_gemm(K.I8, K.I8, dev(a), dev(b), m, n, k)
    ref = oracle.gemm_i8_i32(a, b, True).astype(np.int8)
    np.testing.assert_array_equal(c.cpu().numpy(), ref)


def test_int8_to_int8_relu_acts_on_the_wrapped_value():
    # sums far outside int8: the result is the sum wrapped to 8 bits, and the ReLU sees that value
    # (acc = 200 wraps to -56, then ReLU gives 0; a ReLU taken on the 32-bit sum would store -56)
    g = rng(25)
    m = n = 128
    k = 256
    a = g.integers(-128, 128, size=(1, m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(1, n, k), dtype=np.int8)
    c, _, _ = run_gemm(K.I8, K.I8, dev(a), dev(b), m, n, k, epilogue=K.EPI_RELU)
    wrapped = oracle.gemm_i8_i32(a, b, True).astype(np.int8)
    assert (wrapped < 0).mean() > 0.3 and (np.abs(oracle.gemm_i8_i32(a, b, True)) > 127).mean() > 0.9
    np.testing.assert_array_equal(c.cpu().numpy(), np.maximum(wrapped, 0))


def test_row_max_of_negative_zero():
    # a row whose largest element is -0.0: the atomic fold must rank it above every negative value
    m, n, k = 128, 512, 64
    a = np.zeros((1, m, k), dtype=np.float32)
    a[:, :, 0] = 1.0
    b = np.full((1, n, k), 0.0, dtype=np.float32)
    b[:, :, 0] = -1.0          # every product is -1 ...
    b[:, 300, :] = -0.0        # ... except one column whose products are all -0.0 (a sum of them stays -0.0)
    at, bt = dev_bf16(a), dev_bf16(b)
    c, rowmax, _ = run_gemm(K.BF16, K.F32, at, bt, m, n, k, epilogue=K.EPI_ROWMAX, want_rowmax=True)
    got = rowmax.cpu().numpy()
    assert np.all(got == 0.0) and np.all(c.cpu().numpy()[0, :, 300] == 0.0)
    assert np.all(c.cpu().numpy()[0, :, 299] == -1.0)


# --- K split over several CTAs per tile (two passes: partial products, then sum + epilogue) -------------

@pytest.mark.parametrize("b_is_nk", [True, False], ids=["B[n][k]", "B[k][n]"])
@pytest.mark.parametrize("out_dtype", [K.F32, K.BF16], ids=["f32_out", "bf16_out"])
def test_split_k_bf16_with_every_epilogue_term(b_is_nk, out_dtype):
    g = rng(40)
    m, n, k = 200, 328, 1024                      # ragged M and N; 16 k-blocks -> 8 parts when forced
    a = dev_bf16(g.standard_normal((1, m, k)))
    b = dev_bf16(g.standard_normal((1, n, k) if b_is_nk else (1, k, n)))
    bias = g.standard_normal(n).astype(np.float32)
    res_f32 = g.standard_normal((1, m, n)).astype(np.float32) * 8
    res = dev(res_f32) if out_dtype == K.F32 else dev_bf16(res_f32)
    epi = K.EPI_BIAS | K.EPI_RESIDUAL | K.EPI_RELU
    outs = {}
    for name, flags in (("split", K.GEMM_SPLIT_K), ("single", K.GEMM_NO_SPLIT_K)):
        c, _, plan = run_gemm(K.BF16, out_dtype, a, b, m, n, k, 1, b_is_nk, epilogue=epi, bias=dev(bias), residual=res, flags=flags)
        assert plan.split_k == (8 if name == "split" else 1)
        outs[name] = as_f32(c)
    ref = oracle.gemm_h16_f32(bits16(a), bits16(b), False, b_is_nk) + bias + as_f32(res)
    ref = np.maximum(ref, 0)
    if out_dtype == K.F32:
        check_close(outs["split"], ref, 1e-4)
        check_close(outs["split"], outs["single"], 1e-5)
    else:
        check_close(outs["split"], oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)


def test_split_k_int8_is_bit_exact_and_chosen_for_few_tiles():
    g = rng(41)
    m, n, k = 256, 256, 4096                      # four 128-wide tiles, 32 k-blocks: the library splits by itself
    a = g.integers(-128, 128, size=(1, m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(1, k, n), dtype=np.int8)
    bias = g.integers(-1000, 1000, size=n).astype(np.int32)
    c, _, plan = run_gemm(K.I8, K.I32, dev(a), dev(b), m, n, k, 1, False, epilogue=K.EPI_BIAS | K.EPI_RELU, bias=dev(bias))
    assert plan.split_k == 8 and plan.scratch_bytes == 8 * m * n * 4
    ref = np.maximum(oracle.gemm_i8_i32(a, b, False) + bias, 0)
    np.testing.assert_array_equal(c.cpu().numpy(), ref)
    # int8 result: the wrapped sum, then the ReLU
    c8, _, plan8 = run_gemm(K.I8, K.I8, dev(a), dev(b), m, n, k, 1, False, epilogue=K.EPI_RELU)
    assert plan8.split_k == 8
    np.testing.assert_array_equal(c8.cpu().numpy(), np.maximum(oracle.gemm_i8_i32(a, b, False).astype(np.int8), 0))
    # many tiles: one pass
    _, _, big = run_gemm(K.I8, K.I32, dev(g.integers(-128, 128, size=(1, 4096, 512), dtype=np.int8)),
                         dev(g.integers(-128, 128, size=(1, 512, 2048), dtype=np.int8)), 4096, 2048, 512, 1, False)
    assert big.split_k == 1


def test_split_k_f16_skinny_fc_shape():
    # the shape of a classifier head at a small batch: 32 x 1000 x 2048, B stored [k][n]
    g = rng(42)
    m, n, k = 32, 1000, 2048
    a16 = g.standard_normal((1, m, k)).astype(np.float16)
    b16 = (g.standard_normal((1, k, n)) * 0.03).astype(np.float16)
    bias = g.standard_normal(n).astype(np.float32)
    c, _, plan = run_gemm(K.F16, K.F32, dev(a16), dev(b16), m, n, k, 1, False, epilogue=K.EPI_BIAS, bias=dev(bias))
    assert plan.split_k == 8
    ref = a16[0].astype(np.float64) @ b16[0].astype(np.float64) + bias
    assert max_rel(c.cpu().numpy()[0], ref) < 1e-5


# --- bounded waits -------------------------------------------------------------------------------------

def test_a_wait_that_runs_out_ends_the_launch_with_a_status_and_the_plan_stays_usable():
    # Every device-side wait of the kernel is bounded.  The plan is armed so that, in its next launch, the first
    # CTA's producer never issues its first operand load and waits give up after 5 ms: the issuer's wait for
    # that stage runs out, the CTA's roles leave through the tear-down (no trap, nothing left spinning), the
    # launch returns and the status word says so.  The launch after it is an ordinary one and must be correct.
    import time
    g = rng(45)
    m, n, k = 512, 256, 512
    a = g.integers(-128, 128, size=(1, m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(1, n, k), dtype=np.int8)
    d = K.GemmDesc()
    d.in_dtype, d.out_dtype = K.I8, K.I32
    d.m, d.n, d.k, d.batch = m, n, k, 1
    d.lda, d.ldb, d.ldc = k, k, n
    d.b_is_nk = 1
    d.flags = K.GEMM_NO_SPLIT_K | K.GEMM_NO_CTA_PAIRS
    plan = K.Plan("gemm", d)
    a_t, b_t = dev(a), dev(b)
    c = empty((1, m, n), K.I32)
    plan.arm_timeout_test(5)
    t0 = time.perf_counter()
    plan.gemm(ptr(a_t), ptr(b_t), ptr(c))
    with pytest.raises(K.KernelError) as err:
        plan.check()
    assert err.value.status == K.ERR_TIMEOUT and "gave up" in str(err.value)
    assert time.perf_counter() - t0 < 2.0            # milliseconds, not the two-second default
    # the context is intact and the same plan computes the right product
    c.fill_(0)
    plan.gemm(ptr(a_t), ptr(b_t), ptr(c))
    plan.check()
    np.testing.assert_array_equal(c.cpu().numpy(), oracle.gemm_i8_i32(a, b, True))


# --- fp32 as 3xTF32 ---------------------------------------------------------------------------

@pytest.mark.parametrize("b_is_nk", [True, False])
def test_f32_3xtf32(b_is_nk):
    g = rng(30)
    m, n, k = 256, 192, 320
    a = g.uniform(-1, 1, size=(1, m, k)).astype(np.float32)
    b = g.uniform(-1, 1, size=(1, n, k) if b_is_nk else (1, k, n)).astype(np.float32)
    c, _, plan = run_gemm(K.F32, K.F32, dev(a), dev(b), m, n, k, 1, b_is_nk)
    assert plan.scratch_bytes > 0
    ref64 = oracle.gemm_f32_acc64(a, b, b_is_nk)
    ref32 = oracle.gemm_f32(a, b, b_is_nk)
    err = max_rel(c.cpu().numpy(), ref64)
    err_cpu = max_rel(ref32, ref64)
    print(f"3xTF32 max-rel vs f64: {err:.3e}; f32 CPU loop vs f64: {err_cpu:.3e}")
    # 1e-5 relative: the tolerance the reference's own f32 Dot test uses (edsl_test.cc:448-486)
    assert err < 1e-5
    check_close(c.cpu().numpy(), ref32, 1e-5)


def test_f32_reference_microkernel_dot_on_the_tensor_cores():
    # the 8 x 8 product printed by the reference's x86 microkernel test (pmlc/target/x86/tests/xsmm_call.mlir):
    # integer-valued operands, so three TF32 products per term reproduce it exactly
    import json
    from pathlib import Path
    kat = {k["name"]: k for k in json.loads((Path(__file__).parent / "golden" / "reference_xsmm_kats.json").read_text())}["xsmm_dot_8x8"]
    a, b = (np.array(v, dtype=np.float32).reshape(1, 8, 8) for v in kat["inputs"])
    c, _, plan = run_gemm(K.F32, K.F32, dev(a), dev(b), 8, 8, 8, 1, False)
    assert plan.kernel == "tc_gemm"
    np.testing.assert_array_equal(c.cpu().numpy()[0], np.array(kat["outputs"][0], dtype=np.float32))


def test_f32_ragged():
    g = rng(31)
    m, n, k = 70, 50, 37
    a = g.uniform(-1, 1, size=(1, m, k)).astype(np.float32)
    b = g.uniform(-1, 1, size=(1, k, n)).astype(np.float32)
    c, _, _ = run_gemm(K.F32, K.F32, dev(a), dev(b), m, n, k, 1, False)
    assert max_rel(c.cpu().numpy(), oracle.gemm_f32_acc64(a, b, False)) < 1e-5


# --- CTA pairs (two CTAs per 256 x 256 tile) -----------------------------------------------------

@pytest.mark.parametrize("b_is_nk", [True, False], ids=["B[n][k]", "B[k][n]"])
def test_cta_pairs_bf16_matches_single_cta_and_oracle(b_is_nk):
    # ragged in M (the second CTA of the last pair has no rows), N and K; more pair tiles than clusters
    g = rng(50)
    m, n, k = 128 * 5 + 24, 256 * 3 + 72, 2048 + 40
    a = dev_bf16(g.standard_normal((1, m, k)))
    b = dev_bf16(g.standard_normal((1, n, k) if b_is_nk else (1, k, n)))
    outs = []
    for flags in (K.GEMM_CTA_PAIRS, K.GEMM_NO_CTA_PAIRS):
        c, _, _ = run_gemm(K.BF16, K.F32, a, b, m, n, k, b_is_nk=b_is_nk, tile_n=256, flags=flags)
        outs.append(c.cpu().numpy())
    ref = oracle.gemm_h16_f32(bits16(a), bits16(b), False, b_is_nk)
    check_close(outs[0], ref, 1e-4)
    np.testing.assert_array_equal(outs[0], outs[1])      # same products in the same order per element


@pytest.mark.parametrize("b_is_nk", [True, False], ids=["B[n][k]", "B[k][n]"])
def test_cta_pairs_int8_bit_exact(b_is_nk):
    g = rng(51)
    m, n, k = 1024 + 128, 512, 4096
    a = g.integers(-128, 128, size=(1, m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(1, n, k) if b_is_nk else (1, k, n), dtype=np.int8)
    c, _, _ = run_gemm(K.I8, K.I32, dev(a), dev(b), m, n, k, b_is_nk=b_is_nk, tile_n=256, flags=K.GEMM_CTA_PAIRS)
    np.testing.assert_array_equal(c.cpu().numpy(), oracle.gemm_i8_i32(a, b, b_is_nk))


def test_cta_pairs_batched_epilogue_bf16_out():
    g = rng(52)
    m, n, k = 384, 512, 1600
    a = dev_bf16(g.standard_normal((3, m, k)))
    b = dev_bf16(g.standard_normal((3, n, k)) * 0.05)
    bias = dev(g.standard_normal(n).astype(np.float32))
    res = dev_bf16(g.standard_normal((3, m, n)))
    c, _, _ = run_gemm(K.BF16, K.BF16, a, b, m, n, k, batch=3, tile_n=256, flags=K.GEMM_CTA_PAIRS,
                       epilogue=K.EPI_BIAS | K.EPI_RESIDUAL | K.EPI_RELU, bias=bias, residual=res)
    ref = oracle.gemm_h16_f32(bits16(a), bits16(b), False, True)
    ref = ref + bias.cpu().numpy()[None, None, :] + as_f32(res)
    ref = oracle.bf16_to_f32(oracle.f32_to_bf16(np.where(ref < 0, 0, ref)))
    check_close(as_f32(c), ref, 1e-2)


def test_large_gemm_chooses_cta_pairs_and_is_exact():
    # the headline shape takes the pair kernel by itself; int8 makes any slip visible
    g = rng(53)
    m = n = k = 4096
    a = g.integers(-128, 128, size=(1, m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(1, k, n), dtype=np.int8)
    c, _, _ = run_gemm(K.I8, K.I32, dev(a), dev(b), m, n, k, b_is_nk=False)
    rows = np.concatenate([np.arange(0, 300), np.arange(4096 - 300, 4096)])
    ref = oracle.gemm_i8_i32(np.ascontiguousarray(a[:, rows]), b, False)
    np.testing.assert_array_equal(c.cpu().numpy()[:, rows], ref)


# --- half-width tiles in a short last wave --------------------------------------------------------

@pytest.mark.parametrize("pairs", [False, True], ids=["one CTA per tile", "CTA pairs"])
@pytest.mark.parametrize("kind", ["bf16 B[n][k]", "bf16 B[k][n]", "int8 B[n][k]", "int8 B[k][n]"])
def test_split_tail_matches_whole_tiles(kind, pairs):
    # 168 tiles of 128 x 256 (84 pair tiles): one full wave on a 148-SM device plus a tail of 20 (10), which
    # is walked as half-width tiles; the result must not depend on it
    g = rng(60)
    m, n, k = 1536, 3584, 320
    b_is_nk = "[n][k]" in kind
    if kind.startswith("bf16"):
        a = dev_bf16(g.standard_normal((1, m, k)))
        b = dev_bf16(g.standard_normal((1, n, k) if b_is_nk else (1, k, n)))
        dt_in, dt_out = K.BF16, K.F32
    else:
        a = dev(g.integers(-128, 128, size=(1, m, k), dtype=np.int8))
        b = dev(g.integers(-128, 128, size=(1, n, k) if b_is_nk else (1, k, n), dtype=np.int8))
        dt_in, dt_out = K.I8, K.I32
    base = K.GEMM_CTA_PAIRS if pairs else K.GEMM_NO_CTA_PAIRS
    outs = []
    for flags in (base, base | K.GEMM_NO_TAIL_SPLIT):
        c, _, _ = run_gemm(dt_in, dt_out, a, b, m, n, k, b_is_nk=b_is_nk, tile_n=256, flags=flags)
        outs.append(c.cpu().numpy())
    np.testing.assert_array_equal(outs[0], outs[1])
    if dt_in == K.I8:
        ref = oracle.gemm_i8_i32(a.cpu().numpy(), b.cpu().numpy(), b_is_nk)
        np.testing.assert_array_equal(outs[0], ref)
    else:
        check_close(outs[0], oracle.gemm_h16_f32(bits16(a), bits16(b), False, b_is_nk), 1e-4)


def test_two_issuers_with_tiles_longer_than_the_ring():
    # 64-wide tiles have two MMA-issuing warps that take alternate tiles; with K = 1024 a tile is 16 stages, more
    # than two revolutions of the ring, and there are ten tiles per CTA.  Every stage is refilled only after both
    # warps have reported on it, so the warp that watches the other's tile go by can never fall a revolution
    # behind.  Repeated launches, bit-identical results, rows checked against the oracle.
    g = rng(4242)
    m, n, k = 50176, 256, 1024
    a = dev_bf16(g.standard_normal((1, m, k)))
    b = dev_bf16(g.standard_normal((1, n, k)) * 0.05)
    first = None
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for rep in range(12):
        flush.fill_(rep)
        c, _, plan = run_gemm(K.BF16, K.BF16, a, b, m, n, k, tile_n=64)
        got = bits16(c)
        if first is None:
            first = got
            assert "tc_gemm" in plan.kernel
        else:
            np.testing.assert_array_equal(got, first)
    rows = np.concatenate([np.arange(0, 256), np.arange(25000, 25128), np.arange(m - 128, m)])
    ref = oracle.gemm_h16_f32(bits16(a)[:, rows], bits16(b), False, True)
    check_close(oracle.bf16_to_f32(first[:, rows]), oracle.bf16_to_f32(oracle.f32_to_bf16(ref)), 1e-2)


@pytest.mark.parametrize("kind,m,n,k1,k2,b_is_nk,epi", [
    ("bf16", 300, 256, 64, 64, False, K.EPI_BIAS | K.EPI_RELU),        # a residual block's last 1x1 layer with its shortcut
    ("bf16", 1000, 512, 128, 256, False, K.EPI_BIAS | K.EPI_RELU),     # several k-blocks per part
    ("bf16", 4096, 1024, 256, 512, True, 0),                            # B as [n][k]; CTA pairs (256-wide tiles, 12 k-blocks)
    ("bf16", 640, 192, 128, 72, False, K.EPI_BIAS),                    # second part ends inside a k-block (zero fill)
    ("i8", 512, 256, 128, 384, False, 0),                               # int8, bit-exact
    ("i8", 4096, 4096, 2048, 2048, True, 0),                            # pairs, 32 k-blocks
])
def test_gemm_with_a_in_two_parts(kind, m, n, k1, k2, b_is_nk, epi):
    # C = [A1 | A2] * B with A1 and A2 separate matrices (own row strides): what sums a shortcut projection and a
    # block's last convolution in one accumulator; against the oracle on the concatenated operand
    g = rng(5200 + m + k2)
    k = k1 + k2
    bshape = (n, k) if b_is_nk else (k, n)
    d = K.GemmDesc()
    d.m, d.n, d.k, d.batch = m, n, k, 1
    d.lda, d.lda2, d.k_first = k1, k2 + 8 * (16 if kind == "i8" else 8), k1     # (the second part with padded rows)
    d.ldb, d.ldc = (k if b_is_nk else n), n
    d.stride_a, d.stride_b, d.stride_c = m * k1, n * k, m * n
    d.b_is_nk, d.epilogue = int(b_is_nk), epi
    d.ldr, d.stride_r = n, m * n
    bias = g.standard_normal(n).astype(np.float32) if epi & K.EPI_BIAS else None
    if kind == "i8":
        d.in_dtype, d.out_dtype = K.I8, K.I32
        a1 = g.integers(-128, 128, size=(m, k1), dtype=np.int8)
        a2 = np.zeros((m, d.lda2), dtype=np.int8)
        a2[:, :k2] = g.integers(-128, 128, size=(m, k2), dtype=np.int8)
        b = g.integers(-128, 128, size=bshape, dtype=np.int8)
        plan = K.Plan("gemm", d)
        out = empty((1, m, n), K.I32)
        a1d, a2d, bd = dev(a1), dev(a2), dev(b)
        plan.gemm_two(ptr(a1d), ptr(a2d), ptr(bd), ptr(out))
        plan.check()
        ref = oracle.gemm_i8_i32(np.concatenate([a1, a2[:, :k2]], axis=1), b, b_is_nk)
        np.testing.assert_array_equal(out.cpu().numpy()[0], ref)
        with pytest.raises(K.KernelError):
            plan.gemm(ptr(a1d), ptr(bd), ptr(out))          # the plain call has no second part to give
        return
    d.in_dtype, d.out_dtype = K.BF16, K.F32
    a1 = dev_bf16(g.standard_normal((m, k1)))
    a2_host = np.zeros((m, d.lda2), dtype=np.float32)
    a2_host[:, :k2] = g.standard_normal((m, k2))
    a2 = dev_bf16(a2_host)
    b = dev_bf16(g.standard_normal(bshape))
    plan = K.Plan("gemm", d)
    out = empty((1, m, n), K.F32)
    bias_dev = dev(bias) if bias is not None else None
    plan.gemm_two(ptr(a1), ptr(a2), ptr(b), ptr(out), ptr(bias_dev))
    plan.check()
    a_cat = np.concatenate([bits16(a1), bits16(a2)[:, :k2]], axis=1)
    ref = oracle.gemm_h16_f32(a_cat[None], bits16(b)[None], False, b_is_nk)[0].astype(np.float64)
    if bias is not None:
        ref = ref + bias[None, :]
    if epi & K.EPI_RELU:
        ref = np.maximum(ref, 0)
    check_close(out.cpu().numpy()[0], ref.astype(np.float32), 1e-4)


@pytest.mark.parametrize("n,h,w,c1,c2,k,stride,pairs", [
    (2, 28, 28, 128, 256, 512, 2, False),      # a block that halves the resolution: 392 rows, the last tile ragged
    (64, 28, 28, 128, 256, 512, 2, True),      # 12544 rows, 6 k-blocks, 256-wide tiles as CTA pairs
    (3, 15, 13, 64, 72, 128, 2, False),        # odd sizes (8 x 7 samples per image), channels ending inside a k-block
    (4, 7, 9, 64, 64, 64, 1, False),           # stride 1: the activation's pixels as they are
    (5, 20, 20, 64, 128, 256, 3, False),       # stride 3
])
def test_gemm_whose_second_part_of_a_is_an_activation_sampled_at_a_stride(n, h, w, c1, c2, k, stride, pairs):
    # C = [Y | sample(X)] * B: Y a matrix of m = n * P * Q rows, X an NHWC activation of which every stride-th pixel in
    # both directions is a row: the shortcut projection of a block that halves the resolution, inside the block's
    # last 1x1 layer
    g = rng(5300 + n + h)
    pp, qq = -(-h // stride), -(-w // stride)
    m = n * pp * qq
    y = dev_bf16(g.standard_normal((m, c1)))
    x = dev_bf16(g.standard_normal((n, h, w, c2)))
    b = dev_bf16(g.standard_normal((c1 + c2, k)) * 0.1)
    bias = g.standard_normal(k).astype(np.float32)
    d = K.GemmDesc()
    d.in_dtype, d.out_dtype = K.BF16, K.F32
    d.m, d.n, d.k, d.batch = m, k, c1 + c2, 1
    d.lda, d.k_first, d.ldb, d.ldc = c1, c1, k, k
    d.a2_stride, d.a2_n, d.a2_h, d.a2_w = stride, n, h, w
    d.stride_a, d.stride_b, d.stride_c = m * c1, (c1 + c2) * k, m * k
    d.b_is_nk, d.epilogue = 0, K.EPI_BIAS | K.EPI_RELU
    d.ldr, d.stride_r = k, m * k
    d.flags = K.GEMM_CTA_PAIRS if pairs else 0
    plan = K.Plan("gemm", d)
    out = empty((1, m, k), K.F32)
    out.fill_(float("nan"))
    bias_dev = dev(bias)
    plan.gemm_two(ptr(y), ptr(x), ptr(b), ptr(out), ptr(bias_dev))
    plan.check()
    sampled = bits16(x)[:, ::stride, ::stride, :].reshape(m, c2)
    a_cat = np.concatenate([bits16(y), sampled], axis=1)
    ref = oracle.gemm_h16_f32(a_cat[None], bits16(b)[None], False, False)[0].astype(np.float64) + bias[None, :]
    check_close(out.cpu().numpy()[0], np.maximum(ref, 0).astype(np.float32), 1e-4)
    # a pixel count that does not match m is refused
    d.a2_h = h + stride
    with pytest.raises(K.KernelError):
        K.Plan("gemm", d)
