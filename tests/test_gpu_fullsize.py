"""The metric's configurations at their full sizes, where the CPU oracle cannot compute the whole
result in seconds: sampled outputs against the oracle, and size-independent properties (two kernel
routes that must agree, a maximum that must equal the maximum of the stored product, a batch entry
whose result must not depend on the batch it travels in)."""

import numpy as np
import pytest

import oracle
from plaidml_b200 import kernels as K
from plaidml_b200 import programs
from plaidml_b200.core import DType, Program, bf16_bits_to_f32, f32_to_bf16_bits
from plaidml_b200.edsl import Contraction, TensorIndexes
from plaidml_b200.exec import Runner

import edsl_programs as P
from gpu_util import as_f32, check_close, dev, dev_bf16, empty, max_rel, ptr, rng

pytestmark = pytest.mark.gpu


def conv_plan(n, h, w, c, k, out_dtype, epilogue, flags):
    d = K.ConvDesc()
    d.in_dtype, d.out_dtype = K.BF16, out_dtype
    d.n, d.h, d.w, d.c, d.r, d.s, d.k, d.p, d.q = n, h, w, c, 3, 3, k, h, w
    d.stride_h = d.stride_w = 1
    d.pad_h = d.pad_w = 1
    d.dil_h = d.dil_w = 1
    d.epilogue, d.tile_n, d.flags = epilogue, 0, flags
    return K.Plan("conv", d)


def test_cfg3_conv_full_size_routes_agree_and_samples_match_oracle():
    # configuration 3: I bf16 [128,56,56,64] ~U[0,1), F ~N(0, sqrt(2/576)), bias, ReLU
    g = rng(1234 + 3)
    n, h, w, c, k = 128, 56, 56, 64, 64
    x = dev_bf16(g.uniform(0, 1, size=(n, h, w, c)))
    f32 = (g.standard_normal((3, 3, c, k)) * np.sqrt(2.0 / 576)).astype(np.float32)
    bias = (g.standard_normal(k) * 0.1).astype(np.float32)
    f_dev, b_dev = dev(f32), dev(bias)
    outs = {}
    for name, flags in (("halo", 0), ("im2col", K.CONV_NO_HALO)):
        plan = conv_plan(n, h, w, c, k, K.F32, K.EPI_BIAS | K.EPI_RELU, flags)
        plan.set_filter(ptr(f_dev), K.F32)
        out = empty((n, h, w, k), K.F32)
        plan.conv(ptr(x), ptr(out), ptr(b_dev), None)
        plan.check()
        outs[name] = (plan.kernel, as_f32(out))
    assert outs["halo"][0] == "tc_conv_halo" and outs["im2col"][0] == "tc_conv"
    # two different kernels (resident weights + shifted windows, im2col TMA): same sums, f32 out
    check_close(outs["halo"][1], outs["im2col"][1], 1e-5)
    # 96 output pixels (corners, edges, interior, first and last image) against the oracle's loop nest
    xf = as_f32(x)
    ff = oracle.bf16_to_f32(oracle.f32_to_bf16(f32))
    picks = [(0, 0, 0), (0, 0, 55), (0, 55, 0), (127, 55, 55), (127, 0, 0), (64, 27, 31)]
    picks += [(int(a), int(b), int(cc)) for a, b, cc in zip(g.integers(0, n, 90), g.integers(0, h, 90), g.integers(0, w, 90))]
    got = np.stack([outs["halo"][1][a, b, cc] for a, b, cc in picks])
    ref = np.zeros((len(picks), k), np.float64)
    for i, (a, b, cc) in enumerate(picks):
        for fr in range(3):
            for fs in range(3):
                y, xx = b + fr - 1, cc + fs - 1
                if 0 <= y < h and 0 <= xx < w:
                    ref[i] += xf[a, y, xx].astype(np.float64) @ ff[fr, fs].astype(np.float64)
    ref = np.maximum(ref + bias, 0.0)
    check_close(got, ref.astype(np.float32), 1e-4)
    # the bf16-output variant of the metric is the f32 result rounded once
    plan = conv_plan(n, h, w, c, k, K.BF16, K.EPI_BIAS | K.EPI_RELU, 0)
    plan.set_filter(ptr(f_dev), K.F32)
    out16 = empty((n, h, w, k), K.BF16)
    plan.conv(ptr(x), ptr(out16), ptr(b_dev), None)
    plan.check()
    np.testing.assert_array_equal(as_f32(out16), oracle.bf16_to_f32(oracle.f32_to_bf16(outs["halo"][1])))


def test_cfg5_full_size_row_max_equals_max_of_stored_product():
    # configuration 5: Q, K bf16 [1024,512,64] ~N(0,1); S = Q K^T (f32), R = row max of S
    g = rng(1234 + 5)
    b, m, k = 1024, 512, 64
    q = f32_to_bf16_bits(g.standard_normal((b, m, k)).astype(np.float32))
    kk = f32_to_bf16_bits(g.standard_normal((b, m, k)).astype(np.float32))
    Q, Kt, S = P.tile_gemm(DType.BFLOAT16, m, m, k, acc=DType.FLOAT32, batch=b, b_transposed=True)
    bb, i, j = TensorIndexes(3)
    R = Contraction(name="rowmax").outShape(b, m).outAccess(bb, i).max(S[bb, i, j]).build()
    s_out, r_out = Runner(Program("qk_rowmax_full", [Q, Kt], [S, R]), "cuda.0").run([q, kk])
    np.testing.assert_array_equal(r_out, s_out.max(axis=2))          # exact given identical S
    only_r = Runner(Program("qk_rowmax_only_full", [Q, Kt], [R]), "cuda.0").run([q, kk])[0]
    np.testing.assert_array_equal(only_r, r_out)                      # S never written: same maxima
    for e in (0, 511, 1023, int(g.integers(1, 1023))):               # whole batch entries against the oracle
        ref = oracle.gemm_h16_f32(q[e:e + 1], kk[e:e + 1], False, True)
        check_close(s_out[e:e + 1], ref, 1e-2)


@pytest.mark.parametrize("split_k", [False, True], ids=["one_pass", "split_k"])
def test_cfg4_resnet50_batch_256_entries_do_not_depend_on_the_batch(split_k, monkeypatch):
    # configuration 4 at its full batch: an image's logits must be the ones it gets in a batch of two (the
    # oracle-checked size of test_gpu_resnet.py).  With every GEMM in one pass the kernel routes differ between
    # the two batch sizes only in tiling, never in the order in which a sum is accumulated; with the library's
    # default, the few-tile layers of the batch of two sum a long K range in parts, which moves f32 sums by a
    # last bit and, after bf16 rounding of the activations layer after layer, the logits by a few 1e-3
    if not split_k:
        monkeypatch.setenv("PMLB_SPLIT_K", "0")
    g = rng(1234 + 4)
    img = g.uniform(0, 1, size=(256, 224, 224, 3)).astype(np.float32)
    bits = f32_to_bf16_bits(img)
    big_prog, _ = programs.resnet50(256)
    big = Runner(big_prog, "cuda.0")
    logits = big.run([bits])[0]
    assert logits.shape == (256, 1000) and np.isfinite(logits).all()
    replay = big.run([bits])[0]                                        # the CUDA-graph replay
    np.testing.assert_array_equal(replay, logits)
    small_prog, _ = programs.resnet50(2)
    small = Runner(small_prog, "cuda.0")
    for first in (0, 254):
        pair = small.run([np.ascontiguousarray(bits[first:first + 2])])[0]
        err = max_rel(logits[first:first + 2], pair)
        print("batch 256 vs batch 2, images", first, first + 1, "max-rel", err)
        assert err < (8e-3 if split_k else 1e-3)
    # images differ, so do their logits (guards against a stuck or broadcast batch index)
    assert np.abs(logits[0] - logits[255]).max() > 1e-3
