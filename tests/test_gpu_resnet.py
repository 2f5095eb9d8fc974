"""ResNet-50 v1.5 built from the op library, run on the cuda device, compared with the CPU oracle
at a small batch (configuration 4's network; logits within 2e-2 relative)."""

import numpy as np
import pytest

import oracle
from plaidml_b200 import programs
from plaidml_b200.core import bf16_bits_to_f32, f32_to_bf16_bits
from plaidml_b200.exec import Runner

from gpu_util import max_rel, rng

pytestmark = pytest.mark.gpu


def bf16_round(x):
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def oracle_resnet50(x_f32, weights):
    """The same graph on the CPU: f32 loops over bf16-rounded activations and weights."""
    def conv(x, name, stride=1, pad=None, relu=True, shortcut=None):
        w, b = weights[name]
        w = bf16_bits_to_f32(w)
        if pad is None:
            pad = (w.shape[0] - 1) // 2
        y = oracle.conv2d_nhwc_f32(x, w, b, shortcut, (stride, stride), (pad, pad), (1, 1), relu)
        return bf16_round(y)

    x = conv(x_f32, "conv1", stride=2, pad=3)
    p = (x.shape[1] + 2 - 3) // 2 + 1
    x = oracle.pool2d_nhwc_f32(x, "max", (3, 3), (2, 2), (1, 1), (p, p))
    for si, (blocks, mid, out, stride) in enumerate(programs.RESNET_STAGES):
        for b in range(blocks):
            name = f"res{si + 2}{chr(ord('a') + b)}"
            s = stride if b == 0 else 1
            shortcut = conv(x, name + "_1", stride=s, relu=False) if b == 0 else x
            y = conv(x, name + "_2a")
            y = conv(y, name + "_2b", stride=s)
            x = conv(y, name + "_2c", shortcut=shortcut)
    pooled = bf16_round(x.astype(np.float32).sum(axis=(1, 2)) / np.float32(x.shape[1] * x.shape[2]))
    w, b = weights["fc"]
    return oracle.gemm_f32(pooled, bf16_bits_to_f32(w)) + b


def test_resnet50_logits_match_oracle():
    batch = 2
    program, weights = programs.resnet50(batch)
    runner = Runner(program, "cuda.0")
    plan = runner.executable.describe()
    lines = plan.strip().splitlines()
    kinds = [ln.split()[0] for ln in lines]
    # 53 convolutions + the FC contraction on tensor cores; pooling and the average on their kernels
    assert kinds.count("tc_conv_s2d_pool") == 1, plan      # the 7x7 / 2 first layer on 3 channels with its max pool
    assert kinds.count("tc_conv_halo") == 3, plan          # the 3x3, 64 -> 64 convolutions of the first stage
    # (50 launches for the 54 contractions: the four shortcut projections run inside their blocks' last 1x1 layers)
    assert kinds.count("tc_conv_s2d_pool") + kinds.count("tc_conv_halo") + kinds.count("tc_conv") + kinds.count("tc_gemm") == 50, plan
    for tag in ("+shortcut(k64)", "+shortcut(k256/2)", "+shortcut(k512/2)", "+shortcut(k1024/2)"):
        assert plan.count(tag) == 1, (tag, plan)
    assert "nhwc_pool" not in kinds and "strided_reduce" in kinds
    assert "generic_contract" not in kinds, plan
    g = rng(1234 + 4)
    img = g.uniform(0, 1, size=(batch, 224, 224, 3)).astype(np.float32)
    x_bits = f32_to_bf16_bits(img)
    logits = runner.run([x_bits])[0]
    assert not runner.executable.uses_graph                 # first pass: direct launches
    again = runner.run([x_bits])[0]                          # second pass: captured and replayed as a CUDA graph
    assert runner.executable.uses_graph
    np.testing.assert_array_equal(again, logits)
    ref = oracle_resnet50(bf16_bits_to_f32(x_bits), weights)
    err = max_rel(logits, ref)
    print("resnet50 logits max-rel error:", err, "steps:", len(lines))
    # 2e-2 relative: the stated tolerance for the network's logits in bf16
    assert err < 2e-2


def test_resnet50_with_softmax_output_plans_and_sums_to_one():
    # fc + bias feeding a softmax: the fc GEMM already has an epilogue term, so the softmax's row maximum
    # stays a reduction step of its own
    batch = 2
    program, _ = programs.resnet50(batch, with_softmax=True)
    runner = Runner(program, "cuda.0")
    assert "+rowmax" not in runner.executable.describe()
    g = rng(1234 + 4)
    x_bits = f32_to_bf16_bits(g.uniform(0, 1, size=(batch, 224, 224, 3)).astype(np.float32))
    logits, probs = runner.run([x_bits])
    e = np.exp(logits - logits.max(axis=1, keepdims=True))
    np.testing.assert_allclose(probs, e / e.sum(axis=1, keepdims=True), rtol=1e-4, atol=1e-7)
    np.testing.assert_allclose(probs.sum(axis=1), 1.0, rtol=1e-5)
