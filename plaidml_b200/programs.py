"""EDSL builders of the benchmark configurations: Tile GEMMs, the NHWC convolution layer and
ResNet-50 v1.5 assembled from the op library (the structure of the reference's
``networks/oplib/resnet50.cc:26-57,223-320`` with the stride moved to the 3x3 convolutions).
"""

from __future__ import annotations

import numpy as np

from . import edsl, op
from .core import DType, Program, f32_to_bf16_bits
from .edsl import Contraction, Placeholder, TensorIndexes, cast


def tile_gemm(dtype_in: DType, m, n, k, acc: DType = None, batch=None, b_transposed=False, out_bf16=False):
    """C[i,j] += A[i,k] * B[k,j], optionally with operands cast to a wider accumulate type
    (``acc``), a leading batch dimension, B stored [j,k], or the result cast to bf16.
    Returns (A, B, C)."""
    ashape = [m, k] if batch is None else [batch, m, k]
    if batch is None:
        bshape = [n, k] if b_transposed else [k, n]
    else:
        bshape = [batch, n, k] if b_transposed else [batch, k, n]
    A = Placeholder(dtype_in, ashape, name="A")
    B = Placeholder(dtype_in, bshape, name="B")
    a = cast(A, acc) if acc is not None else A
    b = cast(B, acc) if acc is not None else B
    i, j, kk, bb = TensorIndexes(4)
    if batch is None:
        rhs = a[i, kk] * (b[j, kk] if b_transposed else b[kk, j])
        C = Contraction(name="gemm").outShape(m, n).outAccess(i, j).sum(rhs).build()
    else:
        rhs = a[bb, i, kk] * (b[bb, j, kk] if b_transposed else b[bb, kk, j])
        C = Contraction(name="bgemm").outShape(batch, m, n).outAccess(bb, i, j).sum(rhs).build()
    if out_bf16:
        C = cast(C, DType.BFLOAT16)
    return A, B, C


def conv_bias_relu(n, h, w, cin, cout, r=3, s=3, out_bf16=True, filt=None, bias=None, stride=1):
    """NHWC convolution as a Tile contraction (op.convolution) + bias + ReLU; bf16 storage,
    f32 accumulate.  ``filt`` holds bf16 bit patterns [r, s, cin, cout], ``bias`` float32."""
    I = Placeholder(DType.BFLOAT16, [n, h, w, cin], name="I")
    F = edsl.Constant(filt, name="F", dtype=DType.BFLOAT16)
    Bz = edsl.Constant(bias, name="bias")
    pads = [(r - 1) // 2, (s - 1) // 2, (r - 1) // 2, (s - 1) // 2]
    O = op.convolution(cast(I, DType.FLOAT32), cast(F, DType.FLOAT32), strides=[stride, stride],
                       autopad_mode=op.AutoPadMode.EXPLICIT, manual_padding=pads, name="conv")
    O = op.relu(O + Bz)
    if out_bf16:
        O = cast(O, DType.BFLOAT16)
    return Program("conv_bias_relu", [I], [O])


# ---------------------------------------------------------------------- ResNet-50 v1.5

RESNET_STAGES = [(3, 64, 256, 1), (4, 128, 512, 2), (6, 256, 1024, 2), (3, 512, 2048, 2)]


def resnet50_weights(seed: int = 1234 + 4):
    """He-normal weights (sigma = sqrt(2 / fan_in)) as bf16 bit patterns and zero float32 biases,
    in layer order; deterministic in ``seed``."""
    g = np.random.Generator(np.random.PCG64(seed))
    weights = {}

    def conv(name, r, s, cin, cout):
        w = g.standard_normal((r, s, cin, cout)).astype(np.float32) * np.sqrt(2.0 / (r * s * cin))
        weights[name] = (f32_to_bf16_bits(w), np.zeros(cout, dtype=np.float32))

    conv("conv1", 7, 7, 3, 64)
    cin = 64
    for si, (blocks, mid, out, _) in enumerate(RESNET_STAGES):
        for b in range(blocks):
            p = f"res{si + 2}{chr(ord('a') + b)}"
            conv(p + "_2a", 1, 1, cin, mid)
            conv(p + "_2b", 3, 3, mid, mid)
            conv(p + "_2c", 1, 1, mid, out)
            if b == 0:
                conv(p + "_1", 1, 1, cin, out)
            cin = out
    w = g.standard_normal((2048, 1000)).astype(np.float32) * np.sqrt(2.0 / 2048)
    weights["fc"] = (f32_to_bf16_bits(w), np.zeros(1000, dtype=np.float32))
    return weights


def resnet50(batch: int, weights=None, with_softmax=False):
    """ResNet-50 v1.5 inference, NHWC, bf16 activations / weights with f32 accumulation.

    The image input is [batch, 224, 224, 3]; the first convolution takes the packed-row route of
    the kernel library, which needs no channel alignment.  Returns (program, weights); output 0
    is the [batch, 1000] float32 logits."""
    if weights is None:
        weights = resnet50_weights()
    f32, bf16 = DType.FLOAT32, DType.BFLOAT16

    def conv_block(x, name, stride=1, pad=None, relu=True, shortcut=None):
        wbits, bias = weights[name]
        r = wbits.shape[0]
        if pad is None:
            pad = (r - 1) // 2
        F = cast(edsl.Constant(wbits, name=name + "_w", dtype=bf16), f32)
        B = edsl.Constant(bias, name=name + "_b")
        y = op.convolution(cast(x, f32), F, strides=[stride, stride], autopad_mode=op.AutoPadMode.EXPLICIT,
                           manual_padding=[pad, pad, pad, pad], name=name) + B
        if shortcut is not None:
            y = y + cast(shortcut, f32)
        if relu:
            y = op.relu(y)
        return cast(y, bf16)

    I = Placeholder(bf16, [batch, 224, 224, 3], name="image")
    x = conv_block(I, "conv1", stride=2, pad=3)
    x = op.pool(x, op.PoolMode.MAX, [3, 3], [2, 2], op.AutoPadMode.EXPLICIT, [1, 1, 1, 1], op.TensorLayout.NXC, name="pool1")
    for si, (blocks, mid, out, stride) in enumerate(RESNET_STAGES):
        for b in range(blocks):
            p = f"res{si + 2}{chr(ord('a') + b)}"
            s = stride if b == 0 else 1
            shortcut = conv_block(x, p + "_1", stride=s, relu=False) if b == 0 else x
            y = conv_block(x, p + "_2a")
            y = conv_block(y, p + "_2b", stride=s)          # v1.5: the 3x3 convolution strides
            x = conv_block(y, p + "_2c", shortcut=shortcut)
    pooled = op.mean(cast(x, f32), axes=[1, 2])               # global average pool -> [batch, 2048]
    wbits, bias = weights["fc"]
    logits = op.dot(cast(cast(pooled, bf16), f32), cast(edsl.Constant(wbits, name="fc_w", dtype=bf16), f32), name="fc")
    logits = logits + edsl.Constant(bias, name="fc_b")
    outputs = [logits]
    if with_softmax:
        outputs.append(op.softmax(logits, axis=1))
    return Program("resnet50_v1_5", [I], outputs), weights


RESNET50_GFLOP_PER_IMAGE = 8.178  # 2 * MACs of the 53 convolutions and the FC layer
