"""Small, self-contained runs of single hot-path configurations, for profilers.

    python tests/profile_cases.py <case> [passes]

Each case builds its program through the EDSL, runs it once through ``plaidml_executable_run``
(inputs seeded, uploaded from host buffers) and then repeats the device-resident kernel
sequence once untimed and then ``passes`` times (default 3) without L2 flushing, so that a profiler sees a handful of
launches of the kernel of interest:

    i8_4k      int8 -> int32 Tile GEMM 4096^3            (tc_contract_kernel, int8, B as [k][n])
    bf16_4k    bf16 Tile GEMM 4096^3, f32 accumulate     (tc_contract_kernel, bf16)
    f32_1k     fp32 Tile GEMM 1024^3 via three TF32 products
    bf16_2a    bf16 GEMM 50176 x 256 x 1024 (the shape of ResNet-50's res4x_2a layers at 256 images: A streamed once)
    bf16_2c    bf16 GEMM 50176 x 1024 x 256 (res4x_2c: short K, 103 MB of output)
    conv3      conv 3x3 56x56 64->64 + bias + ReLU, batch 16
    conv3_full the same at batch 128
    conv1x1    conv 1x1 56x56 64->256 + bias + ReLU, batch 64 (HBM-bound: 26 MB in, 103 MB out)
    qk         batched Q.K^T 128 x (512x512x64) + row max (folded into the GEMM's epilogue)
    qk_r       the same at the full batch of 1024 with only the row maxima as output (the product is never written:
               134 MB read, 2 MB written)
    rowmax     row max alone over a 256 x 512 x 512 f32 tensor (row_reduce_kernel, 256 MiB)
    stem       the first two layers of ResNet-50 at batch 32: 7x7 / 2 convolution on 3 channels + bias + ReLU and the
               3x3 / 2 max pool as one kernel (s2d_pack_kernel, then conv_s2d_pool_kernel); with
               PLAIDML_CUDA_NO_POOL_FUSION=1 in the environment the two-kernel form (tc_contract_kernel on the
               space-to-depth route, pool16_kernel)
    stem_full  the same at batch 256 (120 MB of packed pixels in, 103 MB out)
    gather_rows   2 M rows of 64 f32 gathered from a table of 1 M rows (gather_kernel: 8 MB of indices, 512 MB read at
               random row granularity, 512 MB written)
    gather_lin    64 M linearly interpolated samples of a 16 M-element f32 signal (256 MB of positions in, 256 MB out)
    scatter_add   16 M f32 updates added into 4 M cells (64 MB + 64 MB in, one 16 MB copy, atomics)
    argsort       4096 lines of 4096 f32 sorted along the line (12 merge passes of argsort_pass_kernel)
    prng          256 M numbers (prng_kernel: 1 GiB written) and the state after them
    resnet N   ResNet-50 v1.5 at batch N
    resnet_steps N   the same, followed by a table of every kernel step on its own (CUDA events around 20 launches
               of the step replayed from a CUDA graph: device time without the host's launch cost) beside the time of
               the whole pass replayed as one graph
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from plaidml_b200 import programs  # noqa: E402
from plaidml_b200.core import DType, Program, f32_to_bf16_bits  # noqa: E402
from plaidml_b200.edsl import Contraction, TensorIndexes  # noqa: E402
from plaidml_b200.exec import Runner  # noqa: E402


def main(argv) -> None:
    from plaidml_b200.core import settings_set
    # one launch per GEMM, as in the device-resident timing of bench.py (plaidml_executable_run would
    # otherwise cut a large single GEMM into four row slices to overlap its host copies)
    settings_set("PLAIDML_CUDA_SLICED_RUN", "0")
    case = argv[1] if len(argv) > 1 else "i8_4k"
    g = np.random.Generator(np.random.PCG64(7))
    passes = 3
    if case == "i8_4k":
        A, B, C = programs.tile_gemm(DType.INT8, 4096, 4096, 4096, acc=DType.INT32)
        r = Runner(Program(case, [A, B], [C]), "cuda.0")
        ins = [g.integers(-128, 128, (4096, 4096), dtype=np.int8) for _ in range(2)]
    elif case == "bf16_4k":
        A, B, C = programs.tile_gemm(DType.BFLOAT16, 4096, 4096, 4096, acc=DType.FLOAT32, out_bf16=True)
        r = Runner(Program(case, [A, B], [C]), "cuda.0")
        ins = [f32_to_bf16_bits(g.standard_normal((4096, 4096))) for _ in range(2)]
    elif case in ("bf16_2a", "bf16_2c"):
        m, n, k = (50176, 256, 1024) if case == "bf16_2a" else (50176, 1024, 256)
        A, B, C = programs.tile_gemm(DType.BFLOAT16, m, n, k, acc=DType.FLOAT32, out_bf16=True)
        r = Runner(Program(case, [A, B], [C]), "cuda.0")
        ins = [f32_to_bf16_bits(g.standard_normal((m, k))), f32_to_bf16_bits(g.standard_normal((k, n)))]
    elif case == "f32_1k":
        A, B, C = programs.tile_gemm(DType.FLOAT32, 1024, 1024, 1024)
        r = Runner(Program(case, [A, B], [C]), "cuda.0")
        ins = [g.uniform(-1, 1, (1024, 1024)).astype(np.float32) for _ in range(2)]
    elif case in ("conv3", "conv3_full"):
        n = 16 if case == "conv3" else 128
        f = f32_to_bf16_bits(g.standard_normal((3, 3, 64, 64)) * np.sqrt(2.0 / 576))
        r = Runner(programs.conv_bias_relu(n, 56, 56, 64, 64, filt=f, bias=np.zeros(64, np.float32)), "cuda.0")
        ins = [f32_to_bf16_bits(g.uniform(0, 1, (n, 56, 56, 64)))]
    elif case == "conv1x1":
        f = f32_to_bf16_bits(g.standard_normal((1, 1, 64, 256)) * np.sqrt(2.0 / 64))
        r = Runner(programs.conv_bias_relu(64, 56, 56, 64, 256, r=1, s=1, filt=f, bias=np.zeros(256, np.float32)),
                   "cuda.0")
        ins = [f32_to_bf16_bits(g.uniform(0, 1, (64, 56, 56, 64)))]
    elif case in ("qk", "qk_r"):
        nb = 128 if case == "qk" else 1024
        Q, Kt, S = programs.tile_gemm(DType.BFLOAT16, 512, 512, 64, acc=DType.FLOAT32, batch=nb, b_transposed=True)
        bb, i, j = TensorIndexes(3)
        R = Contraction(name="rowmax").outShape(nb, 512).outAccess(bb, i).max(S[bb, i, j]).build()
        r = Runner(Program(case, [Q, Kt], [S, R] if case == "qk" else [R]), "cuda.0")
        ins = [f32_to_bf16_bits(g.standard_normal((nb, 512, 64))) for _ in range(2)]
    elif case == "rowmax":
        from plaidml_b200.edsl import Placeholder
        S = Placeholder(DType.FLOAT32, [256, 512, 512])
        bb, i, j = TensorIndexes(3)
        R = Contraction(name="rowmax").outShape(256, 512).outAccess(bb, i).max(S[bb, i, j]).build()
        r = Runner(Program(case, [S], [R]), "cuda.0")
        ins = [g.standard_normal((256, 512, 512)).astype(np.float32)]
    elif case in ("stem", "stem_full"):
        from plaidml_b200 import edsl, op
        from plaidml_b200.edsl import Placeholder, cast
        w = f32_to_bf16_bits(g.standard_normal((7, 7, 3, 64)) * np.sqrt(2.0 / 147))
        nimg = 32 if case == "stem" else 256
        I = Placeholder(DType.BFLOAT16, [nimg, 224, 224, 3])
        F = cast(edsl.Constant(w, name="w", dtype=DType.BFLOAT16), DType.FLOAT32)
        y = op.convolution(cast(I, DType.FLOAT32), F, strides=[2, 2], autopad_mode=op.AutoPadMode.EXPLICIT,
                           manual_padding=[3, 3, 3, 3]) + edsl.Constant(np.zeros(64, np.float32), name="b")
        y = cast(op.relu(y), DType.BFLOAT16)
        y = op.pool(y, op.PoolMode.MAX, [3, 3], [2, 2], op.AutoPadMode.EXPLICIT, [1, 1, 1, 1], op.TensorLayout.NXC)
        r = Runner(Program(case, [I], [y]), "cuda.0")
        ins = [f32_to_bf16_bits(g.uniform(0, 1, (nimg, 224, 224, 3)).astype(np.float32))]
    elif case in ("gather_rows", "gather_lin", "scatter_add", "argsort", "prng"):
        from plaidml_b200 import edsl
        from plaidml_b200.edsl import Placeholder
        if case == "gather_rows":
            T, I = Placeholder(DType.FLOAT32, [1 << 20, 64]), Placeholder(DType.INT32, [1 << 21])
            r = Runner(Program(case, [T, I], [edsl.gather(T, I)]), "cuda.0")
            ins = [g.standard_normal((1 << 20, 64), dtype=np.float32), g.integers(0, 1 << 20, 1 << 21, dtype=np.int32)]
        elif case == "gather_lin":
            T, I = Placeholder(DType.FLOAT32, [1 << 24]), Placeholder(DType.FLOAT32, [1 << 26])
            r = Runner(Program(case, [T, I], [edsl.gather(T, I, interpolation_mode=edsl.InterpolationMode.LINEAR)]), "cuda.0")
            pos = (np.arange(1 << 26, dtype=np.float64) * 0.25 + g.uniform(0, 0.25, 1 << 26)).astype(np.float32)
            ins = [g.standard_normal(1 << 24, dtype=np.float32), pos]
        elif case == "scatter_add":
            D, I, U = (Placeholder(DType.FLOAT32, [1 << 22]), Placeholder(DType.INT32, [1 << 24]),
                       Placeholder(DType.FLOAT32, [1 << 24]))
            r = Runner(Program(case, [D, I, U], [edsl.scatter(D, I, U)]), "cuda.0")
            ins = [np.zeros(1 << 22, np.float32), g.integers(0, 1 << 22, 1 << 24, dtype=np.int32),
                   g.standard_normal(1 << 24, dtype=np.float32)]
        elif case == "argsort":
            X = Placeholder(DType.FLOAT32, [4096, 4096])
            r = Runner(Program(case, [X], [edsl.argsort(X, 1)]), "cuda.0")
            ins = [g.standard_normal((4096, 4096), dtype=np.float32)]
        else:
            S = Placeholder(DType.UINT32, [3])
            r = Runner(Program(case, [S], list(edsl.prng(S, [1 << 28]))), "cuda.0")
            ins = [np.array([5, 6, 7], dtype=np.uint32)]
    elif case in ("resnet", "resnet_steps"):
        batch = int(argv[2]) if len(argv) > 2 else 32
        prog, _ = programs.resnet50(batch)
        r = Runner(prog, "cuda.0")
        img = g.uniform(0, 1, (batch, 224, 224, 3)).astype(np.float32)
        ins = [f32_to_bf16_bits(img)]
        passes = 1
    else:
        raise SystemExit(__doc__)
    if len(argv) > 2 and case not in ("resnet", "resnet_steps"):
        passes = int(argv[2])
    r.run(ins)
    r.executable.time_steps(1, False)      # first use of the kernels of the resident path (module loading)
    ms = r.executable.time_steps(passes, False)
    print(f"{case}: {ms:.4f} ms per pass over {passes} passes; {r.executable.launch_count} launches per pass")
    if case == "resnet_steps":
        r.executable.time_steps(5, False)
        whole = np.median(r.executable.time_passes(30, False))
        rows = r.executable.time_each_step(20, False)
        print(f"whole pass (one graph, L2 not flushed): {whole * 1e3:.1f} us; sum of the steps: {sum(t for _, t in rows) * 1e3:.1f} us")
        for line, t in rows:
            print(f"{t * 1e3:8.1f} us  {line}")
    else:
        print(r.executable.describe())
        if case in ("gather_rows", "gather_lin", "scatter_add", "argsort", "prng"):
            for line, t in r.executable.time_each_step(20, False):
                print(f"{t * 1e3:8.1f} us  {line}")


if __name__ == "__main__":
    main(sys.argv)
