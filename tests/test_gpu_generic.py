"""Parity of the general contraction, element-wise and aggregation kernels with the oracle."""

import ctypes

import numpy as np
import pytest
import torch

import oracle
from plaidml_b200 import kernels as K
from gpu_util import as_f32, check_close, dev, dev_bf16, empty, ptr, rng

pytestmark = pytest.mark.gpu

NP_OF = {K.F32: np.float32, K.F64: np.float64, K.I8: np.int8, K.I32: np.int32, K.I64: np.int64, K.U8: np.uint8,
         K.F16: np.float16, K.I16: np.int16, K.BOOL: np.uint8}


def run_contract(desc, srcs, out_shape, out_dtype, init=None):
    """Runs one descriptor on the GPU and through the definition-order CPU walker."""
    plan = K.Plan("contract", desc)
    d_srcs = [dev(s) for s in srcs]
    d_init = dev(init) if init is not None else None
    out = empty(out_shape, out_dtype)
    plan.contract([ptr(s) for s in d_srcs], ptr(out), ptr(d_init))
    torch.cuda.synchronize()
    ref = np.empty(out_shape, dtype=NP_OF[out_dtype])
    oracle.contract(desc, srcs, init, ref)
    return out.cpu().numpy(), ref


def gemm_desc(dt, m, n, k):
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_MUL, 3, 2
    d.range[0], d.range[1], d.range[2] = m, n, k
    d.out = K.make_access(dt, [m, n], [{0: 1}, {1: 1}])
    d.src[0] = K.make_access(dt, [m, k], [{0: 1}, {2: 1}])
    d.src[1] = K.make_access(dt, [k, n], [{2: 1}, {1: 1}])
    return d


def test_contract_gemm_f32():
    g = rng(1)
    a = g.standard_normal((8, 16)).astype(np.float32)
    b = g.standard_normal((16, 32)).astype(np.float32)
    out, ref = run_contract(gemm_desc(K.F32, 8, 32, 16), [a, b], (8, 32), K.F32)
    np.testing.assert_array_equal(out, ref)  # same order of additions as the CPU walker


def test_contract_gemm_int8_wraps():
    g = rng(2)
    a = g.integers(-128, 128, size=(9, 33), dtype=np.int8)
    b = g.integers(-128, 128, size=(33, 7), dtype=np.int8)
    out, ref = run_contract(gemm_desc(K.I8, 9, 7, 33), [a, b], (9, 7), K.I8)
    np.testing.assert_array_equal(out, ref)
    np.testing.assert_array_equal(out, (a.astype(np.int32) @ b.astype(np.int32)).astype(np.int8))


def test_contract_conv_with_oob_rule():
    # O[n,x,y,co] += I[n, x+i-1, y+j-1, ci] * F[i,j,ci,co]: taps outside the image are skipped
    g = rng(3)
    n, h, w, ci, co = 2, 6, 5, 3, 4
    x = g.standard_normal((n, h, w, ci)).astype(np.float32)
    f = g.standard_normal((3, 3, ci, co)).astype(np.float32)
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_MUL, 7, 2
    for i, r in enumerate([n, h, w, co, 3, 3, ci]):
        d.range[i] = r
    d.out = K.make_access(K.F32, [n, h, w, co], [{0: 1}, {1: 1}, {2: 1}, {3: 1}])
    d.src[0] = K.make_access(K.F32, [n, h, w, ci], [{0: 1}, {1: 1, 4: 1}, {2: 1, 5: 1}, {6: 1}], offs=[0, -1, -1, 0])
    d.src[1] = K.make_access(K.F32, [3, 3, ci, co], [{4: 1}, {5: 1}, {6: 1}, {3: 1}])
    out, ref = run_contract(d, [x, f], (n, h, w, co), K.F32)
    np.testing.assert_array_equal(out, ref)
    check_close(out, oracle.conv2d_nhwc_f32(x, f, pad=(1, 1)), 1e-5)


def test_contract_maxpool_with_constraint():
    # O[x] >= I[2x + i], i < 2 as a constraint on a wider index range
    x = np.array([1, -5, 3, 9, -2, -7, 4, 0], dtype=np.float32)
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_MAX, K.COMBO_NONE, 2, 1
    d.range[0], d.range[1] = 4, 8
    d.out = K.make_access(K.F32, [4], [{0: 1}])
    d.src[0] = K.make_access(K.F32, [8], [{0: 2, 1: 1}])
    d.n_cons = 1
    d.cons_coef[0][1] = 1
    d.cons_range[0] = 2
    out, ref = run_contract(d, [x], (4,), K.F32)
    np.testing.assert_array_equal(out, ref)
    np.testing.assert_array_equal(out, np.array([1, 9, -2, 4], dtype=np.float32))


def test_contract_non_injective_output_and_fraction():
    # O[i + j] += A[i] * B[j]  (output coordinate is not a single index) and
    # O[i] += A[i / 2] (only even i contribute)
    a = np.arange(1, 5, dtype=np.int32)
    b = np.arange(1, 4, dtype=np.int32)
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_MUL, 2, 2
    d.range[0], d.range[1] = 4, 3
    d.out = K.make_access(K.I32, [6], [{0: 1, 1: 1}])
    d.src[0] = K.make_access(K.I32, [4], [{0: 1}])
    d.src[1] = K.make_access(K.I32, [3], [{1: 1}])
    out, ref = run_contract(d, [a, b], (6,), K.I32)
    np.testing.assert_array_equal(out, ref)
    np.testing.assert_array_equal(out, np.convolve(a, b))
    d2 = K.ContractDesc()
    d2.agg, d2.combo, d2.n_idx, d2.n_src = K.AGG_SUM, K.COMBO_NONE, 1, 1
    d2.range[0] = 8
    d2.out = K.make_access(K.I32, [8], [{0: 1}])
    d2.src[0] = K.make_access(K.I32, [4], [{0: 1}], dens=[2])
    out, ref = run_contract(d2, [a], (8,), K.I32)
    np.testing.assert_array_equal(out, ref)
    np.testing.assert_array_equal(out, np.array([1, 0, 2, 0, 3, 0, 4, 0], dtype=np.int32))


@pytest.mark.parametrize("seed", range(12))
def test_contract_output_dims_that_mix_variables(seed):
    # O[n, s*y + i - p, t*x - j + q, k] += I[n, y, x, c] * F[i, j, c, k] with random strides, signs, offsets and
    # an output that may be cropped: every thread solves for (y, x) from its element and walks the taps only.
    g = rng(900 + seed)
    n, h, w, c, k = (int(v) for v in g.integers(1, 5, 5))
    h, w = h + 2, w + 3
    fi, fj = int(g.integers(1, 4)), int(g.integers(1, 4))
    s, t = int(g.integers(1, 4)), int(g.integers(1, 4))
    po, qo = int(g.integers(0, 2)), int(g.integers(0, 3))
    oh = s * (h - 1) + fi - po - int(g.integers(0, 2))
    ow = t * (w - 1) + qo + 1 - int(g.integers(0, 2))
    x = g.integers(-4, 5, (n, h, w, c)).astype(np.int32)
    f = g.integers(-4, 5, (fi, fj, c, k)).astype(np.int32)
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_MUL, 7, 2
    for i, r in enumerate([n, h, w, k, fi, fj, c]):
        d.range[i] = r
    d.out = K.make_access(K.I32, [n, oh, ow, k], [{0: 1}, {1: s, 4: 1}, {2: t, 5: -1}, {3: 1}], offs=[0, -po, qo, 0])
    d.src[0] = K.make_access(K.I32, [n, h, w, c], [{0: 1}, {1: 1}, {2: 1}, {6: 1}])
    d.src[1] = K.make_access(K.I32, [fi, fj, c, k], [{4: 1}, {5: 1}, {6: 1}, {3: 1}])
    out, ref = run_contract(d, [x, f], (n, oh, ow, k), K.I32)
    np.testing.assert_array_equal(out, ref)
    want = np.zeros((n, oh, ow, k), dtype=np.int64)
    for y in range(h):
        for xx in range(w):
            for i in range(fi):
                for j in range(fj):
                    oy, ox = s * y + i - po, t * xx - j + qo
                    if 0 <= oy < oh and 0 <= ox < ow:
                        want[:, oy, ox, :] += x[:, y, xx, :].astype(np.int64) @ f[i, j].astype(np.int64)
    np.testing.assert_array_equal(out, want.astype(np.int32))


def test_contract_shared_variable_across_output_dims():
    # O[i, i + j] = A[i, j]: the second dim's only free variable follows from the first
    a = np.arange(12, dtype=np.int32).reshape(3, 4) + 1
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_NONE, 2, 1
    d.range[0], d.range[1] = 3, 4
    d.out = K.make_access(K.I32, [3, 6], [{0: 1}, {0: 1, 1: 1}])
    d.src[0] = K.make_access(K.I32, [3, 4], [{0: 1}, {1: 1}])
    out, ref = run_contract(d, [a], (3, 6), K.I32)
    np.testing.assert_array_equal(out, ref)
    want = np.zeros((3, 6), dtype=np.int32)
    for i in range(3):
        want[i, i:i + 4] = a[i]
    np.testing.assert_array_equal(out, want)


def test_contract_init_tensor_and_min_and_cond():
    g = rng(4)
    a = g.standard_normal((5, 6)).astype(np.float32)
    bias = g.standard_normal(5).astype(np.float32)
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_MIN, K.COMBO_NONE, 2, 1
    d.range[0], d.range[1] = 5, 6
    d.out = K.make_access(K.F32, [5], [{0: 1}])
    d.src[0] = K.make_access(K.F32, [5, 6], [{0: 1}, {1: 1}])
    d.has_init = 1
    d.init = K.make_access(K.F32, [5], None)
    out, ref = run_contract(d, [a], (5,), K.F32, init=bias)
    np.testing.assert_array_equal(out, ref)
    np.testing.assert_array_equal(out, np.minimum(a.min(axis=1), bias))
    # cond: O[i] += (A[i] == B[i]) ? C[i] : 0
    x = np.array([1, 2, 3, 4], dtype=np.int32)
    y = np.array([1, 0, 3, 0], dtype=np.int32)
    z = np.array([10, 20, 30, 40], dtype=np.float32)
    d = K.ContractDesc()
    d.agg, d.combo, d.n_idx, d.n_src = K.AGG_SUM, K.COMBO_COND, 1, 3
    d.range[0] = 4
    d.out = K.make_access(K.F32, [1], [{}])
    for s, dt in enumerate([K.I32, K.I32, K.F32]):
        d.src[s] = K.make_access(dt, [4], [{0: 1}])
    out, ref = run_contract(d, [x, y, z], (1,), K.F32)
    np.testing.assert_array_equal(out, ref)
    assert out[0] == 40.0


# --- element-wise -------------------------------------------------------------------------

def run_eltwise(op, ins, out_shape, out_dtype, in_dtypes):
    d = K.EltwiseDesc()
    d.op = op.encode()
    d.n_in, d.rank, d.out_dtype = len(ins), len(out_shape), out_dtype
    for i, s in enumerate(out_shape):
        d.sizes[i] = s
    devs = []
    for k, (a, dt) in enumerate(zip(ins, in_dtypes)):
        d.in_dtype[k] = dt
        shape = (1,) * (len(out_shape) - a.ndim) + a.shape
        stride = 1
        for i in range(len(out_shape) - 1, -1, -1):
            d.in_strides[k][i] = 0 if shape[i] == 1 and out_shape[i] != 1 else stride
            stride *= shape[i]
        devs.append(dev(a))
    plan = K.Plan("eltwise", d)
    out = empty(out_shape, out_dtype)
    plan.eltwise([ptr(t) for t in devs], ptr(out))
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_eltwise_add_broadcast_and_relu():
    g = rng(5)
    x = g.standard_normal((4, 5, 6)).astype(np.float32)
    b = g.standard_normal(6).astype(np.float32)
    np.testing.assert_array_equal(run_eltwise("add", [x, b], (4, 5, 6), K.F32, [K.F32, K.F32]), x + b)
    np.testing.assert_array_equal(run_eltwise("relu", [x], (4, 5, 6), K.F32, [K.F32]), np.where(x < 0, 0, x))


def test_eltwise_casts_and_compare_select():
    g = rng(6)
    x = (g.standard_normal(100) * 50).astype(np.float32)
    np.testing.assert_array_equal(run_eltwise("cast", [x], (100,), K.I32, [K.F32]), x.astype(np.int32))
    i = g.integers(-1000, 1000, size=100, dtype=np.int32)
    np.testing.assert_array_equal(run_eltwise("cast", [i], (100,), K.I8, [K.I32]), i.astype(np.int8))
    np.testing.assert_array_equal(run_eltwise("cast", [i], (100,), K.F32, [K.I32]), i.astype(np.float32))
    y = g.standard_normal(100).astype(np.float32) * 50
    lt = run_eltwise("cmp_lt", [x, y], (100,), K.BOOL, [K.F32, K.F32])
    np.testing.assert_array_equal(lt, (x < y).astype(np.uint8))
    sel = run_eltwise("select", [lt, x, y], (100,), K.F32, [K.BOOL, K.F32, K.F32])
    np.testing.assert_array_equal(sel, np.where(x < y, x, y))


def test_eltwise_int_wrap_and_exp():
    a = np.array([120, -120, 5], dtype=np.int8)
    b = np.array([10, -10, 7], dtype=np.int8)
    np.testing.assert_array_equal(run_eltwise("add", [a, b], (3,), K.I8, [K.I8, K.I8]), (a + b).astype(np.int8))
    np.testing.assert_array_equal(run_eltwise("mul", [a, b], (3,), K.I8, [K.I8, K.I8]), (a * b).astype(np.int8))
    x = np.linspace(-3, 3, 64).astype(np.float32)
    np.testing.assert_allclose(run_eltwise("exp", [x], (64,), K.F32, [K.F32]), np.exp(x), rtol=1e-6)


# --- aggregation kernels ----------------------------------------------------------------------

@pytest.mark.parametrize("agg,name", [(K.AGG_MAX, "max"), (K.AGG_MIN, "min"), (K.AGG_SUM, "sum")])
@pytest.mark.parametrize("shape", [(64, 512, 1), (33, 100, 1), (8, 49, 2048), (5, 7, 3), (1, 1000, 1)])
def test_reduce_f32(agg, name, shape):
    g = rng(7)
    x = g.standard_normal(shape).astype(np.float32)
    d = K.ReduceDesc()
    d.agg, d.dtype, d.out_dtype = agg, K.F32, K.F32
    d.outer, d.reduce, d.inner = shape
    d.scale = 1.0
    plan = K.Plan("reduce", d)
    xd = dev(x)
    out = empty((shape[0], shape[2]), K.F32)
    plan.reduce(ptr(xd), ptr(out))
    torch.cuda.synchronize()
    ref = oracle.reduce_f32(x, name)
    if agg == K.AGG_SUM:
        check_close(out.cpu().numpy(), ref, 1e-5)   # order of additions differs
    else:
        np.testing.assert_array_equal(out.cpu().numpy(), ref)


def test_reduce_bf16_mean_to_f32():
    g = rng(8)
    x = dev_bf16(g.uniform(0, 1, size=(4, 49, 256)))
    d = K.ReduceDesc()
    d.agg, d.dtype, d.out_dtype = K.AGG_SUM, K.BF16, K.F32
    d.outer, d.reduce, d.inner = 4, 49, 256
    d.scale = 1.0 / 49
    plan = K.Plan("reduce", d)
    out = empty((4, 256), K.F32)
    plan.reduce(ptr(x), ptr(out))
    torch.cuda.synchronize()
    check_close(out.cpu().numpy(), oracle.reduce_f32(as_f32(x), "sum") / 49, 1e-5)


@pytest.mark.parametrize("dtype", [K.F32, K.BF16])
def test_maxpool_3x3_s2_pad1(dtype):
    g = rng(9)
    n, h, w, c = 2, 16, 16, 64
    x32 = g.standard_normal((n, h, w, c)).astype(np.float32)
    xd = dev(x32) if dtype == K.F32 else dev_bf16(x32)
    d = K.PoolDesc()
    d.agg, d.dtype = K.AGG_MAX, dtype
    d.n, d.h, d.w, d.c, d.r, d.s, d.p, d.q = n, h, w, c, 3, 3, 8, 8
    d.stride_h = d.stride_w = 2
    d.pad_h = d.pad_w = 1
    plan = K.Plan("pool", d)
    out = empty((n, 8, 8, c), dtype)
    plan.pool(ptr(xd), ptr(out))
    torch.cuda.synchronize()
    ref = oracle.pool2d_nhwc_f32(as_f32(xd), "max", (3, 3), (2, 2), (1, 1), (8, 8))
    np.testing.assert_array_equal(as_f32(out), ref)   # max is exact in any element type


def test_avgpool_excludes_padding():
    g = rng(10)
    x = g.standard_normal((1, 7, 7, 5)).astype(np.float32)
    d = K.PoolDesc()
    d.agg, d.dtype = K.AGG_SUM, K.F32
    d.n, d.h, d.w, d.c, d.r, d.s, d.p, d.q = 1, 7, 7, 5, 3, 3, 7, 7
    d.stride_h = d.stride_w = 1
    d.pad_h = d.pad_w = 1
    d.average = 1
    plan = K.Plan("pool", d)
    xd = dev(x)
    out = empty((1, 7, 7, 5), K.F32)
    plan.pool(ptr(xd), ptr(out))
    torch.cuda.synchronize()
    ref = oracle.pool2d_nhwc_f32(x, "sum", (3, 3), (1, 1), (1, 1), (7, 7), average=True)
    check_close(out.cpu().numpy(), ref, 1e-6)


def test_eltwise_dense_f32_form_gives_the_bits_of_the_general_form():
    # f32 in and out, operands dense or one value: eight elements per thread as two 16-byte pieces.  The same
    # operation on a view that is not a multiple of four elements takes the general kernel; both call one
    # arithmetic function, so the common part of their results must be equal bit for bit.
    g = rng(31)
    n = 4 * 1000 + 8
    a = g.standard_normal(n).astype(np.float32)
    b = g.uniform(0.5, 2.0, n).astype(np.float32)
    one = np.array([1.5], dtype=np.float32)
    for op_name, ins in (("add", [a, b]), ("div", [a, b]), ("max", [a, b]), ("relu", [a]), ("exp", [a]), ("tanh", [a]),
                         ("mul", [a, one]), ("sub", [one, b]), ("sqrt", [b]), ("pow", [b, a])):
        outs = []
        for count in (n, n - 3):          # dense form; general form
            arrays = [x if x.size == 1 else x[:count] for x in ins]
            strides = [[0] if x.size == 1 else [1] for x in arrays]
            d = K.EltwiseDesc()
            d.op = op_name.encode()
            d.n_in, d.rank, d.out_dtype = len(arrays), 1, K.F32
            d.sizes[0] = count
            for k, x in enumerate(arrays):
                d.in_dtype[k] = K.F32
                d.in_strides[k][0] = strides[k][0]
            plan = K.Plan("eltwise", d)
            devs = [dev(x) for x in arrays]
            out = empty((count,), K.F32)
            plan.eltwise([ptr(t) for t in devs], ptr(out))
            torch.cuda.synchronize()
            outs.append(out.cpu().numpy())
        np.testing.assert_array_equal(outs[0][:n - 3].view(np.uint32), outs[1].view(np.uint32), err_msg=op_name)
    np.testing.assert_array_equal(outs[0][:4], np.power(b[:4].astype(np.float64), a[:4].astype(np.float64)).astype(np.float32))


def test_dense_casts_between_f32_and_16_bit_floats_match_the_general_kernel():
    g = rng(32)
    n = 8 * 513
    x = (g.standard_normal(n) * 100).astype(np.float32)
    x[:6] = [np.inf, -np.inf, 0.0, -0.0, 65504.0, 1e-8]
    for narrow_dt, torch_dt in ((K.F16, torch.float16), (K.BF16, torch.bfloat16)):
        results = []
        for count in (n, n - 5):            # eight at a time; general kernel
            d = K.EltwiseDesc()
            d.op = b"cast"
            d.n_in, d.rank, d.out_dtype = 1, 1, narrow_dt
            d.sizes[0] = count
            d.in_dtype[0] = K.F32
            d.in_strides[0][0] = 1
            down = K.Plan("eltwise", d)
            src = dev(x[:count])
            half = torch.empty(count, dtype=torch_dt, device="cuda")
            down.eltwise([ptr(src)], ptr(half))
            u = K.EltwiseDesc()
            u.op = b"cast"
            u.n_in, u.rank, u.out_dtype = 1, 1, K.F32
            u.sizes[0] = count
            u.in_dtype[0] = narrow_dt
            u.in_strides[0][0] = 1
            up = K.Plan("eltwise", u)
            back = torch.empty(count, dtype=torch.float32, device="cuda")
            up.eltwise([ptr(half)], ptr(back))
            torch.cuda.synchronize()
            results.append((half.view(torch.int16).cpu().numpy(), back.cpu().numpy()))
            np.testing.assert_array_equal(back.cpu().numpy().view(np.uint32), src.to(torch_dt).to(torch.float32).cpu().numpy().view(np.uint32))
        np.testing.assert_array_equal(results[0][0][:n - 5], results[1][0])
        np.testing.assert_array_equal(results[0][1][:n - 5].view(np.uint32), results[1][1].view(np.uint32))


@pytest.mark.parametrize("dt,torch_dt", [(K.F16, torch.float16), (K.BF16, torch.bfloat16)])
def test_eltwise_dense_16_bit_form_gives_the_bits_of_the_general_form(dt, torch_dt):
    g = rng(33)
    n = 8 * 700 + 16
    a = torch.from_numpy(g.standard_normal(n).astype(np.float32)).cuda().to(torch_dt)
    b = torch.from_numpy(g.uniform(0.5, 2.0, n).astype(np.float32)).cuda().to(torch_dt)
    one = torch.tensor([1.5], device="cuda").to(torch_dt)
    for op_name, ins in (("add", [a, b]), ("mul", [a, b]), ("div", [a, b]), ("relu", [a]), ("exp", [a]), ("sub", [one, b]),
                         ("max", [a, one]), ("sqrt", [b])):
        outs = []
        for count in (n, n - 3):          # dense form; general form
            arrays = [x if x.numel() == 1 else x[:count].contiguous() for x in ins]
            d = K.EltwiseDesc()
            d.op = op_name.encode()
            d.n_in, d.rank, d.out_dtype = len(arrays), 1, dt
            d.sizes[0] = count
            for k, x in enumerate(arrays):
                d.in_dtype[k] = dt
                d.in_strides[k][0] = 0 if x.numel() == 1 else 1
            plan = K.Plan("eltwise", d)
            out = torch.empty(count, dtype=torch_dt, device="cuda")
            plan.eltwise([ptr(t) for t in arrays], ptr(out))
            torch.cuda.synchronize()
            outs.append(out.view(torch.int16).cpu().numpy())
        np.testing.assert_array_equal(outs[0][:n - 3], outs[1], err_msg=op_name)
    # and against torch for an operation whose rounding is unambiguous
    d = K.EltwiseDesc()
    d.op = b"add"
    d.n_in, d.rank, d.out_dtype = 2, 1, dt
    d.sizes[0] = n
    for k in range(2):
        d.in_dtype[k] = dt
        d.in_strides[k][0] = 1
    out = torch.empty(n, dtype=torch_dt, device="cuda")
    K.Plan("eltwise", d).eltwise([ptr(a), ptr(b)], ptr(out))
    torch.cuda.synchronize()
    assert torch.equal(out, (a.float() + b.float()).to(torch_dt))


def test_eltwise_dense_f32_with_bias_and_column_operands():
    # an operand repeated over the leading dims (a bias) or holding one value per run of the trailing dims (a column)
    # stays on the 16-byte path; +, -, *, / are correctly rounded, so numpy's float32 results are the expected bits
    from plaidml_b200.core import DType, Program
    from plaidml_b200.edsl import Placeholder
    from plaidml_b200.exec import Runner
    g = rng(34)
    cases = [((64, 256), (256,)), ((64, 256), (64, 1)), ((4, 8, 16), (8, 16)), ((4, 8, 16), (4, 8, 1)), ((4, 8, 16), (4, 1, 16)),
             ((6, 20), (20,)), ((5, 8), (5, 1))]
    for big, small in cases:
        x = g.standard_normal(big).astype(np.float32)
        y = g.uniform(0.5, 2.0, small).astype(np.float32)
        X, Y = Placeholder(DType.FLOAT32, list(big)), Placeholder(DType.FLOAT32, list(small))
        outs = Runner(Program("bcast", [X, Y], [X + Y, X * Y, Y - X, X / Y]), "cuda.0").run([x, y])
        for got, want in zip(outs, (x + y, x * y, y - x, x / y)):
            np.testing.assert_array_equal(got.view(np.uint32), want.astype(np.float32).view(np.uint32), err_msg=f"{big} {small}")
