"""gather / scatter / argsort / prng on the device: the reference's own test cases built through the EDSL, the
kernels against the CPU restatement on seeded inputs, and properties at sizes the restatement cannot reach."""

import numpy as np
import pytest
import torch

import special_cases as SC
from oracle import special as S
from plaidml_b200 import edsl, op
from plaidml_b200 import kernels as K
from plaidml_b200.core import DType, Program
from plaidml_b200.edsl import Constant, Placeholder
from plaidml_b200.exec import Runner
from gpu_util import dev, ptr, rng

pytestmark = pytest.mark.gpu

DT = {"FLOAT16": DType.FLOAT16, "FLOAT32": DType.FLOAT32, "FLOAT64": DType.FLOAT64, "INT32": DType.INT32}
K_OF = {np.dtype(np.float16): K.F16, np.dtype(np.float32): K.F32, np.dtype(np.float64): K.F64,
        np.dtype(np.int8): K.I8, np.dtype(np.int16): K.I16, np.dtype(np.int32): K.I32, np.dtype(np.int64): K.I64,
        np.dtype(np.uint8): K.U8}


# ------------------------------------------------------------------ the reference's cases through the EDSL

def build_case(name):
    kind, kw, _ = SC.CASES[name]
    arrays = SC.inputs(name)
    if kind == "prng":
        state = Constant(arrays[0], name="S")
        return Program("prng", [], list(edsl.prng(state, kw["dims"]))), []
    holders = SC.KATS[name]["placeholders"]
    ins = [Placeholder(DT[h["dtype"]], h["shape"]) for h in holders.values()]
    if kind == "gather":
        out = edsl.gather(ins[0], ins[1], axis=kw["axis"], interpolation_mode=kw.get("interpolation", S.NONE),
                          nearest_mode=kw.get("nearest", 0), cube_coeff=kw.get("cube_coeff", -0.75),
                          out_of_bounds_mode=kw.get("out_of_bounds", 0))
    elif kind == "gather_nd":
        out = op.gatherND(ins[0], ins[1], batch_dims=kw["batch_dims"])
    elif kind == "scatter":
        out = edsl.scatter(ins[0], ins[1], ins[2], axis=kw["axis"], mode=kw["mode"])
    else:
        out = edsl.argsort(ins[0], kw["axis"], edsl.SortDirection.DESC if kw["descending"] else edsl.SortDirection.ASC)
    return Program(name, ins, [out]), arrays


@pytest.mark.parametrize("name", sorted(SC.CASES))
def test_reference_case_on_the_device(name):
    program, arrays = build_case(name)
    got = Runner(program, "cuda.0").run(arrays)
    SC.check(name, got)
    # ... and, beyond the test's own tolerance, the device agrees with the CPU restatement bit for bit
    for g, want in zip(got, SC.run_oracle(name)):
        np.testing.assert_array_equal(np.asarray(g).reshape(-1), np.asarray(want).reshape(-1), err_msg=name)


# ------------------------------------------------------------------ kernels against the restatement

def run_special(desc, ins, out_shape, out_np_dtype, second=None):
    plan = K.Plan("special", desc)
    d_ins = [dev(a) for a in ins]
    out = torch.empty(out_shape, dtype=torch.from_numpy(np.empty(0, dtype=out_np_dtype)).dtype, device="cuda")
    out2 = None if second is None else torch.empty(second[0], dtype=torch.int32, device="cuda")
    plan.special([ptr(t) for t in d_ins], ptr(out), ptr(out2))
    torch.cuda.synchronize()
    return (out.cpu().numpy(), None if out2 is None else out2.cpu().numpy())


@pytest.mark.parametrize("seed", range(24))
def test_gather_along_an_axis_matches_the_restatement(seed):
    g = rng(4000 + seed)
    rank = int(g.integers(1, 5))
    shape = [int(v) for v in g.integers(1, 7, rank)]
    axis = int(g.integers(0, rank))
    shape[axis] = int(g.integers(1, 40))
    idx_shape = [int(v) for v in g.integers(1, 6, int(g.integers(1, 4)))]
    tdt = [np.float32, np.float64, np.float16, np.int32, np.int8, np.int64][seed % 6]
    float_idx = seed % 2 == 0
    if np.issubdtype(tdt, np.floating):
        t = g.standard_normal(shape).astype(tdt)
    else:
        t = g.integers(-100, 100, shape).astype(tdt)
    if float_idx:
        idt = tdt if np.issubdtype(tdt, np.floating) else np.float32
        idx = g.uniform(-2.0, shape[axis] + 1.0, idx_shape).astype(idt)
        idx.reshape(-1)[::3] = np.floor(idx.reshape(-1)[::3]) + 0.5     # halves exercise the rounding rules
        idx.reshape(-1)[1::5] = np.floor(idx.reshape(-1)[1::5])         # ... and whole numbers the floor == ceil case
    else:
        idx = g.integers(-2, shape[axis] + 2, idx_shape).astype([np.int32, np.int64][seed % 4 // 2])
    interp = int(g.integers(0, 3)) if float_idx else S.NONE
    nearest = int(g.integers(0, 5))
    oob = int(g.integers(0, 2))
    coeff = float(g.choice([-0.75, -0.5, -1.0]))
    d = K.special_desc(K.SPECIAL_GATHER, K_OF[np.dtype(tdt)], shape, K_OF[idx.dtype], idx_shape, axis=axis, mode=0,
                       interpolation=interp, nearest=nearest, out_of_bounds=oob, cube_coeff=coeff)
    want = S.gather(t, idx, axis, interp, nearest, coeff, oob)
    got, _ = run_special(d, [t, idx], want.shape, tdt)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("seed", range(10))
def test_gather_nd_matches_the_restatement(seed):
    g = rng(4100 + seed)
    rank = int(g.integers(1, 6))
    shape = [int(v) for v in g.integers(1, 6, rank)]
    batch = int(g.integers(0, rank))
    k = int(g.integers(1, rank - batch + 1)) if rank - batch >= 1 else 0
    if k == 0:
        batch, k = 0, 1
    mid = [int(v) for v in g.integers(1, 5, int(g.integers(0, 3)))]
    idx_shape = shape[:batch] + mid + [k]
    idx = np.stack([g.integers(-1, shape[batch + i] + 1, idx_shape[:-1]) for i in range(k)], axis=-1).astype(np.int32)
    t = g.integers(-1000, 1000, shape).astype([np.float32, np.int16, np.float64][seed % 3])
    d = K.special_desc(K.SPECIAL_GATHER, K_OF[t.dtype], shape, K.I32, idx_shape, mode=1, batch_dims=batch)
    want = S.gather_nd(t, idx, batch)
    got, _ = run_special(d, [t, idx], want.shape, t.dtype)
    np.testing.assert_array_equal(got, want)


def scatter_case(seed):
    """Seeded data / indices / updates for one scatter mode; storing modes get distinct destinations (with equal
    destinations one of the updates stays, which no comparison can pin), the adding mode gets duplicates."""
    g = rng(4200 + seed)
    mode = seed % 4
    tdt = [np.float32, np.int32, np.float16, np.int8, np.float64, np.int64, np.int16, np.uint8][seed % 8]
    if mode == 0:
        rank = int(g.integers(1, 4))
        data_shape = [int(v) for v in g.integers(2, 9, rank)]
        axis = int(g.integers(0, rank))
        upd_shape = [int(g.integers(1, n + 1)) for n in data_shape]
        idx_shape = upd_shape[:int(g.integers(1, rank + 1))]
        idx = g.integers(-1, data_shape[axis] + 1, idx_shape).astype(np.int32)      # duplicates add up, some land outside
    elif mode == 2:
        rank = int(g.integers(1, 4))
        data_shape = [int(v) for v in g.integers(2, 9, rank)]
        axis = int(g.integers(0, rank))
        upd_shape = [int(g.integers(1, n + 1)) for n in data_shape]
        idx_rank = int(g.integers(1, rank + 1))
        if axis >= idx_rank:
            upd_shape[axis] = 1          # the index does not depend on the axis coordinate: one update per line
        idx_shape = upd_shape[:idx_rank]
        perm = g.permutation(data_shape[axis] + 1)       # (one value points outside)
        along = np.arange(idx_shape[axis]) if axis < idx_rank else np.zeros(1, dtype=np.int64)
        shape = [1] * idx_rank
        if axis < idx_rank:
            shape[axis] = idx_shape[axis]
        idx = np.broadcast_to(perm[along].reshape(shape), idx_shape).astype(np.int32)
    elif mode == 1:
        rank = int(g.integers(1, 4))
        data_shape = [int(v) for v in g.integers(2, 9, rank)]
        axis = int(g.integers(0, rank))
        data_shape[axis] = int(g.integers(6, 12))
        idx_shape = [[2], [3], [2, 2], [5], [3, 2]][int(g.integers(0, 5))]
        upd_shape = [int(g.integers(1, n + 1)) for n in data_shape[:axis]] + idx_shape + \
                    [int(g.integers(1, n + 1)) for n in data_shape[axis + 1:]]
        n = int(np.prod(idx_shape))
        idx = g.permutation(data_shape[axis] + 1)[:n].reshape(idx_shape).astype(np.int32)
    else:
        rank = int(g.integers(1, 5))
        data_shape = [int(v) for v in g.integers(2, 7, rank)]
        axis = 0
        k = int(g.integers(1, rank + 1))
        cells = int(np.prod(data_shape[:k]))
        lead = [int(v) for v in g.integers(1, 5, int(g.integers(1, 3)))]
        while int(np.prod(lead)) > cells + 1:
            lead = lead[:-1] if len(lead) > 1 else [cells]
        idx_shape = lead + [k]
        upd_shape = lead + [int(g.integers(1, n + 1)) for n in data_shape[k:]]
        rows = int(np.prod(lead))
        pick = g.permutation(cells + 1)[:rows]
        coords = np.stack(np.unravel_index(np.minimum(pick, cells - 1), data_shape[:k]), axis=-1)
        coords[pick == cells] = data_shape[0]          # one row may point outside: dropped
        idx = coords.reshape(idx_shape).astype(np.int32)
    # small integer values: sums are exact in every type and order
    data = g.integers(0, 3, data_shape).astype(tdt)
    upd = g.integers(1, 4, upd_shape).astype(tdt)
    return data, idx, upd, axis, mode


@pytest.mark.parametrize("seed", range(16))
def test_scatter_matches_the_restatement(seed):
    data, idx, upd, axis, mode = scatter_case(seed)
    want = S.scatter(data, idx, upd, axis, mode)
    d = K.special_desc(K.SPECIAL_SCATTER, K_OF[data.dtype], list(data.shape), K.I32, list(idx.shape), list(upd.shape),
                       axis=axis, mode=mode)
    got, _ = run_special(d, [data, idx, upd], data.shape, data.dtype)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("seed", range(12))
def test_argsort_matches_the_restatement(seed):
    g = rng(4300 + seed)
    rank = int(g.integers(1, 4))
    shape = [int(v) for v in g.integers(1, 6, rank)]
    axis = int(g.integers(0, rank))
    shape[axis] = int(g.choice([1, 2, 3, 17, 64, 100, 257, 1000]))
    tdt = [np.float32, np.int32, np.float16, np.int8, np.float64, np.int64][seed % 6]
    x = g.integers(-20, 20, shape).astype(tdt)        # few distinct values: many ties
    if np.issubdtype(tdt, np.floating) and seed % 2:
        x = g.standard_normal(shape).astype(tdt)
    desc = bool(seed % 2)
    d = K.special_desc(K.SPECIAL_ARGSORT, K_OF[np.dtype(tdt)], shape, axis=axis, mode=int(desc))
    got, _ = run_special(d, [x], shape, np.int32)
    np.testing.assert_array_equal(got, S.argsort(x, axis, desc))


def test_argsort_of_long_lines_is_a_stable_sort():
    g = rng(4400)
    x = g.integers(0, 1000, (3, 200_001, 2)).astype(np.int32)
    d = K.special_desc(K.SPECIAL_ARGSORT, K.I32, list(x.shape), axis=1, mode=0)
    got, _ = run_special(d, [x], x.shape, np.int32)
    np.testing.assert_array_equal(got, np.argsort(x, axis=1, kind="stable").astype(np.int32))
    d = K.special_desc(K.SPECIAL_ARGSORT, K.I32, list(x.shape), axis=1, mode=1)
    got, _ = run_special(d, [x], x.shape, np.int32)
    np.testing.assert_array_equal(got, np.argsort(-x, axis=1, kind="stable").astype(np.int32))


def test_prng_in_parallel_is_the_sequential_generator():
    state = np.array([123456789, 362436069, 521288629, 77], dtype=np.uint32)
    for count in (0, 1, 63, 64, 65, 100_003):
        d = K.special_desc(K.SPECIAL_PRNG, sizes=[count] if count else [0], state_elems=4)
        want, after = S.prng(state, count)
        got, new_state = run_special(d, [state.view(np.int32)], (count,), np.float32, second=((4,),))
        np.testing.assert_array_equal(got, want)
        np.testing.assert_array_equal(new_state.view(np.uint32), after)


def test_prng_of_many_numbers_continues_from_its_own_state():
    # 40 million numbers in one launch == 10 million, then 30 million from the state the first launch left
    state = np.array([5, 6, 7], dtype=np.uint32)
    whole, end = run_special(K.special_desc(K.SPECIAL_PRNG, sizes=[40_000_000], state_elems=3), [state.view(np.int32)],
                             (40_000_000,), np.float32, second=((3,),))
    a, mid = run_special(K.special_desc(K.SPECIAL_PRNG, sizes=[10_000_000], state_elems=3), [state.view(np.int32)],
                         (10_000_000,), np.float32, second=((3,),))
    b, end2 = run_special(K.special_desc(K.SPECIAL_PRNG, sizes=[30_000_000], state_elems=3), [mid],
                          (30_000_000,), np.float32, second=((3,),))
    np.testing.assert_array_equal(whole[:10_000_000], a)
    np.testing.assert_array_equal(whole[10_000_000:], b)
    np.testing.assert_array_equal(end, end2)
    want, _ = S.prng(state, 1000)
    np.testing.assert_array_equal(whole[:1000], want)
    assert 0.49 < float(whole.mean()) < 0.51


def test_inconsistent_descriptors_are_refused():
    bad = [
        K.special_desc(K.SPECIAL_GATHER, K.F32, [4, 4], K.I32, [3], axis=2),
        K.special_desc(K.SPECIAL_GATHER, K.F32, [4, 4], K.F32, [3], axis=0, interpolation=3),
        K.special_desc(K.SPECIAL_GATHER, K.F32, [4, 4], K.F32, [3, 1], mode=1),
        K.special_desc(K.SPECIAL_GATHER, K.F32, [4, 4], K.I32, [3, 3], mode=1),
        K.special_desc(K.SPECIAL_SCATTER, K.F32, [4, 4], K.I64, [2], [2, 4]),
        K.special_desc(K.SPECIAL_SCATTER, K.F32, [4, 4], K.I32, [2], [2, 4, 4]),
        K.special_desc(K.SPECIAL_ARGSORT, K.F32, [4, 4], axis=2),
        K.special_desc(K.SPECIAL_PRNG, sizes=[8], state_elems=2),
    ]
    for d in bad:
        with pytest.raises(K.KernelError):
            K.Plan("special", d)


# ------------------------------------------------------------------ the op library on top of them

def run_op(build, *arrays, dtypes=None):
    dtypes = dtypes or [DType.FLOAT32] * len(arrays)
    ins = [Placeholder(dt, list(a.shape)) for dt, a in zip(dtypes, arrays)]
    out = build(*ins)
    outs = list(out) if isinstance(out, (list, tuple)) else [out]
    res = Runner(Program("op", ins, outs), "cuda.0").run(list(arrays))
    return res if isinstance(out, (list, tuple)) else res[0]


def test_sort_and_topk():
    g = rng(4500)
    x = g.integers(-50, 50, (4, 9, 5)).astype(np.float32)
    np.testing.assert_array_equal(run_op(lambda X: op.sort(X, 1), x), np.sort(x, axis=1))
    np.testing.assert_array_equal(run_op(lambda X: op.sort(X, -1, edsl.SortDirection.DESC), x), -np.sort(-x, axis=-1))
    vals, pos = run_op(lambda X: op.topk(X, 3, axis=1), x)
    order = S.argsort(x, 1, True)[:, :3, :]
    np.testing.assert_array_equal(pos, order)
    np.testing.assert_array_equal(vals, np.take_along_axis(x, order.astype(np.int64), axis=1))
    vals, pos = run_op(lambda X: op.topk(X, 3, axis=1, sort_type=op.TopKSortType.INDEX), x)
    by_index = np.sort(order, axis=1)
    np.testing.assert_array_equal(pos, by_index)
    np.testing.assert_array_equal(vals, np.take_along_axis(x, by_index.astype(np.int64), axis=1))


def test_gather_nd_with_linear_interpolation_blends_the_corners_of_zero_padded_data():
    g = rng(4600)
    x = g.standard_normal((5, 6)).astype(np.float32)
    rows = g.uniform(-1.5, 6.5, (7, 2)).astype(np.float32)
    rows[:, 0] = np.clip(rows[:, 0], -1.5, 5.4)
    got = run_op(lambda X, I: op.gatherND(X, I, interpolation_mode=edsl.InterpolationMode.LINEAR), x, rows)
    padded = np.zeros((9, 10), dtype=np.float64)
    padded[2:7, 2:8] = x
    want = np.zeros(7)
    for r, (a, b) in enumerate(rows.astype(np.float64) + 2):
        a0, b0 = int(np.floor(a)), int(np.floor(b))
        for da in (0, 1):
            for db in (0, 1):
                w = (a - a0 if da else a0 + 1 - a) * (b - b0 if db else b0 + 1 - b)
                want[r] += w * padded[a0 + da, b0 + db]
    np.testing.assert_allclose(got.reshape(-1), want, rtol=1e-5, atol=1e-6)


def test_programs_mix_them_with_contractions():
    # scores = A . B; the three best columns per row, their scores scattered back into a zero matrix
    g = rng(4700)
    a = g.standard_normal((6, 16)).astype(np.float32)
    b = g.standard_normal((16, 10)).astype(np.float32)

    def build(A, B):
        scores = op.dot(A, B)
        vals, pos = op.topk(scores, 3, axis=1)
        rows = edsl.index([6, 3], 0)
        where = op.concatenate([op.unsqueeze(rows, [2]), op.unsqueeze(pos, [2])], axis=-1)
        zeros = scores * 0.0
        return edsl.scatter(zeros, where, vals, mode=edsl.ScatterMode.UPDATE_ND)

    got = run_op(build, a, b)
    s = (a.astype(np.float64) @ b.astype(np.float64))
    want = np.zeros_like(s)
    order = np.argsort(-s, axis=1, kind="stable")[:, :3]
    np.put_along_axis(want, order, np.take_along_axis(s, order, axis=1), axis=1)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)


# ------------------------------------------------------------------ non-maximum suppression (parity unpinned: see the oracle)

def nms_case(seed, nb=2, nc=3, nx=24):
    g = rng(4800 + seed)
    centre = g.uniform(0.1, 0.9, (nb, nx, 2))
    size = g.uniform(0.05, 0.4, (nb, nx, 2))
    corners = np.concatenate([centre - size / 2, centre + size / 2], axis=-1).astype(np.float32)   # y1 x1 y2 x2
    scores = g.uniform(0.0, 1.0, (nb, nc, nx)).astype(np.float32)
    return corners, scores


def run_nms(boxes, scores, iou_thr, score_thr, k, **kw):
    B = Placeholder(DType.FLOAT32, list(boxes.shape))
    S_ = Placeholder(DType.FLOAT32, list(scores.shape))
    I = Placeholder(DType.FLOAT32, [1])
    T = Placeholder(DType.FLOAT32, [1])
    outs = op.nms(B, S_, I, T, k, **kw)
    return Runner(Program("nms", [B, S_, I, T], list(outs)), "cuda.0").run(
        [boxes, scores, np.array([iou_thr], np.float32), np.array([score_thr], np.float32)])


@pytest.mark.parametrize("style", [op.NmsStyle.OV, op.NmsStyle.CAFFE, op.NmsStyle.MXNET])
@pytest.mark.parametrize("sort_desc", [True, False])
def test_nms_matches_the_restatement(style, sort_desc):
    boxes, scores = nms_case(int(style) * 2 + int(sort_desc))
    got_b, got_s, got_v = run_nms(boxes, scores, 0.4, 0.3, 5, nms_style=style, sort_result_descending=sort_desc)
    want_b, want_s, want_v = S.nms(boxes, scores, 0.4, 0.3, 5, style=int(style), sort_descending=sort_desc)
    np.testing.assert_array_equal(got_b, want_b)
    np.testing.assert_array_equal(got_s, want_s)
    assert int(got_v.reshape(-1)[0]) == want_v
    # what any non-maximum suppression guarantees: picks of one (batch, class) overlap each other by less than the
    # threshold, score above the score threshold, and no box is picked twice
    y1, x1, y2, x2 = (boxes[..., i] for i in range(4))
    rows = got_b[got_b[:, 0] >= 0]
    assert len(rows) == want_v and len({tuple(r) for r in rows}) == len(rows)
    for b_, c_ in {(r[0], r[1]) for r in rows}:
        picked = [r[2] for r in rows if r[0] == b_ and r[1] == c_]
        assert all(scores[b_, c_, p] > 0.3 for p in picked)
        for i, p in enumerate(picked):
            for q in picked[i + 1:]:
                ih = max(0.0, min(y2[b_, p], y2[b_, q]) - max(y1[b_, p], y1[b_, q]))
                iw = max(0.0, min(x2[b_, p], x2[b_, q]) - max(x1[b_, p], x1[b_, q]))
                union = (y2[b_, p] - y1[b_, p]) * (x2[b_, p] - x1[b_, p]) + (y2[b_, q] - y1[b_, q]) * (x2[b_, q] - x1[b_, q]) - ih * iw
                assert ih * iw / union < 0.4 + 1e-6


def test_nms_centre_boxes_clipping_soft_suppression():
    boxes, scores = nms_case(9, nb=1, nc=2, nx=16)
    centre = np.concatenate([(boxes[..., 1:2] + boxes[..., 3:4]) / 2, (boxes[..., 0:1] + boxes[..., 2:3]) / 2,
                             boxes[..., 3:4] - boxes[..., 1:2], boxes[..., 2:3] - boxes[..., 0:1]], axis=-1).astype(np.float32)
    kw = dict(center_point_box=True, clip_before_nms=True, soft_nms_sigma=0.5, hard_suppression=False)
    got_b, got_s, got_v = run_nms(centre, scores, 0.5, 0.2, 4, **kw)
    want_b, want_s, want_v = S.nms(centre, scores, 0.5, 0.2, 4, soft_sigma=0.5, center_point_box=True, clip_before=True,
                                   hard_suppression=False)
    np.testing.assert_array_equal(got_b, want_b)
    np.testing.assert_allclose(got_s, want_s, rtol=1e-5, atol=1e-6)
    assert int(got_v.reshape(-1)[0]) == want_v


def test_gather_of_whole_rows_moves_16_byte_pieces():
    # rows of 64 f32 and of 24 int8 x 2 (48 bytes): the 16-byte path, four pieces per thread, counts that are not
    # multiples of four, positions outside the table on both sides
    g = rng(4900)
    for dtype, tail, n_rows, n_idx in ((np.float32, (64,), 1000, 4099), (np.int8, (24, 2), 77, 1001), (np.float64, (3, 2), 50, 7)):
        table = g.integers(-100, 100, (n_rows,) + tail).astype(dtype)
        idx = g.integers(-3, n_rows + 3, n_idx).astype(np.int32)
        d = K.special_desc(K.SPECIAL_GATHER, K_OF[np.dtype(dtype)], list(table.shape), K.I32, [n_idx], axis=0)
        got, _ = run_special(d, [table, idx], (n_idx,) + tail, dtype)
        np.testing.assert_array_equal(got, table[np.clip(idx, 0, n_rows - 1)])
    # an outer dimension in front of the axis
    table = g.standard_normal((5, 40, 8)).astype(np.float32)
    idx = g.integers(0, 40, (6, 3)).astype(np.int64)
    d = K.special_desc(K.SPECIAL_GATHER, K.F32, list(table.shape), K.I64, list(idx.shape), axis=1)
    got, _ = run_special(d, [table, idx], (5, 6, 3, 8), np.float32)
    np.testing.assert_array_equal(got, table[:, idx, :])


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_scatter_of_whole_rows(mode):
    # data [rows][5][3], a list of row numbers, updates [n][5][3]: the four-updates-per-thread form
    g = rng(4950 + mode)
    for dtype in (np.float32, np.int16, np.float64):
        data = g.integers(0, 5, (37, 5, 3)).astype(dtype)
        n = 33 if mode else 201
        idx = (g.permutation(39)[:n] - 1 if mode else g.integers(-1, 38, n)).astype(np.int32)    # storing modes: distinct rows
        upd = g.integers(1, 4, (n, 5, 3)).astype(dtype)
        d = K.special_desc(K.SPECIAL_SCATTER, K_OF[np.dtype(dtype)], list(data.shape), K.I32, [n], list(upd.shape), axis=0, mode=mode)
        got, _ = run_special(d, [data, idx, upd], data.shape, dtype)
        np.testing.assert_array_equal(got, S.scatter(data, idx, upd, 0, mode))
