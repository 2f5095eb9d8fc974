"""CPU restatement of the four tile operations that are not contractions -- TEST INFRASTRUCTURE ONLY.

gather / scatter / argsort follow the loops their lowering emits
(pmlc/conversion/linalg_to_pxa/tile_to_pxa_special_patterns.cc: ArgSortOpConversion :30-245, GatherOpConversion
:305-766, ScatterOpConversion :768-931); prng follows the runtime function the x86 target links
(pmlc/rt/prng.cc:8-40).  numpy evaluates one operation at a time in the array's own type, so the float arithmetic
of the interpolations rounds after every operation, as scalar code in that type does (nothing is fused).

Pinned by tests/test_oracle_special.py against the expected vectors of the reference's own tests for these
operations (plaidml/edsl/tests/edsl_test.cc: Prng :1138, Gather :1490, InterpolatedGather* :1510-1615, Scatter*
:1874-2112, ArgSort* :2400-2720), read as text.
"""

from __future__ import annotations

import numpy as np

NEAREST, LINEAR, CUBIC, NONE = range(4)
ROUND_PREFER_FLOOR, ROUND_PREFER_CEIL, FLOOR, CEIL, SIMPLE = range(5)
EDGE_PADDED, RETURN_ZERO = range(2)
SCATTER_ADD, SCATTER_SLICE, SCATTER_ELT, SCATTER_ND = range(4)


def _to_i32(x: np.ndarray) -> np.ndarray:
    """fptosi to 32 bits; out-of-range values (undefined in the lowering) saturate."""
    x = np.nan_to_num(np.asarray(x, dtype=np.float64), nan=0.0)
    return np.clip(np.trunc(x), -2147483648.0, 2147483647.0).astype(np.int64)


def gather(tensor: np.ndarray, indices: np.ndarray, axis: int = 0, interpolation: int = NONE,
           nearest: int = ROUND_PREFER_FLOOR, cube_coeff: float = -0.75, out_of_bounds: int = EDGE_PADDED) -> np.ndarray:
    """out[o.., j.., i..] = tensor[o.., indices[j..], i..] along ``axis`` (GatherMode::normal, :350-405)."""
    axis = axis % tensor.ndim
    t = np.moveaxis(tensor, axis, 0)            # [len, rest...]
    hi = t.shape[0] - 1
    flat = indices.reshape(-1)

    def take(pos):                               # pos: int64 [n] -> [n, rest...]
        return t[np.clip(pos, 0, hi)]

    if not np.issubdtype(indices.dtype, np.floating):
        got = take(flat.astype(np.int64))
    elif not np.issubdtype(tensor.dtype, np.floating):
        got = take(_to_i32(flat))
    else:
        T = tensor.dtype.type
        idx = flat.astype(T)
        shape = (-1,) + (1,) * (t.ndim - 1)
        fl = np.floor(idx)
        if interpolation == NEAREST:
            half = idx == (fl + T(0.5))
            rounded = _to_i32(np.floor(idx + T(0.5)))
            if nearest == ROUND_PREFER_FLOOR:
                pos = np.where(half, _to_i32(fl), rounded)
            elif nearest == ROUND_PREFER_CEIL:
                pos = np.where(half, _to_i32(np.ceil(idx)), rounded)
            elif nearest == FLOOR:
                pos = _to_i32(fl)
            elif nearest == CEIL:
                pos = _to_i32(np.ceil(idx))
            else:
                pos = _to_i32(idx)
            got = take(pos)
        elif interpolation == LINEAR:
            g0 = take(_to_i32(np.ceil(idx)))
            g1 = take(_to_i32(fl))
            c0 = (idx - fl).reshape(shape)
            c1 = T(1) - c0
            got = c0 * g0 + c1 * g1
        elif interpolation == CUBIC:
            a = T(cube_coeff)
            fi, ci = _to_i32(fl), _to_i32(np.ceil(idx))
            g = [take(fi - 1), take(fi), take(ci), take(ci + 1)]
            s = (idx - fl).reshape(shape)
            s2 = s * s
            s3 = s2 * s
            s_a, s2_a, s3_a = a * s, a * s2, a * s3
            s3_a2 = (a + T(2)) * s3
            s2_a3 = (a + T(3)) * s2
            s2_2a3 = ((a + a) + T(3)) * s2
            p = [(s3_a - s2_a * T(2)) + s_a, (s3_a2 - s2_a3) + T(1), (s2_2a3 - s3_a2) - s_a, s2_a - s3_a]
            got = ((p[0] * g[0] + p[1] * g[1]) + p[2] * g[2]) + p[3] * g[3]
        else:
            raise ValueError("float indices need an interpolation mode")
        got = got.astype(tensor.dtype)
        if out_of_bounds == RETURN_ZERO:
            outside = ((idx > T(hi)) | (idx < T(0))).reshape(shape)
            got = np.where(outside, T(0), got)
    got = got.reshape(indices.shape + t.shape[1:])          # [idx dims..., rest...]
    # the index dims take the place of the axis
    lead = list(range(indices.ndim, indices.ndim + axis))
    order = lead + list(range(indices.ndim)) + list(range(indices.ndim + axis, got.ndim))
    return np.ascontiguousarray(np.transpose(got, order))


def gather_nd(tensor: np.ndarray, indices: np.ndarray, batch_dims: int = 0) -> np.ndarray:
    """GatherMode::nd (:407-433): the last dim of indices addresses dims [batch_dims, batch_dims + K)."""
    k = indices.shape[-1]
    out_shape = indices.shape[:-1] + tensor.shape[batch_dims + k:]
    out = np.empty(out_shape, dtype=tensor.dtype)
    for pos in np.ndindex(*indices.shape[:-1]):
        row = [int(np.clip(indices[pos + (i,)], 0, tensor.shape[batch_dims + i] - 1)) for i in range(k)]
        out[pos] = tensor[pos[:batch_dims] + tuple(row)]
    return out


def scatter(data: np.ndarray, indices: np.ndarray, updates: np.ndarray, axis: int = 0, mode: int = SCATTER_ADD) -> np.ndarray:
    """The result starts as ``data``; every element of ``updates`` is added (mode 0) or stored (:768-931).
    Updates are applied in element order, so with equal destinations in a storing mode the last one stays."""
    out = data.copy()
    ir = indices.ndim
    for c in np.ndindex(*updates.shape):
        if mode == SCATTER_ND:
            k = indices.shape[-1]
            dst = tuple(int(indices[c[:ir - 1] + (i,)]) for i in range(k)) + c[ir - 1:]
        elif mode == SCATTER_SLICE:
            dst = list(c[:axis] + c[axis + ir - 1:])
            dst[axis] = int(indices[c[axis:axis + ir]])
            dst = tuple(dst)
        else:
            dst = list(c)
            dst[axis] = int(indices[c[:ir]])
            dst = tuple(dst)
        if len(dst) != data.ndim:
            raise ValueError("updates and indices do not address the data's dimensions")
        if any(d < 0 or d >= n for d, n in zip(dst, data.shape)):
            continue
        if mode == SCATTER_ADD:
            out[dst] = out[dst] + updates[c]
        else:
            out[dst] = updates[c]
    return out


def argsort(x: np.ndarray, axis: int = -1, descending: bool = False) -> np.ndarray:
    """Positions that sort ``x`` along ``axis``, ties in their original order (the stable selection sort of
    :130-204 with a strict comparison)."""
    moved = np.moveaxis(x, axis, -1)
    out = np.empty(moved.shape, dtype=np.int32)
    for pos in np.ndindex(*moved.shape[:-1]):
        line = moved[pos]
        _, rank = np.unique(line, return_inverse=True)     # ascending rank, equal values share one
        key = -rank if descending else rank
        out[pos] = np.argsort(key, kind="stable").astype(np.int32)
    return np.ascontiguousarray(np.moveaxis(out, -1, axis))


def prng(state: np.ndarray, count: int):
    """(numbers f32[count], new state) of the three-word generator (pmlc/rt/prng.cc:26-39)."""
    s0, s1, s2 = (int(v) & 0xFFFFFFFF for v in state.reshape(-1)[:3])
    m = 0xFFFFFFFF
    out = np.empty(count, dtype=np.float32)
    for i in range(count):
        out[i] = np.float32((s0 ^ s1 ^ s2) / 4294967296.0)
        s0 = (((s0 & 4294967294) << 12) & m) ^ ((((s0 << 13) & m) ^ s0) >> 19)
        s1 = (((s1 & 4294967288) << 4) & m) ^ ((((s1 << 2) & m) ^ s1) >> 25)
        s2 = (((s2 & 4294967280) << 17) & m) ^ ((((s2 << 3) & m) ^ s2) >> 11)
    new_state = state.copy().reshape(-1)
    new_state[:3] = np.array([s0, s1, s2], dtype=np.uint64).astype(state.dtype)
    return out, new_state.reshape(state.shape)


def nms(boxes: np.ndarray, scores: np.ndarray, iou_threshold: float, score_threshold: float, max_per_class: int,
        soft_sigma: float = 0.0, center_point_box: bool = False, sort_descending: bool = True, clip_before: bool = False,
        style: int = 2, share_location: bool = True, hard_suppression: bool = True):
    """Non-maximum suppression as the op library builds it (plaidml/op/lib/ops.cc:2034-2419, NMS box decoding), as plain
    loops in float32.  PARITY UNPINNED: the reference's tests hold no expected values for this operation; this
    restatement follows the reference's sequence of operations (so that float results agree) and pins only that the
    device and the CPU compute the same thing, plus properties any NMS has (tests/test_gpu_special.py).

    boxes [batch, boxes, 4], scores [batch, classes, boxes].  Returns (rows of (batch, class, box) int32, rows of
    (batch, class, score) float32, number of valid picks); rows that found nothing hold -1.  style: 0 CAFFE (only a
    class's best `max_per_class` boxes compete), 1 MXNET (a box competes in its best class only), 2 OV."""
    f = np.float32
    nb, nc, nx = scores.shape
    b = boxes.astype(f)
    if center_point_box:
        xc, yc, hw, hh = b[..., 0], b[..., 1], b[..., 2] / f(2), b[..., 3] / f(2)
        x1, x2, y1, y2 = xc - hw, xc + hw, yc - hh, yc + hh
    else:
        y1, y2 = np.minimum(b[..., 0], b[..., 2]), np.maximum(b[..., 0], b[..., 2])
        x1, x2 = np.minimum(b[..., 1], b[..., 3]), np.maximum(b[..., 1], b[..., 3])
    if clip_before:
        y1, x1, y2, x2 = (np.clip(v, f(0), f(1)) for v in (y1, x1, y2, x2))
    if not share_location:
        raise ValueError("boxes per class need boxes of shape [batch, classes * boxes, 4]; not restated")
    area = (y2 - y1) * (x2 - x1)
    ygap = np.minimum(y2[:, :, None], y2[:, None, :]) - np.maximum(y1[:, :, None], y1[:, None, :])
    xgap = np.minimum(x2[:, :, None], x2[:, None, :]) - np.maximum(x1[:, :, None], x1[:, None, :])
    inter = np.where(ygap > 0, ygap, f(0)) * np.where(xgap > 0, xgap, f(0))
    denom = area[:, :, None] + area[:, None, :] - inter
    with np.errstate(divide="ignore", invalid="ignore"):
        iou = inter * np.where(denom <= 0, f(0), f(1) / denom)          # [batch, boxes, boxes]
    per_class = min(nx, max_per_class) if max_per_class else nx
    live = np.where(scores.astype(f) > f(score_threshold), scores.astype(f), f(0))

    def stable_desc(line):
        return argsort(line, 0, True)

    if style == 0:
        kept = np.zeros_like(live)
        for bi in range(nb):
            for ci in range(nc):
                top = stable_desc(live[bi, ci])[:per_class]
                kept[bi, ci, top] = live[bi, ci, top]
        live = kept
    elif style == 1:
        kept = np.zeros_like(live)
        for bi in range(nb):
            best_class = np.array([stable_desc(live[bi, :, x])[0] for x in range(nx)])
            best_score = live[bi, best_class, np.arange(nx)]
            top = np.sort(stable_desc(best_score)[:per_class])
            kept[bi, best_class[top], top] = best_score[top]
        live = kept
    weight = f(-0.5 / soft_sigma) if soft_sigma else f(0)
    box_rows = np.full((nb, nc, per_class, 3), -1, dtype=np.int32)
    score_rows = np.full((nb, nc, per_class, 3), -1, dtype=f)
    valid = 0
    for k in range(per_class):
        for bi in range(nb):
            for ci in range(nc):
                cand = int(stable_desc(live[bi, ci])[0])
                score = live[bi, ci].max()
                if score != 0:
                    valid += 1
                if score > 0:
                    box_rows[bi, ci, k] = (bi, ci, cand)
                    score_rows[bi, ci, k] = (bi, ci, score)
                live[bi, ci, cand] = 0
                overlap = iou[bi, cand]
                hit = overlap >= f(iou_threshold) if hard_suppression else overlap > f(iou_threshold)
                live[bi, ci] = np.where(hit, f(0), live[bi, ci])
                if soft_sigma:
                    live[bi, ci] = live[bi, ci] * np.exp(overlap * overlap * weight).astype(f)
                    live[bi, ci] = np.where(live[bi, ci] > f(score_threshold), live[bi, ci], f(0))
    box_rows = box_rows.reshape(-1, 3)
    score_rows = score_rows.reshape(-1, 3)
    if sort_descending:
        order = argsort(score_rows[:, 2], 0, True)
    else:
        order = np.argsort(np.where(score_rows[:, 2] != -1, np.arange(len(score_rows)), len(score_rows)), kind="stable")
    return box_rows[order], score_rows[order], valid
