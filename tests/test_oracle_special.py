"""The CPU restatement of gather / scatter / argsort / prng (oracle/special.py) against the expected vectors of the
reference's own tests for these operations (30 tests of plaidml/edsl/tests/edsl_test.cc, read as text)."""

import numpy as np
import pytest

import special_cases as SC
from oracle import special as S


@pytest.mark.parametrize("name", sorted(SC.CASES))
def test_oracle_reproduces_the_reference_tests_expected_values(name):
    SC.check(name, SC.run_oracle(name))


def test_every_extracted_test_is_covered():
    assert sorted(SC.CASES) == sorted(SC.KATS)


def test_prng_state_after_n_numbers_continues_the_sequence():
    state = np.array([123456789, 362436069, 521288629], dtype=np.uint32)
    whole, after = S.prng(state, 300)
    first, mid = S.prng(state, 113)
    rest, end = S.prng(mid, 187)
    np.testing.assert_array_equal(np.concatenate([first, rest]), whole)
    np.testing.assert_array_equal(end, after)
    assert whole.min() >= 0.0 and whole.max() < 1.0 or whole.max() == 1.0   # (x / 2^32 can round up to 1.0 in f32)


def test_argsort_keeps_the_order_of_equal_elements_in_both_directions():
    x = np.array([3, 1, 3, 2, 1, 3], dtype=np.int32)
    np.testing.assert_array_equal(S.argsort(x, 0, False), [1, 4, 3, 0, 2, 5])
    np.testing.assert_array_equal(S.argsort(x, 0, True), [0, 2, 5, 3, 1, 4])


def test_scatter_drops_updates_outside_the_data_and_gather_clamps():
    data = np.zeros(4, dtype=np.float32)
    out = S.scatter(data, np.array([1, 7, -1], dtype=np.int32), np.array([5, 6, 7], dtype=np.float32))
    np.testing.assert_array_equal(out, [0, 5, 0, 0])
    got = S.gather(np.arange(4, dtype=np.float32), np.array([-3, 2, 9], dtype=np.int32))
    np.testing.assert_array_equal(got, [0, 2, 3])


def test_nms_restatement_agrees_with_textbook_greedy_suppression():
    # an independent formulation: per (batch, class) walk the boxes by falling score and keep a box unless it overlaps
    # an already kept one by the threshold or more; then the best `k` per class, all rows by falling score
    g = np.random.default_rng(5)
    nb, nc, nx, k, iou_thr, score_thr = 2, 3, 30, 6, 0.35, 0.25
    centre = g.uniform(0.1, 0.9, (nb, nx, 2))
    size = g.uniform(0.05, 0.4, (nb, nx, 2))
    boxes = np.concatenate([centre - size / 2, centre + size / 2], axis=-1).astype(np.float32)
    scores = g.uniform(0, 1, (nb, nc, nx)).astype(np.float32)

    def iou(a, b):
        ih = max(np.float32(0), min(a[2], b[2]) - max(a[0], b[0]))
        iw = max(np.float32(0), min(a[3], b[3]) - max(a[1], b[1]))
        inter = ih * iw
        union = (a[2] - a[0]) * (a[3] - a[1]) + (b[2] - b[0]) * (b[3] - b[1]) - inter
        return inter * (np.float32(1) / union) if union > 0 else np.float32(0)

    rows = []
    for b in range(nb):
        for c in range(nc):
            kept = []
            for x in S.argsort(scores[b, c], 0, True):
                if scores[b, c, x] <= score_thr or len(kept) == k:
                    break
                if all(iou(boxes[b, x], boxes[b, y]) < np.float32(iou_thr) for y in kept):
                    kept.append(int(x))
            rows += [(b, c, x, scores[b, c, x]) for x in kept]
    rows.sort(key=lambda r: -r[3])
    got_b, got_s, valid = S.nms(boxes, scores, iou_thr, score_thr, k)
    assert valid == len(rows)
    np.testing.assert_array_equal(got_b[:valid], np.array([r[:3] for r in rows], dtype=np.int32))
    np.testing.assert_array_equal(got_s[:valid, 2], np.array([r[3] for r in rows], dtype=np.float32))
    assert (got_b[valid:] == -1).all() and (got_s[valid:] == -1).all()
