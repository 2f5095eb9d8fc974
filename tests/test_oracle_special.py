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
