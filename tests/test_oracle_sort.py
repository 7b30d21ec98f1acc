"""CPU: the oracle's sort rule (stable, -0 = +0, NaN placement) on hand-written cases."""
import numpy as np

import oracle as O


def test_sort_rule_on_small_cases():
    x = np.array([[3, 1, 2, 1, 3]], dtype=np.int32)
    v, i = O.sort_last_axis(O.I32, x)
    assert v.tolist() == [[1, 1, 2, 3, 3]] and i.tolist() == [[1, 3, 2, 0, 4]]
    v, i = O.sort_last_axis(O.I32, x, descending=True)
    assert v.tolist() == [[3, 3, 2, 1, 1]] and i.tolist() == [[0, 4, 2, 1, 3]]          # ties keep the source order
    f = np.array([[0.0, np.nan, -0.0, -1.0, np.inf]], dtype=np.float32)
    v, i = O.sort_last_axis(O.F32, f)
    assert i.tolist() == [[3, 0, 2, 4, 1]] and np.isnan(v[0, -1])
    v, i = O.sort_last_axis(O.F32, f, descending=True)
    assert i.tolist() == [[1, 4, 0, 2, 3]]


def test_sort_agrees_with_numpy_on_random_rows():
    rng = np.random.default_rng(1)
    x = rng.integers(-50, 50, size=(20, 257)).astype(np.int16)
    v, i = O.sort_last_axis(O.I16, x)
    assert np.array_equal(i, np.argsort(x, axis=1, kind="stable").astype(np.int32))
    assert np.array_equal(v, np.sort(x, axis=1))
