"""CPU: the oracle's sort.  `sort_last_axis_loops` runs the reference's lowering of hfusion.sort literally (n-1 bubble passes
of n-1 compare-and-swaps on `cmpf ugt` / `ult`, DecomposeOpInterfaceImpl.cpp:742-838); `sort_last_axis` is its closed
form, used at sizes the loops cannot reach.  The two must agree everywhere, NaN and signed zeros included."""
import numpy as np

import oracle as O


def test_sort_rule_on_small_cases():
    x = np.array([[3, 1, 2, 1, 3]], dtype=np.int32)
    for fn in (O.sort_last_axis, O.sort_last_axis_loops):
        v, i = fn(O.I32, x)
        assert v.tolist() == [[1, 1, 2, 3, 3]] and i.tolist() == [[1, 3, 2, 0, 4]]
        v, i = fn(O.I32, x, descending=True)
        assert v.tolist() == [[3, 3, 2, 1, 1]] and i.tolist() == [[0, 4, 2, 1, 3]]          # ties keep the source order
    # a NaN at position p ends at (p + 1) mod n, whatever the direction; zeros of either sign tie in source order
    f = np.array([[0.0, np.nan, -0.0, -1.0, np.inf]], dtype=np.float32)
    for fn in (O.sort_last_axis, O.sort_last_axis_loops):
        v, i = fn(O.F32, f)
        assert i.tolist() == [[3, 0, 1, 2, 4]] and np.isnan(v[0, 2])
        v, i = fn(O.F32, f, descending=True)
        assert i.tolist() == [[4, 0, 1, 2, 3]] and np.isnan(v[0, 2])
    # the NaN at the end of a row is carried round to the front
    g = np.array([[2.0, 1.0, np.nan]], dtype=np.float32)
    for fn in (O.sort_last_axis, O.sort_last_axis_loops):
        assert fn(O.F32, g)[1].tolist() == [[2, 1, 0]]


def test_closed_form_equals_the_loops_on_random_rows_with_nan():
    rng = np.random.default_rng(7)
    for trial in range(400):
        n = int(rng.integers(1, 40))
        x = rng.integers(-3, 4, size=(3, n)).astype(np.float32)
        x[rng.random((3, n)) < 0.2] = np.nan
        x[rng.random((3, n)) < 0.1] = -0.0
        x[rng.random((3, n)) < 0.05] = np.inf
        for dt, src in ((O.F32, x), (O.BF16, O.f32_to_bf16(x)), (O.F16, x.astype(np.float16).view(np.uint16))):
            for desc in (False, True):
                v1, i1 = O.sort_last_axis_loops(dt, src, desc)
                v2, i2 = O.sort_last_axis(dt, src, desc)
                assert np.array_equal(i1, i2), (trial, dt, desc)
                assert np.array_equal(v1.view(np.uint8), v2.view(np.uint8))


def test_sort_agrees_with_numpy_on_random_rows():
    rng = np.random.default_rng(1)
    x = rng.integers(-50, 50, size=(20, 257)).astype(np.int16)
    for fn in (O.sort_last_axis, O.sort_last_axis_loops):
        v, i = fn(O.I16, x)
        assert np.array_equal(i, np.argsort(x, axis=1, kind="stable").astype(np.int32))
        assert np.array_equal(v, np.sort(x, axis=1))
