"""CPU: the oracle's cumulative ops (vcumsum / vcumprod / vcummax / vcummin) against hand-computed cases that
follow the reference's loop nest (test/Dialect/HIVM/hivm-lower-to-loops-op.mlir:1558-1599: dst[0] = src[0],
dst[i] = src[i] + dst[i-1]) and against properties that do not depend on the size."""
import numpy as np

import oracle as O


def test_cumsum_i16_follows_the_loop_nest_and_wraps():
    x = np.array([[1, 2, 3, 4], [32767, 1, -5, 7]], dtype=np.int16)
    got = O.cumulative("sum", O.I16, x, axis=1)
    assert got.tolist() == [[1, 3, 6, 10], [32767, -32768, 32763, -32766]]
    rev = O.cumulative("sum", O.I16, x[:1], axis=1, reverse=True)
    assert rev.tolist() == [[10, 9, 7, 4]]
    col = O.cumulative("sum", O.I16, np.array([[1, 10], [2, 20], [3, 30]], dtype=np.int16), axis=0)
    assert col.tolist() == [[1, 10], [3, 30], [6, 60]]


def test_cumprod_max_min_small_cases():
    x = np.array([[2, -3, 4, -1]], dtype=np.int32)
    assert O.cumulative("prod", O.I32, x).tolist() == [[2, -6, -24, 24]]
    assert O.cumulative("max", O.I32, x).tolist() == [[2, 2, 4, 4]]
    assert O.cumulative("min", O.I32, x).tolist() == [[2, -3, -3, -3]]
    assert O.cumulative("min", O.I32, x, reverse=True).tolist() == [[-3, -3, -1, -1]]


def test_f32_cumsum_is_sequential_left_to_right():
    # (1e8 + 1) + -1e8 = 0 in f32 when summed left to right; a tree would give other answers
    x = np.array([[1e8, 1.0, -1e8, 1.0]], dtype=np.float32)
    assert O.cumulative("sum", O.F32, x).tolist() == [[1e8, 1e8, 0.0, 1.0]]


def test_16_bit_floats_keep_an_f32_running_value():
    # 2048 + 1 is not representable in f16 (spacing 2 there): with a running f16 value the ones would be lost
    # for ever, with an f32 running value the fourth output is round(2051) = 2052
    x = np.array([[2048.0, 1.0, 1.0, 1.0, 1.0]], dtype=np.float16).view(np.uint16)
    got = O.cumulative("sum", O.F16, x).view(np.float16).astype(np.float32)
    assert got.tolist() == [[2048.0, 2048.0, 2050.0, 2052.0, 2052.0]]


def test_nan_modes_of_cummax():
    x = np.array([[1.0, np.nan, 3.0, 2.0]], dtype=np.float32)
    poisoned = O.cumulative("max", O.F32, x, propagate_nan=True)
    assert poisoned[0, 0] == 1.0 and np.isnan(poisoned[0, 1:]).all()
    ignored = O.cumulative("max", O.F32, x, propagate_nan=False)
    assert ignored.tolist() == [[1.0, 1.0, 3.0, 3.0]]


def test_last_element_of_a_cumulative_sum_is_the_reduction():
    rng = np.random.default_rng(0)
    x = rng.integers(-1000, 1000, size=(17, 301)).astype(np.int32)
    assert np.array_equal(O.cumulative("sum", O.I32, x)[:, -1], O.reduce_last_axis("sum", O.I32, x))
    assert np.array_equal(O.cumulative("max", O.I32, x, axis=0)[-1], O.reduce_first_axis("max", O.I32, x))
    f = rng.standard_normal((9, 257)).astype(np.float32)
    assert np.array_equal(O.cumulative("sum", O.F32, f)[:, -1], O.reduce_last_axis("sum", O.F32, f))    # the same order of additions
    assert np.array_equal(O.cumulative("sum", O.F32, f, reverse=True)[:, ::-1], O.cumulative("sum", O.F32, np.ascontiguousarray(f[:, ::-1])))
