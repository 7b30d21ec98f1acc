"""CPU: the restated seeded-input generator and dump format of the reference's runner
(bishengir/lib/ExecutionEngine/BiShengIRRunnerUtils.cpp:63-125)."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "ascendnpu-ir_b200"))
from bsir import runner_data as R  # noqa: E402


def test_mersenne_twister_is_the_standard_one():
    g = np.random.MT19937()
    g._legacy_seeding(5489)                                    # the default seed of std::mt19937
    assert int(g.random_raw(10000)[-1]) == 4123659995           # the value the C++ standard requires of the 10000th draw
    g._legacy_seeding(1)
    assert [int(v) for v in g.random_raw(2)] == [1791095845, 4282876139]


def test_real_distributions():
    d = R.RunnerData()
    x = d.get_data("f32", [4, 5])
    assert x.dtype == np.float32 and x.shape == (4, 5) and np.all((x >= -1000) & (x < 1000))
    # first draw 1791095845: float(.) / 2^32 * 2000 - 1000, every step in f32
    u = np.float32(np.float32(1791095845) / np.float32(4294967296.0))
    assert x[0, 0] == np.float32(u * np.float32(2000.0) + np.float32(-1000.0))
    y = d.get_data("f32", [3])                                 # the f32 generator goes on where it stopped
    again = R.RunnerData().get_data("f32", [23])
    assert np.array_equal(np.concatenate([x.reshape(-1), y]), again)
    h = R.RunnerData().get_data("bf16", [1000])                # its own generator, values in [-100, 100)
    hf = (h.astype(np.uint32) << 16).view(np.float32)
    assert h.dtype == np.uint16 and np.all(np.abs(hf) <= 100)
    f = R.RunnerData().get_data("f32", [1000]) / 10            # same draws as f32, another range
    assert np.allclose(hf, f, rtol=2 ** -8)


def test_integer_distribution_is_lemire_on_32_bit_draws():
    d = R.RunnerData()
    x = d.get_data("i32", [1000])
    assert x.min() >= -10000 and x.max() <= 10000
    assert int(x[0]) == ((1791095845 * 20001) >> 32) - 10000
    b = R.RunnerData().get_data("i1", [64])
    assert b.dtype == np.bool_ and b.any() and not b.all()
    # rejections are consumed draws: a tiny range with a large rejection zone still yields n values in range
    assert R.RunnerData().get_data("i8", [5000]).min() >= -100


def test_dump_format_round_trip():
    a = np.array([[1.5, -2.25e-3, 1000.0]], dtype=np.float32)
    text = R.print_data("f32", a)
    assert text == "2\n1 3\n1.500000000e+00 -2.249999903e-03 1.000000000e+03\n"
    i = np.arange(6, dtype=np.int32).reshape(2, 3) - 2
    both = text + R.print_data("i32", i)
    back = R.read_data(both)
    assert back[0][0] == [1, 3] and back[1] == ([2, 3], ["-2", "-1", "0", "1", "2", "3"])
    assert R.print_data("bf16", np.array([0x3FC0], dtype=np.uint16)) == "1\n1\n1.500000000e+00\n"
