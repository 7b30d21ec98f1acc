"""GPU parity: hivm.hir.vcumsum / vcumprod / vcummax / vcummin through the C ABI against the oracle, bit for bit
(the scan is sequential along its axis on both sides, so float sums agree exactly too)."""
import numpy as np
import pytest
import torch

import oracle as O
from conftest import assert_bits_equal, oracle_dtype, to_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bsir():
    import bsir as B
    B.lib()
    return B


def _data(shape, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.randn(shape, device="cuda", generator=g) * 0.5 + 0.05).to(dtype)
    hi = {torch.int8: 5, torch.int16: 300, torch.int32: 2 ** 20, torch.int64: 2 ** 40}[dtype]
    return torch.randint(-hi, hi, shape, device="cuda", generator=g, dtype=torch.int64).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.int8, torch.int16, torch.int32, torch.int64])
@pytest.mark.parametrize("kind", ["sum", "prod", "max", "min"])
@pytest.mark.parametrize("rows,cols", [(64, 16), (70, 256), (33, 1000), (5, 17), (1, 640), (300, 1)])
def test_cumulative_ops_both_axes(bsir, dtype, kind, rows, cols):
    x = _data((rows, cols), dtype, rows * 7 + cols)
    if kind == "prod" and dtype.is_floating_point:
        x = (1 + 0.01 * x.float()).to(dtype)                     # keeps the products finite
    dt = oracle_dtype(x)
    for axis in (0, 1):
        for reverse in (False, True):
            y = bsir.cumulative(kind, x, dim=axis, reverse=reverse)
            assert_bits_equal(y, O.cumulative(kind, dt, to_bits(x), axis=axis, reverse=reverse),
                              f"cum{kind} {dtype} [{rows},{cols}] axis {axis} reverse {reverse}")


def test_cumulative_nan_modes_and_strided_rows(bsir):
    x = torch.randn(40, 128, device="cuda")
    x[3, 5] = float("nan")
    for nanp in (True, False):
        y = bsir.cumulative("max", x, propagate_nan=nanp)
        w = O.cumulative("max", O.F32, to_bits(x), propagate_nan=nanp)
        assert np.array_equal(to_bits(y), w, equal_nan=True)
        assert bool(torch.isnan(y[3, 5:]).all()) == nanp
    big = torch.randn(50, 400, device="cuda").to(torch.bfloat16)
    view = big[:, 8:264]                                         # 256 columns, row stride 400: the tiled path
    out_big = torch.zeros(50, 300, device="cuda", dtype=torch.bfloat16)
    bsir.cumulative("sum", view, out=out_big[:, :256])
    assert_bits_equal(out_big[:, :256].contiguous(), O.cumulative("sum", O.BF16, to_bits(view.contiguous())), "strided cumsum")
    assert out_big[:, 256:].abs().sum().item() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int8])
@pytest.mark.parametrize("reverse", [False, True])
def test_row_scan_with_many_rows_and_without_tensor_maps(bsir, monkeypatch, dtype, reverse):
    """So many rows that ten warps share an SM (the ring of tiles per warp is then short and one tile wide), and the
    same problem through the kernel that copies its tiles without a tensor map."""
    rows, cols = 48000, 384
    x = _data((rows, cols), dtype, 11)
    want = O.cumulative("sum", oracle_dtype(x), to_bits(x), axis=1, reverse=reverse)
    assert_bits_equal(bsir.cumulative("sum", x, dim=1, reverse=reverse), want, f"cumsum {dtype} many rows")
    monkeypatch.setenv("BSIR_CUM_NO_TMA", "1")
    assert_bits_equal(bsir.cumulative("sum", x, dim=1, reverse=reverse), want, f"cumsum {dtype} many rows, no tensor map")
    monkeypatch.delenv("BSIR_CUM_NO_TMA")
    monkeypatch.setenv("BSIR_CUM_WIDE", "1")
    y = bsir.cumulative("sum", x[:200].contiguous(), dim=1, reverse=reverse)
    assert_bits_equal(y, want[:200], f"cumsum {dtype} one tile a step")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int8, torch.int16, torch.int32])
@pytest.mark.parametrize("kind", ["sum", "max"])
def test_first_axis_scan_of_tall_problems(bsir, dtype, kind):
    """Down the rows through tiles of 128 rows: a last tile of 44 rows, a last column group of 32 bytes (a strided
    view), both directions; and a problem tall enough for the ring to wrap many times."""
    big = _data((300, 1024), dtype, 21)
    eb = big.element_size()
    view = big[:, :1024 - 96 // eb]                              # row pitch stays 1024 elements
    out = torch.zeros_like(big)
    for reverse in (False, True):
        bsir.cumulative(kind, view, dim=0, reverse=reverse, out=out[:, :view.shape[1]])
        assert_bits_equal(out[:, :view.shape[1]].contiguous(),
                          O.cumulative(kind, oracle_dtype(big), to_bits(view.contiguous()), axis=0, reverse=reverse),
                          f"cum{kind} {dtype} first axis, reverse {reverse}")
        assert out[:, view.shape[1]:].abs().sum().item() == 0
    tall = _data((5000, 96), dtype, 22)
    assert_bits_equal(bsir.cumulative(kind, tall, dim=0), O.cumulative(kind, oracle_dtype(tall), to_bits(tall), axis=0), "tall")
    wide = _data((300, 65536 // eb), dtype, 23)                  # 512 column groups: four warps an SM, tiles of 64 rows
    for reverse in (False, True):
        assert_bits_equal(bsir.cumulative(kind, wide, dim=0, reverse=reverse),
                          O.cumulative(kind, oracle_dtype(wide), to_bits(wide), axis=0, reverse=reverse), f"wide, reverse {reverse}")


def test_cumulative_config_shape_and_validation(bsir):
    """A decode-time top-p shape: many rows, sorted probabilities along the row."""
    p = torch.softmax(torch.randn(2048, 4096, device="cuda"), dim=1).sort(dim=1, descending=True).values.contiguous()
    c = bsir.cumulative("sum", p)
    assert_bits_equal(c[:64].contiguous(), O.cumulative("sum", O.F32, to_bits(p[:64].contiguous())), "top-p cumsum")
    assert (c[:, -1] - 1).abs().max().item() < 1e-4
    with pytest.raises(bsir.BsirError):
        bsir.cumulative("sum", torch.zeros(4, 4, device="cuda", dtype=torch.bool))


@pytest.mark.parametrize("dtype,cols", [(torch.bfloat16, 16384), (torch.float32, 8192), (torch.int8, 32768), (torch.int16, 16384)])
@pytest.mark.parametrize("kind", ["sum", "max"])
def test_first_axis_scan_of_wide_problems(bsir, dtype, cols, kind):
    """Wide, short problems scanned down the rows (37 rows: the thread-per-column kernel)."""
    x = _data((37, cols), dtype, cols)
    for reverse in (False, True):
        y = bsir.cumulative(kind, x, dim=0, reverse=reverse)
        assert_bits_equal(y, O.cumulative(kind, oracle_dtype(x), to_bits(x), axis=0, reverse=reverse), f"cum{kind} axis 0 {dtype} reverse {reverse}")
