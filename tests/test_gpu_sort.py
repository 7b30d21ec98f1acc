"""GPU parity: hivm.hir.vsort through the C ABI against the oracle (values bit for bit, indices exactly: the result of the
reference's compare-and-swap passes is unique, ties and NaN included)."""
import numpy as np
import pytest
import torch

import oracle as O
from conftest import oracle_dtype, to_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bsir():
    import bsir as B
    B.lib()
    return B


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.int8, torch.int16, torch.int32])
@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 2), (64, 100), (17, 1000), (5, 4096), (2, 8192), (300, 33)])
@pytest.mark.parametrize("descending", [False, True])
def test_sort_values_and_indices(bsir, dtype, rows, cols, descending):
    g = torch.Generator(device="cuda").manual_seed(rows * 31 + cols)
    if dtype.is_floating_point:
        x = (torch.randn(rows, cols, device="cuda", generator=g) * 4).round().div(2).to(dtype)     # many ties
    else:
        hi = 100 if dtype == torch.int8 else 500
        x = torch.randint(-hi, hi, (rows, cols), device="cuda", generator=g).to(dtype)
    val, idx = bsir.sort(x, descending=descending)
    wv, wi = O.sort_last_axis(oracle_dtype(x), to_bits(x), descending=descending)
    assert np.array_equal(idx.cpu().numpy(), wi)
    assert np.array_equal(to_bits(val), wv)


def test_sort_special_values(bsir):
    """The reference's compare-and-swap passes swap every pair that holds a NaN, so a NaN that starts at position p ends
    at (p + 1) mod n in either direction; zeros of either sign tie in source order and keep their own bits."""
    x = torch.tensor([[3.0, float("nan"), -0.0, 0.0, float("-inf"), float("inf"), -0.0, 1.0]], device="cuda")
    for desc in (False, True):
        val, idx = bsir.sort(x, descending=desc)
        wv, wi = O.sort_last_axis_loops(O.F32, to_bits(x), descending=desc)
        assert np.array_equal(idx.cpu().numpy(), wi)
        assert np.array_equal(to_bits(val).view(np.uint32), wv.view(np.uint32))
    val, idx = bsir.sort(x)
    assert idx.tolist() == [[4, 2, 1, 3, 6, 7, 0, 5]] and torch.isnan(val[0, 2])
    assert torch.signbit(val[0, [1, 3, 4]]).tolist() == [True, False, True]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(40, 1), (40, 2), (33, 7), (16, 100), (9, 1000), (4, 8192), (3, 8193), (2, 40000)])
@pytest.mark.parametrize("descending", [False, True])
def test_sort_rows_with_nan(bsir, dtype, rows, cols, descending):
    """Rows holding no, one, a few and many NaNs (first and last positions among them), against the literal loops where
    they finish in time and their closed form beyond."""
    g = torch.Generator(device="cuda").manual_seed(rows * 131 + cols)
    x = (torch.randn(rows, cols, device="cuda", generator=g) * 4).round().div(2).to(dtype)
    frac = torch.linspace(0, 0.6, rows, device="cuda")[:, None]
    x[torch.rand(rows, cols, device="cuda", generator=g) < frac] = float("nan")
    x[1::4, 0] = float("nan")
    x[2::4, -1] = float("nan")
    if rows > 3:
        x[3] = float("nan")                                  # a row of nothing else
    val, idx = bsir.sort(x, descending=descending)
    fn = O.sort_last_axis_loops if cols <= 1000 else O.sort_last_axis
    wv, wi = fn(oracle_dtype(x), to_bits(x), descending=descending)
    assert np.array_equal(idx.cpu().numpy(), wi)
    assert np.array_equal(to_bits(val).view(np.uint8), wv.view(np.uint8))         # bits: NaN is not equal to itself


def test_sort_limits_and_strides(bsir):
    big = torch.randn(10, 300, device="cuda")
    view = big[:, 10:210]                                      # row stride 300
    val, idx = bsir.sort(view)
    assert torch.equal(val, torch.sort(view, dim=1, stable=True).values)
    assert torch.equal(idx.long(), torch.sort(view, dim=1, stable=True).indices)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.int8, torch.int16, torch.int32])
@pytest.mark.parametrize("rows,cols", [(2, 8193), (3, 20000), (5, 65536), (2, 152064), (2, 200001)])
@pytest.mark.parametrize("descending", [False, True])
def test_sort_rows_longer_than_shared_memory(bsir, dtype, rows, cols, descending):
    """Keys in device scratch, sorted by stable radix passes: the same rule, the same bits."""
    g = torch.Generator(device="cuda").manual_seed(cols)
    if dtype.is_floating_point:
        x = (torch.randn(rows, cols, device="cuda", generator=g) * 8).round().div(4).to(dtype)
    else:
        hi = 100 if dtype == torch.int8 else 3000
        x = torch.randint(-hi, hi, (rows, cols), device="cuda", generator=g).to(dtype)
    val, idx = bsir.sort(x, descending=descending)
    wv, wi = O.sort_last_axis(oracle_dtype(x), to_bits(x), descending=descending)
    assert np.array_equal(idx.cpu().numpy(), wi)
    assert np.array_equal(to_bits(val), wv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int32])
def test_sort_long_rows_every_digit(bsir, dtype):
    """Values that differ in every byte of the key (the whole range of the type, infinities, both zeros), rows that
    do not fill their last tile, a strided source: every radix pass has work to do."""
    g = torch.Generator(device="cuda").manual_seed(5)
    rows, cols = 3, 70001
    if dtype == torch.int32:
        x = torch.randint(-2**31, 2**31 - 1, (rows, cols + 7), device="cuda", generator=g, dtype=torch.int64).to(torch.int32)
    else:
        bits = torch.randint(0, 2**16, (rows, cols + 7), device="cuda", generator=g)
        if dtype == torch.float16:
            x = bits.to(torch.int16).view(torch.float16)
        else:
            lo = torch.randint(0, 2**16, (rows, cols + 7), device="cuda", generator=g)
            x = ((bits << 16) | lo).to(torch.int32).view(torch.float32)
        x = torch.where(torch.isnan(x), torch.zeros_like(x), x)
        x[:, 5] = float("inf"); x[:, 9] = float("-inf"); x[:, 11] = -0.0; x[:, 12] = 0.0
    view = x[:, :cols]
    for descending in (False, True):
        val, idx = bsir.sort(view, descending=descending)
        wv, wi = O.sort_last_axis(oracle_dtype(x), to_bits(view.contiguous()), descending=descending)
        assert np.array_equal(idx.cpu().numpy(), wi)
        assert np.array_equal(to_bits(val), wv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.int8, torch.int16, torch.int32])
@pytest.mark.parametrize("rows,cols", [(3, 2), (7, 33), (64, 100), (5, 512), (9, 513), (17, 1000), (3, 2048), (4, 2049), (5, 4096), (2, 5000)])
@pytest.mark.parametrize("descending", [False, True])
def test_sort_radix_in_one_cta(bsir, monkeypatch, dtype, rows, cols, descending):
    """Every row length through the radix kernels (the switch moves the point from which they are used down to 2):
    ties, NaNs at random places, both directions, the same bits as the reference's rule."""
    monkeypatch.setenv("BSIR_SORT_RADIX_FROM", "2")
    g = torch.Generator(device="cuda").manual_seed(rows * 77 + cols)
    if dtype.is_floating_point:
        x = (torch.randn(rows, cols, device="cuda", generator=g) * 4).round().div(2).to(dtype)
        x[torch.rand(rows, cols, device="cuda", generator=g) < 0.02] = float("nan")
        x[0, 0] = -0.0
    else:
        hi = 100 if dtype == torch.int8 else 3000
        x = torch.randint(-hi, hi, (rows, cols), device="cuda", generator=g).to(dtype)
    val, idx = bsir.sort(x, descending=descending)
    wv, wi = O.sort_last_axis(oracle_dtype(x), to_bits(x), descending=descending)
    assert np.array_equal(idx.cpu().numpy(), wi)
    assert np.array_equal(to_bits(val).view(np.uint8), wv.view(np.uint8))         # bits: NaN is not equal to itself


def test_sort_refuses_to_write_values_over_the_source(bsir):
    x = torch.randn(4, 100, device="cuda")
    keep = x.clone()
    with pytest.raises(bsir.BsirError):
        bsir.sort(x, out_val=x)
    assert torch.equal(x, keep)
