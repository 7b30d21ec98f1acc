"""GPU parity: hivm.hir.vsort through the C ABI against the oracle (values bit for bit, indices exactly: the sort is
stable on both sides)."""
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
    """NaN after the numbers ascending and before them descending; zeros of either sign tie in source order."""
    x = torch.tensor([[3.0, float("nan"), -0.0, 0.0, float("-inf"), float("inf"), -0.0, 1.0]], device="cuda")
    val, idx = bsir.sort(x)
    assert idx.tolist() == [[4, 2, 3, 6, 7, 0, 5, 1]]
    assert torch.isnan(val[0, -1]) and val[0, 0] == float("-inf")
    assert torch.signbit(val[0, 1:4]).tolist() == [True, False, True]         # the zeros keep their own bits
    val, idx = bsir.sort(x, descending=True)
    assert idx.tolist() == [[1, 5, 0, 7, 2, 3, 6, 4]]
    wv, wi = O.sort_last_axis(O.F32, to_bits(x), descending=True)
    assert np.array_equal(idx.cpu().numpy(), wi)


def test_sort_limits_and_strides(bsir):
    big = torch.randn(10, 300, device="cuda")
    view = big[:, 10:210]                                      # row stride 300
    val, idx = bsir.sort(view)
    assert torch.equal(val, torch.sort(view, dim=1, stable=True).values)
    assert torch.equal(idx.long(), torch.sort(view, dim=1, stable=True).indices)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
@pytest.mark.parametrize("rows,cols", [(2, 8193), (3, 20000), (5, 65536), (2, 152064)])
@pytest.mark.parametrize("descending", [False, True])
def test_sort_rows_longer_than_shared_memory(bsir, dtype, rows, cols, descending):
    """Keys in device scratch, the wide steps of the network on global memory: the same rule, the same bits."""
    g = torch.Generator(device="cuda").manual_seed(cols)
    if dtype.is_floating_point:
        x = (torch.randn(rows, cols, device="cuda", generator=g) * 8).round().div(4).to(dtype)
    else:
        x = torch.randint(-3000, 3000, (rows, cols), device="cuda", generator=g).to(dtype)
    val, idx = bsir.sort(x, descending=descending)
    wv, wi = O.sort_last_axis(oracle_dtype(x), to_bits(x), descending=descending)
    assert np.array_equal(idx.cpu().numpy(), wi)
    assert np.array_equal(to_bits(val), wv)
