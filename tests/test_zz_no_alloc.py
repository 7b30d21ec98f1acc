"""GPU: the allocation-free argmax entry point (bsir_reduce_with_index_static).

Some hosts give all device memory to their own pool at start-up, or call from places where the CUDA
allocator must not be entered, so a library call that reaches cudaMalloc is not an option for them.
This entry point keeps its scratch in a fixed array inside the library image.  The test drives it
through the C ABI and checks it against the ordinary entry point and against the CPU oracle (bit-exact:
indices and values) on two calls in a row, because the array is shared between calls and keeps the
previous call's contents.
The file sorts last on purpose, so a run that stops at the first failure has already run every other
test; it also passes on its own in a fresh process."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import oracle as O
from conftest import floats_from_bits, oracle_dtype, to_bits

pytestmark = pytest.mark.gpu


def _call_static(B, x, kind, left, nan_mode):
    rows, cols = x.shape
    val = torch.empty(rows, dtype=x.dtype, device=x.device)
    idx = torch.empty(rows, dtype=torch.int32, device=x.device)
    rc = B.lib().bsir_reduce_with_index_static(
        C.c_int32(B.RWI_KIND[kind]), C.c_int32(B._TORCH2DT[x.dtype]), C.c_int32(int(left)),
        C.c_int32({"region": 0, "nan_first": 1}[nan_mode]), C.c_int64(rows), C.c_int64(cols),
        C.c_void_p(x.data_ptr()), C.c_int64(x.stride(0)), C.c_void_p(val.data_ptr()), C.c_void_p(idx.data_ptr()),
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, val, idx


def _same_bits(a, b):
    if a.dtype in (torch.float16, torch.bfloat16):
        ia, ib = a.view(torch.int16), b.view(torch.int16)
    elif a.dtype == torch.float32:
        ia, ib = a.view(torch.int32), b.view(torch.int32)
    else:
        ia, ib = a, b
    both_nan = torch.isnan(a.float()) & torch.isnan(b.float()) if a.is_floating_point() else torch.zeros_like(ia, dtype=torch.bool)
    return bool(((ia == ib) | both_nan).all())


def _check_against_oracle(x, kind, left, nan_mode, val, idx):
    ov, oi = O.reduce_with_index(kind, oracle_dtype(x), to_bits(x), tie_break_left=left, nan_mode=nan_mode)
    assert np.array_equal(idx.cpu().numpy(), oi), f"indices differ from the oracle for {tuple(x.shape)} {kind}"
    got, want = val.float().cpu().numpy(), floats_from_bits(ov, x.dtype)
    assert np.array_equal(got, want, equal_nan=True), f"values differ from the oracle for {tuple(x.shape)} {kind}"


def test_static_scratch_matches_the_allocating_entry_point_twice_in_a_row():
    import bsir as B
    from bsir import workloads as W
    B.lib()
    # call 1: the benchmark shape (bf16 256 x 152064, several segments per row), with ties, a NaN row
    # and an all -inf row planted
    x1 = W.argmax_input(256, 152064, seed=11)
    x1[3, [17, 90000, 152063]] = 9.0
    x1[4, 70000] = float("nan")
    x1[5] = -float("inf")
    # call 2: a different shape and dtype right behind it, so stale partial results and counters of
    # call 1 are still sitting in the shared array
    x2 = W.argmax_input(37, 65536, seed=12, dtype=torch.float32)
    x2[0, [5, 6]] = 7.5
    for x, kind, left, nm in ((x1, "max", True, "region"), (x2, "min", False, "nan_first"),
                              (x1, "max", False, "nan_first"), (x2, "max", True, "region")):
        rc, val, idx = _call_static(B, x, kind, left, nm)
        assert rc == 0, B.lib().bsir_last_error().decode()
        want_val, want_idx = B.reduce_with_index(kind, x, tie_break_left=left, nan_mode=nm)
        torch.cuda.synchronize()
        assert torch.equal(idx, want_idx), f"indices differ for {tuple(x.shape)} {kind} left={left} {nm}"
        assert _same_bits(val, want_val), f"values differ for {tuple(x.shape)} {kind} left={left} {nm}"
        _check_against_oracle(x, kind, left, nm, val, idx)


def test_static_scratch_small_and_unaligned_shapes():
    import bsir as B
    B.lib()
    g = torch.Generator(device="cuda").manual_seed(5)
    for shape, dtype in (((1, 8), torch.bfloat16), ((9, 1000), torch.float16), ((5, 33), torch.float32)):
        x = torch.randn(shape, generator=g, device="cuda").to(dtype)
        rc, val, idx = _call_static(B, x, "max", True, "region")
        assert rc == 0
        wv, wi = B.reduce_with_index("max", x)
        assert torch.equal(idx, wi) and _same_bits(val, wv)
        _check_against_oracle(x, "max", True, "region", val, idx)


def test_static_scratch_refuses_what_does_not_fit():
    import bsir as B
    B.lib()
    x = torch.zeros(4097, 8, dtype=torch.bfloat16, device="cuda")            # more rows than counters
    rc, _, _ = _call_static(B, x, "max", True, "region")
    assert rc == -10 and b"4096" in B.lib().bsir_last_error()
    # rows x segments too large: with segments capped at 256 vectors, 4000 rows of 2048 vectors make 8 segments each,
    # 32000 partial results against room for 31744
    y = torch.zeros(4000, 8192, dtype=torch.float32, device="cuda")
    os.environ["BSIR_RWI_SEGVECS"] = "256"
    try:
        rc, val, idx = _call_static(B, y, "max", True, "region")
        text = B.lib().bsir_last_error()
    finally:
        del os.environ["BSIR_RWI_SEGVECS"]
    assert rc == -10 and b"partial results" in text
    z = torch.randn(2, 4096, device="cuda")                                 # the library still works afterwards
    rc, val, idx = _call_static(B, z, "max", True, "region")
    assert rc == 0 and torch.equal(idx.long(), z.argmax(dim=1))
