"""Shared test plumbing: import paths, the `gpu` marker, bit-pattern helpers."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for sub in ("ascendnpu-ir_b200", "oracle"):
    p = os.path.join(ROOT, sub)
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on the GPU box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


# ---- helpers shared by the GPU parity tests -------------------------------------------------
def to_bits(t):
    """torch tensor (any dtype, any device) -> numpy array the oracle understands."""
    import torch
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.bool:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def oracle_dtype(t):
    import oracle as O
    import torch
    return {torch.float32: O.F32, torch.float16: O.F16, torch.bfloat16: O.BF16, torch.int8: O.I8,
            torch.int16: O.I16, torch.int32: O.I32, torch.int64: O.I64, torch.uint8: O.U8,
            torch.bool: O.BOOL}[t.dtype]


def floats_from_bits(bits, torch_dtype):
    """numpy bit array from the oracle -> float32 numpy values."""
    import oracle as O
    import torch
    if torch_dtype == torch.bfloat16:
        return O.bf16_to_f32(bits)
    if torch_dtype == torch.float16:
        return O.f16_to_f32(bits)
    return np.asarray(bits, np.float32)


def assert_bits_equal(got_t, want_bits, what=""):
    """Bit-exact comparison (NaNs compare equal to NaNs of any payload for float types)."""
    import torch
    got = to_bits(got_t)
    want = np.asarray(want_bits).reshape(got.shape)
    if got_t.dtype in (torch.bfloat16, torch.float16, torch.float32):
        gf = floats_from_bits(got, got_t.dtype)
        wf = floats_from_bits(want, got_t.dtype)
        both_nan = np.isnan(gf) & np.isnan(wf)
        eq = (got.view(np.uint16 if got.dtype.itemsize == 2 else np.uint32) ==
              want.view(np.uint16 if want.dtype.itemsize == 2 else np.uint32)) | both_nan
    else:
        eq = got == want
    if not eq.all():
        bad = np.argwhere(~eq)
        i = tuple(bad[0])
        raise AssertionError(f"{what}: {len(bad)} of {eq.size} elements differ; first at {i}: got {got[i]} want {want[i]}")


def assert_close(got_t, want_bits, rtol, atol, what=""):
    gf = floats_from_bits(to_bits(got_t), got_t.dtype).astype(np.float64)
    wf = floats_from_bits(np.asarray(want_bits).reshape(gf.shape), got_t.dtype).astype(np.float64)
    nan_ok = np.isnan(gf) == np.isnan(wf)
    assert nan_ok.all(), f"{what}: NaN pattern differs"
    m = ~np.isnan(wf)
    inf = np.isinf(wf) & m
    assert (gf[inf] == wf[inf]).all(), f"{what}: infinities differ"
    m &= ~np.isinf(wf)
    err = np.abs(gf[m] - wf[m])
    tol = atol + rtol * np.abs(wf[m])
    if not (err <= tol).all():
        k = np.argmax(err - tol)
        raise AssertionError(f"{what}: max violation got {gf[m][k]} want {wf[m][k]} (err {err[k]:.3e} > tol {tol[k]:.3e}); "
                             f"{int((err > tol).sum())} of {err.size} outside")
