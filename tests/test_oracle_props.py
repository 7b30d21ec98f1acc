"""CPU: internal consistency of the oracle where the reference pins nothing, checked against
independent computations (numpy / torch in float64), plus the arithmetic identities the CUDA
kernels rely on."""
import numpy as np
import pytest
import torch

import oracle as O


def _bf16(x):
    return O.f32_to_bf16(np.asarray(x, np.float32))


def test_bf16_rounding_matches_torch():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(100000).astype(np.float32) * np.exp(rng.uniform(-30, 30, 100000)).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(_bf16(x), want)


def test_softmax_against_float64():
    rng = np.random.default_rng(1)
    x = (3 * rng.standard_normal((7, 1000))).astype(np.float32)
    xb = _bf16(x)
    xf = O.bf16_to_f32(xb).astype(np.float64)
    want = np.exp(xf - xf.max(1, keepdims=True))
    want /= want.sum(1, keepdims=True)
    got = O.bf16_to_f32(O.softmax(O.BF16, xb))
    assert np.allclose(got, want, rtol=2 ** -8, atol=1e-30)
    got32 = O.softmax(O.F32, O.bf16_to_f32(xb))
    assert np.allclose(got32, want, rtol=1e-5)


def test_rms_norm_against_float64():
    rng = np.random.default_rng(2)
    x = rng.standard_normal((5, 4096)).astype(np.float32)
    w = (1 + 0.02 * rng.standard_normal(4096)).astype(np.float32)
    y, rstd = O.rms_norm(O.F32, x, w, 1e-6, want_rstd=True)
    r = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(1) + 1e-6)
    assert np.allclose(rstd, r, rtol=1e-5)
    assert np.allclose(y, x * r[:, None] * w, rtol=1e-5, atol=1e-7)


def test_quant_properties():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((64, 512)).astype(np.float32)
    x[rng.random(x.shape) < 1e-2] *= 20
    xb = _bf16(x)
    xf = O.bf16_to_f32(xb)
    q, s = O.quant_per_token_i8(O.BF16, xb)
    assert np.array_equal(s, (np.abs(xf).max(1) / np.float32(127)).astype(np.float32))
    assert np.abs(q.astype(np.float32) * s[:, None] - xf).max() <= 0.5001 * s.max()
    assert q.max() == 127 or q.min() == -127          # the row maximum maps to +-127
    # all-zero row: scale 0, 0/0 = NaN saturates to 0
    q0, s0 = O.quant_per_token_i8(O.BF16, np.zeros((1, 16), np.uint16))
    assert s0[0] == 0 and not q0.any()


def test_reciprocal_division_identity_over_every_scale():
    """The CUDA quantiser replaces x / s by r = RN(1/s), q0 = x r, q = fma(fma(-q0, s, x), r, q0) when 2^-60 < s < 2^60.
    A row's scale is s = RN(amax / 127) with amax a positive finite bf16 (f16) value: 32,639 (31,743) scales in all.
    For every one of them inside that range and every x of the type with |x| <= amax, the rounded integer must equal that
    of the IEEE quotient.  Last run: bf16 526,844,418 pairs, f16 1,007,713,278 pairs, 0 mismatches."""
    import ctypes as C
    fn = O.lib().orc_check_recip_division_all
    fn.restype = C.c_int64
    O.set_threads(O.max_threads())
    try:
        for is_f16, pairs in ((0, 526844418), (1, 1007713278)):
            n = C.c_int64(0)
            assert fn(is_f16, C.byref(n)) == 0
            assert n.value == pairs
    finally:
        O.set_threads(1)


def test_reciprocal_division_identity_on_other_scales():
    """Scales a row cannot produce (random f32): the identity holds there too for |x / s| <= 127.5."""
    rng = np.random.default_rng(0)
    scales = np.exp(rng.uniform(np.log(2.0 ** -59), np.log(2.0 ** 59), 200)).astype(np.float32)
    assert sum(O.lib().orc_check_recip_division(float(s), 1) for s in scales) == 0
    am = rng.integers(1, 0x7c00, 100).astype(np.uint16).view(np.float16).astype(np.float32)
    assert sum(O.lib().orc_check_recip_division_f16(float(s), 1) for s in (am / np.float32(127)).astype(np.float32)) == 0


def test_w8a8_against_int64():
    rng = np.random.default_rng(4)
    a = rng.integers(-127, 128, (9, 300), dtype=np.int8)
    w = rng.integers(-127, 128, (300, 40), dtype=np.int8)
    sa = rng.uniform(1e-3, 1e-2, 9).astype(np.float32)
    sw = rng.uniform(1e-3, 1e-2, 40).astype(np.float32)
    out, acc = O.matmul_w8a8(a, w, sa, sw, want_acc=True)
    want = a.astype(np.int64) @ w.astype(np.int64)
    assert np.array_equal(acc, want)
    ref = _bf16((want.astype(np.float32) * sa[:, None]) * sw[None, :])
    assert np.array_equal(out, ref)
    out_t = O.matmul_w8a8(a, np.ascontiguousarray(w.T), sa, sw, transpose_b=True)
    assert np.array_equal(out_t, out)


def test_w4a16_against_float64():
    rng = np.random.default_rng(5)
    m, n, k, g = 3, 32, 256, 128
    a = _bf16(rng.standard_normal((m, k)))
    q = rng.integers(0, 16, (k, n))
    z = rng.integers(0, 16, (k // g, n))
    s = _bf16(rng.uniform(1e-3, 1e-2, (k // g, n)))
    qw = np.zeros((k // 8, n), np.uint32)
    for t in range(8):
        qw |= (q[t::8].astype(np.uint32) << (4 * t))
    zw = np.zeros((k // g, n // 8), np.uint32)
    for t in range(8):
        zw |= (z[:, t::8].astype(np.uint32) << (4 * t))
    out = O.bf16_to_f32(O.matmul_w4a16(a, qw.view(np.int32), s, zw.view(np.int32), g))
    wdeq = O.bf16_to_f32(_bf16((q - np.repeat(z, g, 0)).astype(np.float32) * np.repeat(O.bf16_to_f32(s), g, 0)))
    want = O.bf16_to_f32(a).astype(np.float64) @ wdeq.astype(np.float64)
    assert np.allclose(out, want, rtol=2 ** -7, atol=1e-3)


def test_thread_count_does_not_change_results():
    rng = np.random.default_rng(6)
    xb = _bf16(rng.standard_normal((37, 333)))
    O.set_threads(1)
    a = O.softmax(O.BF16, xb), O.quant_per_token_i8(O.BF16, xb)[0], O.rms_norm(O.BF16, xb, xb[0], 1e-6)
    O.set_threads(4)
    b = O.softmax(O.BF16, xb), O.quant_per_token_i8(O.BF16, xb)[0], O.rms_norm(O.BF16, xb, xb[0], 1e-6)
    O.set_threads(1)
    for u, v in zip(a, b):
        assert np.array_equal(u, v)
