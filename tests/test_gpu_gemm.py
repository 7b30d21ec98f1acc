"""GPU parity: W8A8 GEMM (int32 accumulators bit-exact, bf16 output within 1e-2 rel) and the
W4A16 group-quantised GEMM (within 2e-2 rel), against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle as O
from conftest import assert_bits_equal, assert_close, to_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bsir():
    import bsir as B
    B.lib()
    O.set_threads(O.max_threads())
    return B


def _w8a8_case(bsir, m, n, k, transpose_b, seed=0, out_dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randint(-127, 128, (m, k), generator=g, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (k, n), generator=g, device="cuda", dtype=torch.int8)
    sa = torch.rand(m, generator=g, device="cuda") * 9e-3 + 1e-3
    sw = torch.rand(n, generator=g, device="cuda") * 9e-3 + 1e-3
    b = w.t().contiguous() if transpose_b else w
    out, acc = bsir.matmul_w8a8(a, b, sa, sw, transpose_b=transpose_b, want_acc=True, out_dtype=out_dtype)
    wout, wacc = O.matmul_w8a8(to_bits(a), to_bits(b), to_bits(sa), to_bits(sw), transpose_b=transpose_b,
                               out_dt=O.BF16 if out_dtype == torch.bfloat16 else O.F16, want_acc=True)
    assert np.array_equal(acc.cpu().numpy(), wacc), f"int32 accumulators differ ({m},{n},{k}) tb={transpose_b}"
    assert_bits_equal(out, wout, f"w8a8 out ({m},{n},{k}) tb={transpose_b}")   # same f32 op order: bit-exact
    assert bsir.device_error() == 0


@pytest.mark.parametrize("transpose_b", [True, False])
@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 128, 512), (16, 256, 4096), (1, 128, 128), (200, 384, 640),
                                   (130, 320, 208), (256, 512, 1024), (128, 1000, 256), (300, 136, 144), (40, 1000, 640),
                                   (48, 14336, 512), (49, 384, 256)])
def test_w8a8_small_shapes_exact(bsir, m, n, k, transpose_b):
    _w8a8_case(bsir, m, n, k, transpose_b, seed=m + n + k)


@pytest.mark.parametrize("transpose_b", [True, False])
@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (512, 512, 1024), (300, 320, 208), (128, 1000, 256), (1024, 768, 4096)])
def test_w8a8_cta_pair_kernel_exact(bsir, m, n, k, transpose_b, monkeypatch):
    monkeypatch.setenv("BSIR_W8A8_PATH", "2")      # force the cta_group::2 kernel on small shapes
    _w8a8_case(bsir, m, n, k, transpose_b, seed=m + n + k + 7)
    monkeypatch.setenv("BSIR_W8A8_PATH", "1")      # and the single-CTA kernel gives the same bits
    _w8a8_case(bsir, m, n, k, transpose_b, seed=m + n + k + 7)


@pytest.mark.parametrize("transpose_b", [True, False])
@pytest.mark.parametrize("m,n,k", [(1, 128, 128), (16, 256, 4096), (7, 1000, 640), (33, 384, 208), (64, 14336, 512),
                                   (100, 320, 1024), (128, 256, 256)])
def test_w8a8_decode_kernel_exact(bsir, m, n, k, transpose_b, monkeypatch):
    monkeypatch.setenv("BSIR_W8A8_PATH", "3")      # operands swapped: weights on the TMEM lanes, rows of a as MMA N
    _w8a8_case(bsir, m, n, k, transpose_b, seed=m + n + k + 11)
    _w8a8_case(bsir, m, n, k, transpose_b, seed=m + n + k + 12, out_dtype=torch.float16)
    monkeypatch.setenv("BSIR_W8A8_PATH", "1")      # the 128-row-tile kernel gives the same bits
    _w8a8_case(bsir, m, n, k, transpose_b, seed=m + n + k + 11)


@pytest.mark.parametrize("m,n,k", [(16, 14336, 4096), (8, 14336 + 72, 4096 + 128), (24, 7168, 4096), (3, 640, 128 * 37), (16, 128 * 147, 256)])
def test_w8a8_decode_k_split_over_ctas(bsir, m, n, k, monkeypatch):
    """Fewer tiles than SMs: a tile's k blocks are shared out over two or more CTAs and the partial tiles meet in
    scratch.  Same bits as whole tiles per CTA, launch after launch on the same scratch, and under a replayed graph."""
    _w8a8_case(bsir, m, n, k, False, seed=5)
    g = torch.Generator(device="cuda").manual_seed(9)
    a = torch.randint(-127, 128, (m, k), generator=g, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (k, n), generator=g, device="cuda", dtype=torch.int8)
    sa = torch.rand(m, generator=g, device="cuda") * 9e-3 + 1e-3
    sw = torch.rand(n, generator=g, device="cuda") * 9e-3 + 1e-3
    outs = [bsir.matmul_w8a8(a, w, sa, sw) for _ in range(6)]
    monkeypatch.setenv("BSIR_W8A8_SPLITK", "0")
    whole = bsir.matmul_w8a8(a, w, sa, sw)
    monkeypatch.delenv("BSIR_W8A8_SPLITK")
    for o in outs:
        assert torch.equal(o.view(torch.int16), whole.view(torch.int16))
    out = torch.empty_like(whole)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        bsir.matmul_w8a8(a, w, sa, sw, out=out)
    for _ in range(3):                                   # the same launch tag every replay: the arrival words were left at zero
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), whole.view(torch.int16))
    assert bsir.device_error() == 0


def test_w8a8_f16_output_and_unaligned_fallback(bsir):
    _w8a8_case(bsir, 64, 256, 256, False, seed=3, out_dtype=torch.float16)
    # k = 100: the row pitch is not a multiple of 16 bytes -> plain path
    _w8a8_case(bsir, 33, 72, 100, False, seed=4)
    _w8a8_case(bsir, 33, 72, 100, True, seed=5)


@pytest.mark.parametrize("m", [16, 128])
def test_w8a8_config_small_m_full_check(bsir, m):
    from bsir import workloads as W
    a, sa, w, sw = W.w8a8_input(m, seed=1)
    out, acc = bsir.matmul_w8a8(a, w, sa, sw, want_acc=True)
    wout, wacc = O.matmul_w8a8(to_bits(a), to_bits(w), to_bits(sa), to_bits(sw), want_acc=True)
    assert np.array_equal(acc.cpu().numpy(), wacc), "int32 accumulators differ"
    assert_close(out, wout, 1e-2, 1e-6, f"w8a8 m={m}")
    assert_bits_equal(out, wout, f"w8a8 m={m} bits")


def test_w8a8_config_m4096(bsir):
    from bsir import workloads as W
    a, sa, w, sw = W.w8a8_input(4096, seed=2)
    out, acc = bsir.matmul_w8a8(a, w, sa, sw, want_acc=True)
    assert bsir.device_error() == 0
    # 48 sampled rows (every tile row block is hit) against the oracle, bit-exact accumulators
    rows = torch.arange(5, 4096, 86, device="cuda")
    wout, wacc = O.matmul_w8a8(to_bits(a[rows]), to_bits(w), to_bits(sa[rows]), to_bits(sw), want_acc=True)
    assert np.array_equal(acc[rows].cpu().numpy(), wacc), "sampled int32 accumulators differ"
    assert_close(out[rows], wout, 1e-2, 1e-6, "w8a8 m=4096 sample")
    # checksum over every output element: row sums of acc == A . (W . 1) in int64
    w1 = w.cpu().numpy().astype(np.int64).sum(axis=1)
    want_rows = a.cpu().numpy().astype(np.int64) @ w1
    got_rows = acc.sum(dim=1, dtype=torch.int64).cpu().numpy()
    assert np.array_equal(got_rows, want_rows), "row checksums differ"
    # and column sums == (1 . A) . W
    a1 = a.cpu().numpy().astype(np.int64).sum(axis=0)
    want_cols = a1 @ w.cpu().numpy().astype(np.int64)
    got_cols = acc.sum(dim=0, dtype=torch.int64).cpu().numpy()
    assert np.array_equal(got_cols, want_cols), "column checksums differ"
    # the output is the accumulator times both scales, rounded once
    ref = (acc.float() * sa[:, None]) * sw[None, :]
    assert torch.equal(out, ref.to(torch.bfloat16))
    # transposed-B entry point gives the same bits
    out_t = bsir.matmul_w8a8(a, w.t().contiguous(), sa, sw, transpose_b=True)
    assert torch.equal(out_t, out)


def test_w8a8_library_symbol(bsir):
    import ctypes as C
    L = bsir.lib()
    L.bsir_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    a = torch.randint(-5, 6, (64, 256), device="cuda", dtype=torch.int8)
    b = torch.randint(-5, 6, (256, 128), device="cuda", dtype=torch.int8)
    c = torch.empty(64, 128, device="cuda", dtype=torch.float16)
    f = L._mlir_ciface_matmul_Xbias_Xdescale_XtransposeA_XtransposeB_TAint8_t_TBint8_t_TChalf
    assert f(C.byref(bsir.memref(a)), C.byref(bsir.memref(b)), C.byref(bsir.memref(c))) == 0
    want = (a.cpu().int() @ b.cpu().int()).to(torch.float16)
    assert torch.equal(c.cpu(), want)


# ---------------------------------------------------------------- W4A16 (2e-2 rel, stated by the config)
def _w4_close(out, want_bits, what):
    """2e-2 relative is the configuration's bar.  The exact-rounding kernels round every dequantised weight to bf16 as
    the oracle does, so only the order of the f32 additions differs; the folded-scale kernel (on request:
    BSIR_W4A16_PATH=f) applies scale and zero point to a group's sum instead and so skips those roundings (a relative
    RMS of about 1.5e-3 against the oracle).  In practice all agree to one bf16 step of the largest output, which is
    asserted as well."""
    wf = O.bf16_to_f32(want_bits)
    # 2e-2 of the value, and for values near zero 1e-2 of the output's RMS (a sum of K terms that cancel to little
    # keeps the absolute error of its terms)
    assert_close(out, want_bits, 2e-2, 1e-2 * float(np.sqrt(np.mean(wf.astype(np.float64) ** 2))) + 1e-6, what)
    assert np.abs(out.float().cpu().numpy() - wf).max() <= 1.0 / 128 * np.abs(wf).max() + 1e-6, what


@pytest.mark.parametrize("m", [1, 2, 3, 8, 16, 5, 33])
@pytest.mark.parametrize("n,k", [(256, 256), (14336, 4096), (1024, 1024), (136, 384)])
def test_w4a16(bsir, m, n, k):
    from bsir import workloads as W
    a, qw, s, z = W.w4a16_input(m, n, k, seed=m + n)
    out = bsir.matmul_w4a16(a, qw, s, z)
    want = O.matmul_w4a16(to_bits(a), to_bits(qw), to_bits(s), to_bits(z))
    _w4_close(out, want, f"w4a16 m={m} n={n} k={k}")


@pytest.mark.parametrize("m", [1, 8, 16])
def test_w4a16_config_shape_error_bounds(bsir, m, monkeypatch):
    """The configuration's shape, all three M: the error against the oracle, stated as numbers -- RMS error below
    3e-3 of the output's RMS (1e-3 for the kernels that round every weight as the oracle does), and 2e-2 relative
    outright wherever |result| >= RMS / 2.  And against what the folded-scale kernel computes by definition -- the
    products of the unrounded weights (q - z) * s, here in float64 -- it is right to the rounding of its bf16 output."""
    from bsir import workloads as W
    a, qw, s, z = W.w4a16_input(m, seed=40 + m)
    want = O.matmul_w4a16(to_bits(a), to_bits(qw), to_bits(s), to_bits(z))
    wf = O.bf16_to_f32(want).astype(np.float64)
    rms = np.sqrt(np.mean(wf ** 2))
    big = np.abs(wf) >= 0.5 * rms
    for path, bound in (("", 1e-3), ("m", 1e-3), ("t", 1e-3), ("f", 3e-3)):
        if path:
            monkeypatch.setenv("BSIR_W4A16_PATH", path)
        out = bsir.matmul_w4a16(a, qw, s, z)
        gf = out.float().cpu().numpy().astype(np.float64)
        assert (np.abs(gf - wf)[big] / np.abs(wf)[big]).max() <= 2e-2, path
        assert np.sqrt(np.mean((gf - wf) ** 2)) <= bound * rms, path
        _w4_close(out, want, f"w4a16 config m={m} path={path}")
    k, n = a.shape[1], s.shape[1]                       # still with BSIR_W4A16_PATH=f
    shifts = torch.arange(8, device="cuda", dtype=torch.int32) * 4
    q = ((qw[:, None, :] >> shifts[None, :, None]) & 15).reshape(k, n).double()
    zz = ((z[:, :, None] >> shifts[None, None, :]) & 15).reshape(z.shape[0], n).double()
    wd = (q - zz.repeat_interleave(128, dim=0)) * s.double().repeat_interleave(128, dim=0)
    ref = (a.double() @ wd).cpu().numpy()
    got = bsir.matmul_w4a16(a, qw, s, z).float().cpu().numpy().astype(np.float64)
    assert np.abs(got - ref).max() <= 2.0 ** -8 * np.abs(ref).max(), "folded-scale kernel against unrounded weights"
    assert np.sqrt(np.mean((got - ref) ** 2)) <= 2e-3 * np.sqrt(np.mean(ref ** 2))        # the bf16 rounding of the output alone (1.65e-3)


@pytest.mark.parametrize("group", [64, 256, 32])
@pytest.mark.parametrize("m,n,k", [(4, 512, 1024), (16, 384, 2048), (9, 136, 768)])
def test_w4a16_other_group_sizes(bsir, m, n, k, group):
    from bsir import workloads as W
    a, qw, s, z = W.w4a16_input(m, n, k, group=group, seed=group + m)
    out = bsir.matmul_w4a16(a, qw, s, z, group=group)
    want = O.matmul_w4a16(to_bits(a), to_bits(qw), to_bits(s), to_bits(z), group)
    _w4_close(out, want, f"w4a16 group={group} m={m} n={n} k={k}")


@pytest.mark.parametrize("path", ["m", "t", "f"])
@pytest.mark.parametrize("m,n,k", [(1, 14336, 4096), (16, 14336, 4096), (7, 1024, 1024), (16, 256, 8192), (3, 136, 384), (9, 128, 2048), (33, 192, 4096)])
def test_w4a16_each_kernel(bsir, m, n, k, path, monkeypatch):
    """The weight-streaming kernels (register dequantisation + mma.sync, tensor-memory + tcgen05, folded scales) on
    the same inputs; shapes a kernel does not take fall through to another one."""
    from bsir import workloads as W
    monkeypatch.setenv("BSIR_W4A16_PATH", path)
    a, qw, s, z = W.w4a16_input(m, n, k, seed=3 * m + n)
    out = bsir.matmul_w4a16(a, qw, s, z)
    want = O.matmul_w4a16(to_bits(a), to_bits(qw), to_bits(s), to_bits(z))
    _w4_close(out, want, f"w4a16 path={path} m={m} n={n} k={k}")


def test_w4a16_twice_gives_the_same_bits(bsir):
    from bsir import workloads as W
    a, qw, s, z = W.w4a16_input(16, seed=77)
    o1 = bsir.matmul_w4a16(a, qw, s, z)
    o2 = bsir.matmul_w4a16(a, qw, s, z)
    assert torch.equal(o1.view(torch.int16), o2.view(torch.int16))
