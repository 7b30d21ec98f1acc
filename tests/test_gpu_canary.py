"""GPU memory safety without a sanitiser: every output lives inside a larger buffer pre-filled with a guard pattern --
bytes before it, after it, and (for 2-D outputs) in the padding between rows -- and the guards must be untouched after
the kernel ran; plus run-twice bit-compares of the kernels that fold partial results across CTAs.  Ragged shapes are
chosen to hit the edge tiles of every kernel family: TMA stores of the GEMMs at m / n that are not tile multiples, odd
lengths of the streaming kernels, sub-warp and two-pass row kernels."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GUARD = 0xA5
PAD = 512          # guard bytes in front and behind


@pytest.fixture(scope="module")
def bsir():
    import bsir as B
    B.lib()
    return B


class Guarded:
    """A [rows, cols] (or 1-D) tensor of `dtype` whose rows sit `pitch` elements apart inside a guarded byte buffer."""

    def __init__(self, shape, dtype, pitch_extra=0):
        self.shape = tuple(shape)
        es = torch.empty(0, dtype=dtype).element_size()
        rows = 1 if len(shape) == 1 else shape[0]
        cols = shape[-1]
        self.pitch = cols + pitch_extra
        nbytes = rows * self.pitch * es
        # start 256-byte aligned inside the raw buffer (torch allocations are), so alignment-dependent fast paths run
        self.raw = torch.full((PAD + nbytes + PAD,), GUARD, dtype=torch.uint8, device="cuda")
        body = self.raw[PAD:PAD + nbytes].view(dtype)
        self.full = body.view(rows, self.pitch)
        self.view = self.full[:, :cols] if len(shape) == 2 else self.full[0, :cols]
        self.rows, self.cols, self.es = rows, cols, es

    def check(self, what):
        torch.cuda.synchronize()
        raw = self.raw.cpu().numpy()
        assert (raw[:PAD] == GUARD).all(), f"{what}: bytes in front of the output were written"
        assert (raw[-PAD:] == GUARD).all(), f"{what}: bytes behind the output were written"
        if self.pitch > self.cols:
            body = raw[PAD:-PAD].reshape(self.rows, self.pitch * self.es)
            assert (body[:, self.cols * self.es:] == GUARD).all(), f"{what}: the padding between rows was written"


# ------------------------------------------------------------------------------------------------ GEMMs
@pytest.mark.parametrize("path", [None, "1", "2", "3"])
@pytest.mark.parametrize("m,n,k", [(300, 1000, 208), (130, 136, 144), (7, 1000, 640), (257, 264, 128)])
def test_w8a8_edge_tiles_stay_inside_the_output(bsir, m, n, k, path, monkeypatch):
    if path:
        monkeypatch.setenv("BSIR_W8A8_PATH", path)
    a = torch.randint(-127, 128, (m, k), device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (k, n), device="cuda", dtype=torch.int8)
    sa, sw = torch.rand(m, device="cuda"), torch.rand(n, device="cuda")
    for extra in (0, 8, 24):                     # ldo = n, and pitches with padding (multiples of 8 keep the TMA store path)
        out = Guarded((m, n), torch.bfloat16, extra)
        acc = Guarded((m, n), torch.int32, 0)
        bsir.lib()      # noqa
        import ctypes as C
        L = bsir.lib()
        rc = L.bsir_matmul_w8a8(C.c_int64(m), C.c_int64(n), C.c_int64(k), C.c_void_p(a.data_ptr()), C.c_int64(k), C.c_void_p(w.data_ptr()),
                                C.c_int64(n), 0, C.c_void_p(sa.data_ptr()), C.c_void_p(sw.data_ptr()), 2, C.c_void_p(out.view.data_ptr()),
                                C.c_int64(out.pitch), C.c_void_p(acc.view.data_ptr()), None, C.c_int64(0),
                                C.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        out.check(f"w8a8 ({m},{n},{k}) path={path} pitch+{extra}")
        acc.check(f"w8a8 accumulators ({m},{n},{k}) path={path}")


@pytest.mark.parametrize("dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float32), (torch.int8, torch.int8), (torch.bfloat16, torch.int8)])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(300, 1000, 208), (130, 136, 144), (1, 40, 64)])
def test_matmul_edge_tiles_stay_inside_the_output(bsir, dtype, out_dtype, ta, tb, m, n, k):
    if dtype == torch.int8:
        a = torch.randint(-127, 128, (k, m) if ta else (m, k), device="cuda", dtype=torch.int8)
        b = torch.randint(-127, 128, (n, k) if tb else (k, n), device="cuda", dtype=torch.int8)
        desc = torch.full((n,), 1e-4, device="cuda")
    else:
        a = torch.randn((k, m) if ta else (m, k), device="cuda").to(dtype)
        b = torch.randn((n, k) if tb else (k, n), device="cuda").to(dtype)
        desc = torch.ones(n, device="cuda")
    for extra in (0, 16):
        out = Guarded((m, n), out_dtype, extra)
        bsir.matmul(a, b, transpose_a=ta, transpose_b=tb, descale=desc, descale_mode="DescalePerChannel", out=out.view)
        out.check(f"matmul {dtype}->{out_dtype} ({m},{n},{k}) ta={ta} tb={tb} pitch+{extra}")


@pytest.mark.parametrize("m", [1, 5, 16, 33])
@pytest.mark.parametrize("n,k", [(136, 384), (1000, 512), (64, 256)])
def test_w4a16_stays_inside_the_output(bsir, m, n, k):
    from bsir import workloads as W
    a, qw, s, z = W.w4a16_input(m, n, k, seed=m)
    for extra in (0, 8):
        out = Guarded((m, n), torch.bfloat16, extra)
        bsir.matmul_w4a16(a, qw, s, z, out=out.view)
        out.check(f"w4a16 ({m},{n},{k}) pitch+{extra}")


# ------------------------------------------------------------------------------------------------ streaming kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int8])
@pytest.mark.parametrize("n", [1, 7, 1000, 4097, 1000003])
def test_stream_kernels_odd_lengths(bsir, dtype, n):
    a = (torch.randn(n, device="cuda") * 10).to(dtype)
    b = (torch.randn(n, device="cuda") * 10).to(dtype)
    out = Guarded((n,), dtype)
    bsir.vadd(a, b, out=out.view)
    out.check(f"vadd {dtype} n={n}")
    if dtype != torch.int8:
        out2 = Guarded((n,), dtype)
        bsir.elemwise_unary("exp", a, out=out2.view)
        out2.check(f"exp {dtype} n={n}")
        q = Guarded((n,), torch.int8)
        bsir.cast(a, torch.int8, round_mode="rint", enable_saturate=True, out=q.view)
        q.check(f"cast {dtype}->i8 n={n}")
        f = Guarded((n,), dtype)
        bsir.elemwise_ternary("fma", a, b, a, out=f.view)
        f.check(f"fma {dtype} n={n}")


# ------------------------------------------------------------------------------------------------ row kernels
@pytest.mark.parametrize("rows,cols", [(1, 8), (37, 24), (300, 64), (5, 1000), (33, 4096), (3, 70000), (2, 152064), (9, 4104)])
def test_row_kernels_stay_inside_their_outputs(bsir, rows, cols):
    x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    w = torch.randn(cols, device="cuda").to(torch.bfloat16)
    for extra in (0, 8, 3):
        y = Guarded((rows, cols), torch.bfloat16, extra)
        bsir.rms_norm(x, w, 1e-6, out=y.view)
        y.check(f"rms_norm ({rows},{cols}) pitch+{extra}")
        s = Guarded((rows, cols), torch.bfloat16, extra)
        bsir.softmax(x, out=s.view)
        s.check(f"softmax ({rows},{cols}) pitch+{extra}")
        q = Guarded((rows, cols), torch.int8, extra)
        sc = Guarded((rows,), torch.float32)
        bsir.quant_per_token_i8(x, q=q.view, scale=sc.view)
        q.check(f"quant q ({rows},{cols}) pitch+{extra}")
        sc.check(f"quant scales ({rows},{cols})")
    v, i = Guarded((rows,), torch.bfloat16), Guarded((rows,), torch.int32)
    bsir.reduce_with_index("max", x, out_val=v.view, out_idx=i.view)
    v.check(f"argmax values ({rows},{cols})")
    i.check(f"argmax indices ({rows},{cols})")
    r = Guarded((rows,), torch.bfloat16)
    bsir.reduce("sum", x, out=r.view)
    r.check(f"reduce sum ({rows},{cols})")
    c = Guarded((cols,), torch.bfloat16)
    bsir.reduce("max", x, dim=0, out=c.view)
    c.check(f"reduce first axis ({rows},{cols})")


@pytest.mark.parametrize("rows,cols", [(3, 2), (64, 100), (7, 1000), (2, 2049), (3, 4096), (5, 8193), (2, 40000)])
def test_sort_cumulative_transpose_stay_inside(bsir, rows, cols):
    x = torch.randn(rows, cols, device="cuda")
    sv, si = Guarded((rows, cols), torch.float32), Guarded((rows, cols), torch.int32)
    bsir.sort(x, out_val=sv.view, out_idx=si.view)
    sv.check(f"sort values ({rows},{cols})")
    si.check(f"sort indices ({rows},{cols})")
    for dim in (0, 1):
        c = Guarded((rows, cols), torch.float32, 5)
        bsir.cumulative("sum", x, dim=dim, out=c.view)
        c.check(f"cumsum dim {dim} ({rows},{cols})")
    t = Guarded((cols, rows), torch.float32, 0)
    bsir.transpose(x, out=t.view)
    t.check(f"transpose ({rows},{cols})")


# ------------------------------------------------------------------------------------------------ determinism
def test_cross_cta_folds_give_the_same_bits_every_time(bsir):
    from bsir import workloads as W
    x = W.argmax_input(64, 152064, seed=1)
    x[3, [100, 90000]] = 9.0
    ref = None
    for _ in range(5):
        v, i = bsir.reduce_with_index("max", x)
        s = bsir.reduce("sum", x.float()[:8].contiguous())                 # few long rows: split sum, partials combined in order
        sm = bsir.softmax(x[:4])                                          # two-pass long rows
        so = bsir.sort(x[:2].float())
        torch.cuda.synchronize()
        cur = [v.view(torch.int16).clone(), i.clone(), s.view(torch.int32).clone(), sm.view(torch.int16).clone(), so[0].view(torch.int32).clone(), so[1].clone()]
        if ref is None:
            ref = cur
        else:
            for a, b in zip(ref, cur):
                assert torch.equal(a, b)
    a8 = torch.randint(-127, 128, (16, 4096), device="cuda", dtype=torch.int8)
    w8 = torch.randint(-127, 128, (4096, 1024), device="cuda", dtype=torch.int8)
    o1 = bsir.matmul_w8a8(a8, w8)
    o2 = bsir.matmul_w8a8(a8, w8)
    assert torch.equal(o1.view(torch.int16), o2.view(torch.int16))
