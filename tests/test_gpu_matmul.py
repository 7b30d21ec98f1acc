"""GPU parity of bsir_matmul -- hivm.hir.matmul "C = descale * (A * B + bias)" with transposed operands, the fixpipe
stages (relu, F322F16 / F322BF16 / S322I8) and batch_matmul -- against the CPU oracle, through the C ABI.
int8 products: accumulators, int32 and int8 outputs bit-exact, 16-bit outputs bit-exact (same f32 op order).
f16 / bf16 products: the tensor core adds the f32 products in another order than the oracle's k loop, so outputs are
compared at 1e-2 relative (plus 1e-2 of the output's RMS for results near zero); small-integer data, where every
partial sum is exact in f32, must agree bit for bit."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O
from conftest import assert_bits_equal, floats_from_bits, to_bits

pytestmark = pytest.mark.gpu

_ODT = {torch.int8: O.I8, torch.float16: O.F16, torch.bfloat16: O.BF16, torch.float32: O.F32, torch.int32: O.I32}


@pytest.fixture(scope="module")
def bsir():
    import bsir as B
    B.lib()
    O.set_threads(O.max_threads())
    return B


def _operands(dtype, m, n, k, ta, tb, seed, small_ints=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype == torch.int8:
        a = torch.randint(-127, 128, (m, k), generator=g, device="cuda", dtype=torch.int8)
        b = torch.randint(-127, 128, (k, n), generator=g, device="cuda", dtype=torch.int8)
    elif small_ints:
        a = torch.randint(-4, 5, (m, k), generator=g, device="cuda").to(dtype)
        b = torch.randint(-4, 5, (k, n), generator=g, device="cuda").to(dtype)
    else:
        a = torch.randn(m, k, generator=g, device="cuda").to(dtype)
        b = (torch.randn(k, n, generator=g, device="cuda") * 0.25).to(dtype)
    return (a.t().contiguous() if ta else a), (b.t().contiguous() if tb else b)


def _check(bsir, dtype, m, n, k, ta=False, tb=False, bias=False, descale=None, relu=False, scale_a=False, out_dtype=None,
           seed=0, small_ints=False, param_dtype=None, exact=None):
    a, b = _operands(dtype, m, n, k, ta, tb, seed, small_ints)
    g = torch.Generator(device="cuda").manual_seed(seed + 1)
    int_in = dtype == torch.int8
    out_dtype = out_dtype or (torch.float16 if int_in else dtype)
    pd = param_dtype or (torch.float32 if int_in else dtype)
    bias_t = None
    if bias:
        bias_t = (torch.randint(-20000, 20000, (n,), generator=g, device="cuda", dtype=torch.int32) if int_in
                  else (torch.randn(n, generator=g, device="cuda") * 2).to(pd))
    mag = 3e-5 if int_in else 0.5
    desc_t, mode = None, None
    if descale == "channel":
        desc_t, mode = (torch.rand(n, generator=g, device="cuda") * mag + mag).to(pd), "DescalePerChannel"
    elif descale == "tensor":
        desc_t, mode = (torch.rand(1, generator=g, device="cuda") * mag + mag).to(pd), "DescalePerTensor"
    sa_t = (torch.rand(m, generator=g, device="cuda") + 0.5) if scale_a else None
    out = bsir.matmul(a, b, transpose_a=ta, transpose_b=tb, bias=bias_t, descale=desc_t, descale_mode=mode, scale_a=sa_t,
                      relu=relu, out_dtype=out_dtype)
    want = O.matmul(_ODT[dtype], to_bits(a), to_bits(b), _ODT[out_dtype], transpose_a=ta, transpose_b=tb,
                    bias=None if bias_t is None else to_bits(bias_t), bias_dt=None if bias_t is None else _ODT[bias_t.dtype],
                    descale=None if desc_t is None else to_bits(desc_t), descale_dt=O.F32 if desc_t is None else _ODT[desc_t.dtype],
                    descale_mode={None: 0, "DescalePerChannel": 1, "DescalePerTensor": 2}[mode],
                    scale_a=None if sa_t is None else sa_t.cpu().numpy(), relu=relu)
    what = f"matmul {dtype} ({m},{n},{k}) ta={ta} tb={tb} bias={bias} descale={descale} relu={relu} -> {out_dtype}"
    if exact is None:
        exact = int_in or small_ints
    if exact:
        assert_bits_equal(out, want, what)
    else:
        gf = floats_from_bits(to_bits(out), out_dtype).astype(np.float64) if out_dtype != torch.int8 else out.cpu().numpy().astype(np.float64)
        wf = floats_from_bits(want, out_dtype).astype(np.float64) if out_dtype != torch.int8 else want.astype(np.float64)
        rms = np.sqrt(np.mean(wf ** 2)) + 1e-30
        err = np.abs(gf - wf)
        tol = 1e-2 * np.abs(wf) + 1e-2 * rms + (1.0 if out_dtype == torch.int8 else 0.0)   # one step of an int8 output
        assert (err <= tol).all(), f"{what}: worst excess {(err - tol).max():.3e}, rms {rms:.3e}"
    assert bsir.device_error() == 0
    return out


SHAPES = [(128, 256, 128), (1, 128, 64), (200, 384, 640), (130, 320, 208), (16, 256, 1024), (300, 136, 144), (256, 512, 1024)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_float_matmul_all_layouts(bsir, dtype, m, n, k, ta, tb):
    _check(bsir, dtype, m, n, k, ta, tb, seed=m + n + k, small_ints=True)     # every partial sum exact: bit for bit
    _check(bsir, dtype, m, n, k, ta, tb, seed=m + n + k + 1)                  # real data: tolerance


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_int8_matmul_all_layouts(bsir, m, n, k, ta, tb):
    _check(bsir, torch.int8, m, n, k, ta, tb, seed=m + n + k, out_dtype=torch.int32)             # raw accumulators
    _check(bsir, torch.int8, m, n, k, ta, tb, seed=m + n + k, descale="channel", out_dtype=torch.float16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.int8])
@pytest.mark.parametrize("bias,descale,relu", [(True, None, False), (False, "channel", False), (False, "tensor", True),
                                               (True, "channel", True), (True, "tensor", False)])
@pytest.mark.parametrize("m,n,k", [(130, 320, 208), (16, 256, 1024), (256, 512, 512)])
def test_matmul_bias_descale_relu(bsir, dtype, bias, descale, relu, m, n, k):
    _check(bsir, dtype, m, n, k, False, True, bias=bias, descale=descale, relu=relu, seed=m + k, small_ints=dtype != torch.int8,
           exact=True)
    _check(bsir, dtype, m, n, k, True, False, bias=bias, descale=descale, relu=relu, seed=m + k + 3)


@pytest.mark.parametrize("dtype,out_dtype", [(torch.bfloat16, torch.float32), (torch.bfloat16, torch.float16), (torch.float16, torch.bfloat16),
                                             (torch.float16, torch.float32), (torch.int8, torch.int8), (torch.int8, torch.bfloat16),
                                             (torch.int8, torch.float32), (torch.bfloat16, torch.int8)])
@pytest.mark.parametrize("m,n,k", [(130, 320, 208), (64, 1000, 512), (512, 768, 1024)])
def test_matmul_output_modes(bsir, dtype, out_dtype, m, n, k):
    """fixpipe pre_quant: F322F16, F322BF16, S322I8 (int32 accumulators scaled into the int8 range, saturating), and the
    unconverted f32."""
    _check(bsir, dtype, m, n, k, False, False, bias=True, descale="channel", relu=(out_dtype == torch.int8), seed=n,
           out_dtype=out_dtype, small_ints=dtype != torch.int8, exact=True,
           param_dtype=torch.float32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.int8])
def test_matmul_with_per_token_scale(bsir, dtype):
    _check(bsir, dtype, 200, 384, 640, False, False, descale="channel", scale_a=True, seed=5, small_ints=dtype != torch.int8,
           exact=True, param_dtype=torch.float32, out_dtype=torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.int8])
@pytest.mark.parametrize("path", ["1", "2"])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_matmul_both_kernels_same_bits(bsir, dtype, path, ta, tb, monkeypatch):
    """The single-CTA kernel and the CTA-pair kernel (forced on a small shape) against the oracle."""
    monkeypatch.setenv("BSIR_W8A8_PATH", path)
    _check(bsir, dtype, 512, 768, 1024, ta, tb, bias=True, descale="channel", seed=9, small_ints=dtype != torch.int8, exact=True,
           param_dtype=torch.float32)
    _check(bsir, dtype, 300, 320, 208, ta, tb, seed=10, small_ints=dtype != torch.int8, exact=True)


def test_batch_matmul(bsir):
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randint(-4, 5, (3, 130, 208), generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randint(-4, 5, (3, 208, 320), generator=g, device="cuda").to(torch.bfloat16)
    out = bsir.matmul(a, b)
    for e in range(3):
        want = O.matmul(O.BF16, to_bits(a[e]), to_bits(b[e]), O.BF16)
        assert_bits_equal(out[e], want, f"batch entry {e}")
    shared = bsir.matmul(a, b[0])                     # one B for every batch entry (batch stride 0)
    for e in range(3):
        assert_bits_equal(shared[e], O.matmul(O.BF16, to_bits(a[e]), to_bits(b[0]), O.BF16), f"shared B, entry {e}")


@pytest.mark.parametrize("dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float32), (torch.int8, torch.float16),
                                             (torch.int8, torch.int8), (torch.int8, torch.int32)])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, True)])
def test_batch_matmul_in_one_launch(bsir, dtype, out_dtype, ta, tb):
    """A batch of small products runs as one launch over rank-3 tensor maps: ragged m (the last tile of a product must
    not reach into the next product's rows), every store path of the epilogue, transposed operands, and operands that
    are views with padded batch strides."""
    g = torch.Generator(device="cuda").manual_seed(8)
    batch, m, n, k = 5, 130, 192, 256
    mk = (lambda *sh: torch.randint(-4, 5, sh, generator=g, device="cuda").to(dtype))
    a_big = mk(batch + 1, *( (k, m) if ta else (m, k) ))
    b_big = mk(batch + 2, *( (n, k) if tb else (k, n) ))
    a, b = a_big[1:], b_big[:batch]                                   # views: the same batch stride, another base
    int_in = dtype == torch.int8
    bias = (torch.randint(-50, 50, (n,), generator=g, device="cuda", dtype=torch.int32) if int_in else mk(n))
    desc = torch.full((1,), 0.01 if int_in else 0.5, device="cuda", dtype=torch.float32 if int_in else dtype)
    out = bsir.matmul(a, b, transpose_a=ta, transpose_b=tb, bias=bias, descale=desc, descale_mode="DescalePerTensor", relu=True,
                      out_dtype=out_dtype)
    for e in range(batch):
        want = O.matmul(_ODT[dtype], to_bits(a[e].contiguous()), to_bits(b[e].contiguous()), _ODT[out_dtype], transpose_a=ta,
                        transpose_b=tb, bias=to_bits(bias), bias_dt=_ODT[bias.dtype], descale=to_bits(desc), descale_dt=_ODT[desc.dtype],
                        descale_mode=2, relu=True)
        assert_bits_equal(out[e], want, f"{dtype} -> {out_dtype} ta={ta} tb={tb}, product {e}")
    assert bsir.device_error() == 0


def test_batch_matmul_many_products(bsir):
    g = torch.Generator(device="cuda").manual_seed(9)
    a = torch.randint(-3, 4, (8, 512, 1024), generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randint(-3, 4, (8, 1024, 512), generator=g, device="cuda").to(torch.bfloat16)
    out = bsir.matmul(a, b)
    assert torch.equal(out.float(), torch.bmm(a.float(), b.float()).to(torch.bfloat16).float())


@pytest.mark.parametrize("dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16), (torch.bfloat16, torch.float32),
                                             (torch.float16, torch.int8)])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(16, 4096, 4096), (1, 1000, 2048), (64, 520, 1024), (33, 4096, 512)])
def test_float_matmul_with_k_split_over_ctas(bsir, dtype, out_dtype, m, n, k, ta, tb):
    """Few tiles and a long K: the k blocks are shared out over 2, 4 or 8 CTAs a tile, the partial results added in
    part order by a second launch that applies bias, scales, relu and the conversion.  Exact on small integers, within
    tolerance on real data, the same bits on every run."""
    _check(bsir, dtype, m, n, k, ta, tb, bias=True, descale="channel", relu=True, scale_a=True, out_dtype=out_dtype, seed=m + n + k,
           small_ints=True, exact=out_dtype != torch.int8, param_dtype=torch.float32)
    first = _check(bsir, dtype, m, n, k, ta, tb, bias=True, descale="tensor", out_dtype=out_dtype, seed=m + n)
    again = _check(bsir, dtype, m, n, k, ta, tb, bias=True, descale="tensor", out_dtype=out_dtype, seed=m + n)
    assert torch.equal(first.view(torch.uint8), again.view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (16, 14336, 1024), (33, 1000, 640), (48, 264, 2048), (7, 136, 128), (24, 7168, 4096),
                                   (3, 640, 64 * 37), (16, 128 * 147, 256)])
def test_float_matmul_of_few_rows_with_swapped_operands(bsir, dtype, tb, m, n, k):
    """Float products of up to 48 rows and a 16-bit result take the decode kernel's form (weights on the tensor-memory
    lanes, four issuing threads with an accumulator each, added in issuer order): both weight layouts, ragged n and m,
    bias + descale + relu + per-row scale; exact on small integers, the same bits on every run, within tolerance on
    real data."""
    _check(bsir, dtype, m, n, k, False, tb, bias=True, descale="channel", relu=True, scale_a=True, seed=m + n + k, small_ints=True,
           exact=True, param_dtype=torch.float32)
    _check(bsir, dtype, m, n, k, False, tb, descale="tensor", seed=m + n, small_ints=True, exact=True)
    first = _check(bsir, dtype, m, n, k, False, tb, bias=True, seed=m + k)
    again = _check(bsir, dtype, m, n, k, False, tb, bias=True, seed=m + k)
    assert torch.equal(first.view(torch.uint8), again.view(torch.uint8))


def test_matmul_unaligned_operands_take_the_plain_kernel(bsir):
    a = torch.randint(-4, 5, (37, 101), device="cuda").to(torch.float16)     # row pitch 202 bytes: not a TMA pitch
    b = torch.randint(-4, 5, (101, 45), device="cuda").to(torch.float16)
    bias = torch.randn(45, device="cuda").to(torch.float16)
    out = bsir.matmul(a, b, bias=bias, relu=True)
    want = O.matmul(O.F16, to_bits(a), to_bits(b), O.F16, bias=to_bits(bias), bias_dt=O.F16, relu=True)
    assert_bits_equal(out, want, "plain kernel")


def test_matmul_rejects_bad_arguments(bsir):
    a = torch.zeros(8, 16, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(16, 8, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(bsir.BsirError):
        bsir.matmul(a, b, out_dtype=torch.int32)                              # int32 output only for int8 products
    with pytest.raises(bsir.BsirError):
        bsir.matmul(a, b, bias=torch.zeros(8, dtype=torch.int32, device="cuda"))   # float product wants a float bias
    with pytest.raises(bsir.BsirError):
        bsir.matmul(a.to(torch.int8), b.to(torch.int8), bias=torch.zeros(8, device="cuda"))


def test_matmul_library_symbols(bsir):
    """The reference's library-call names: operands as memref descriptors in the op's order."""
    L = bsir.lib()
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randint(-4, 5, (64, 96), generator=g, device="cuda").to(torch.float16)
    b = torch.randint(-4, 5, (96, 48), generator=g, device="cuda").to(torch.float16)
    bias = torch.randint(-4, 5, (48,), generator=g, device="cuda").to(torch.float16)
    desc = torch.tensor([0.5], device="cuda", dtype=torch.float16)
    c = torch.empty(64, 48, dtype=torch.float16, device="cuda")
    at, bt = a.t().contiguous(), b.t().contiguous()
    mr = bsir.memref
    rc = L._mlir_ciface_matmul_Xbias_Xdescale_XtransposeA_XtransposeB_TAhalf_TBhalf_TChalf(C.byref(mr(a)), C.byref(mr(b)), C.byref(mr(c)))
    assert rc == 0
    assert_bits_equal(c, O.matmul(O.F16, to_bits(a), to_bits(b), O.F16), "plain symbol")
    rc = L._mlir_ciface_matmul_bias_TBIAShalf_descalePerTensor_TDESCALEhalf_transposeA_transposeB_TAhalf_TBhalf_TChalf(
        C.byref(mr(at)), C.byref(mr(bt)), C.byref(mr(bias)), C.byref(mr(desc)), C.byref(mr(c)))
    assert rc == 0, L.bsir_last_error()
    want = O.matmul(O.F16, to_bits(at), to_bits(bt), O.F16, transpose_a=True, transpose_b=True, bias=to_bits(bias), bias_dt=O.F16,
                    descale=to_bits(desc), descale_dt=O.F16, descale_mode=2)
    assert_bits_equal(c, want, "bias + per-tensor descale symbol, both operands transposed")
    ai = torch.randint(-127, 128, (64, 96), generator=g, device="cuda", dtype=torch.int8)
    bi = torch.randint(-127, 128, (96, 48), generator=g, device="cuda", dtype=torch.int8)
    rc = L._mlir_ciface_matmul_Xbias_Xdescale_transposeA_XtransposeB_TAint8_t_TBint8_t_TChalf(
        C.byref(mr(ai.t().contiguous())), C.byref(mr(bi)), C.byref(mr(c)))
    assert rc == 0
    assert_bits_equal(c, O.matmul(O.I8, to_bits(ai.t().contiguous()), to_bits(bi), O.F16, transpose_a=True), "int8 transposeA symbol")
