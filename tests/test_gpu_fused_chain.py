"""GPU: chains of elementwise ops run as one kernel (bsir_fused_elementwise) against the oracle's op-by-op f32
evaluation with a single final rounding -- the numerics HFusion's bf16 legalisation gives a fused chain
(LegalizeBF16.cpp:243-275 + SimplifyOps.cpp:105-230).  Every case runs on both execution paths: the kernel
compiled for the chain (NVRTC) and the tape interpreter kernel."""
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


@pytest.fixture(params=["compiled", "interpreted"])
def path(request, monkeypatch):
    """Selects the execution path through BSIR_CHAIN_JIT; 'compiled' falls back to the interpreter only where the
    compiled path does not apply (ragged rows), which the tests check through FusedChain.last_path()."""
    monkeypatch.setenv("BSIR_CHAIN_JIT", "0" if request.param == "interpreted" else "2")
    return request.param


def _expect_path(bsir, path, vector_ok):
    assert bsir.FusedChain.last_path() == ("compiled" if path == "compiled" and vector_ok else "interpreted")


def _f32(t):
    return t.float().cpu().numpy().astype(np.float32)


def _round_to(x32, dtype):
    """f32 numpy -> storage bits of dtype (one RNE)."""
    if dtype == torch.float32:
        return x32.astype(np.float32)
    return O.cast(O.F32, oracle_dtype(torch.empty(0, dtype=dtype)), np.ascontiguousarray(x32), "rint")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,cols", [(64, 4096), (7, 40), (1, 8), (333, 1000), (5, 17)])
def test_rms_norm_tail_chain(bsir, path, dtype, rows, cols):
    """y = gamma * (rstd * x): full tensor, per-row vector, per-column vector -- bit-exact against the f32 evaluation."""
    g = torch.Generator(device="cuda").manual_seed(rows + cols)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(dtype)
    gamma = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).to(dtype)
    rstd = (0.5 + torch.rand(rows, 1, device="cuda", generator=g)).to(torch.float32)
    ch = bsir.FusedChain()
    hx, hg, hr = ch.operand(x), ch.operand(gamma, "row_vector"), ch.operand(rstd, "col_vector")
    ch.load(ch.op(hr)).binary("mul", ch.op(hx)).rbinary("mul", ch.op(hg))
    y = ch.run(rows, cols, out_dtype=dtype)
    _expect_path(bsir, path, cols % 8 == 0)
    want32 = O.elemwise_binary("mul", O.F32, np.broadcast_to(_f32(gamma)[None, :], (rows, cols)).copy(),
                               O.elemwise_binary("mul", O.F32, np.broadcast_to(_f32(rstd), (rows, cols)).copy(), _f32(x)))
    assert_bits_equal(y, _round_to(want32, dtype).reshape(rows, cols), f"chain {dtype} {rows}x{cols}")


def test_gelu_like_chain_with_temporaries_and_two_outputs(bsir, path):
    """0.5 x (1 + tanh(0.79788456 (x + 0.044715 x^3))) with a saved temporary, plus a second output (x^2)."""
    rows, cols = 48, 2048
    x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    ch = bsir.FusedChain()
    hx = ch.operand(x)
    (ch.load(ch.op(hx)).unary("square").save(1)                      # t1 = x^2
       .binary("mul", ch.op(hx)).binary("mul", 0.044715).binary("add", ch.op(hx)).binary("mul", 0.7978845608)
       .unary("tanh").binary("add", 1.0).binary("mul", ch.op(hx)).binary("mul", 0.5))
    y, sq = ch.run(outs=[(torch.bfloat16, -1), (torch.float32, 1)])
    _expect_path(bsir, path, True)
    x32 = _f32(x)
    f = lambda fn, a, b: O.elemwise_binary(fn, O.F32, a, b)
    c = lambda v: np.full_like(x32, np.float32(v))
    x2 = O.elemwise_unary("square", O.F32, x32)
    t = f("mul", f("add", f("mul", f("mul", x2, x32), c(0.044715)), x32), c(0.7978845608))
    want = f("mul", f("mul", f("add", O.elemwise_unary("tanh", O.F32, t), c(1.0)), x32), c(0.5))
    assert np.array_equal(sq.cpu().numpy(), x2)
    got = _f32(y)
    ref = O.bf16_to_f32(O.f32_to_bf16(want))
    assert np.abs(got - ref).max() <= 2 ** -7 * np.abs(ref).max()      # tanh: device libm vs host libm, then bf16


def test_chain_equals_separate_launches_in_f32(bsir, path):
    """For f32 data the fused chain and the op-by-op library calls give the same bits."""
    a = torch.randn(100, 513, device="cuda")
    b = torch.rand(100, 513, device="cuda") + 0.5
    s = torch.tensor([1.5], device="cuda")
    ch = bsir.FusedChain()
    ha, hb, hs = ch.operand(a), ch.operand(b), ch.operand(s)
    ch.load(ch.op(ha)).binary("div", ch.op(hb)).unary("abs").unary("sqrt").rbinary("sub", ch.op(hs)).binary("maxf", 0.25)
    y = ch.run()
    w = bsir.elemwise_binary("maxf", bsir.elemwise_binary("sub", 1.5, bsir.elemwise_unary(
        "sqrt", bsir.elemwise_unary("abs", bsir.elemwise_binary("div", a, b)))), 0.25)
    assert torch.equal(y, w)


def test_chain_validation(bsir):
    x = torch.randn(4, 8, device="cuda")
    ch = bsir.FusedChain()
    h = ch.operand(x)
    ch.load(ch.op(h)).unary("vnot")                                   # no f32 form
    with pytest.raises(bsir.BsirError):
        ch.run()
    ch2 = bsir.FusedChain()
    ch2.operand(x)
    ch2.load(("operand", 3))                                          # operand out of range
    with pytest.raises(bsir.BsirError):
        ch2.run()


def test_both_paths_give_the_same_bits(bsir, monkeypatch):
    """Transcendentals included: the compiled kernel and the interpreter spell the arithmetic alike."""
    rows, cols = 96, 1024
    x = torch.randn(rows, cols, device="cuda").to(torch.float16)
    w = torch.rand(rows, cols, device="cuda") + 0.25
    bias = torch.randn(cols, device="cuda").to(torch.bfloat16)
    res = {}
    for mode in ("2", "0"):
        monkeypatch.setenv("BSIR_CHAIN_JIT", mode)
        ch = bsir.FusedChain()
        hx, hw, hb = ch.operand(x), ch.operand(w), ch.operand(bias, "row_vector")
        (ch.load(ch.op(hx)).binary("add", ch.op(hb)).save(0).unary("exp").binary("div", ch.op(hw)).unary("log")
           .rbinary("sub", ("tmp", 0)).unary("erf").binary("powf", 2.0).unary("sin").binary("minnumf", ch.op(hw)).save(2)
           .unary("rsqrt").binary("maxf", ("tmp", 2)))
        res[mode] = ch.run(outs=[(torch.float16, -1), (torch.float32, 0), (torch.bfloat16, 2)])
        assert bsir.FusedChain.last_path() == ("compiled" if mode == "2" else "interpreted")
    for a, b in zip(res["2"], res["0"]):
        assert np.array_equal(to_bits(a), to_bits(b))


def test_compiled_chain_in_place_and_strided(bsir, monkeypatch):
    """An output that is also an operand, and row strides wider than the row."""
    monkeypatch.setenv("BSIR_CHAIN_JIT", "1")           # the compiled path or an error
    big = torch.randn(50, 96, device="cuda")
    before = big.clone()
    x = big[:, 16:80]                                    # 64 columns, row stride 96, 16-byte aligned
    keep = x.clone()
    ch = bsir.FusedChain()
    h = ch.operand(x)
    ch.load(ch.op(h)).binary("mul", 2.0).binary("add", ch.op(h))
    ch.run(50, 64, outs=[(x, -1)])
    assert bsir.FusedChain.last_path() == "compiled"
    assert torch.equal(x, keep * 2.0 + keep)
    assert torch.equal(big[:, :16], before[:, :16]) and torch.equal(big[:, 80:], before[:, 80:])


def test_compiled_path_refuses_ragged_rows_when_required(bsir, monkeypatch):
    monkeypatch.setenv("BSIR_CHAIN_JIT", "1")
    x = torch.randn(5, 17, device="cuda")
    ch = bsir.FusedChain()
    ch.load(ch.op(ch.operand(x)))
    with pytest.raises(bsir.BsirError):
        ch.run()


# ---------------------------------------------------------------------------- chains with last-axis reductions
def _rms_chain(bsir, x, gamma, eps):
    ch = bsir.FusedChain()
    hx, hg = ch.op(ch.operand(x)), ch.op(ch.operand(gamma, "row_vector"))
    (ch.load(hx).unary("square").reduce("sum").binary("div", float(x.shape[1])).binary("add", eps).unary("sqrt").unary("rec")
       .save(0).binary("mul", hx).rbinary("mul", hg))
    return ch


@pytest.mark.parametrize("dtype,rows,cols", [(torch.bfloat16, 64, 4096), (torch.float16, 40, 512), (torch.float32, 1001, 64),
                                             (torch.bfloat16, 7, 8192), (torch.bfloat16, 3, 32768), (torch.float16, 300, 8),
                                             (torch.bfloat16, 600, 32768)])
def test_rms_norm_as_a_chain_with_a_reduction(bsir, dtype, rows, cols):
    """A whole RMSNorm (LAST_AXIS_PBR): square, row sum, scalar tail, two multiplies, the per-row rstd as a second
    output -- one kernel, against the oracle's RMSNorm (the row sum associates differently: tolerance as for the
    hand-written kernel)."""
    g = torch.Generator(device="cuda").manual_seed(cols)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(dtype)
    gamma = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).to(dtype)
    n0 = bsir.launch_count()
    y, rstd = _rms_chain(bsir, x, gamma, 1e-6).run(outs=[(dtype, -1), (torch.empty(rows, dtype=dtype, device="cuda"), 0)])
    assert bsir.launch_count() - n0 == 1 and bsir.FusedChain.last_path() == "compiled"
    dt = oracle_dtype(x)
    wy, wr = O.rms_norm(dt, to_bits(x), to_bits(gamma), 1e-6, want_rstd=True)
    from conftest import assert_close
    assert_close(y, wy, 1e-2, 1e-3, "rms-norm chain")
    assert_close(rstd, wr, 1e-2, 1e-3, "rstd of the chain")


@pytest.mark.parametrize("dtype,rows,cols", [(torch.bfloat16, 33, 4096), (torch.float32, 257, 1000), (torch.float16, 5, 32768),
                                             (torch.bfloat16, 700, 32768), (torch.float32, 333, 24576)])
def test_softmax_as_a_chain_with_two_reductions(bsir, dtype, rows, cols):
    """The last two shapes: rows that fill an SM's registers run as persistent blocks fed by a ring of bulk copies,
    each block going through four or five rows (every buffer of the ring is reused)."""
    g = torch.Generator(device="cuda").manual_seed(rows)
    x = (4 * torch.randn(rows, cols, device="cuda", generator=g)).to(dtype)
    ch = bsir.FusedChain()
    hx = ch.op(ch.operand(x))
    ch.load(hx).reduce("max").save(0).load(hx).binary("sub", ("tmp", 0)).unary("exp").save(1).reduce("sum").rbinary("div", ("tmp", 1))
    y = ch.run(out_dtype=dtype)
    assert bsir.FusedChain.last_path() == "compiled"
    from conftest import assert_close
    assert_close(y, O.softmax(oracle_dtype(x), to_bits(x)), 2e-2, 1e-6, "softmax chain")
    assert abs(y.float().sum(dim=1) - 1).max().item() < 2e-2


def test_row_maximum_of_absolute_values_is_exact(bsir):
    """max is associative: the per-row output equals the op-by-op result exactly (a NaN row gives NaN in both; the
    payload of a NaN that went through max.NaN is not compared)."""
    x = torch.randn(500, 2048, device="cuda").to(torch.bfloat16)
    x[7, 100] = float("nan")
    x[9, :] = float("-inf")
    ch = bsir.FusedChain()
    ch.load(ch.op(ch.operand(x))).unary("abs").reduce("max")
    amax = ch.run(outs=[(torch.empty(500, dtype=torch.float32, device="cuda"), -1)])
    want = bsir.reduce("max", bsir.elemwise_unary("abs", x.float()), dim=1)
    assert np.array_equal(to_bits(amax), to_bits(want), equal_nan=True)
    assert torch.isnan(amax[7]) and amax[9] == float("inf")


def test_chains_with_reductions_need_the_compiled_path(bsir, monkeypatch):
    x = torch.randn(4, 20, device="cuda")                 # 20 columns: not a multiple of 8
    ch = bsir.FusedChain()
    ch.load(ch.op(ch.operand(x))).reduce("sum")
    with pytest.raises(bsir.BsirError):
        ch.run()
    monkeypatch.setenv("BSIR_CHAIN_JIT", "0")
    x = torch.randn(4, 64, device="cuda")
    ch = bsir.FusedChain()
    ch.load(ch.op(ch.operand(x))).reduce("sum")
    with pytest.raises(bsir.BsirError):
        ch.run()
    ch = bsir.FusedChain()                                 # a per-row output without a reduction
    ch.load(ch.op(ch.operand(x)))
    monkeypatch.setenv("BSIR_CHAIN_JIT", "2")
    with pytest.raises(bsir.BsirError):
        ch.run(outs=[(torch.empty(4, device="cuda"), -1)])
