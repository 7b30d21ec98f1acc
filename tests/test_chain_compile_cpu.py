"""CPU: the code generator behind bsir_fused_elementwise and its NVRTC build for sm_100a (no device is touched:
source text and cubin only)."""
import pytest
import torch

import bsir


def _rms_tail():
    ch = bsir.FusedChain()
    x = ch.operand(torch.zeros(4, 16, dtype=torch.bfloat16))
    g = ch.operand(torch.zeros(16, dtype=torch.bfloat16), "row_vector")
    r = ch.operand(torch.zeros(4, 1), "col_vector")
    ch.load(ch.op(r)).binary("mul", ch.op(x)).rbinary("mul", ch.op(g))
    return ch


def test_source_is_straight_line_code_for_the_tape():
    src = _rms_tail().source(outs=[(torch.bfloat16, -1)], contiguous=False)
    assert 'extern "C" __global__ void __launch_bounds__(256) bsir_chain' in src
    assert src.count("__fmul_rn(x, y)") == 2                     # one line per binary instruction
    assert "ld_stream((const u16 *)a.in[0]" in src               # the tensor: streaming 16-byte loads
    assert "ld_keep((const u16 *)a.in[1] + c0)" in src           # the [cols] vector stays in L1
    assert "one_f32(a.in[2], row)" in src                        # the [rows] vector: one value per row
    assert "pk_bf16(acc[0], acc[1])" in src
    assert "switch" not in src[src.index("bsir_chain"):]         # nothing is decoded at run time


def test_source_depends_on_the_chain_not_on_unused_fields():
    a, b = bsir.FusedChain(), bsir.FusedChain()
    for ch, junk in ((a, 0.0), (b, 7.0)):
        h = ch.operand(torch.zeros(2, 8))
        ch.load(ch.op(h)).unary("exp")
        ch._tape[-1] = ch._tape[-1][:4] + (junk,)                # the immediate of a unary is never read
    assert a.source() == b.source()
    c = bsir.FusedChain()
    h = c.operand(torch.zeros(2, 8))
    c.load(c.op(h)).unary("log")
    assert c.source() != a.source()


def test_in_place_chains_use_coherent_loads():
    ch = bsir.FusedChain()
    h = ch.operand(torch.zeros(2, 8))
    ch.load(ch.op(h)).binary("add", 1.0)
    assert "ld_plain(" in ch.source(in_place=True).split("bsir_chain")[1]
    assert "ld_plain(" not in ch.source(in_place=False).split("bsir_chain")[1]


def test_invalid_tapes_are_refused_before_code_generation():
    ch = bsir.FusedChain()
    h = ch.operand(torch.zeros(2, 8))
    ch.load(ch.op(h)).binary("add", ("tmp", 2))                  # read before any save
    with pytest.raises(bsir.BsirError):
        ch.source()
    ch2 = bsir.FusedChain()
    ch2.operand(torch.zeros(2, 8))
    ch2.load(("operand", 0)).unary("vnot")                       # no f32 form
    with pytest.raises(bsir.BsirError):
        ch2.source()


def _nvrtc_available():
    ch = bsir.FusedChain()
    ch.load(ch.op(ch.operand(torch.zeros(2, 8))))
    try:
        ch.compile()
        return True
    except bsir.BsirError as e:
        return "libnvrtc" not in str(e)


@pytest.mark.skipif(not _nvrtc_available(), reason="no NVRTC library in this environment")
def test_every_function_compiles_for_sm_100a():
    ch = bsir.FusedChain()
    x = ch.operand(torch.zeros(4, 16, dtype=torch.float16))
    w = ch.operand(torch.zeros(4, 16))
    ch.load(ch.op(x))
    for fn in ("relu", "sqrt", "rsqrt", "rec", "tanh", "exp", "log", "abs", "ceil", "floor", "negf", "round"):
        ch.unary(fn)
    ch.save(0)
    for i, fn in enumerate(("add", "sub", "mul", "div", "maxf")):
        (ch.rbinary if i % 2 else ch.binary)(fn, ch.op(w))
    assert ch.compile(outs=[(torch.float16, -1), (torch.float32, 0)], contiguous=False) > 1000
    ch2 = bsir.FusedChain()
    x = ch2.operand(torch.zeros(4, 16, dtype=torch.bfloat16))
    s = ch2.operand(torch.zeros(1, dtype=torch.bfloat16))
    ch2.load(ch2.op(s)).binary("minf", ch2.op(x))
    for fn in ("square", "erf", "sin", "cos", "exp2", "log2", "reciprocal"):
        ch2.unary(fn)
    for fn in ("minnumf", "maxnumf", "powf", "divfhp"):
        ch2.binary(fn, 1.25)
    assert ch2.compile(outs=[(torch.bfloat16, -1)]) > 1000
    assert _rms_tail().compile(outs=[(torch.bfloat16, -1)], contiguous=False) > 1000


@pytest.mark.skipif(not _nvrtc_available(), reason="no NVRTC library in this environment")
def test_chains_with_reductions_compile_for_short_and_long_rows():
    """A LAST_AXIS_PBR chain: the generated kernel keeps the row in registers (threads per row and groups per thread
    follow the row length)."""
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    ch = bsir.FusedChain()
    hx, hg = ch.op(ch.operand(x)), ch.op(ch.operand(torch.zeros(64, dtype=torch.bfloat16), "row_vector"))
    (ch.load(hx).unary("square").reduce("sum").binary("div", 64.0).binary("add", 1e-6).unary("sqrt").unary("rec").save(0)
       .binary("mul", hx).rbinary("mul", hg))
    outs = [(torch.bfloat16, -1), (torch.zeros(4), 0)]
    short, mid = ch.source(outs=outs, cols=64), ch.source(outs=outs, cols=4096)
    assert "#define TPR 4\n" in short and "#define VPT 2\n" in short
    assert "#define TPR 256\n" in mid and "#define VPT 2\n" in mid       # one temporary: two groups per thread
    assert "row_sum(p, red)" in mid and "((float *)a.out[1])[row] = t0[0][0]" in mid
    for cols in (64, 4096, 32768):
        assert ch.compile(outs=outs, cols=cols) > 1000
    # rows that fill an SM's registers: persistent blocks, rows through a ring of bulk copies; not when in place
    long_rows = ch.source(outs=outs, cols=32768)
    assert "#define TPR 1024\n" in long_rows and "#define NBUF 3\n" in long_rows and "cp.async.bulk.shared::cluster.global" in long_rows
    assert "NBUF" not in mid and "NBUF" not in ch.source(outs=outs, cols=32768, in_place=True)
    with pytest.raises(bsir.BsirError):
        ch.source(outs=outs, cols=1 << 20)                       # a row that no block can hold
    ch2 = bsir.FusedChain()
    ch2.load(ch2.op(ch2.operand(x))).reduce("any")               # not a float reduction
    with pytest.raises(bsir.BsirError):
        ch2.source()
