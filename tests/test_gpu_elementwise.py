"""GPU parity: elementwise / compare / select / cast against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle as O
from conftest import assert_bits_equal, assert_close, oracle_dtype, to_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bsir():
    import bsir as B
    B.lib()
    return B


def _rand(shape, dtype, seed, lo=-4.0, hi=4.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(shape, generator=g, device="cuda") * (hi - lo) + lo).to(dtype)
    info = torch.iinfo(dtype)
    return torch.randint(max(info.min, -1000), min(info.max, 1000) + 1, shape, generator=g, device="cuda", dtype=dtype)


# --- config 0: HIVM VecAdd, fp32 and fp16, length 2^24, bit-exact -------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_vecadd_full_size_bit_exact(bsir, dtype):
    from bsir import workloads as W
    a, b = W.vecadd(1 << 24, dtype, seed=0)
    out = bsir.vadd(a, b)
    want = O.elemwise_binary("add", oracle_dtype(a), to_bits(a), to_bits(b))
    assert_bits_equal(out, want, f"vadd {dtype}")


def test_vecadd_reference_e2e_vector(bsir):
    # bishengir/test/Integration/HIVM/VecAdd/main.cpp:141-158: {0..15} + {1,...} -> {1..16}, i16, N = 16
    a = torch.arange(16, dtype=torch.int16, device="cuda")
    b = torch.ones(16, dtype=torch.int16, device="cuda")
    assert bsir.vadd(a, b).cpu().tolist() == list(range(1, 17))


@pytest.mark.parametrize("n", [0, 1, 3, 7, 8, 9, 255, 256, 1023, 4097, 100003])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.int16, torch.int32])
def test_vadd_ragged_lengths(bsir, n, dtype):
    a, b = _rand((n,), dtype, 1), _rand((n,), dtype, 2)
    out = bsir.vadd(a, b)
    if n == 0:
        assert out.numel() == 0
        return
    want = O.elemwise_binary("add", oracle_dtype(a), to_bits(a), to_bits(b))
    assert_bits_equal(out, want, f"vadd n={n} {dtype}")


EXACT_BINARY = ["add", "sub", "mul", "div", "maxf", "minf", "maxnumf", "minnumf", "copysign"]


@pytest.mark.parametrize("fn", EXACT_BINARY)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_binary_float_exact(bsir, fn, dtype):
    a, b = _rand((257, 129), dtype, 3), _rand((257, 129), dtype, 4)
    # plant special values
    a.view(-1)[:8] = torch.tensor([0.0, -0.0, float("nan"), float("inf"), -float("inf"), 1.0, -0.0, 0.0], device="cuda").to(dtype)
    b.view(-1)[:8] = torch.tensor([-0.0, 0.0, 1.0, float("inf"), 2.0, float("nan"), -0.0, 0.0], device="cuda").to(dtype)
    out = bsir.elemwise_binary(fn, a, b)
    want = O.elemwise_binary(fn, oracle_dtype(a), to_bits(a), to_bits(b))
    assert_bits_equal(out, want, f"{fn} {dtype}")


@pytest.mark.parametrize("fn", ["add", "sub", "mul", "div", "max_signed", "min_signed", "vand", "vor", "vxor",
                                "mod", "shli", "shrsi", "shrui", "floordivsi", "ceildivsi"])
@pytest.mark.parametrize("dtype", [torch.int8, torch.int16, torch.int32, torch.int64])
def test_binary_int_exact(bsir, fn, dtype):
    a, b = _rand((1000,), dtype, 5), _rand((1000,), dtype, 6)
    if fn in ("shli", "shrsi", "shrui"):
        b = b.abs() % 9
    if fn in ("div", "mod", "floordivsi", "ceildivsi"):
        b = torch.where(b == 0, torch.ones_like(b), b)
    out = bsir.elemwise_binary(fn, a, b)
    want = O.elemwise_binary(fn, oracle_dtype(a), to_bits(a), to_bits(b))
    assert_bits_equal(out, want, f"{fn} {dtype}")


@pytest.mark.parametrize("fn,lo,hi", [("exp", -10, 10), ("log", 0.01, 100), ("abs", -4, 4), ("sqrt", 0, 100),
                                      ("rsqrt", 0.01, 100), ("rec", 0.1, 10), ("relu", -4, 4), ("tanh", -4, 4),
                                      ("sin", -6, 6), ("cos", -6, 6), ("erf", -3, 3), ("floor", -9, 9),
                                      ("ceil", -9, 9), ("negf", -4, 4), ("exp2", -8, 8), ("log2", 0.01, 100),
                                      ("log1p", -0.5, 10), ("square", -4, 4), ("nearbyint", -9, 9), ("sinh", -4, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unary_float(bsir, fn, lo, hi, dtype):
    x = _rand((4099,), dtype, 7, lo, hi)
    out = bsir.elemwise_unary(fn, x)
    want = O.elemwise_unary(fn, oracle_dtype(x), to_bits(x))
    if fn in ("abs", "sqrt", "rsqrt", "rec", "relu", "floor", "ceil", "negf", "square", "nearbyint"):
        assert_bits_equal(out, want, f"{fn} {dtype}")      # correctly rounded ops: bit-exact
    else:
        # transcendental: device libm vs host libm; tolerance of the reference's own convention
        # (docs/source/en/developer_guide/conversion/triton_interface.md:88-99)
        tol = 1e-4 if dtype == torch.float32 else 1e-2
        assert_close(out, want, tol, tol, f"{fn} {dtype}")


def test_scalar_and_broadcast_operands(bsir):
    a = _rand((33, 65), torch.float32, 8)
    out = bsir.elemwise_binary("mul", a, 2.5)
    want = O.elemwise_binary("mul", O.F32, to_bits(a), np.array([2.5], np.float32))
    assert_bits_equal(out, want, "mul scalar")
    out = bsir.elemwise_binary("sub", 1.0, a)
    want = O.elemwise_binary("sub", O.F32, np.array([1.0], np.float32), to_bits(a))
    assert_bits_equal(out, want, "scalar sub")
    row = _rand((1, 65), torch.float32, 9)      # inline broadcast along dim 0
    out = bsir.elemwise_binary("add", a, row)
    want = O.elemwise_binary("add", O.F32, to_bits(a), to_bits(row.expand(33, 65).contiguous()))
    assert_bits_equal(out, want, "add broadcast")
    col = _rand((33, 1), torch.float32, 10)     # inline broadcast along dim 1
    out = bsir.elemwise_binary("add", a, col)
    want = O.elemwise_binary("add", O.F32, to_bits(a), to_bits(col.expand(33, 65).contiguous()))
    assert_bits_equal(out, want, "add broadcast col")


def test_strided_views(bsir):
    big = _rand((64, 96), torch.float16, 11)
    a = big[::2, 1:65]           # non-contiguous, misaligned base
    b = big.t()[1:65, :32].t()   # transposed view
    out = bsir.elemwise_binary("add", a, b)
    want = O.elemwise_binary("add", O.F16, to_bits(a.contiguous()), to_bits(b.contiguous()))
    assert_bits_equal(out, want, "strided add")


def test_rank3(bsir):
    a, b = _rand((5, 7, 24), torch.bfloat16, 12), _rand((5, 7, 24), torch.bfloat16, 13)
    out = bsir.elemwise_binary("mul", a, b)
    want = O.elemwise_binary("mul", O.BF16, to_bits(a), to_bits(b))
    assert_bits_equal(out, want, "rank3 mul")


@pytest.mark.parametrize("fn", ["veq", "vne", "vlt", "vle", "vgt", "vge"])
def test_compare_and_select(bsir, fn):
    a, b = _rand((1000,), torch.float32, 14), _rand((1000,), torch.float32, 15)
    a[:4] = torch.tensor([float("nan"), 1.0, 0.0, -0.0], device="cuda")
    b[:4] = torch.tensor([1.0, float("nan"), -0.0, 0.0], device="cuda")
    b[10:20] = a[10:20]
    c = bsir.compare(fn, a, b)
    want = O.compare(fn, O.F32, to_bits(a), to_bits(b))
    assert_bits_equal(c, want, f"compare {fn}")
    s = bsir.select(c, a, b)
    wants = O.select(O.F32, want, to_bits(a), to_bits(b))
    assert_bits_equal(s, wants, "select")


def test_copy_strided(bsir):
    x = _rand((40, 50), torch.int32, 16)
    out = bsir.copy(x.t())
    assert torch.equal(out, x.t())


# --- hfusion.cast ------------------------------------------------------------------------------
MODES = ["rint", "round", "floor", "ceil", "trunc", "odd"]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("sat", [False, True])
@pytest.mark.parametrize("dst", [torch.int8, torch.int16, torch.int32, torch.int64])
def test_cast_float_to_int(bsir, mode, sat, dst):
    x = _rand((5003,), torch.float32, 17, -300.0, 300.0)
    ties = torch.arange(-140, 140, device="cuda", dtype=torch.float32) + 0.5
    x[:ties.numel()] = ties
    x[300:306] = torch.tensor([float("nan"), float("inf"), -float("inf"), 3e9, -3e9, 1e20], device="cuda")
    out = bsir.cast(x, dst, round_mode=mode, enable_saturate=sat)
    want = O.cast(O.F32, {torch.int8: O.I8, torch.int16: O.I16, torch.int32: O.I32, torch.int64: O.I64}[dst], to_bits(x),
                  mode, "saturate" if sat else "wrap")
    assert_bits_equal(out, want, f"cast f32->{dst} {mode} sat={sat}")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("dst", [torch.float16, torch.bfloat16])
def test_cast_float_narrowing(bsir, mode, dst):
    x = _rand((8191,), torch.float32, 18, -70000.0, 70000.0)
    x[:6] = torch.tensor([0.0, -0.0, float("nan"), float("inf"), 1e-8, -1e-8], device="cuda")
    out = bsir.cast(x, dst, round_mode=mode)
    want = O.cast(O.F32, O.F16 if dst == torch.float16 else O.BF16, to_bits(x), mode)
    assert_bits_equal(out, want, f"cast f32->{dst} {mode}")


def test_cast_reference_known_answers(bsir):
    # test/Dialect/HFusion/canonicalize.mlir:149-166: i64 2 -> 2.0f; f32 2.8 -> 3.0 (default rint)
    assert bsir.cast(torch.full((16,), 2, dtype=torch.int64, device="cuda"), torch.float32).cpu().tolist() == [2.0] * 16
    assert bsir.cast(torch.full((16,), 2.8, device="cuda"), torch.float32).cpu().tolist() == [3.0] * 16
    # Normalize.cpp:3806-3811 saturate example
    x = torch.tensor([128.7, 127.5, 100.3, -129.2, -128.4], device="cuda")
    got = bsir.cast(x, torch.int8, overflow_mode="ascend_saturate_trunc_via_f16").cpu().tolist()
    assert got == [127, 127, 100, -128, -128]
    # double rounding through f16 vs single rounding
    y = torch.tensor([2.5 + 2.0 ** -20], device="cuda")
    assert bsir.cast(y, torch.int8, enable_saturate=True).item() == 3
    assert bsir.cast(y, torch.int8, overflow_mode="ascend_double_round_via_f16").item() == 2


@pytest.mark.parametrize("src,dst", [(torch.bfloat16, torch.float32), (torch.float16, torch.float32),
                                     (torch.int8, torch.float16), (torch.int32, torch.float32),
                                     (torch.int64, torch.float32), (torch.int32, torch.int8),
                                     (torch.int64, torch.int32), (torch.int16, torch.int8),
                                     (torch.bool, torch.float32), (torch.uint8, torch.int32),
                                     (torch.int32, torch.bfloat16), (torch.bfloat16, torch.int32)])
def test_cast_other_pairs(bsir, src, dst):
    if src == torch.bool:
        x = _rand((1000,), torch.int8, 19) > 0
    elif src.is_floating_point:
        x = _rand((1000,), src, 19, -1000, 1000)
    elif src == torch.uint8:
        x = _rand((1000,), torch.int16, 19).abs().clamp(max=255).to(torch.uint8)
    else:
        x = _rand((1000,), src, 19)
        if src in (torch.int32, torch.int64):
            x = x * 70001
    out = bsir.cast(x, dst, round_mode="trunc" if (src.is_floating_point and not dst.is_floating_point) else "rint")
    code = lambda d: oracle_dtype(torch.empty(0, dtype=d))
    want = O.cast(code(src), code(dst), to_bits(x), "trunc" if (src.is_floating_point and not dst.is_floating_point) else "rint", "wrap")
    assert_bits_equal(out, want, f"cast {src}->{dst}")


# ---------------------------------------------------------------- hivm.hir.load (padding) / hivm.hir.store (atomic)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int8, torch.int64])
@pytest.mark.parametrize("shape,dst_last,left,right", [((5, 37), 64, -1, -1), ((5, 37), 64, 3, -1), ((5, 37), 64, -1, 7),
                                                      ((5, 37), 64, 3, 7), ((1000,), 1024, 8, 16), ((3, 4, 100), 128, 28, 0),
                                                      ((70000, 3), 8, 2, 3)])
@pytest.mark.parametrize("pad_mode", ["value", "first_elem"])
def test_load_with_padding(bsir, dtype, shape, dst_last, left, right, pad_mode):
    """Left / right padding with the paddings given or deduced (reference CPU lowering:
    ConvertHIVMToUpstream.cpp:1140-1166), value or first-element pad, untouched tail."""
    x = _rand(shape, dtype, seed=sum(shape) + dst_last)
    out = _rand(shape[:-1] + (dst_last,), dtype, seed=1)          # recognisable initial contents
    before = out.clone()
    pv = 3 if not dtype.is_floating_point else 2.5
    bsir.load(x, out, pad_mode=pad_mode, pad_value=pv, left_padding_num=left, right_padding_num=right)
    want = O.load_pad(oracle_dtype(x), to_bits(x), to_bits(before), pad_mode, to_bits(torch.tensor([pv], dtype=dtype)),
                      left, right)
    assert_bits_equal(out, want.reshape(out.shape), f"load {pad_mode} {shape}->{dst_last} l={left} r={right}")


def test_load_plain_and_errors(bsir):
    x = _rand((7, 33), torch.float16, seed=2)
    out = torch.empty_like(x)
    bsir.load(x, out)                                            # no pad_mode: shapes must match, plain copy
    assert torch.equal(out, x)
    with pytest.raises(bsir.BsirError):
        bsir.load(x, torch.empty(7, 40, dtype=torch.float16, device="cuda"))            # pad needed but no pad_mode
    with pytest.raises(bsir.BsirError):
        bsir.load(x, torch.empty(7, 40, dtype=torch.float16, device="cuda"), pad_mode="value", pad_value=0.0,
                  left_padding_num=5, right_padding_num=5)                               # 5 + 33 + 5 > 40


@pytest.mark.parametrize("dtype,kinds", [(torch.float32, ["add", "max", "min"]), (torch.float16, ["add"]), (torch.bfloat16, ["add"]),
                                         (torch.int32, ["add", "max", "min", "and", "or", "xor", "umax", "umin"]),
                                         (torch.int64, ["add", "max", "min", "and", "or", "xor", "umax", "umin"])])
def test_store_atomic_kinds(bsir, dtype, kinds):
    for kind in kinds:
        src = _rand((9, 1000), dtype, seed=3)
        dst = _rand((9, 1000), dtype, seed=4)
        if dtype == torch.float32:
            src[0, 5] = float("nan")
            dst[1, 6] = float("nan")
        before = dst.clone()
        bsir.store(src, dst, atomic=kind)
        want = O.store_atomic(oracle_dtype(src), kind, to_bits(src), to_bits(before))
        assert_bits_equal(dst, want.reshape(dst.shape), f"store atomic={kind} {dtype}")
    out = torch.zeros(9, 1000, dtype=dtype, device="cuda")
    bsir.store(src, out)                                         # atomic none: a copy
    assert torch.equal(out.view(torch.uint8), src.view(torch.uint8))
    with pytest.raises(bsir.BsirError):
        bsir.store(src, out, atomic="cas")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_load_and_atomic_add_on_row_strided_views(bsir, dtype):
    """Rows of wider tensors on both sides (16-byte aligned: the vector kernels) and from an odd column (the element
    kernels): a padded load and an adding store, against the oracle; nothing outside the views changes."""
    src_wide = _rand((50, 640), dtype, seed=11)
    for c0 in (64, 3):
        src = src_wide[:, c0:c0 + 256]
        dst_wide = _rand((50, 512), dtype, seed=12)
        before = dst_wide.clone()
        bsir.load(src, dst_wide[:, 128:448], pad_mode="value", pad_value=1.5, left_padding_num=32, right_padding_num=32)
        want = O.load_pad(oracle_dtype(src), to_bits(src.contiguous()), to_bits(before[:, 128:448].contiguous()), "value",
                          to_bits(torch.tensor([1.5], dtype=dtype)), 32, 32)
        assert_bits_equal(dst_wide[:, 128:448].contiguous(), want.reshape(50, 320), f"strided load from column {c0}")
        assert torch.equal(dst_wide[:, :128], before[:, :128]) and torch.equal(dst_wide[:, 448:], before[:, 448:])
        acc_wide = _rand((50, 512), dtype, seed=13)
        before = acc_wide.clone()
        bsir.store(src, acc_wide[:, 64:320], atomic="add")
        want = O.store_atomic(oracle_dtype(src), "add", to_bits(src.contiguous()), to_bits(before[:, 64:320].contiguous()))
        assert_bits_equal(acc_wide[:, 64:320].contiguous(), want.reshape(50, 256), f"strided adding store from column {c0}")
        assert torch.equal(acc_wide[:, :64], before[:, :64]) and torch.equal(acc_wide[:, 320:], before[:, 320:])


def test_store_atomic_adds_up_over_calls(bsir):
    acc = torch.zeros(4, 257, dtype=torch.int32, device="cuda")
    parts = [torch.randint(-100, 100, (4, 257), dtype=torch.int32, device="cuda") for _ in range(5)]
    for p in parts:
        bsir.store(p, acc, atomic="add")
    assert torch.equal(acc, sum(parts))


# ---------------------------------------------------------------- transposition (a copy from a transposed view)
@pytest.mark.parametrize("dtype", [torch.int8, torch.bfloat16, torch.float32, torch.int64])
@pytest.mark.parametrize("shape", [(64, 128), (256, 512), (1000, 72), (65, 33), (3, 200, 136), (2, 64, 64), (1, 7), (513, 1024)])
def test_transpose_of_the_last_two_axes(bsir, dtype, shape):
    """Bit-exact against the permutation itself: full tiles, ragged edges, batches, every element size."""
    g = torch.Generator(device="cuda").manual_seed(sum(shape))
    x = torch.randint(-2 ** 15, 2 ** 15, shape, device="cuda", generator=g).to(dtype) if not dtype.is_floating_point \
        else torch.randn(shape, device="cuda", generator=g).to(dtype)
    y = bsir.transpose(x)
    assert y.shape == x.transpose(-1, -2).shape and y.is_contiguous()
    assert torch.equal(y, x.transpose(-1, -2))


def test_transpose_with_row_strides_and_unaligned_views(bsir):
    big = torch.randn(300, 700, device="cuda").to(torch.float16)
    x = big[4:260, 8:520]                                       # 256 x 512, row stride 700 (16-byte aligned rows)
    out_big = torch.zeros(600, 400, device="cuda", dtype=torch.float16)
    out = out_big[:512, 16:272]
    bsir.transpose(x, out=out)
    assert torch.equal(out, x.t())
    assert out_big[:, :16].abs().sum().item() == 0 and out_big[:, 272:].abs().sum().item() == 0 and out_big[512:].abs().sum().item() == 0
    odd = big[1:258, 3:200]                                     # unaligned start, odd sizes: the element path
    assert torch.equal(bsir.transpose(odd), odd.t())


# ---------------------------------------------------------------- gather along an axis
@pytest.mark.parametrize("dtype", [torch.int8, torch.float16, torch.float32, torch.int64])
@pytest.mark.parametrize("idx_dtype", [torch.int16, torch.int32, torch.int64])
@pytest.mark.parametrize("shape,dim,n", [((100, 7, 4), 1, 6), ((512,), 0, 300), ((33, 1000), 1, 17), ((50, 9), 0, 64), ((2, 3, 5, 8), 2, 11)])
def test_gather_along_an_axis(bsir, dtype, idx_dtype, shape, dim, n):
    """hivm.hir.vgather: bit-exact against the indexing rule itself (the [100,7,4] -> [100,6,4] case is the one of
    test/Dialect/HIVM/hivm-flatten-ops.mlir:1036-1045)."""
    g = torch.Generator(device="cuda").manual_seed(n)
    x = torch.randint(-100, 100, shape, device="cuda", generator=g).to(dtype)
    ishape = list(shape)
    ishape[dim] = n
    idx = torch.randint(0, shape[dim], ishape, device="cuda", generator=g).to(idx_dtype)
    y = bsir.gather(x, idx, dim=dim)
    assert torch.equal(y, torch.gather(x, dim, idx.long()))
    assert bsir.device_error() == 0


def test_gather_reports_indices_outside_the_axis(bsir):
    x = torch.arange(10, device="cuda", dtype=torch.float32)
    idx = torch.tensor([0, 9, 10, -1, 3], device="cuda", dtype=torch.int32)
    out = torch.full((5,), -7.0, device="cuda")
    bsir.gather(x, idx, out=out)
    assert bsir.device_error() == 0x100                          # BSIR_DEVERR_GATHER_INDEX
    assert out.tolist() == [0.0, 9.0, -7.0, -7.0, 3.0]           # the bad ones are left untouched
    assert bsir.device_error() == 0                              # reading clears it


@pytest.mark.parametrize("dtype", [torch.int8, torch.bfloat16, torch.float32, torch.int64])
@pytest.mark.parametrize("idx_dtype", [torch.int16, torch.int32, torch.int64])
@pytest.mark.parametrize("rows,axis,n", [(5, 3000, 5000), (300, 4096, 4096), (3, 6144, 100), (2, 6145, 70), (700, 129, 64)])
def test_gather_along_the_last_axis_from_rows_in_shared_memory(bsir, dtype, idx_dtype, rows, axis, n):
    """Source rows of up to 48 KB are staged in shared memory (6144 int64 = 48 KB: the largest; 6145: the general kernel
    again); few rows share their destination row out over several CTAs; bad indices leave their elements alone."""
    g = torch.Generator(device="cuda").manual_seed(n + axis)
    x = torch.randint(-100, 100, (rows, axis), device="cuda", generator=g).to(dtype)
    idx = torch.randint(0, axis, (rows, n), device="cuda", generator=g).to(idx_dtype)
    y = bsir.gather(x, idx, dim=1)
    assert torch.equal(y, torch.gather(x, 1, idx.long()))
    assert bsir.device_error() == 0
    idx[0, 3] = -1
    idx[rows - 1, n - 1] = axis
    out = torch.full((rows, n), 77, device="cuda").to(dtype)
    bsir.gather(x, idx, dim=1, out=out)
    assert bsir.device_error() == 0x100
    want = torch.gather(x, 1, idx.long().clamp(0, axis - 1))
    want[0, 3] = 77
    want[rows - 1, n - 1] = 77
    assert torch.equal(out, want)


# ---------------------------------------------------------------- varange, vinterleave, vdeinterleave
def test_arange_example_of_the_op_definition(bsir):
    """HIVMVectorOps.td:1518-1522: offset 1, strides [1, 2], shape 2x4 -> [[1, 3, 5, 7], [2, 4, 6, 8]]."""
    y = bsir.arange([2, 4], [1, 2], offset=1, dtype=torch.int32)
    assert y.tolist() == [[1, 3, 5, 7], [2, 4, 6, 8]]


@pytest.mark.parametrize("dtype", [torch.int16, torch.int32, torch.int64, torch.float16, torch.float32])
@pytest.mark.parametrize("shape,strides,offset", [((1000,), (3,), -7), ((17, 33), (100, 1), 5), ((4, 5, 6), (30, 6, 1), 0)])
def test_arange_shapes_and_types(bsir, dtype, shape, strides, offset):
    y = bsir.arange(shape, strides, offset=offset, dtype=dtype)
    want = torch.full(shape, offset, dtype=torch.int64, device="cuda")
    for d, (n, s) in enumerate(zip(shape, strides)):
        view = [1] * len(shape)
        view[d] = n
        want = want + (torch.arange(n, device="cuda") * s).view(view)
    assert torch.equal(y, want.to(dtype))


@pytest.mark.parametrize("dtype", [torch.int8, torch.bfloat16, torch.float32, torch.int64])
@pytest.mark.parametrize("channels", [1, 2, 3, 8])
@pytest.mark.parametrize("shape", [(64, 128), (7, 33), (1, 1000), (2, 5, 16)])
def test_interleave_and_deinterleave_are_inverse_bit_moves(bsir, dtype, channels, shape):
    g = torch.Generator(device="cuda").manual_seed(channels)
    srcs = [torch.randint(-100, 100, shape, device="cuda", generator=g).to(dtype) for _ in range(channels)]
    y = bsir.interleave(srcs)
    assert torch.equal(y, torch.stack(srcs, dim=-1).reshape(*shape[:-1], shape[-1] * channels))
    back = bsir.deinterleave(y, channels)
    assert all(torch.equal(b, s) for b, s in zip(back, srcs))
    only = bsir.deinterleave(y, channels, keep=[channels - 1])
    assert torch.equal(only[channels - 1], srcs[-1]) and all(o is None for o in only[:-1])


@pytest.mark.parametrize("dtype", [torch.int8, torch.float16, torch.float32])
def test_interleave_two_channels_at_any_alignment(bsir, dtype):
    """Two channels take 16-byte vectors when every operand is 16-byte aligned; operands that start on an odd element
    take the element path.  Both must move the same bits."""
    n = 100003
    g = torch.Generator(device="cuda").manual_seed(3)
    pool = [torch.randint(-100, 100, (n + 8,), device="cuda", generator=g).to(dtype) for _ in range(2)]
    for off in (0, 1, 3):
        a, b = pool[0][off:off + n], pool[1][off:off + n]
        y = bsir.interleave([a, b])
        assert torch.equal(y, torch.stack([a, b], dim=-1).reshape(-1))
        src = torch.zeros(2 * n + 8, device="cuda", dtype=dtype)
        src[off:off + 2 * n] = y
        back = bsir.deinterleave(src[off:off + 2 * n], 2)
        assert torch.equal(back[0], a) and torch.equal(back[1], b)


def _in_fresh_thread(fn):
    """Runs fn in a new thread and returns (its result, the fused-chain path that thread used: "none" when the chain
    executor, and with it the runtime compiler, was never entered)."""
    import threading
    box = {}

    def run():
        try:
            box["out"] = fn()
        except BaseException as e:                                   # noqa: BLE001 - re-raised in the caller's thread
            box["err"] = e
        box["path"] = bsir_mod().FusedChain.last_path()
    t = threading.Thread(target=run)
    t.start()
    t.join()
    if "err" in box:
        raise box["err"]
    return box["out"], box["path"]


def bsir_mod():
    import bsir
    return bsir


def test_broadcast_binary_ops_use_the_precompiled_vector_kernel(bsir):
    """A binary op with a per-column or per-row operand (hivm's inline broadcast), an immediate or an in-memory scalar
    runs the library's own 16-byte-vector kernel: no fused-chain call, no runtime compiler.  Bits as the oracle's;
    ragged rows still go to the indexed kernel."""
    x = torch.randn(300, 1024, device="cuda").to(torch.bfloat16)
    bias = torch.randn(1024, device="cuda").to(torch.bfloat16)
    scale = (torch.rand(300, 1, device="cuda") + 0.5).to(torch.bfloat16)
    one = torch.full((1, 1), 1.5, device="cuda", dtype=torch.bfloat16)
    for fn, other in (("add", bias.view(1, -1).expand(300, 1024)), ("mul", scale.expand(300, 1024)), ("sub", bias.view(1, -1).expand(300, 1024)),
                      ("div", one.expand(300, 1024)), ("maxf", scale.expand(300, 1024)), ("powf", one.expand(300, 1024))):
        y, path = _in_fresh_thread(lambda: bsir.elemwise_binary(fn, x, other))
        assert path == "none"
        want = O.elemwise_binary(fn, O.BF16, to_bits(x), to_bits(other.contiguous()))
        assert_bits_equal(y, want, f"broadcast {fn}")
        z = bsir.elemwise_binary(fn, other, x)                     # the broadcast operand on the left
        assert_bits_equal(z, O.elemwise_binary(fn, O.BF16, to_bits(other.contiguous()), to_bits(x)), f"broadcast r{fn}")
    # row vector against column vector: both operands broadcast
    outer = bsir.elemwise_binary("mul", bias.view(1, -1).expand(300, 1024), scale.expand(300, 1024))
    assert_bits_equal(outer, O.elemwise_binary("mul", O.BF16, to_bits(bias.view(1, -1).expand(300, 1024).contiguous()),
                                               to_bits(scale.expand(300, 1024).contiguous())), "outer mul")
    # f32 and integers take the same kernel
    xf = torch.randn(64, 260, device="cuda")
    bf = torch.randn(260, device="cuda")
    assert_bits_equal(bsir.elemwise_binary("add", xf, bf.view(1, -1).expand(64, 260)),
                      O.elemwise_binary("add", O.F32, to_bits(xf), to_bits(bf.view(1, -1).expand(64, 260).contiguous())), "f32 bias")
    xi = torch.randint(-1000, 1000, (70, 64), device="cuda", dtype=torch.int32)
    ci = torch.randint(-1000, 1000, (70, 1), device="cuda", dtype=torch.int32)
    for fn in ("add", "mul", "max_signed"):
        assert torch.equal(bsir.elemwise_binary(fn, xi, ci.expand(70, 64)).cpu(),
                           torch.from_numpy(O.elemwise_binary(fn, O.I32, xi.cpu().numpy(), ci.expand(70, 64).contiguous().cpu().numpy())))
    ragged = torch.randn(50, 1001, device="cuda")
    rb = torch.randn(1001, device="cuda").view(1, -1).expand(50, 1001)
    assert_bits_equal(bsir.elemwise_binary("add", ragged, rb), O.elemwise_binary("add", O.F32, to_bits(ragged), to_bits(rb.contiguous())), "ragged")


def test_row_strided_views_use_the_precompiled_vector_kernel(bsir):
    """Slices of wider tensors (row stride > row length, 16-byte aligned rows) as operands and as the result."""
    big_a = torch.randn(200, 512, device="cuda").to(torch.float16)
    big_b = torch.randn(200, 640, device="cuda").to(torch.float16)
    a, b = big_a[:, 64:320], big_b[:, 128:384]                     # 256 columns each
    out_big = torch.zeros(200, 400, device="cuda", dtype=torch.float16)
    out = out_big[:, 8:264]
    _, path = _in_fresh_thread(lambda: bsir.elemwise_binary("mul", a, b, out=out))
    assert path == "none"
    assert_bits_equal(out.contiguous(), O.elemwise_binary("mul", O.F16, to_bits(a.contiguous()), to_bits(b.contiguous())), "strided mul")
    assert out_big[:, :8].abs().sum().item() == 0 and out_big[:, 264:].abs().sum().item() == 0
    y, path = _in_fresh_thread(lambda: bsir.elemwise_unary("exp", a))
    assert path == "none"
    assert_bits_equal(y, O.elemwise_unary("exp", O.F16, to_bits(a.contiguous())), "strided exp")
    z = bsir.elemwise_binary("add", a, 2.5)                         # strided tensor and an immediate
    assert_bits_equal(z, O.elemwise_binary("add", O.F16, to_bits(a.contiguous()), to_bits(torch.full_like(a, 2.5).contiguous())), "strided + imm")
    odd = big_a[:, 3:259]                                          # rows not 16-byte aligned: the indexed kernel
    assert_bits_equal(bsir.elemwise_unary("abs", odd), O.elemwise_unary("abs", O.F16, to_bits(odd.contiguous())), "unaligned abs")


# ---------------------------------------------------------------- elemwise_ternary {fma}, unary ilogb
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1 << 16,), (33, 100), (5, 7, 64), (3, 1000)])
def test_ternary_fma_bit_exact(bsir, dtype, shape):
    """math.fma: one rounding of a * b + c (then the storage rounding of 16-bit types), against the oracle's fmaf."""
    g = torch.Generator(device="cuda").manual_seed(len(shape) * 7 + shape[-1])
    a, b, c = (torch.randn(shape, generator=g, device="cuda").to(dtype) for _ in range(3))
    out = bsir.elemwise_ternary("fma", a, b, c)
    want = O.elemwise_fma(oracle_dtype(a), to_bits(a), to_bits(b), to_bits(c))
    assert_bits_equal(out, want, f"fma {dtype} {shape}")


@pytest.mark.parametrize("dtype", [torch.int8, torch.bfloat16, torch.float32, torch.int64])
def test_copies_of_strided_and_broadcast_views(bsir, dtype):
    """Slices of a wider tensor, destinations with padded rows, and broadcasts of a row, a column and one element
    (hivm.hir.vbrc arrives as a copy from a stride-0 view) move 16-byte vectors; ragged or misaligned rows take the
    element kernel.  Same bits either way, nothing outside the destination's rows."""
    g = torch.Generator(device="cuda").manual_seed(9)
    wide = torch.randint(-100, 100, (300, 512), device="cuda", generator=g).to(dtype)
    for view in (wide[:, 64:320], wide[:, 3:200], wide[5:6].expand(300, 512), wide[:, 7:8].expand(300, 512),
                 wide[2:3, 9:10].expand(300, 512), wide[:, 64:320].reshape(10, 30, 256)):
        assert torch.equal(bsir.copy(view), view.contiguous())
    padded = torch.full((300, 600), 55, device="cuda").to(dtype)
    bsir.copy(wide, out=padded[:, 16:528])
    assert torch.equal(padded[:, 16:528], wide)
    assert (padded[:, :16] == 55).all() and (padded[:, 528:] == 55).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
def test_broadcasts_over_three_axes_take_the_vector_kernel(bsir, dtype):
    """[n0, n1, cols] against [n0, 1, cols], [1, n1, cols], [n0, 1, 1], [1, n1, 1], [n0, n1, 1], a strided column of a
    wider tensor, and a batch-padded full operand: the operand's outer and row strides (either may be 0) go into the
    kernel; results are the element kernel's bits."""
    g = torch.Generator(device="cuda").manual_seed(4)
    mk = (lambda *sh: torch.randint(-50, 50, sh, device="cuda", generator=g).to(dtype))
    x = mk(6, 40, 256)
    fn, tf = ("add", torch.add) if dtype == torch.int32 else ("mul", torch.mul)
    for other in (mk(6, 1, 256), mk(1, 40, 256), mk(6, 1, 1), mk(1, 40, 1), mk(6, 40, 1), mk(1, 1, 256), mk(1, 1, 1),
                  mk(6, 40, 300)[:, :, 7:8], mk(6, 64, 256)[:, :40, :], mk(8, 40, 512)[1:7, :, 256:]):
        want = tf(x, other.expand_as(x) if other.shape != x.shape else other)
        assert torch.equal(bsir.elemwise_binary(fn, x, other.expand_as(x)), want), f"{tuple(other.shape)} {other.stride()}"
        assert torch.equal(bsir.elemwise_binary(fn, other.expand_as(x), x), want), f"{tuple(other.shape)} first"
    rowv, colv = mk(1, 1, 256), mk(6, 40, 1)                    # two broadcast operands: an outer sum
    want = tf(rowv.expand_as(x), colv.expand_as(x))
    assert torch.equal(bsir.elemwise_binary(fn, rowv.expand_as(x), colv.expand_as(x)), want)
    assert torch.equal(bsir.elemwise_binary(fn, colv.expand_as(x), rowv.expand_as(x)), want)
    r3, c3 = mk(6, 1, 256), mk(1, 40, 1)                        # the same with an outer index on the row vector
    assert torch.equal(bsir.elemwise_binary(fn, r3.expand_as(x), c3.expand_as(x)), tf(r3.expand_as(x), c3.expand_as(x)))
    wide = mk(240, 512)
    col = wide[:, 5:6]                                          # one value per row, 512 elements apart
    y = mk(240, 256)
    assert torch.equal(bsir.elemwise_binary(fn, y, col.expand_as(y)), tf(y, col))
    out = torch.zeros(6, 48, 256, device="cuda").to(dtype)      # a result with padded outer stride
    bsir.elemwise_binary(fn, x, mk(6, 1, 256).expand_as(x), out=out[:, :40, :])
    assert (out[:, 40:, :] == 0).all()


def test_unary_ops_on_broadcast_operands(bsir):
    x = torch.randn(200, 256, device="cuda")
    for view in (x[3:4].expand(200, 256), x[:, 5:6].expand(200, 256), x[1:2, 2:3].expand(200, 256)):
        for dt in (torch.float32, torch.bfloat16):
            v = view.to(dt) if dt == torch.float32 else view.to(dt)
            got = bsir.elemwise_unary("abs", v)
            assert torch.equal(got, v.contiguous().abs())


def test_ternary_fma_scalars_broadcasts_and_views(bsir):
    g = torch.Generator(device="cuda").manual_seed(2)
    a = torch.randn(40, 96, generator=g, device="cuda")
    row = torch.randn(1, 96, generator=g, device="cuda")
    col = torch.randn(40, 1, generator=g, device="cuda")
    out = bsir.elemwise_ternary("fma", a, row, col)                       # inline broadcasts (stride 0)
    ref = O.elemwise_fma(O.F32, a.cpu().numpy(), row.expand(40, 96).contiguous().cpu().numpy(), col.expand(40, 96).contiguous().cpu().numpy())
    assert np.array_equal(out.cpu().numpy(), ref)
    out = bsir.elemwise_ternary("fma", a, 2.5, -1.25)                     # scalar operands
    ref = O.elemwise_fma(O.F32, a.cpu().numpy(), np.array([2.5], np.float32), np.array([-1.25], np.float32))
    assert np.array_equal(out.cpu().numpy(), ref)
    view = torch.randn(40, 200, generator=g, device="cuda")[:, 3:99]       # strided, unaligned view
    out = bsir.elemwise_ternary("fma", view, a, a)
    ref = O.elemwise_fma(O.F32, view.contiguous().cpu().numpy(), a.cpu().numpy(), a.cpu().numpy())
    assert np.array_equal(out.cpu().numpy(), ref)
    with pytest.raises(bsir.BsirError):
        bsir.elemwise_ternary("fma", a.to(torch.int32), a.to(torch.int32), a.to(torch.int32))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_unary_ilogb(bsir, dtype):
    """ilogb(x) = floor(log2(|x|)) (Normalize.cpp:6782-6830): the exponent, -inf at zero, +inf at infinities, NaN kept."""
    x = torch.tensor([1.0, 1.5, 2.0, 3.99, 4.0, 0.75, -0.3, 1e-3, 1000.0, 0.0, -0.0, float("inf"), -float("inf"), float("nan"), 6e-8, 255.0],
                     device="cuda").to(dtype)
    out = bsir.elemwise_unary("ilogb", x)
    want = O.elemwise_unary("ilogb", oracle_dtype(x), to_bits(x))
    assert_bits_equal(out, want, f"ilogb {dtype}")
    f = out.float().cpu().numpy()
    assert f[:5].tolist() == [0.0, 0.0, 1.0, 1.0, 2.0] and f[9] == -np.inf and f[11] == np.inf and np.isnan(f[13])
    big = (torch.randn(1 << 16, device="cuda") * 100).to(dtype)
    assert_bits_equal(bsir.elemwise_unary("ilogb", big), O.elemwise_unary("ilogb", oracle_dtype(big), to_bits(big)), "ilogb random")
