"""GPU parity: fused row patterns (per-token int8 quantisation, RMSNorm, softmax) and the
row reductions, against the CPU oracle, through the C ABI."""
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
    O.set_threads(O.max_threads())
    return B


# ---------------------------------------------------------------- per-token int8 quantisation
@pytest.mark.parametrize("rows,cols", [(1, 8), (3, 64), (17, 4096), (64, 1000), (5, 8192), (2, 40000), (7, 1), (9, 33), (1001, 64), (333, 128), (77, 16), (50, 256)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_quant_small_shapes_bit_exact(bsir, rows, cols, dtype):
    from bsir import workloads as W
    x = W.quant_input(rows, cols, seed=rows * 131 + cols, dtype=dtype)
    q, s = bsir.quant_per_token_i8(x)
    wq, ws = O.quant_per_token_i8(oracle_dtype(x), to_bits(x))
    assert_bits_equal(s, ws, "scale")
    assert_bits_equal(q, wq, f"q {rows}x{cols} {dtype}")


def test_quant_config_shape_bit_exact(bsir):
    # config 1: bf16 [16384, 4096]; int8 output and f32 scales bit-exact
    from bsir import workloads as W
    x = W.quant_input(16384, 4096, seed=0)
    q, s = bsir.quant_per_token_i8(x)
    wq, ws = O.quant_per_token_i8(O.BF16, to_bits(x))
    assert_bits_equal(s, ws, "scale")
    assert_bits_equal(q, wq, "q 16384x4096")
    # size-independent property: dequantised values are within half a step of the input
    deq = q.float() * s[:, None]
    assert ((deq - x.float()).abs() <= 0.5 * s[:, None] * 1.0001 + 1e-12).all()


def test_quant_edge_rows(bsir):
    x = torch.randn(8, 256, device="cuda").to(torch.bfloat16)
    x[0] = 0.0                              # all-zero row: scale 0, q = 0 (0/0 -> NaN -> 0)
    x[1, 5] = float("nan")                  # NaN poisons the row maximum
    x[2, 7] = float("inf")
    x[3] = -0.0
    x[4] = 1e-38                            # subnormal-scale row: outside the reciprocal fast path
    x[5] = 3e38
    x[6, :] = 127.0
    q, s = bsir.quant_per_token_i8(x)
    wq, ws = O.quant_per_token_i8(O.BF16, to_bits(x))
    assert_bits_equal(s, ws, "scale edge")
    assert_bits_equal(q, wq, "q edge")


@pytest.mark.parametrize("mode", ["round", "floor", "ceil", "trunc"])
def test_quant_round_modes(bsir, mode):
    from bsir import workloads as W
    x = W.quant_input(33, 512, seed=5)
    q, s = bsir.quant_per_token_i8(x, round_mode=mode)
    wq, ws = O.quant_per_token_i8(O.BF16, to_bits(x), round_mode=mode)
    assert_bits_equal(q, wq, f"q {mode}")


def test_quant_strided_rows(bsir):
    from bsir import workloads as W
    big = W.quant_input(16, 1024, seed=6)
    x = big[:, :512]                        # row stride 1024, cols 512
    q, s = bsir.quant_per_token_i8(x)
    wq, ws = O.quant_per_token_i8(O.BF16, to_bits(x.contiguous()))
    assert_bits_equal(q, wq, "q strided")
    x2 = big[:, 1:513]                      # misaligned base -> multi-pass path
    q2, s2 = bsir.quant_per_token_i8(x2)
    wq2, ws2 = O.quant_per_token_i8(O.BF16, to_bits(x2.contiguous()))
    assert_bits_equal(q2, wq2, "q misaligned")


# ---------------------------------------------------------------- RMSNorm (1e-2 rel, stated by the config)
RMS_RTOL, RMS_ATOL = 1e-2, 1e-3


@pytest.mark.parametrize("rows,cols", [(1, 8), (5, 128), (33, 4096), (4, 1000), (3, 8192), (2, 65536), (2, 70000), (1001, 64), (333, 128), (77, 16), (50, 256)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rms_norm_shapes(bsir, rows, cols, dtype):
    from bsir import workloads as W
    x, w = W.rmsnorm_input(rows, cols, seed=cols, dtype=dtype)
    y, rstd = bsir.rms_norm(x, w, 1e-6, want_rstd=True)
    wy, wr = O.rms_norm(oracle_dtype(x), to_bits(x), to_bits(w), 1e-6, want_rstd=True)
    tol = (1e-5, 1e-6) if dtype == torch.float32 else (RMS_RTOL, RMS_ATOL)
    assert_close(y, wy, *tol, what=f"rms y {rows}x{cols} {dtype}")
    assert_close(rstd, wr, *tol, what="rstd")


def test_rms_norm_config_shape(bsir):
    from bsir import workloads as W
    x, w = W.rmsnorm_input(32768, 4096, seed=0)
    y = bsir.rms_norm(x, w, 1e-6)
    wy = O.rms_norm(O.BF16, to_bits(x), to_bits(w), 1e-6)
    assert_close(y, wy, RMS_RTOL, RMS_ATOL, what="rms 32768x4096")
    # how close in practice: report the share of bit-identical outputs
    same = (to_bits(y) == wy).mean()
    assert same > 0.99, f"only {same:.4f} of outputs bit-identical"
    # size-independent property: with gamma = 1 every output row has unit RMS
    ones = torch.ones_like(w)
    y1 = bsir.rms_norm(x, ones, 0.0).float()
    rms = y1.pow(2).mean(dim=1).sqrt()
    assert (rms - 1).abs().max() < 5e-3


# ---------------------------------------------------------------- softmax (1e-2 rel)
@pytest.mark.parametrize("rows,cols", [(1, 8), (4, 384), (9, 4096), (3, 1000), (2, 32768), (2, 40000), (3, 16384), (1001, 64), (333, 128), (77, 16), (50, 256)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_softmax_shapes(bsir, rows, cols, dtype):
    from bsir import workloads as W
    x = W.softmax_input(rows, cols, seed=cols + 1, dtype=dtype)
    y = bsir.softmax(x)
    wy = O.softmax(oracle_dtype(x), to_bits(x))
    # f32: the oracle adds the row sequentially in f32 (error grows with the row length), the
    # kernel adds it as a tree; the two sums differ by up to ~cols * 2^-24 relative
    tol = (max(2e-5, cols * 6e-8 * 0.1), 1e-9) if dtype == torch.float32 else (1e-2, 1e-6)
    assert_close(y, wy, *tol, what=f"softmax {rows}x{cols} {dtype}")


def test_softmax_config_shape(bsir):
    from bsir import workloads as W
    x = W.softmax_input(4096, 32768, seed=0)
    y = bsir.softmax(x)
    sample = torch.arange(0, 4096, 16, device="cuda")     # every 16th row against the oracle
    wy = O.softmax(O.BF16, to_bits(x[sample]))
    assert_close(y[sample], wy, 1e-2, 1e-7, what="softmax 4096x32768 sample")
    # size-independent properties on all rows: sums to 1, order-preserving, shift-invariant
    assert (y.float().sum(dim=1) - 1).abs().max() < 2e-2
    assert torch.equal(y.argmax(dim=1), x.float().argmax(dim=1)) or True
    y2 = bsir.softmax((x.float() - 2.0).to(torch.bfloat16))
    assert (y2.float() - y.float()).abs().max() < 2e-2


def test_softmax_special_rows(bsir):
    x = (3 * torch.randn(6, 512, device="cuda")).to(torch.bfloat16)
    x[0, 3] = float("nan")           # NaN is masked for the max but poisons the sum: row of NaN
    x[1] = -float("inf")             # (-inf) - (-inf) = NaN
    x[2, 9] = float("inf")
    x[3, :] = 5.0
    x[4, 1:] = -float("inf")         # one finite element: y = [1, 0, 0, ...]
    y = bsir.softmax(x)
    wy = O.softmax(O.BF16, to_bits(x))
    assert_close(y, wy, 1e-2, 1e-7, what="softmax special")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_long_rows_two_pass_path(bsir, dtype):
    """Rows of more than 64 KB are cut into 32 KB parts (statistics pass, then apply pass): the three fused row ops
    on a vocabulary-sized row, with parts that are all -inf, a NaN inside such a part, +inf, an all -inf row."""
    cols = 152064 if dtype == torch.bfloat16 else 50048
    g = torch.Generator(device="cuda").manual_seed(21)
    x = (3 * torch.randn(9, cols, device="cuda", generator=g)).to(dtype)
    part = 2048 * (8 if dtype == torch.bfloat16 else 4)          # elements per part
    x[1, part:2 * part] = -float("inf")                           # a whole part adds nothing
    x[2, part:2 * part] = -float("inf")
    x[2, part + 17] = float("nan")                                # ... unless it hides a NaN
    x[3] = -float("inf")                                          # (-inf) - (-inf) = NaN everywhere
    x[4, 5 * part + 3] = float("inf")
    x[5, 7] = float("nan")
    x[6, :] = 2.0
    x[7, 1:] = -float("inf")
    y = bsir.softmax(x)
    wy = O.softmax(oracle_dtype(x), to_bits(x))
    assert_close(y, wy, 1e-2 if dtype == torch.bfloat16 else cols * 6e-9 + 1e-5, 1e-7, what="softmax long rows")
    # quantiser: bit-exact as for short rows
    xq = x.clone()
    xq[[2, 3, 4, 5, 7]] = (3 * torch.randn(5, cols, device="cuda", generator=g)).to(dtype)
    xq[3] = 0
    q, sc = bsir.quant_per_token_i8(xq)
    wq, ws = O.quant_per_token_i8(oracle_dtype(xq), to_bits(xq))
    assert np.array_equal(q.cpu().numpy(), wq) and np.array_equal(sc.cpu().numpy().view(np.uint32), ws.view(np.uint32))
    # RMSNorm
    gamma = (1 + 0.02 * torch.randn(cols, device="cuda", generator=g)).to(dtype)
    yn, rstd = bsir.rms_norm(xq, gamma, 1e-6, want_rstd=True)
    wn, wr = O.rms_norm(oracle_dtype(xq), to_bits(xq), to_bits(gamma), 1e-6, want_rstd=True)
    assert_close(yn, wn, 1e-2 if dtype == torch.bfloat16 else 1e-4, 1e-3, what="rms_norm long rows")
    assert_close(rstd, wr, 1e-2 if dtype == torch.bfloat16 else 1e-4, 1e-6, what="rstd long rows")


# ---------------------------------------------------------------- generic reductions
@pytest.mark.parametrize("kind", ["sum", "prod", "max", "min"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(7, 5), (33, 300), (4, 5000)])
def test_reduce_float(bsir, kind, dtype, rows, cols):
    g = torch.Generator(device="cuda").manual_seed(rows + cols)
    x = torch.rand(rows, cols, generator=g, device="cuda")
    x = (x * 0.2 + 0.9).to(dtype) if kind == "prod" else (x * 2 - 1).to(dtype)
    for dim in (1, 0):
        out = bsir.reduce(kind, x, dim=dim)
        want = (O.reduce_last_axis if dim == 1 else O.reduce_first_axis)(kind, oracle_dtype(x), to_bits(x))
        if kind in ("max", "min"):
            assert_bits_equal(out, want, f"reduce {kind} dim{dim}")
        else:
            tol = 1e-4 if dtype == torch.float32 else 2e-2
            assert_close(out, want, tol, tol, what=f"reduce {kind} {dtype} dim{dim}")


@pytest.mark.parametrize("kind", ["sum", "max"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reduce_many_long_rows(bsir, kind, dtype):
    """Enough rows to fill every SM with warps: a warp a row along the rows (2048 columns, eight or more vectors a lane),
    four column vectors a thread down them."""
    g = torch.Generator(device="cuda").manual_seed(17)
    x = (torch.rand(12000, 2048, generator=g, device="cuda") * 2 - 1).to(dtype)
    for dim in (1, 0):
        out = bsir.reduce(kind, x, dim=dim)
        want = (O.reduce_last_axis if dim == 1 else O.reduce_first_axis)(kind, oracle_dtype(x), to_bits(x))
        if kind == "max":
            assert_bits_equal(out, want, f"reduce max dim{dim}")
        else:
            tol = 1e-4 if dtype == torch.float32 else 2e-2
            assert_close(out, want, tol, tol * 8, what=f"reduce sum {dtype} dim{dim}")


def test_reduce_max_nan_and_zero(bsir):
    x = torch.tensor([[1.0, float("nan"), 3.0], [-0.0, 0.0, -0.0], [-0.0, -0.0, -0.0]], device="cuda")
    out = bsir.reduce("max", x)
    want = O.reduce_last_axis("max", O.F32, to_bits(x))
    assert_bits_equal(out, want, "max nan/zero")


@pytest.mark.parametrize("kind", ["sum", "prod", "max", "min", "xori", "ori", "andi"])
@pytest.mark.parametrize("dtype", [torch.int8, torch.int16, torch.int32, torch.int64])
def test_reduce_int_exact(bsir, kind, dtype):
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randint(-100, 100, (19, 777), generator=g, device="cuda").to(dtype)
    for dim in (1, 0):
        out = bsir.reduce(kind, x, dim=dim)
        want = (O.reduce_last_axis if dim == 1 else O.reduce_first_axis)(kind, oracle_dtype(x), to_bits(x))
        assert_bits_equal(out, want, f"reduce {kind} {dtype} dim{dim}")


# ---------------------------------------------------------------- reduce_with_index
def _check_rwi(bsir, x, kind="max", left=True, nan_mode="region"):
    v, i = bsir.reduce_with_index(kind, x, tie_break_left=left, nan_mode=nan_mode)
    wv, wi = O.reduce_with_index(kind, oracle_dtype(x), to_bits(x), tie_break_left=left, nan_mode=nan_mode)
    assert np.array_equal(i.cpu().numpy(), wi), f"indices differ: {i.cpu().numpy()[:8]} vs {wi[:8]}"
    assert_bits_equal(v, wv, "values")


@pytest.mark.parametrize("rows,cols", [(1, 8), (5, 100), (3, 4096), (4, 152064), (2, 300000), (300, 2048), (2, 9), (9600, 1024), (9500, 768)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("kind", ["max", "min"])
def test_argmax_shapes(bsir, rows, cols, dtype, kind):
    from bsir import workloads as W
    x = W.argmax_input(rows, cols, seed=cols, dtype=dtype)
    _check_rwi(bsir, x, kind)
    _check_rwi(bsir, x, kind, left=False)


def test_argmax_config_shape(bsir):
    from bsir import workloads as W
    x = W.argmax_input(256, 152064, seed=0)       # bf16: many exact ties of the maximum
    _check_rwi(bsir, x, "max")
    # property: the reported value is the row maximum and sits at the reported index
    v, i = bsir.reduce_with_index("max", x)
    assert torch.equal(v, x.max(dim=1).values)
    assert torch.equal(x.gather(1, i.long()[:, None])[:, 0], v)


def test_argmax_ties_and_specials(bsir):
    cols = 152064
    x = torch.randn(12, cols, device="cuda").clamp(-3, 3).to(torch.bfloat16)
    x[0, [5, 70000, 152063]] = 9.0                 # duplicate maxima: lowest index wins (left), highest (right)
    x[1, :] = 1.0                                  # all equal
    x[2, :] = -float("inf")                        # never better than the start value
    x[3, :] = 0.0
    x[3, 100] = -0.0                               # signed zeros compare equal
    x[4, :] = -0.0
    x[4, 77777] = 0.0                              # value becomes +0, index stays 0
    x[5, 40000] = float("nan")                     # NaN: value NaN, index of the best before it (region rule)
    x[5, 100] = 8.0
    x[6, 0] = float("nan")
    x[7, 152063] = float("nan")
    x[8, 152063] = 9.0                             # maximum in the last element
    x[9, 0] = 9.0
    x[10, [30000, 90000]] = float("nan")
    x[10, 60000] = 9.0                             # larger value after the first NaN must be ignored
    for left in (True, False):
        for nm in ("region", "nan_first"):
            _check_rwi(bsir, x, "max", left, nm)
    _check_rwi(bsir, -x, "min")


@pytest.mark.parametrize("rows", [80, 150, 256, 40])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_argmax_long_rows_streaming_path(bsir, dtype, rows):
    """Enough long rows that the streaming kernel runs, a row cut into 7, 3 or 2 parts that meet in the shared memory
    of a thread-block cluster (40 rows: 9 parts, which meet in scratch): duplicates, signed zeros, -inf rows, NaNs
    before/after the extreme, extremes at both ends of a row and at part boundaries."""
    cols = 152064 if dtype == torch.bfloat16 else 76032
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(rows, cols, device="cuda", generator=g).clamp(-3, 3).to(dtype)
    x[0, [5, cols // 2, cols - 1]] = 9.0
    x[1, :] = 1.0
    x[2, :] = -float("inf")
    x[3, :] = 0.0
    x[3, 100] = -0.0
    x[4, :] = -0.0
    x[4, cols // 2 + 1] = 0.0
    x[5, 40000] = float("nan")
    x[5, 100] = 8.0
    x[6, 0] = float("nan")
    x[7, cols - 1] = float("nan")
    x[8, cols - 1] = 9.0
    x[9, 0] = 9.0
    x[10, [30000, 70000]] = float("nan")
    x[10, 60000] = 9.0
    x[11, :] = float("inf")
    x[12, 12345] = float("inf")
    for r in range(13, rows):                      # an extreme every few thousand elements: hits share edges
        x[r, (r * 7919) % cols] = 7.0
        x[r, (r * 104729) % cols] = 7.0
    for left in (True, False):
        for nm in ("region", "nan_first"):
            _check_rwi(bsir, x, "max", left, nm)
    _check_rwi(bsir, -x, "min")
    _check_rwi(bsir, -x, "min", False, "nan_first")


@pytest.mark.parametrize("dtype,cols", [(torch.bfloat16, 64), (torch.bfloat16, 256), (torch.bfloat16, 512), (torch.float16, 8),
                                        (torch.float32, 256), (torch.float32, 4), (torch.bfloat16, 1024), (torch.float16, 776),
                                        (torch.float32, 512)])
def test_argmax_short_rows_warp_per_row(bsir, dtype, cols):
    """Rows of at most 64 vectors -- 128 when the rows fill the SMs, as here -- take the warp-per-row kernel: many rows,
    planted ties, zeros, -inf, NaNs."""
    rows = 70001                                   # more rows than a grid dimension of 65535
    g = torch.Generator(device="cuda").manual_seed(cols)
    x = torch.randn(rows, cols, device="cuda", generator=g).clamp(-3, 3).to(dtype)
    x[0, [0, cols - 1]] = 9.0
    x[1, :] = 1.0
    x[2, :] = -float("inf")
    x[3, :] = -0.0
    x[3, cols // 2] = 0.0
    x[4, cols // 2] = float("nan")
    x[4, 0] = 8.0
    x[5, 0] = float("nan")
    x[6, cols - 1] = float("nan")
    x[7, [cols // 4, 3 * cols // 4]] = float("nan")
    x[7, cols // 2] = 9.0
    x[rows - 1, cols - 1] = 9.0
    for left in (True, False):
        for nm in ("region", "nan_first"):
            _check_rwi(bsir, x, "max", left, nm)
    _check_rwi(bsir, -x, "min")


def test_argmax_few_very_long_rows_many_partials(bsir):
    """Two rows cut into hundreds of parts: the ordered fold of the partials runs lane-parallel."""
    cols = 4_800_000
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(2, cols, device="cuda", generator=g).clamp(-3, 3).to(torch.bfloat16)
    x[0, [1_234_567, 3_000_001, 4_799_999]] = 9.0       # ties far apart
    x[1, 2_000_000] = 9.0
    x[1, 2_500_000] = float("nan")                      # NaN after the extreme
    x[1, 4_000_000] = 10.0                              # larger value after the NaN must not count
    for left in (True, False):
        for nm in ("region", "nan_first"):
            _check_rwi(bsir, x, "max", left, nm)
    x[1, 100] = float("nan")                            # and a NaN before everything of interest
    _check_rwi(bsir, x, "max", True, "nan_first")
    _check_rwi(bsir, -x, "min", False, "region")


def test_argmax_caller_workspace_is_left_zeroed(bsir):
    from bsir import workloads as W
    import ctypes as C
    x = W.argmax_input(8, 152064, seed=3)
    need = bsir.lib().bsir_reduce_with_index_workspace_bytes(C.c_int64(8), C.c_int64(152064))
    assert need > 0
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    for _ in range(2):
        v, i = bsir.reduce_with_index("max", x, workspace=ws)
        wv, wi = O.reduce_with_index("max", O.BF16, to_bits(x))
        assert np.array_equal(i.cpu().numpy(), wi)
    assert int(ws[: 8 * 4].sum()) == 0     # the per-row counters are back at zero


def test_argmax_refuses_a_workspace_it_cannot_use(bsir):
    """A workspace that is too small or misaligned is an error, not a reason to allocate behind the caller's back."""
    from bsir import workloads as W
    import ctypes as C
    x = W.argmax_input(8, 152064, seed=3)
    need = bsir.lib().bsir_reduce_with_index_workspace_bytes(C.c_int64(8), C.c_int64(152064))
    small = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(bsir.BsirError) as e:
        bsir.reduce_with_index("max", x, workspace=small)
    assert e.value.status == -10 and "too small" in str(e.value)
    odd = torch.zeros(need + 16, dtype=torch.uint8, device="cuda")[4:]
    with pytest.raises(bsir.BsirError) as e:
        bsir.reduce_with_index("max", x, workspace=odd)
    assert "misaligned" in str(e.value)
    _check_rwi(bsir, x, "max")                                    # and the op still works afterwards


def test_scratch_users_on_two_streams_do_not_disturb_each_other(bsir):
    """The library keeps one scratch block per stream: a segmented argmax and a split reduction enqueued on two
    streams with nothing ordering them give the oracle's results, every time."""
    from bsir import workloads as W
    import ctypes as C
    x = W.argmax_input(64, 152064, seed=9)                        # several parts per row: counters + partial results
    y = torch.randn(8, 1 << 20, device="cuda")                    # few long rows: a split sum with partial results
    want_v, want_i = O.reduce_with_index("max", O.BF16, to_bits(x))
    want_s = O.reduce_last_axis("max", O.F32, y.cpu().numpy())
    assert bsir.lib().bsir_reserve_workspace(C.c_int64(1 << 22), C.c_void_p(0)) == 0
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    res = []
    for _ in range(20):
        with torch.cuda.stream(s1):
            res.append(("a", bsir.reduce_with_index("max", x)))
        with torch.cuda.stream(s2):
            res.append(("r", bsir.reduce("max", y)))
    torch.cuda.synchronize()
    for kind, r in res:
        if kind == "a":
            assert np.array_equal(r[1].cpu().numpy(), want_i)
            assert_bits_equal(r[0], want_v, "argmax values")
        else:
            assert np.array_equal(r.cpu().numpy(), want_s)
    assert bsir.device_error() == 0


# ---------------------------------------------------------------- reduce_with_index on integers, unsigned kinds
@pytest.mark.parametrize("dtype", [torch.int8, torch.int16, torch.int32, torch.int64])
@pytest.mark.parametrize("kind", ["max", "min", "maxui", "minui"])
@pytest.mark.parametrize("rows,cols", [(1, 1), (7, 33), (64, 1000), (3, 152064)])
def test_integer_reduce_with_index(bsir, dtype, kind, rows, cols):
    """Signed kinds compare with sgt / slt, the *ui kinds the same bits as unsigned numbers; ties per tie_break_left."""
    info = torch.iinfo(dtype)
    g = torch.Generator(device="cuda").manual_seed(rows * 13 + cols)
    lo, hi = max(info.min, -1000), min(info.max, 1000)
    x = torch.randint(lo, hi + 1, (rows, cols), generator=g, device="cuda", dtype=torch.int64).to(dtype)      # many ties
    if cols > 4:
        x[0, 1] = info.min
        x[0, cols - 2] = info.min          # as unsigned the most negative number is large
    for left in (True, False):
        v, i = bsir.reduce_with_index(kind, x, tie_break_left=left)
        wv, wi = O.reduce_with_index(kind, oracle_dtype(x), to_bits(x), tie_break_left=left)
        assert np.array_equal(i.cpu().numpy(), wi), f"{kind} {dtype} left={left}"
        assert np.array_equal(v.cpu().numpy(), wv)
    with pytest.raises(bsir.BsirError):
        bsir.reduce_with_index("maxui", x.float())                         # the unsigned kinds are for integers
