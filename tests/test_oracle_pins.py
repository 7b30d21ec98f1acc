"""CPU: the oracle against every known answer the reference holds for the hot path.

Each case names the reference file:line it restates.  What the reference does NOT pin (it has no
numeric test for softmax, RMSNorm, per-token quantisation or the GEMMs) is checked for internal
consistency in test_oracle_props.py instead."""
import numpy as np
import pytest

import oracle as O


def test_f16_conversions_match_compiler():
    assert O.lib().orc_selftest_f16(500000) == 0


def test_cast_folder_known_answers():
    # bishengir/test/Dialect/HFusion/canonicalize.mlir:149-157: dense<2> : i64 -> dense<2.0> : f32 (default round mode)
    assert O.cast(O.I64, O.F32, np.full(16, 2, np.int64)).tolist() == [2.0] * 16
    # canonicalize.mlir:159-166: same-type f32 cast of 2.8 folds to 3.0 (default rint)
    assert O.cast(O.F32, O.F32, np.full(16, 2.8, np.float32)).tolist() == [3.0] * 16
    # canonicalize.mlir:74-81: i64 1 -> bf16 1.0 under trunc
    assert O.cast(O.I64, O.BF16, np.array([1], np.int64), "trunc").tolist() == [0x3F80]


def test_round_mode_meanings():
    # bishengir/include/bishengir/Dialect/HFusion/IR/HFusionEnums.td:122-141 (rint = ties to even, round = ties
    # away, floor, ceil, trunc, odd); exact results as the folder computes them with
    # APFloat::convertToInteger(rm), bishengir/lib/Dialect/HFusion/IR/HFusionOps.cpp:1951-1994
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 2.3, -2.3, 2.7, -2.7, 3.0], np.float32)
    want = {
        "rint": [0, 2, 2, 0, -2, -2, 2, -2, 3, -3, 3],
        "round": [1, 2, 3, -1, -2, -3, 2, -2, 3, -3, 3],
        "floor": [0, 1, 2, -1, -2, -3, 2, -3, 2, -3, 3],
        "ceil": [1, 2, 3, 0, -1, -2, 3, -2, 3, -2, 3],
        "trunc": [0, 1, 2, 0, -1, -2, 2, -2, 2, -2, 3],
        "odd": [1, 1, 3, -1, -1, -3, 3, -3, 3, -3, 3],
    }
    for mode, w in want.items():
        assert O.cast(O.F32, O.I32, x, mode).tolist() == w, mode


def test_saturate_example_vector():
    # bishengir/lib/Dialect/HFusion/Transforms/Normalize.cpp:3806-3811:
    # [128.7, 127.5, 100.3, -129.2, -128.4] -> [127, 127, 100, -128, -128] (f32 -> f16 trunc -> i8 trunc, saturating)
    x = np.array([128.7, 127.5, 100.3, -129.2, -128.4], np.float32)
    assert O.cast(O.F32, O.I8, x, "rint", "ascend_saturate_trunc_via_f16").tolist() == [127, 127, 100, -128, -128]
    # the attribute semantics (round_mode = rint, enable_saturate) give the same vector here
    assert O.cast(O.F32, O.I8, x, "rint", "saturate").tolist() == [127, 127, 100, -128, -128]
    # enable_saturate = false wraps
    assert O.cast(O.F32, O.I8, x, "rint", "wrap").tolist() == [-127, -128, 100, 127, -128]


def test_double_rounding_variant_differs_only_where_expected():
    # bishengir/lib/Dialect/HIVM/Transforms/HIVMDecomposeOp.cpp:101-127,160-190: f32 -> f16 -> i8, mode applied twice
    x = np.array([2.5 + 2.0 ** -20, 2.5, 3.5, 100.25], np.float32)
    assert O.cast(O.F32, O.I8, x, "rint", "saturate").tolist() == [3, 2, 4, 100]
    assert O.cast(O.F32, O.I8, x, "rint", "ascend_double_round_via_f16").tolist() == [2, 2, 4, 100]


def test_default_round_mode_table():
    # bishengir/unittests/Dialect/Utils/SelectRoundModeTest.cpp:40-78 over
    # bishengir/include/bishengir/Dialect/Utils/Util.h:186-215: float -> int defaults to trunc, all else rint.
    # The oracle takes the mode explicitly; this pins that the two defaults behave as named.
    x = np.array([2.7, -2.7], np.float32)
    assert O.cast(O.F32, O.I16, x, "trunc").tolist() == [2, -2]          # (4-TRUNC) float -> int
    assert O.bf16_to_f32(O.cast(O.F32, O.BF16, np.array([1.00390625], np.float32), "rint")).tolist() == [1.0]   # tie -> even
    assert O.cast(O.I32, O.F32, np.array([16777217], np.int32), "rint").tolist() == [16777216.0]               # (5-RINT)


def test_vecadd_e2e_vector():
    # bishengir/test/Integration/HIVM/VecAdd/main.cpp:141-158 with the expected output of :27-42:
    # in0 = {0..15}, in1 = {1,...,1} (i16, N = 16) -> {1..16}
    a = np.arange(16, dtype=np.int16)
    b = np.ones(16, np.int16)
    assert O.elemwise_binary("add", O.I16, a, b).tolist() == list(range(1, 17))


def test_argmax_combiner_truth_table():
    # bishengir/test/Conversion/LinalgToHFusion/linalg-to-hfusion.mlir:224-241: the Triton combiner that is
    # recognised as reduce_with_index {tie_break_left = true} <max>: take `in` when it is greater, or when
    # it is NaN and the accumulator is not, or on a tie (equal, or both NaN) with the lower index.
    nan = np.nan
    rows = np.array([[1, 3, 3, 2], [3, 1, 3, 0], [1, nan, 5, 0], [nan, 9, 9, 9], [2, 2, 2, 2], [1, 5, nan, nan]], np.float32)
    v, i = O.reduce_with_index("max", O.F32, rows, tie_break_left=True, nan_mode="nan_first")
    assert i.tolist() == [1, 0, 1, 0, 0, 2]
    assert np.isnan(v[2]) and np.isnan(v[3]) and np.isnan(v[5]) and v[0] == 3 and v[4] == 2
    # the op's own region (HFusionOps.cpp:1506-1523): maximumf + strict OGT -> ties keep the first index,
    # a NaN poisons the value and freezes the index
    v, i = O.reduce_with_index("max", O.F32, rows, nan_mode="region")
    assert i.tolist() == [1, 0, 0, 0, 0, 1]
    assert np.isnan(v[2]) and np.isnan(v[3]) and np.isnan(v[5])


def test_compare_predicates_are_ordered_except_vne():
    # bishengir/lib/Dialect/HFusion/IR/HFusionOps.cpp:642-720: OEQ/OLE/OLT/OGE/OGT, vne = UNE
    a = np.array([np.nan, 1.0, 1.0], np.float32)
    b = np.array([1.0, np.nan, 1.0], np.float32)
    assert O.compare("veq", O.F32, a, b).tolist() == [0, 0, 1]
    assert O.compare("vne", O.F32, a, b).tolist() == [1, 1, 0]
    for fn in ("vlt", "vle", "vgt", "vge"):
        assert O.compare(fn, O.F32, a, b).tolist()[:2] == [0, 0]


def test_relu_rec_vnot_bodies():
    # HFusionOps.cpp:495-535: relu = maximumf(0, x) (NaN propagates), rec = 1 / x, vnot = x xor -1
    x = np.array([-1.0, 2.0, np.nan, -0.0], np.float32)
    r = O.elemwise_unary("relu", O.F32, x)
    assert r[0] == 0 and r[1] == 2 and np.isnan(r[2]) and r[3] == 0 and not np.signbit(r[3])
    assert O.elemwise_unary("rec", O.F32, np.array([4.0, -0.5], np.float32)).tolist() == [0.25, -2.0]
    assert O.elemwise_unary("vnot", O.I16, np.array([0, -1, 5], np.int16)).tolist() == [-1, 0, -6]


def test_reduce_identities_and_nan_propagation():
    # init values bishengir/lib/Dialect/HIVM/IR/HIVMVectorOps.cpp:571-640; "min/max propagate NaN"
    # bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:1344
    empty = np.zeros((2, 0), np.float32)
    assert O.reduce_last_axis("sum", O.F32, empty).tolist() == [0, 0]
    assert O.reduce_last_axis("prod", O.F32, empty).tolist() == [1, 1]
    assert O.reduce_last_axis("max", O.F32, empty).tolist() == [-np.inf, -np.inf]
    assert O.reduce_last_axis("min", O.I16, np.zeros((1, 0), np.int16)).tolist() == [32767]
    x = np.array([[1, np.nan, 3]], np.float32)
    assert np.isnan(O.reduce_last_axis("max", O.F32, x)[0]) and np.isnan(O.reduce_last_axis("min", O.F32, x)[0])
