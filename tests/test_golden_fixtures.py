"""The committed known-answer fixtures of the reference (tests/golden/reference_kats.json): the CPU oracle
must reproduce them (CPU test) and so must the CUDA library through its C ABI (GPU test)."""
import json
import os

import numpy as np
import pytest

import oracle as O

with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kats.json"), encoding="utf-8") as f:
    CASES = json.load(f)["cases"]

_ODT = {"f32": O.F32, "f16": O.F16, "bf16": O.BF16, "i8": O.I8, "i16": O.I16, "i32": O.I32, "i64": O.I64}
_NP = {"f32": np.float32, "i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64}


def _values(dtype, vals):
    return np.array([float(v) for v in vals], np.float32).astype(_NP[dtype]) if dtype in _NP else None


def _expected_bits(dtype, vals):
    """Expected values as the storage the oracle returns (raw 16-bit patterns for f16 / bf16)."""
    x = np.array([float(v) for v in vals], np.float32)
    if dtype == "bf16":
        return O.f32_to_bf16(x)
    if dtype == "f16":
        return x.astype(np.float16).view(np.uint16)
    return x.astype(_NP[dtype])


def test_fixture_file_is_complete():
    names = {c["name"] for c in CASES}
    assert {"vecadd_i16_e2e", "test_cast_rank0", "test_cst_folding", "test_cst_folding_same_type",
            "saturate_overflow_mode_example", "default_round_mode_table", "isnan_runner_output",
            "cumsum_2d_dim1", "cumsum_2d_dim0_reverse", "interleave_runner_output", "deinterleave_even_runner_output",
            "deinterleave_odd_runner_output", "sort_2d_ascending_runner_output",
            "sort_3d_descending_runner_output"} <= names
    assert len(CASES) >= 12
    assert all(c.get("source") for c in CASES)


@pytest.mark.parametrize("case", [c for c in CASES if c["op"] == "cast"], ids=lambda c: c["name"])
def test_oracle_cast_fixtures(case):
    x = _values(case["src_dtype"], case["input"])
    for ov in [case["overflow"]] + case.get("also_holds_for_overflow", []):
        got = O.cast(_ODT[case["src_dtype"]], _ODT[case["dst_dtype"]], x, case["round_mode"], ov)
        assert np.array_equal(got, _expected_bits(case["dst_dtype"], case["expected"])), (case["name"], ov)


def test_oracle_vadd_and_isnan_fixtures():
    c = next(c for c in CASES if c["op"] == "vadd")
    got = O.elemwise_binary("add", _ODT[c["dtype"]], np.array(c["a"], _NP[c["dtype"]]), np.array(c["b"], _NP[c["dtype"]]))
    assert got.tolist() == c["expected"]
    c = next(c for c in CASES if c["op"] == "isnan")
    x = np.array([float(v) for v in c["input"]], np.float32)
    assert O.compare("vne", O.F32, x, x).tolist() == c["expected"]     # isnan(x) == (x != x), unordered-or-unequal


def test_default_round_mode_fixture():
    import importlib.util
    import torch
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("bsir", os.path.join(here, "..", "ascendnpu-ir_b200", "bsir", "__init__.py"))
    bsir = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bsir)
    t = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "i8": torch.int8, "i16": torch.int16,
         "i32": torch.int32, "i64": torch.int64}
    c = next(c for c in CASES if c["op"] == "default_round_mode")
    assert len(c["table"]) >= 12
    for row in c["table"]:
        assert bsir.default_round_mode(t[row["src"]], t[row["dst"]]) == row["mode"], row


def _f32(tokens):
    return np.array([[float(v) for v in row] for row in tokens] if isinstance(tokens[0], list) else [float(v) for v in tokens],
                    np.float32)


def _same_f32(got, want):
    """Equal as the runner prints them: same numbers, NaN where NaN is expected."""
    return got.shape == want.shape and bool(np.all((got == want) | (np.isnan(got) & np.isnan(want))))


@pytest.mark.parametrize("case", [c for c in CASES if c["op"] == "cumsum"], ids=lambda c: c["name"])
def test_oracle_cumsum_runner_goldens(case):
    got = O.cumulative("sum", O.F32, _f32(case["input"]), axis=case["axis"], reverse=case["reverse"])
    assert _same_f32(got, _f32(case["expected"]))


def test_oracle_interleave_runner_goldens():
    c = next(c for c in CASES if c["op"] == "interleave")
    assert _same_f32(O.interleave([_f32(c["a"]), _f32(c["b"])]), _f32(c["expected"]))
    for c in (c for c in CASES if c["op"] == "deinterleave"):
        assert _same_f32(O.deinterleave(_f32(c["input"]), c["channel"]), _f32(c["expected"]))


@pytest.mark.parametrize("case", [c for c in CASES if c["op"] == "sort"], ids=lambda c: c["name"])
def test_oracle_sort_runner_goldens(case):
    """Both forms of the oracle's sort -- the literal compare-and-swap passes and their closed form."""
    x = _f32(case["input"])
    for fn in (O.sort_last_axis_loops, O.sort_last_axis):
        val, idx = fn(O.F32, x, descending=case["descending"])
        assert _same_f32(val, _f32(case["expected"])), fn.__name__
        assert _same_f32(np.take_along_axis(x, idx.astype(np.int64), axis=-1), val)


# ------------------------------------------------------------------------------------------------ GPU
@pytest.fixture(scope="module")
def bsir():
    import bsir as B
    B.lib()
    return B


@pytest.mark.gpu
@pytest.mark.parametrize("case", [c for c in CASES if c["op"] == "cast"], ids=lambda c: c["name"])
def test_gpu_cast_fixtures(bsir, case):
    import torch
    from conftest import to_bits
    t = {"f32": torch.float32, "bf16": torch.bfloat16, "i8": torch.int8, "i64": torch.int64}
    x = torch.tensor([float(v) for v in case["input"]], dtype=torch.float32).to(t[case["src_dtype"]]).cuda()
    for ov in [case["overflow"]] + case.get("also_holds_for_overflow", []):
        y = bsir.cast(x, t[case["dst_dtype"]], round_mode=case["round_mode"], overflow_mode=ov)
        assert np.array_equal(to_bits(y), _expected_bits(case["dst_dtype"], case["expected"])), (case["name"], ov)


@pytest.mark.gpu
def test_gpu_vadd_and_isnan_fixtures(bsir):
    import torch
    c = next(c for c in CASES if c["op"] == "vadd")
    a = torch.tensor(c["a"], dtype=torch.int16, device="cuda")
    b = torch.tensor(c["b"], dtype=torch.int16, device="cuda")
    assert bsir.vadd(a, b).tolist() == c["expected"]
    c = next(c for c in CASES if c["op"] == "isnan")
    x = torch.tensor([float(v) for v in c["input"]], device="cuda")
    assert bsir.compare("vne", x, x).to(torch.int32).tolist() == c["expected"]


@pytest.mark.gpu
@pytest.mark.parametrize("case", [c for c in CASES if c["op"] == "cumsum"], ids=lambda c: c["name"])
def test_gpu_cumsum_runner_goldens(bsir, case):
    import torch
    x = torch.from_numpy(_f32(case["input"])).cuda()
    got = bsir.cumulative("sum", x, dim=case["axis"], reverse=case["reverse"])
    assert _same_f32(got.cpu().numpy(), _f32(case["expected"]))


@pytest.mark.gpu
def test_gpu_interleave_runner_goldens(bsir):
    import torch
    c = next(c for c in CASES if c["op"] == "interleave")
    got = bsir.interleave([torch.from_numpy(_f32(c["a"])).cuda(), torch.from_numpy(_f32(c["b"])).cuda()])
    assert _same_f32(got.cpu().numpy(), _f32(c["expected"]))
    for c in (c for c in CASES if c["op"] == "deinterleave"):
        outs = bsir.deinterleave(torch.from_numpy(_f32(c["input"])).cuda(), 2, keep=[c["channel"]])
        assert _same_f32(outs[c["channel"]].cpu().numpy(), _f32(c["expected"]))


@pytest.mark.gpu
@pytest.mark.parametrize("case", [c for c in CASES if c["op"] == "sort"], ids=lambda c: c["name"])
def test_gpu_sort_runner_goldens(bsir, case):
    import torch
    x = torch.from_numpy(_f32(case["input"])).cuda()
    val, idx = bsir.sort(x, descending=case["descending"])
    assert _same_f32(val.cpu().numpy(), _f32(case["expected"]))
    assert _same_f32(torch.gather(x, 1, idx.long()).cpu().numpy(), val.cpu().numpy())
