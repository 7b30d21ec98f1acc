"""Extracts the known answers the reference's own tests and comments hold for the hot path and writes them
to reference_kats.json (next to this file).

Run where a checkout of the reference is available:
    python tests/golden/make_reference_kats.py --reference <path to the AscendNPU-IR checkout>
The JSON that is committed was made this way; the tests only read the JSON.

Every case keeps the reference file and line range it was read from.  Only literal values are taken
(arrays in C++ sources, `dense<...>` constants and FileCheck lines in .mlir tests, a documented example
vector in a comment, the arguments of unit-test expectations); nothing is computed here.
"""
import argparse
import json
import os
import re


def _lines(path):
    with open(path, encoding="utf-8") as f:
        return f.read().split("\n")


def _line_of(lines, needle, start=0):
    for i in range(start, len(lines)):
        if needle in lines[i]:
            return i
    raise SystemExit(f"'{needle}' not found")


def _c_array(lines, name):
    """int16_t <name>[] = {...}; -> (values, first line, last line), 1-based lines."""
    i = _line_of(lines, f"{name}[] = {{")
    j = i
    text = lines[i]
    while "}" not in lines[j]:
        j += 1
        text += lines[j]
    vals = [int(v) for v in re.findall(r"-?\d+", text.split("{", 1)[1].split("}", 1)[0])]
    return vals, i + 1, j + 1


def vecadd(ref):
    rel = "bishengir/test/Integration/HIVM/VecAdd/main.cpp"
    lines = _lines(os.path.join(ref, rel))
    exp, e0, e1 = _c_array(lines, "expectedValue")
    a, a0, a1 = _c_array(lines, "input0Value")
    b, b0, b1 = _c_array(lines, "input1Value")
    # the FileCheck lines of the same test: "i<k> Expect: <v> Result: <v>"
    checks = [(int(m.group(1)), int(m.group(2)), int(m.group(3)))
              for m in (re.search(r"CHECK: i(\d+)\s+Expect: (-?\d+)\s+Result: (-?\d+)", l) for l in lines) if m]
    assert [c[1] for c in checks] == exp and [c[2] for c in checks] == exp
    return [{"name": "vecadd_i16_e2e", "op": "vadd", "dtype": "i16", "a": a, "b": b, "expected": exp,
             "source": f"{rel}:{a0}-{b1} (inputs), :{e0}-{e1} and the CHECK lines (expected)"}]


def cast_folds(ref):
    rel = "bishengir/test/Dialect/HFusion/canonicalize.mlir"
    lines = _lines(os.path.join(ref, rel))
    out = []
    for fn in ("test_cast_rank0", "test_cst_folding", "test_cst_folding_same_type"):
        i = _line_of(lines, f"func.func @{fn}(")
        j = _line_of(lines, "  return %", i)
        body = "\n".join(l for l in lines[i:j + 1] if "CHECK" not in l)
        head = "\n".join(l for l in lines[max(0, i - 4):j + 1] if "CHECK" in l)   # above or just inside the function
        src = re.search(r"arith\.constant dense<([^>]+)> : tensor<(?:(\d+)x)?(\w+)>", body)
        chk = re.search(r"CHECK:.*arith\.constant dense<([^>]+)> : tensor<(?:(\d+)x)?(\w+)>", head)
        mode = re.search(r"round_mode = #hfusion\.round_mode<(\w+)>", body)
        n = int(src.group(2) or 1)
        out.append({"name": fn, "op": "cast", "src_dtype": src.group(3), "dst_dtype": chk.group(3),
                    "round_mode": mode.group(1) if mode else "rint", "overflow": "wrap",
                    "input": [float(src.group(1))] * n, "expected": [float(chk.group(1))] * n,
                    "source": f"{rel}:{max(1, i - 2)}-{j + 1}"})
    return out


def saturate_example(ref):
    rel = "bishengir/lib/Dialect/HFusion/Transforms/Normalize.cpp"
    lines = _lines(os.path.join(ref, rel))
    i = _line_of(lines, "e.g. Input (float32): tensor([")
    text = " ".join(l.strip().lstrip("/ ") for l in lines[i:i + 3])
    m = re.search(r"Input \(float32\): tensor\(\[([^\]]+)\]\), Output\(int8\): tensor\(\[([^\]]+)\]", text)
    x = [float(v) for v in m.group(1).split(",")]
    y = [int(v) for v in m.group(2).split(",")]
    return [{"name": "saturate_overflow_mode_example", "op": "cast", "src_dtype": "f32", "dst_dtype": "i8",
             "round_mode": "rint", "overflow": "ascend_saturate_trunc_via_f16", "input": x, "expected": y,
             "also_holds_for_overflow": ["saturate"], "source": f"{rel}:{i + 1}-{i + 3}"}]


def default_round_modes(ref):
    rel = "bishengir/unittests/Dialect/Utils/SelectRoundModeTest.cpp"
    text = "\n".join(_lines(os.path.join(ref, rel)))
    names = {"F32": "f32", "F16": "f16", "BF16": "bf16", "I8": "i8", "I16": "i16", "I32": "i32", "I64": "i64"}
    table = []
    for m in re.finditer(r"expectRoundMode\(builder\.get(\w+)Type\(\),\s*builder\.get(\w+)Type\(\),\s*(?:hivm::)?RoundMode::(\w+)\)", text):
        table.append({"src": names[m.group(1)], "dst": names[m.group(2)], "mode": m.group(3).lower()})
    first = text[:text.index("expectRoundMode(builder")].count("\n") + 1
    last = text[:text.rindex("expectRoundMode(builder")].count("\n") + 3
    return [{"name": "default_round_mode_table", "op": "default_round_mode", "table": table,
             "source": f"{rel}:{first}-{last} (selector: bishengir/include/bishengir/Dialect/Utils/Util.h:180-213)"}]


def isnan_runner_golden(ref):
    rel = "bishengir/test/Dialect/HFusion/test_isnan.mlir"
    lines = _lines(os.path.join(ref, rel))
    i = _line_of(lines, "// CHECK: [1, nan, inf, -inf]")
    assert "// CHECK: [0, 1, 0, 0]" in lines[i + 1]
    return [{"name": "isnan_runner_output", "op": "isnan", "dtype": "f32", "input": ["1", "nan", "inf", "-inf"],
             "expected": [0, 1, 0, 0], "source": f"{rel}:{i + 1}-{i + 2}"}]


_HF = "bishengir/test/Dialect/HFusion/"


def _check_rows(lines):
    """`// CHECK: [a, b, ...]` lines of a runner test -> [(1-based line, [tokens])], in file order."""
    out = []
    for i, l in enumerate(lines):
        m = re.search(r"//\s*CHECK:\s*\[([^\]]*)\]", l)
        if m:
            out.append((i + 1, [t.strip() for t in m.group(1).split(",")]))
    return out


def _stored_buffer(lines, buf):
    """Rebuilds what `memref.store %const, %<buf>[%ci, ...]` lines put into a buffer from the literal
    `arith.constant` each one names (index constants %c<k> are the integer k) -> ({index tuple: token}, first, last)."""
    consts = {}
    for l in lines:
        m = re.match(r"\s*(%[\w.]+)\s*=\s*arith\.constant\s+(\S+)\s*:\s*f32", l)
        if m:
            consts[m.group(1)] = {"0x7F800000": "inf", "0xFF800000": "-inf", "0x7FC00000": "nan"}.get(m.group(2), m.group(2))
    cells, first, last = {}, None, None
    for i, l in enumerate(lines):
        m = re.match(r"\s*memref\.store\s+(%[\w.]+),\s*%" + buf + r"\[([^\]]*)\]", l)
        if m:
            idx = tuple(int(t.strip().lstrip("%c")) for t in m.group(2).split(","))
            cells[idx] = consts[m.group(1)]
            first = first or i + 1
            last = i + 1
    return cells, first, last


def _matrix(cells):
    dims = [max(k[d] for k in cells) + 1 for d in range(len(next(iter(cells))))]
    if len(dims) == 1:
        return [cells[(j,)] for j in range(dims[0])]
    return [[cells[(i, j)] for j in range(dims[1])] for i in range(dims[0])]


def cumsum_runner_golden(ref):
    rel = _HF + "test_cumsum_2d.mlir"
    lines = _lines(os.path.join(ref, rel))
    rows = _check_rows(lines)
    cells, s0, s1 = _stored_buffer(lines, "m")
    x = _matrix(cells)
    assert [r[1] for r in rows[:2]] == [[v.rstrip("0").rstrip(".") for v in row] for row in x]   # the printed input
    src = f"{rel}:{rows[0][0]}-{rows[-1][0]} (printed output), :{s0}-{s1} (input)"
    return [{"name": "cumsum_2d_dim1", "op": "cumsum", "dtype": "f32", "axis": 1, "reverse": False, "input": x,
             "expected": [rows[2][1], rows[3][1]], "source": src},
            {"name": "cumsum_2d_dim0_reverse", "op": "cumsum", "dtype": "f32", "axis": 0, "reverse": True, "input": x,
             "expected": [rows[4][1], rows[5][1]], "source": src}]


def interleave_runner_goldens(ref):
    rel = _HF + "test_interleave.mlir"
    lines = _lines(os.path.join(ref, rel))
    rows = _check_rows(lines)
    a, a0, _ = _stored_buffer(lines, "a")
    b, _, b1 = _stored_buffer(lines, "b")
    assert [v.rstrip("0").rstrip(".") for v in _matrix(a)] == rows[0][1] and [v.rstrip("0").rstrip(".") for v in _matrix(b)] == rows[1][1]
    out = [{"name": "interleave_runner_output", "op": "interleave", "dtype": "f32", "a": rows[0][1], "b": rows[1][1],
            "expected": rows[2][1], "source": f"{rel}:{rows[0][0]}-{rows[2][0]} (printed), :{a0}-{b1} (inputs)"}]
    rel = _HF + "test_deinterleave.mlir"
    lines = _lines(os.path.join(ref, rel))
    rows = _check_rows(lines)
    src = f"{rel}:{rows[0][0]}-{rows[2][0]}"
    out.append({"name": "deinterleave_even_runner_output", "op": "deinterleave", "dtype": "f32", "channel": 0,
                "input": rows[0][1], "expected": rows[1][1], "source": src})
    out.append({"name": "deinterleave_odd_runner_output", "op": "deinterleave", "dtype": "f32", "channel": 1,
                "input": rows[0][1], "expected": rows[2][1], "source": src})
    return out


def sort_runner_goldens(ref):
    rel = _HF + "test_sort_2d_asc.mlir"
    lines = _lines(os.path.join(ref, rel))
    rows = _check_rows(lines)
    cells, s0, s1 = _stored_buffer(lines, "m")
    x = _matrix(cells)
    assert [[v.rstrip("0").rstrip(".") for v in r] for r in x[:2]] == [rows[0][1], rows[1][1]]
    out = [{"name": "sort_2d_ascending_runner_output", "op": "sort", "dtype": "f32", "descending": False,
            "input": [rows[0][1], rows[1][1]], "expected": [rows[2][1], rows[3][1]],
            "note": "the first two rows of the 4x4 tensor: the ones the test checks",
            "source": f"{rel}:{rows[0][0]}-{rows[3][0]} (printed), :{s0}-{s1} (input)"}]
    rel = _HF + "test_sort_3d_des.mlir"
    lines = _lines(os.path.join(ref, rel))
    rows = _check_rows(lines)
    out.append({"name": "sort_3d_descending_runner_output", "op": "sort", "dtype": "f32", "descending": True,
                "input": [rows[0][1]], "expected": [rows[1][1]],
                "note": "row [0, 0, :] of the 2x3x4 tensor: the one the test checks",
                "source": f"{rel}:{rows[0][0]}-{rows[1][0]}"})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    cases = vecadd(args.reference) + cast_folds(args.reference) + saturate_example(args.reference) + \
        default_round_modes(args.reference) + isnan_runner_golden(args.reference) + cumsum_runner_golden(args.reference) + \
        interleave_runner_goldens(args.reference) + sort_runner_goldens(args.reference)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kats.json")
    with open(out, "w", encoding="utf-8") as f:
        json.dump({"cases": cases}, f, indent=1)
        f.write("\n")
    print(f"{len(cases)} cases -> {out}")


if __name__ == "__main__":
    main()
