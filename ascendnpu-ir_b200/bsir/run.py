"""`python -m bsir.run kernel.mlir` -- run one function of an MLIR test file on the GPU the way the reference's CPU
runner runs it: every memref / tensor argument is filled with the runner's seeded data (runner_data.py), all arguments
are dumped to the input file, the function runs through the CUDA library (mlir_text.py), and the outputs are dumped to
the output file in the reference's printData format (bishengir/lib/ExecutionEngine/CreateHostMain.cpp builds exactly
this main around a kernel: getData for every argument, print all to argv[1], call, print the outputs to argv[2];
checked by bishengir/test/ExecutionEngine/wrap-kernel-bufferized-no-return.mlir:22-67).  Outputs are the arguments
marked `hacc.arg_type<output>`; a function without such marks reports what it returns.

    python -m bsir.run add.mlir --func add --input-file in.txt --output-file out.txt [--dyn 128 ...] [--scalar %eps=1e-6]
"""
from __future__ import annotations

import argparse
import re
import sys

import numpy as np

_TORCH = {"f32": "float32", "f16": "float16", "bf16": "bfloat16", "i1": "bool", "i8": "int8", "i16": "int16", "i32": "int32", "i64": "int64"}


def _specialise(text: str, func, dyn):
    """Dynamic sizes are fixed before the run, as the reference's host main fixes them from its command line: each `?`
    of the function's argument types takes the next --dyn value, and the resulting static type replaces the dynamic
    one throughout the module.  Two arguments that spell the same dynamic type must get the same sizes."""
    from . import mlir_text
    if "?" not in text:
        return text
    fns = mlir_text.parse(re.sub(r"\?x", "1x", text))          # only to read names and argument order
    name = func or next((n for n, f in fns.items() if re.search(r"hacc\.(entry|function_kind)", f.attrs)), next(iter(fns)))
    m = re.search(r"func\.func\s+(?:private\s+)?@" + re.escape(name) + r"\s*\(", text)
    end = mlir_text._balanced(text, m.end() - 1, "(", ")")
    chosen = {}
    for a in mlir_text._split_top(text[m.end():end - 1]):
        ty = re.sub(r"\{[^}]*\}\s*$", "", a.split(":", 1)[1]).strip()
        if "?" not in ty:
            continue
        static = ty
        while "?" in static:
            if not dyn:
                raise SystemExit(f"{ty}: a dynamic size needs a --dyn value")
            static = static.replace("?", str(dyn.pop(0)), 1)
        if chosen.setdefault(ty, static) != static:
            raise SystemExit(f"{ty} is used with two different sets of sizes; give the arguments distinct types")
    for ty, static in chosen.items():
        text = text.replace(ty, static)
    if "?" in text:
        raise SystemExit("a dynamic size remains that no argument type fixes")
    return text


def run_file(path: str, func=None, input_file=None, output_file=None, dyn=(), scalars=None, device="cuda"):
    """Runs the function; returns (argument arrays as generated, output arrays as numpy, element types of the outputs)."""
    import torch
    from . import mlir_text, runner_data
    text = _specialise(open(path, encoding="utf-8").read(), func, list(dyn))
    fns = mlir_text.parse(text)
    if func is None:
        marked = [n for n, f in fns.items() if re.search(r"hacc\.(entry|function_kind)", f.attrs)]
        func = marked[0] if marked else next(iter(fns))
    fn = fns[func]
    attrs = fn.arg_attrs
    data = runner_data.RunnerData()
    scalars = dict(scalars or {})
    args_np, args_t, elems = [], [], []
    for (name, ty), _ in zip(fn.args, attrs):
        if ty.startswith(("tensor", "memref")):
            st = mlir_text.ShapedType(ty)
            a = data.get_data(st.elem, st.shape)
            args_np.append(a)
            elems.append(st.elem)
            if st.elem in ("bf16", "f16"):
                t = torch.from_numpy(a.view(np.int16).copy()).to(device).view(getattr(torch, _TORCH[st.elem]))
            else:
                t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
            args_t.append(t)
        else:
            if name not in scalars:
                raise SystemExit(f"argument {name} : {ty} is a scalar: pass --scalar {name}=<value>")
            v = float(scalars[name]) if ty.startswith(("f", "bf")) else int(scalars[name])
            args_np.append(None)
            elems.append(None)
            args_t.append(v)
    if input_file:
        with open(input_file, "w", encoding="utf-8") as f:
            for a, e in zip(args_np, elems):
                if a is not None:
                    f.write(runner_data.print_data(e, a))
    res = fn(*args_t)
    torch.cuda.synchronize()
    out_idx = [i for i, at in enumerate(attrs) if "arg_type<output>" in at]
    if out_idx:
        outs = [(elems[i], args_t[i]) for i in out_idx]
    else:
        res = res if isinstance(res, tuple) else (() if res is None else (res,))
        rev = {v: k for k, v in _TORCH.items()}
        outs = [(rev[str(t.dtype).replace("torch.", "")], t) for t in res if isinstance(t, torch.Tensor)]
    outs_np = []
    for e, t in outs:
        t = t.detach().contiguous().cpu()
        outs_np.append((e, t.view(torch.int16).numpy().view(np.uint16) if e in ("bf16", "f16") else t.numpy()))
    if output_file:
        with open(output_file, "w", encoding="utf-8") as f:
            for e, a in outs_np:
                f.write(runner_data.print_data(e, a))
    return args_np, [a for _, a in outs_np], [e for e, _ in outs_np]


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m bsir.run", description=__doc__.split("\n\n")[0])
    ap.add_argument("file")
    ap.add_argument("--func", default=None, help="function to run (default: the one marked as entry, else the first)")
    ap.add_argument("--input-file", default=None, help="where to dump all arguments before the run")
    ap.add_argument("--output-file", default=None, help="where to dump the outputs after the run (default: stdout)")
    ap.add_argument("--dyn", type=int, nargs="*", default=[], help="values for dynamic dimensions, in order of appearance")
    ap.add_argument("--scalar", action="append", default=[], help="%%name=value for a scalar argument")
    a = ap.parse_args(argv)
    scalars = dict(s.split("=", 1) for s in a.scalar)
    _, outs, elems = run_file(a.file, a.func, a.input_file, a.output_file, a.dyn, scalars)
    if not a.output_file:
        from . import runner_data
        for e, o in zip(elems, outs):
            sys.stdout.write(runner_data.print_data(e, o))
    return 0


if __name__ == "__main__":
    sys.exit(main())
