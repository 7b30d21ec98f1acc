"""A small front end for the MLIR assembly of the hot-path ops: it reads a `func.func` written the way the
reference's tests write them (HFusion / linalg named ops on tensors, HIVM ops on memrefs, the scalar `arith`
ops around them) and runs it op by op through the CUDA library.

    fn = parse(open("rms_norm.mlir").read())["rms_norm_f16"]
    y, rstd = fn(x, gamma, out0, out1)            # torch CUDA tensors in the order of the signature

Covered (attribute spellings as in the reference):
  hfusion.cast {round_mode | mode = #hfusion.round_mode<..>, enable_saturate, overflow_mode}      HFusionNamedStructuredOps.yaml:373-432
  hfusion.elemwise_unary / elemwise_binary {fun = #hfusion.unary_fn<..>}, linalg.elemwise_unary / elemwise_binary
  hfusion.compare {compare_fn = #hfusion.compare_fn<..>}, hfusion.select, hfusion.isnan, hfusion.elemwise_ternary {fun = select | fma},
  hfusion.bitcast, hfusion.load / store
  hfusion.reduce_with_index {tie_break_left} <max|min>
  linalg.fill, linalg.broadcast dimensions = [..], linalg.reduce {arith.<combiner>} dimensions = [k] (short form and a
  region with one combiner op), linalg.matmul / matmul_transpose_a / matmul_transpose_b / batch_matmul (i8 -> i32, f16, bf16),
  linalg.copy, linalg.generic (elementwise bodies over identity maps: one fused kernel; last-axis reductions of one combiner)
  hivm.hir.load (pad_mode / pad_value / left_padding_num / right_padding_num), hivm.hir.store (atomic = <kind>),
  hivm.hir.copy, hivm.hir.vadd / vsub / vmul / vdiv / vmax / vmin / vand / vor / vxor / vpow / vmod / vmodui / vshl / vshr,
  hivm.hir.vexp / vln / vabs / vsqrt / vrsqrt / vrelu / vnot / vrec / vtanh / verf / vsin / vcos, vcmp [compare_mode = <..>], vsel,
  vbrc, vtranspose permutation = [..], varange offset[..] strides[..], vinterleave, vdeinterleave, hivm.hir.vcast, hivm.hir.vreduce <kind>,
  hivm.hir.vcumsum / vcumprod / vcummax / vcummin (and hfusion.cumsum ...) cum_dims = [k] reverse = <bool>,
  hivm.hir.vgather ins(..) indices(..) outs(..) gather_axis = k, hivm.hir.vsort ins(..) outs(%v, %i) descending = <bool>
  tensor.empty, tensor.dim, tensor.collapse_shape / expand_shape / reshape, tensor.extract_slice (static), linalg.transpose, memref.alloc, arith.constant (scalars, splat `dense<..>`), arith.{addf,subf,mulf,divf,addi,subi,muli},
  arith.{index_cast,index_castui,uitofp,sitofp,extf,truncf}, arith.{divsi,divui,remsi,remui,ceildivsi,floordivsi,maxsi,minsi,andi,ori,xori,cmpi,select}
  on scalars, tensor.from_elements, tensor.concat, return
Scalar arithmetic is done in the scalar's own type (f32 ops round to f32).  Anything else raises MlirTextError
with the op's name, so an unsupported file fails loudly instead of computing something different.

Fusion (``Function.fuse``, on by default): elementwise ops, fills, broadcasts and last-axis reductions on f32 tensors,
with the casts at the edges of such a region, are not launched one by one; they are recorded (fusion.py) and every
value the function needs in memory is produced by one fused kernel per [rows, cols] problem -- an outlined
LAST_AXIS_PBR function such as RMSNorm or softmax is one launch.  Elementwise regions keep the bits of op-by-op
execution; a fused row sum associates as a tree.
"""
import re
from typing import Dict, List, Optional, Sequence

import numpy as np

__all__ = ["parse", "Function", "MlirTextError"]


class MlirTextError(ValueError):
    pass


_TORCH_NAMES = {"f32": "float32", "f16": "float16", "bf16": "bfloat16", "i8": "int8", "i16": "int16", "i32": "int32",
                "i64": "int64", "i1": "bool", "ui8": "uint8", "index": "int64"}
_REDUCE_COMBINERS = {"arith.addf": "sum", "arith.addi": "sum", "arith.mulf": "prod", "arith.muli": "prod",
                     "arith.maximumf": "max", "arith.maxsi": "max", "arith.minimumf": "min", "arith.minsi": "min",
                     "arith.ori": "ori", "arith.andi": "andi", "arith.xori": "xori"}
_HIVM_BINARY = {"vadd": "add", "vsub": "sub", "vmul": "mul", "vdiv": "div", "vmax": "maxf", "vmin": "minf", "vand": "vand",
                "vor": "vor", "vxor": "vxor", "vpow": "powf", "vmod": "mod", "vmodui": "modui", "vshl": "shli", "vshr": "shrsi"}
_HIVM_INT_BINARY = {"vmax": "max_signed", "vmin": "min_signed"}     # vmax / vmin of integers
_HIVM_UNARY = {"vexp": "exp", "vln": "log", "vabs": "abs", "vsqrt": "sqrt", "vrsqrt": "rsqrt", "vrelu": "relu", "vnot": "vnot",
               "vrec": "rec", "vtanh": "tanh", "verf": "erf", "vsin": "sin", "vcos": "cos"}
_HIVM_COMPARE = {"eq": "veq", "ne": "vne", "le": "vle", "lt": "vlt", "ge": "vge", "gt": "vgt"}
_LINALG_UNARY = {"exp", "log", "abs", "ceil", "floor", "negf", "reciprocal", "round", "sqrt", "rsqrt", "square", "tanh", "erf"}


class ShapedType:
    def __init__(self, text: str):
        m = re.match(r"(tensor|memref)<(.*)>$", text.strip(), re.S)
        if not m:
            raise MlirTextError(f"not a tensor/memref type: {text}")
        inner = m.group(2).split(",")[0].strip()          # drops the memory space of a memref
        m2 = re.match(r"((?:(?:\d+|\?)x)*)(.*)$", inner)        # sizes, then the element type ("index" has an x of its own)
        self.elem = m2.group(2)
        self.shape = []
        for p in m2.group(1).split("x")[:-1]:
            if p == "?":
                raise MlirTextError("dynamic shapes are not supported by this front end")
            self.shape.append(int(p))
        if self.elem not in _TORCH_NAMES:
            raise MlirTextError(f"element type {self.elem}")


class Scalar:
    """An SSA scalar: a value and its MLIR type (f32 / i32 / index ...)."""

    def __init__(self, value, ty: str):
        self.ty = ty
        if ty == "f32":
            self.value = float(np.float32(value))
        elif ty in ("f16", "bf16", "f64"):
            self.value = float(value)
        else:
            self.value = int(value)


def _float_literal(text: str, ty: str) -> float:
    """A float constant as MLIR prints it: decimal, or the bit pattern in hex (`0xFF800000 : f32` is -inf)."""
    if text.lower().startswith("0x"):
        bits = int(text, 16)
        if ty == "f32":
            return float(np.array([bits], dtype=np.uint32).view(np.float32)[0])
        if ty == "f16":
            return float(np.array([bits], dtype=np.uint16).view(np.float16)[0])
        if ty == "bf16":
            return float(np.array([bits << 16], dtype=np.uint32).view(np.float32)[0])
        return float(np.array([bits], dtype=np.uint64).view(np.float64)[0])
    return float(text)


def _strip_comments(text: str) -> str:
    return "\n".join(line.split("//", 1)[0] for line in text.split("\n"))


def _split_top(text: str, sep: str = ",") -> List[str]:
    """Splits at `sep` outside any brackets."""
    out, depth, cur = [], 0, ""
    for ch in text:
        if ch in "([{<":
            depth += 1
        elif ch in ")]}>":
            depth -= 1
        if ch == sep and depth == 0:
            out.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur.strip())
    return out


def _balanced(text: str, start: int, open_ch: str, close_ch: str) -> int:
    """Index just past the bracket group that opens at `start`."""
    depth = 0
    for i in range(start, len(text)):
        if text[i] == open_ch:
            depth += 1
        elif text[i] == close_ch:
            depth -= 1
            if depth == 0:
                return i + 1
    raise MlirTextError("unbalanced brackets")


class Op:
    def __init__(self, results: List[str], name: str, text: str):
        self.results, self.name, self.text = results, name, text

    # ins(%a, %b : t1, t2)  ->  (["%a", "%b"], ["t1", "t2"])
    def group(self, key: str):
        m = re.search(rf"\b{key}\s*\(", self.text)
        if not m:
            return [], []
        end = _balanced(self.text, m.end() - 1, "(", ")")
        inner = self.text[m.end():end - 1]
        if ":" not in inner:
            return [], []
        names, types = inner.split(":", 1)
        return [n.strip() for n in _split_top(names)], _split_top(types)

    def attr(self, key: str, default=None):
        m = re.search(rf"\b{key}\s*=\s*(#[\w.]+<(\w+)>|true|false|-?[\d.eE+-]+|\"[^\"]*\")", self.text)
        if not m:
            return default
        if m.group(2):
            return m.group(2)
        v = m.group(1)
        return {"true": True, "false": False}.get(v, v.strip('"'))

    def int_list(self, key: str) -> Optional[List[int]]:
        m = re.search(rf"\b{key}\s*=\s*\[([^\]]*)\]", self.text)
        if not m:
            m = re.search(rf"\b{key}\s*=\s*array<i64(?::\s*([^>]*))?>", self.text)
            if not m:
                return None
        body = (m.group(1) or "").strip()
        return [int(v) for v in body.split(",")] if body else []


_OP_START = re.compile(r"(?:(?P<res>%[\w.#:]+(?:\s*,\s*%[\w.#:]+)*)\s*=\s*)?(?P<name>(?:[a-z_][\w]*\.)+[a-z_][\w]*|return)\b")


def _statements(body: str) -> List[Op]:
    """Cuts a function body into ops.  An op starts at `[%r =] dialect.name` at bracket depth 0."""
    ops, depth, i, starts = [], 0, 0, []
    n = len(body)
    while i < n:
        ch = body[i]
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        elif ch == "<" and i > 0 and (body[i - 1].isalnum() or body[i - 1] in "_."):
            end = _balanced(body, i, "<", ">")             # a type or attribute parameter list: skip as a whole
            i = end
            continue
        if depth == 0 and (i == 0 or body[i - 1] in " \n\t"):
            m = _OP_START.match(body, i)
            if m and (m.group("res") or "." in m.group("name") or m.group("name") == "return"):
                # names inside `ins(... : ...)` never match here because depth > 0 there
                starts.append((i, m))
                i = m.end()
                continue
        i += 1
    for k, (pos, m) in enumerate(starts):
        end = starts[k + 1][0] if k + 1 < len(starts) else n
        res = [r.strip().split(":")[0] for r in m.group("res").split(",")] if m.group("res") else []
        ops.append(Op(res, m.group("name"), body[m.end():end].strip()))
    return ops


class Function:
    def __init__(self, name: str, args: List[tuple], ops: List[Op]):
        self.name, self.args, self.ops = name, args, ops
        self.fuse = True          # f32 elementwise ops are deferred and run as fused chains (see fusion.py)
        self.uses: Dict[str, int] = {}
        for o in ops:
            for m in re.finditer(r"%[\w.]+", o.text):
                self.uses[m.group(0)] = self.uses.get(m.group(0), 0) + 1

    def op_names(self) -> List[str]:
        return [o.name for o in self.ops]

    # ------------------------------------------------------------------ execution
    def __call__(self, *tensors):
        import torch
        from . import (arange, cast, compare, copy, cumulative, deinterleave, elemwise_binary, elemwise_ternary, elemwise_unary, gather,
                       interleave,
                       load, matmul, reduce, reduce_with_index, select, sort, store, transpose)
        if len(tensors) != len(self.args):
            raise MlirTextError(f"@{self.name} takes {len(self.args)} arguments, got {len(tensors)}")
        env: Dict[str, object] = {}
        for (name, ty), t in zip(self.args, tensors):
            if ty.startswith(("tensor", "memref")):
                st = ShapedType(ty)
                if list(t.shape) != st.shape or str(t.dtype) != "torch." + _TORCH_NAMES[st.elem]:
                    raise MlirTextError(f"argument {name}: expected {ty}, got {tuple(t.shape)} {t.dtype}")
                env[name] = t
            else:
                env[name] = Scalar(t, ty)
        dev = next((t.device for t in tensors if isinstance(t, torch.Tensor)), torch.device("cuda"))

        def tdtype(elem):
            return getattr(torch, _TORCH_NAMES[elem])

        from . import fusion
        arg_ptrs = {t.data_ptr() for t in tensors if isinstance(t, torch.Tensor)}
        uninitialised = set()                                  # results of tensor.empty: values without contents
        requests: List[tuple] = []                             # (Lazy, destination) pairs waiting to run together
        consumed = set()                                       # deferred values folded into another expression

        def flush():
            """Runs what is waiting: all requests over one [rows, cols] problem as one kernel (four outputs at most)."""
            groups: Dict[tuple, list] = {}
            for lz, dst in requests:
                groups.setdefault(lz.prob, []).append((lz, dst))
            requests.clear()
            for prob, group in groups.items():
                for i in range(0, len(group), fusion.MAX_OUTPUTS):
                    fusion.run(group[i:i + fusion.MAX_OUTPUTS], prob)

        def request(lz, dst=None):
            """Asks for a deferred value in memory (in dst, in the op's own destination, or in a new f32 tensor)."""
            if dst is None:
                dst = lz.dst if lz.dst is not None else torch.empty(lz.shape, dtype=torch.float32, device=dev)
            requests.append((lz, dst))
            return dst

        def val(name):
            if name not in env:
                raise MlirTextError(f"use of undefined value {name}")
            if isinstance(env[name], fusion.Lazy):            # needed in memory now
                env[name] = request(env[name])
            if requests and isinstance(env[name], torch.Tensor):
                flush()
            return env[name]

        def node_of(name, shape, prob, per_row, touched):
            """The chain node for an operand of a fusible op whose result has this shape in this problem, or None."""
            v = env.get(name)
            if isinstance(v, Scalar):
                return ("imm", float(v.value))
            if isinstance(v, fusion.Lazy):
                if v.shape != list(shape):
                    return None
                if per_row and not v.per_row and v.node[0] == "leaf" and v.node[2] == "full":
                    return ("leaf", v.node[1].reshape(-1), "col_vector")      # a widened [rows] vector
                if v.prob != tuple(prob) or v.per_row != per_row:
                    return None
                touched.append(name)
                return v.node
            if isinstance(v, torch.Tensor) and list(v.shape) == list(shape) and v.dtype == torch.float32 and v.is_contiguous():
                if requests and any(d.data_ptr() == v.data_ptr() for _, d in requests):
                    flush()                                    # it is about to be written
                return ("leaf", v, "col_vector") if per_row else ("leaf", v.view(*prob), "full")
            return None

        def defer(op, node, shape, prob, per_row, touched):
            """Defines the op's result as a deferred expression (nothing is launched)."""
            if not fusion.fits(node):
                return False
            consumed.update(touched)
            dst = None
            outs_names = op.group("outs")[0]
            if outs_names and self.uses.get(outs_names[0], 0) == 1 and isinstance(env.get(outs_names[0]), torch.Tensor):
                cand = env[outs_names[0]]                      # the op's own destination, when no other op writes it
                if cand.dtype == torch.float32 and list(cand.shape) == list(shape) and cand.is_contiguous():
                    dst = cand
            env[op.results[0]] = fusion.Lazy(node, list(shape), prob, per_row, dst)
            return True

        def try_fuse(op, name, ins, outs) -> bool:
            """f32 elementwise ops, fills, broadcasts, last-axis reductions and the casts at the edges of an f32 region
            are deferred; True when the op was taken care of."""
            if len(op.results) != 1 or not outs:
                return False
            init = env.get(outs[0])
            if name == "linalg.reduce" and isinstance(init, fusion.Lazy) and init.node[0] == "imm" and len(init.shape) == 1:
                # the accumulator was filled with a constant: the reduction starts from it
                src = env.get(ins[0]) if ins else None
                comb = next((c for c in _REDUCE_COMBINERS if re.search(rf"\b{re.escape(c)}\b", op.text)), None)
                kind = _REDUCE_COMBINERS.get(comb)
                if kind in fusion.REDUCE and isinstance(src, fusion.Lazy) and not src.per_row and len(src.shape) == 2 and \
                        src.shape[0] == init.shape[0] and op.int_list("dimensions") == [1]:
                    fold = {"sum": "add", "prod": "mul", "max": "maxf", "min": "minf"}[kind]
                    return defer(op, ("bin", fold, ("red", kind, src.node), init.node), init.shape, src.prob, True, [ins[0]])
                return False
            if not isinstance(init, torch.Tensor):
                return False
            dst = init
            if not dst.is_contiguous() or dst.numel() == 0 or dst.dim() not in (1, 2):
                return False
            shape, touched = list(dst.shape), []
            if name == "hfusion.cast":
                src = env.get(ins[0])
                if isinstance(src, fusion.Lazy) and dst.dtype in (torch.float16, torch.bfloat16) and src.shape == shape and \
                        (op.attr("round_mode") or op.attr("mode") or "rint") == "rint" and not op.attr("enable_saturate", False) and \
                        op.attr("overflow_mode") is None:
                    consumed.add(ins[0])
                    env[op.results[0]] = request(src, dst)     # the chain's single rounding
                    return True
                if isinstance(src, torch.Tensor) and src.dtype in (torch.float16, torch.bfloat16) and dst.dtype == torch.float32 and \
                        list(src.shape) == shape and src.is_contiguous():
                    if requests and any(d.data_ptr() == src.data_ptr() for _, d in requests):
                        flush()
                    prob = fusion.problem(shape)               # a widening cast is exact: the chain reads the 16-bit storage
                    return defer(op, ("leaf", src.view(*prob), "full"), shape, prob, False, touched)
                return False
            if dst.dtype != torch.float32:
                return False
            # the problem the op lives in: that of a per-row operand, else the result's own shape
            per_row_src = next((env[n] for n in ins if isinstance(env.get(n), fusion.Lazy) and env[n].per_row and env[n].shape == shape), None)
            prob, per_row = (per_row_src.prob, True) if per_row_src is not None else (fusion.problem(shape), False)
            if name in ("linalg.elemwise_unary", "hfusion.elemwise_unary"):
                fun = op.attr("fun") or "exp"
                if fun not in fusion.UNARY or (name.startswith("linalg") and fun not in _LINALG_UNARY):
                    return False
                a = node_of(ins[0], shape, prob, per_row, touched)
                return a is not None and defer(op, ("un", fun, a), shape, prob, per_row, touched)
            if name in ("linalg.elemwise_binary", "hfusion.elemwise_binary"):
                fun = op.attr("fun") or "add"
                if fun not in fusion.BINARY or len(ins) < 2:
                    return False
                a, b = node_of(ins[0], shape, prob, per_row, touched), node_of(ins[1], shape, prob, per_row, touched)
                return a is not None and b is not None and defer(op, ("bin", fun, a, b), shape, prob, per_row, touched)
            if name == "linalg.fill" and isinstance(env.get(ins[0]), Scalar):
                return defer(op, ("imm", float(env[ins[0]].value)), shape, prob, False, touched)
            if name == "linalg.broadcast" and dst.dim() == 2:
                dims = op.int_list("dimensions") or []
                src = env.get(ins[0])
                if dims == [1] and isinstance(src, fusion.Lazy) and src.per_row and src.prob == tuple(shape):
                    touched.append(ins[0])
                    return defer(op, src.node, shape, tuple(shape), False, touched)   # already uniform along the row
                vec = src.node[1].reshape(-1) if isinstance(src, fusion.Lazy) and src.node[0] == "leaf" and src.node[2] == "full" \
                    and len(src.shape) == 1 else src if isinstance(src, torch.Tensor) and src.dim() == 1 and src.is_contiguous() \
                    and src.dtype == torch.float32 else None
                if vec is not None and dims in ([0], [1]) and vec.shape[0] == shape[1 - dims[0]]:
                    return defer(op, ("leaf", vec, "row_vector" if dims == [0] else "col_vector"), shape, tuple(shape), False, touched)
                return False
            if name == "linalg.reduce" and dst.dim() == 1 and op.int_list("dimensions") == [1]:
                comb = next((c for c in _REDUCE_COMBINERS if re.search(rf"\b{re.escape(c)}\b", op.text)), None)
                kind = _REDUCE_COMBINERS.get(comb)
                src = env.get(ins[0])
                if kind not in fusion.REDUCE or not isinstance(src, fusion.Lazy) or src.per_row or len(src.shape) != 2 or \
                        src.shape[0] != shape[0]:
                    return False                               # a reduction of a tensor in memory stays a plain reduce
                touched.append(ins[0])
                return defer(op, ("red", kind, src.node), shape, src.prob, True, touched)
            return False

        def operand(name):
            v = val(name)
            return v.value if isinstance(v, Scalar) else v

        def define(op, values):
            if len(op.results) > len(values):
                raise MlirTextError(f"{op.name}: {len(op.results)} results, {len(values)} produced")
            for r, v in zip(op.results, values):
                env[r] = v

        def write_out(dst, src):
            """Destination-style result: the value lands in the outs buffer."""
            if dst.data_ptr() != src.data_ptr():
                copy(src, out=dst)
            return dst

        for op in self.ops:
            name = op.name
            ins, in_types = op.group("ins")
            outs, out_types = op.group("outs")
            if self.fuse and try_fuse(op, name, ins, outs):
                continue
            if name == "return" or name == "func.return":
                names = [n.strip() for n in _split_top(op.text.split(":")[0])] if op.text.strip() else []
                for k in list(env):                            # results, and deferred values whose destination is an argument
                    if isinstance(env[k], fusion.Lazy) and (k in names or (k not in consumed and env[k].dst is not None and
                                                                            env[k].dst.data_ptr() in arg_ptrs)):
                        env[k] = request(env[k])
                flush()                                        # everything that is still waiting, together
                res = tuple(operand(n) for n in names)
                return res[0] if len(res) == 1 else (res if res else None)
            if name == "arith.constant":
                m = re.match(r"\s*dense<([^>]+)>\s*:\s*(.+)$", op.text, re.S)
                if m:
                    st = ShapedType(m.group(2))
                    define(op, [torch.full(st.shape, float(m.group(1)), dtype=tdtype(st.elem), device=dev)])
                else:
                    v, ty = op.text.rsplit(":", 1)
                    v = v.strip()
                    define(op, [Scalar({"true": 1, "false": 0}.get(v, v) if ty.strip() in ("i1",) else _float_literal(v, ty.strip()) if ty.strip().startswith("f") else int(float(v)), ty.strip())])
            elif name in ("arith.addf", "arith.subf", "arith.mulf", "arith.divf", "arith.addi", "arith.subi", "arith.muli"):
                a, b = [val(n.strip()) for n in _split_top(op.text.split(":")[0])]
                ty = op.text.rsplit(":", 1)[1].strip()
                f = {"add": lambda x, y: x + y, "sub": lambda x, y: x - y, "mul": lambda x, y: x * y, "div": lambda x, y: x / y}[name[6:9]]
                if ty == "f32":
                    define(op, [Scalar(f(np.float32(a.value), np.float32(b.value)), ty)])
                else:
                    define(op, [Scalar(f(a.value, b.value), ty)])
            elif name in ("arith.divsi", "arith.divui", "arith.remsi", "arith.remui", "arith.ceildivsi", "arith.floordivsi", "arith.maxsi",
                          "arith.minsi", "arith.andi", "arith.ori", "arith.xori"):
                a, b = [val(n.strip()) for n in _split_top(op.text.split(":")[0])]
                ty = op.text.rsplit(":", 1)[1].strip()
                x, y = int(a.value), int(b.value)
                if name in ("arith.divsi", "arith.divui", "arith.remsi", "arith.remui", "arith.ceildivsi", "arith.floordivsi") and y == 0:
                    raise MlirTextError(f"{name}: division by zero")
                trunc_div = lambda p, q: abs(p) // abs(q) * (1 if (p >= 0) == (q >= 0) else -1)   # C division: toward zero
                r = {"arith.divsi": lambda: trunc_div(x, y), "arith.divui": lambda: x // y, "arith.remsi": lambda: x - trunc_div(x, y) * y,
                     "arith.remui": lambda: x % y, "arith.ceildivsi": lambda: -((-x) // y), "arith.floordivsi": lambda: x // y,
                     "arith.maxsi": lambda: max(x, y), "arith.minsi": lambda: min(x, y), "arith.andi": lambda: x & y,
                     "arith.ori": lambda: x | y, "arith.xori": lambda: x ^ y}[name]()
                define(op, [Scalar(r, ty)])
            elif name == "arith.cmpi":
                # `%p = arith.cmpi slt, %a, %b : index`
                parts = [n.strip() for n in _split_top(op.text.split(":")[0])]
                a, b = int(val(parts[1]).value), int(val(parts[2]).value)
                pred = parts[0]
                if pred in ("ult", "ule", "ugt", "uge") and (a < 0 or b < 0):
                    raise MlirTextError("arith.cmpi: unsigned predicate on a negative scalar")
                r = {"eq": a == b, "ne": a != b, "slt": a < b, "sle": a <= b, "sgt": a > b, "sge": a >= b,
                     "ult": a < b, "ule": a <= b, "ugt": a > b, "uge": a >= b}[pred]
                define(op, [Scalar(1 if r else 0, "i1")])
            elif name == "arith.select" and isinstance(env.get(_split_top(op.text.split(":")[0])[0].strip()), Scalar):
                c, a, b = [val(n.strip()) for n in _split_top(op.text.split(":")[0])]
                define(op, [a if int(c.value) else b])
            elif name == "tensor.from_elements":
                # `%t = tensor.from_elements %a, %b : tensor<2xindex>`: a small tensor made of scalars
                st = ShapedType(op.text.rsplit(":", 1)[1])
                vals = [val(n.strip()).value for n in _split_top(op.text.rsplit(":", 1)[0]) if n.strip()]
                define(op, [torch.tensor(vals, dtype=tdtype(st.elem), device=dev).reshape(st.shape)])
            elif name == "tensor.concat":
                # `%r = tensor.concat dim(1) %a, %b : (tensor<4x8xf32>, tensor<4x8xf32>) -> tensor<4x16xf32>`: strided copies
                dim = int(re.search(r"dim\((\d+)\)", op.text).group(1))
                srcs = [val(n) for n in re.findall(r"%[\w.]+", op.text.split(":")[0])]
                st = ShapedType(op.text.rsplit("->", 1)[1])
                res = torch.empty(st.shape, dtype=tdtype(st.elem), device=dev)
                off = 0
                for t in srcs:
                    copy(t, out=res.narrow(dim, off, t.shape[dim]))
                    off += t.shape[dim]
                if off != st.shape[dim]:
                    raise MlirTextError("tensor.concat: the operands do not fill the result")
                define(op, [res])
            elif name in ("arith.index_cast", "arith.index_castui", "arith.uitofp", "arith.sitofp", "arith.extf", "arith.truncf",
                          "arith.extsi", "arith.extui", "arith.trunci"):
                src = val(op.text.split(":")[0].strip())
                ty = op.text.rsplit(" to ", 1)[1].strip()
                define(op, [Scalar(src.value, ty)])
            elif name in ("tensor.empty", "memref.alloc"):
                st = ShapedType(op.text.split(":", 1)[1])
                define(op, [torch.empty(st.shape, dtype=tdtype(st.elem), device=dev)])
                if name == "tensor.empty":                     # a tensor value is never written again; a memref may be
                    uninitialised.add(op.results[0])
            elif name == "tensor.dim":
                t_name, i_name = [n.strip() for n in _split_top(op.text.split(":")[0])]
                src = env.get(t_name)
                shape = src.shape if isinstance(src, fusion.Lazy) else val(t_name).shape
                define(op, [Scalar(shape[val(i_name).value], "index")])
            elif name in ("tensor.collapse_shape", "tensor.expand_shape", "tensor.reshape"):
                # `%r = tensor.collapse_shape %x [[0, 1], [2]] : tensor<AxBxCxf32> into tensor<ABxCxf32>`: a view
                src = val(re.match(r"\s*(%[\w.]+)", op.text).group(1))
                st = ShapedType(re.split(r"\binto\b|->", op.text)[-1])
                define(op, [src.reshape(st.shape)])
            elif name == "tensor.extract_slice":
                m = re.match(r"\s*(%[\w.]+)\s*\[([^\]]*)\]\s*\[([^\]]*)\]\s*\[([^\]]*)\]", op.text)
                if not m or "%" in m.group(2) + m.group(3) + m.group(4):
                    raise MlirTextError("tensor.extract_slice: static offsets / sizes / strides are supported")
                src = val(m.group(1))
                offs, sizes, strides = ([int(v) for v in m.group(i).split(",")] for i in (2, 3, 4))
                view = src[tuple(slice(o, o + n * st_, st_) for o, n, st_ in zip(offs, sizes, strides))]
                st = ShapedType(op.text.rsplit(" to ", 1)[1])
                define(op, [view.reshape(st.shape)])
            elif name == "linalg.transpose":
                perm = op.int_list("permutation")
                define(op, [copy(val(ins[0]).permute(perm), out=val(outs[0]))])
            elif name == "hfusion.cast" or name == "hivm.hir.vcast":
                dst = val(outs[0])
                mode = op.attr("round_mode") or op.attr("mode") or "rint"
                ov = op.attr("overflow_mode")
                y = cast(val(ins[0]), dst.dtype, round_mode=mode, enable_saturate=bool(op.attr("enable_saturate", False)),
                         overflow_mode=ov if isinstance(ov, str) and ov in ("saturate", "wrap") else None, out=dst)
                define(op, [y])
            elif name in ("linalg.elemwise_unary", "hfusion.elemwise_unary"):
                fun = op.attr("fun") or "exp"
                if name.startswith("linalg") and fun not in _LINALG_UNARY:
                    raise MlirTextError(f"linalg.elemwise_unary fun {fun}")
                define(op, [elemwise_unary(fun, val(ins[0]), out=val(outs[0]))])
            elif name in ("linalg.elemwise_binary", "hfusion.elemwise_binary"):
                fun = op.attr("fun") or "add"
                define(op, [elemwise_binary(fun, operand(ins[0]), operand(ins[1]), out=val(outs[0]))])
            elif name.startswith("hivm.hir.") and name[9:] in _HIVM_BINARY:
                dst = val(outs[0])
                fun = _HIVM_BINARY[name[9:]]
                if not dst.dtype.is_floating_point and name[9:] in _HIVM_INT_BINARY:
                    fun = _HIVM_INT_BINARY[name[9:]]
                define(op, [elemwise_binary(fun, operand(ins[0]), operand(ins[1]), out=dst)])
            elif name.startswith("hivm.hir.") and name[9:] in _HIVM_UNARY:
                x, dst = val(ins[0]), val(outs[0])
                fun = _HIVM_UNARY[name[9:]]
                if fun == "abs" and not x.dtype.is_floating_point:
                    fun = "absi"
                define(op, [elemwise_unary(fun, x, out=dst)])
            elif name == "hivm.hir.vcmp":
                # `hivm.hir.vcmp ins(%a, %b : T, T) outs(%o : Ti1) [compare_mode = <lt>]` (eq when absent)
                m = re.search(r"compare_mode\s*=\s*(?:#hivm\.compare_mode)?<(\w+)>", op.text)
                mode = m.group(1) if m else "eq"
                if mode not in _HIVM_COMPARE:
                    raise MlirTextError(f"hivm.hir.vcmp: compare_mode {mode}")
                define(op, [write_out(val(outs[0]), compare(_HIVM_COMPARE[mode], operand(ins[0]), operand(ins[1])))])
            elif name == "hivm.hir.vsel":
                cond = operand(ins[0])
                if not isinstance(cond, torch.Tensor):                 # a scalar i1 picks one operand whole
                    dst = val(outs[0])
                    pick = operand(ins[1]) if int(cond) else operand(ins[2])
                    define(op, [copy(pick, out=dst) if isinstance(pick, torch.Tensor) else
                                elemwise_binary("add", torch.zeros_like(dst), pick, out=dst)])
                else:
                    define(op, [write_out(val(outs[0]), select(cond, operand(ins[1]), operand(ins[2])))])
            elif name == "hivm.hir.vbrc":
                # a scalar, or a tensor with unit axes listed in broadcast_dims, spread over the destination
                dst = val(outs[0])
                src = operand(ins[0])
                if isinstance(src, torch.Tensor):
                    if src.dim() != dst.dim():
                        raise MlirTextError("hivm.hir.vbrc: source and destination ranks differ")
                    define(op, [copy(src.expand(dst.shape), out=dst)])
                elif dst.dtype == torch.bool:
                    define(op, [dst.fill_(bool(src))])
                else:
                    define(op, [elemwise_binary("add", torch.zeros_like(dst), src, out=dst)])
            elif name == "hivm.hir.vtranspose":
                src, dst = val(ins[0]), val(outs[0])
                perm = op.int_list("permutation")
                if perm is None or sorted(perm) != list(range(src.dim())):
                    raise MlirTextError("hivm.hir.vtranspose: permutation = [..] expected")
                if perm[:-2] == list(range(src.dim() - 2)) and perm[-2:] == [src.dim() - 1, src.dim() - 2]:
                    lead = int(np.prod(src.shape[:-2])) if src.dim() > 2 else 1     # the last two axes swapped: tiled kernel
                    transpose(src.reshape(lead, src.shape[-2], src.shape[-1]), out=dst.view(lead, dst.shape[-2], dst.shape[-1]))
                    define(op, [dst])
                elif src.dim() <= 3:
                    define(op, [copy(src.permute(perm), out=dst)])
                else:
                    raise MlirTextError("hivm.hir.vtranspose: beyond rank 3 only the last two axes may be swapped")
            elif name == "hivm.hir.varange":
                # `hivm.hir.varange offset[%o] strides[%s0, %s1] outs(%d : T)`
                dst = val(outs[0])
                mo = re.search(r"offset\[([^\]]*)\]", op.text)
                ms = re.search(r"strides\[([^\]]*)\]", op.text)
                off = int(val(mo.group(1).strip()).value) if mo and mo.group(1).strip() else 0
                strides = [int(val(t.strip()).value) for t in ms.group(1).split(",")] if ms and ms.group(1).strip() else None
                if strides is None:                                    # row-major positions
                    strides, acc_s = [], 1
                    for d in reversed(dst.shape):
                        strides.insert(0, acc_s)
                        acc_s *= d
                define(op, [arange(list(dst.shape), strides, off, dtype=dst.dtype, out=dst)])
            elif name == "hivm.hir.vinterleave":
                define(op, [interleave([val(n) for n in ins], out=val(outs[0]))])
            elif name == "hivm.hir.vdeinterleave":
                # `... channel_num = 32 index_mode = <CHANNEL_0>`: the even (CHANNEL_0) or odd (CHANNEL_1) elements, or both
                src = val(ins[0])
                m = re.search(r"index_mode\s*=\s*(?:#hivm\.deinterleave_mode)?<(\w+)>", op.text)
                mode = m.group(1) if m else "ALL_CHANNELS"
                dsts = [val(n) for n in outs]
                if mode == "ALL_CHANNELS":
                    parts = deinterleave(src, 2)
                    define(op, [write_out(d, ptn) for d, ptn in zip(dsts, parts)])
                elif mode in ("CHANNEL_0", "CHANNEL_1"):
                    ch = int(mode[-1])
                    define(op, [write_out(dsts[0], deinterleave(src, 2, keep=[ch])[ch])])
                else:
                    raise MlirTextError(f"hivm.hir.vdeinterleave: index_mode {mode}")
            elif name == "hfusion.compare":
                define(op, [write_out(val(outs[0]), compare(op.attr("compare_fn") or "veq", operand(ins[0]), operand(ins[1])))])
            elif name == "hfusion.isnan":
                x = val(op.text.split(":")[0].strip())
                define(op, [compare("vne", x, x)])
            elif name == "hfusion.select":
                define(op, [write_out(val(outs[0]), select(val(ins[0]), operand(ins[1]), operand(ins[2])))])
            elif name == "linalg.fill":
                dst = val(outs[0])
                define(op, [elemwise_binary("add", torch.zeros_like(dst), operand(ins[0]), out=dst)
                            if dst.dtype.is_floating_point or dst.dtype != torch.bool else dst.fill_(bool(operand(ins[0])))])
            elif name == "linalg.broadcast":
                src, dst = val(ins[0]), val(outs[0])
                dims = op.int_list("dimensions") or []
                view = src
                for d in sorted(dims):
                    view = view.unsqueeze(d)
                define(op, [copy(view.expand(dst.shape), out=dst)])
            elif name in ("linalg.copy", "hivm.hir.copy", "hfusion.load", "hfusion.store"):
                define(op, [copy(val(ins[0]), out=val(outs[0]))])
            elif name == "hfusion.bitcast":
                src, dst = val(ins[0]), val(outs[0])
                if src.element_size() != dst.element_size():
                    raise MlirTextError("hfusion.bitcast: element sizes differ")
                define(op, [copy(src.view(dst.dtype), out=dst)])
            elif name == "hfusion.elemwise_ternary":
                fun = op.attr("fun") or "select"                      # #hfusion.ternary_fn<select | fma>
                if fun == "select":
                    define(op, [write_out(val(outs[0]), select(val(ins[0]), operand(ins[1]), operand(ins[2])))])
                elif fun == "fma":
                    define(op, [write_out(val(outs[0]), elemwise_ternary("fma", operand(ins[0]), operand(ins[1]), operand(ins[2])))])
                else:
                    raise MlirTextError(f"hfusion.elemwise_ternary: fun {fun}")
            elif name == "hivm.hir.load":
                pm = op.attr("pad_mode")
                if pm is None:
                    define(op, [copy(val(ins[0]), out=val(outs[0]))])
                else:
                    pv = re.search(r"pad_value\s*=\s*(%[\w.]+)", op.text)
                    lp = re.search(r"left_padding_num\s*=\s*(%[\w.]+)", op.text)
                    rp = re.search(r"right_padding_num\s*=\s*(%[\w.]+)", op.text)
                    define(op, [load(val(ins[0]), val(outs[0]), pad_mode={"PadValue": "value", "PadFirstElem": "first_elem", "PadNull": "null"}[pm],
                                     pad_value=operand(pv.group(1)) if pv else None,
                                     left_padding_num=operand(lp.group(1)) if lp else -1,
                                     right_padding_num=operand(rp.group(1)) if rp else -1)])
            elif name == "hivm.hir.store":
                m = re.search(r"atomic\s*=\s*<(\w+)>", op.text)
                define(op, [store(val(ins[0]), val(outs[0]), atomic=m.group(1) if m else "none")])
            elif name == "linalg.generic":
                define(op, [self._generic(op, ins, outs, val, operand)])
            elif name == "linalg.reduce" or name == "hivm.hir.vreduce":
                src, dst = val(ins[0]), val(outs[0])
                if name == "linalg.reduce":
                    comb = next((c for c in _REDUCE_COMBINERS if re.search(rf"\b{re.escape(c)}\b", op.text)), None)
                    if comb is None:
                        raise MlirTextError("linalg.reduce: combiner not recognised")
                    kind = _REDUCE_COMBINERS[comb]
                    dims = op.int_list("dimensions")
                else:
                    kind = re.search(r"<(\w+)>", op.text).group(1)
                    dims = op.int_list("reduce_dims")
                if src.dim() != 2 or dims not in ([0], [1]):
                    raise MlirTextError(f"{name}: a 2-D source reduced over one axis is supported, got rank {src.dim()} dims {dims}")
                define(op, [write_out(dst.view(-1) if dst.dim() != 1 else dst, reduce(kind, src, dim=dims[0])).view(dst.shape)])
            elif name in ("hivm.hir.vcumsum", "hivm.hir.vcumprod", "hivm.hir.vcummax", "hivm.hir.vcummin",
                          "hfusion.cumsum", "hfusion.cumprod", "hfusion.cummax", "hfusion.cummin"):
                # `hivm.hir.vcumsum ins(%s : T) outs(%d : T) cum_dims = [k] reverse = false`, or the value form
                # `hfusion.cumsum %s : T cum_dims = [k] reverse = false -> T`
                src = val(ins[0]) if ins else val(re.match(r"\s*(%[\w.]+)", op.text).group(1))
                dims = op.int_list("cum_dims")
                if src.dim() not in (1, 2) or dims is None or len(dims) != 1 or dims[0] >= src.dim():
                    raise MlirTextError(f"{name}: one cumulative axis of a 1-D or 2-D operand is supported")
                two_d = src if src.dim() == 2 else src.view(1, -1)
                axis = dims[0] if src.dim() == 2 else 1
                dst = val(outs[0]) if outs else torch.empty_like(src)
                pn = op.attr("propagate_nan", True)
                y = cumulative(name.rsplit("cum", 1)[1], two_d, dim=axis, reverse=bool(op.attr("reverse", False)),
                               propagate_nan=bool(pn), out=dst if dst.dim() == 2 else dst.view(1, -1))
                define(op, [y.view(src.shape)])
            elif name == "hivm.hir.vsort":
                # `hivm.hir.vsort ins(%s : T) outs(%v, %i : T, Ti) descending = <bool> sort_axis = k` (the last axis)
                src = val(ins[0])
                axis = re.search(r"sort_axis\s*=\s*(-?\d+)", op.text)
                if axis and int(axis.group(1)) not in (-1, src.dim() - 1):
                    raise MlirTextError("hivm.hir.vsort: only the last axis is sorted")
                v, i = sort(src, descending=bool(op.attr("descending", False)))
                res = [write_out(val(outs[0]), v)]
                if len(outs) > 1:
                    dst_i = val(outs[1])
                    res.append(write_out(dst_i, i if dst_i.dtype == torch.int32 else cast(i, dst_i.dtype)))
                define(op, res[:max(len(op.results), 0)] if op.results else [])
            elif name == "hivm.hir.vgather":
                # `hivm.hir.vgather ins(%s : T) indices(%i : Ti) outs(%d : T) [gather_axis = k]` (-1 / absent: the last axis)
                idx_names, _ = op.group("indices")
                if not idx_names:
                    raise MlirTextError("hivm.hir.vgather: indices(...) expected")
                src = val(ins[0])
                m = re.search(r"gather_axis\s*=\s*(-?\d+)", op.text)
                define(op, [gather(src, val(idx_names[0]), dim=int(m.group(1)) if m else -1, out=val(outs[0]))])
            elif name == "hfusion.reduce_with_index":
                kind = re.search(r"<(max|min)>", op.text).group(1)
                v, i = reduce_with_index(kind, val(ins[0]), tie_break_left=bool(op.attr("tie_break_left", True)))
                define(op, [write_out(val(outs[0]), v), write_out(val(outs[1]), i)])
            elif name in ("linalg.matmul", "linalg.matmul_transpose_a", "linalg.matmul_transpose_b", "linalg.batch_matmul"):
                # C = C + A.B (the op accumulates onto its init; an init that is a bare tensor.empty counts as zero).
                # i8 x i8 -> i32 exactly; f16 / bf16 products are accumulated in f32 on the tensor core and rounded
                # once to the result type (the device rule: bishengir/lib/Dialect/HFusion/Transforms/Normalize.cpp:8224-8257)
                a, b, c = val(ins[0]), val(ins[1]), val(outs[0])
                ta, tb = name.endswith("transpose_a"), name.endswith("transpose_b")
                if a.dtype != b.dtype or a.dtype not in (torch.int8, torch.float16, torch.bfloat16):
                    raise MlirTextError(f"{name}: operands {a.dtype} x {b.dtype} (i8, f16 or bf16 pairs are supported)")
                acc_t = torch.int32 if a.dtype == torch.int8 else torch.float32
                if c.dtype not in (acc_t, a.dtype) or (a.dtype == torch.int8 and c.dtype != torch.int32):
                    raise MlirTextError(f"{name}: result type {c.dtype} for {a.dtype} operands")
                fresh = outs[0] in uninitialised
                prod = matmul(a, b, transpose_a=ta, transpose_b=tb, out_dtype=(c.dtype if fresh else acc_t))
                if fresh:
                    define(op, [write_out(c, prod)])
                else:
                    init = c if c.dtype == acc_t else cast(c, acc_t)
                    total = elemwise_binary("add", prod, init)
                    define(op, [write_out(c, total if c.dtype == acc_t else cast(total, c.dtype))])
            else:
                raise MlirTextError(f"op {name} is not supported by this front end")
        return None


_GENERIC_UNARY = {"math.exp": "exp", "math.log": "log", "math.sqrt": "sqrt", "math.rsqrt": "rsqrt", "math.tanh": "tanh", "math.absf": "abs",
                  "math.ceil": "ceil", "math.floor": "floor", "math.erf": "erf", "math.sin": "sin", "math.cos": "cos", "math.exp2": "exp2",
                  "math.log2": "log2", "arith.negf": "negf"}
_GENERIC_BINARY = {"arith.addf": "add", "arith.subf": "sub", "arith.mulf": "mul", "arith.divf": "div", "arith.maximumf": "maxf",
                   "arith.minimumf": "minf", "arith.maxnumf": "maxnumf", "arith.minnumf": "minnumf", "math.powf": "powf"}


def _generic(self, op, ins, outs, val, operand):
    """linalg.generic in the two shapes the reference's tests write by hand: an elementwise body over identity maps
    (all iterators parallel; f32; the body becomes one fused kernel) and a reduction of the last axis whose body is a
    single combiner of the input element and the accumulator (what linalg.reduce says in short)."""
    import torch
    from . import fusion, reduce as reduce_op
    maps = re.findall(r"affine_map<\(([^)]*)\)\s*->\s*\(([^)]*)\)>", op.text)
    iters = re.findall(r'"(parallel|reduction)"', op.text.split("ins(")[0].split("outs(")[0])
    m = re.search(r"\{\s*\^bb0\(([^)]*)\)\s*:(.*)\}\s*(?:->.*)?$", op.text, re.S)
    if not maps or not m:
        raise MlirTextError("linalg.generic: indexing_maps and a region with ^bb0 expected")
    args = [a.split(":")[0].strip() for a in m.group(1).split(",") if a.strip()]
    body = _statements(m.group(2))
    dst = val(outs[0])
    srcs = [val(n) for n in ins]
    ident = lambda mp: [d.strip() for d in mp[0].split(",")] == [d.strip() for d in mp[1].split(",")]
    if len(maps) != len(srcs) + 1 or len(args) != len(srcs) + 1:
        raise MlirTextError("linalg.generic: one indexing map and one block argument per operand expected")
    local = {}                                              # SSA names of the body -> fusion nodes

    def node(name):
        if name in local:
            return local[name]
        v = operand(name)                                   # a value from outside the region
        if isinstance(v, torch.Tensor):
            raise MlirTextError("linalg.generic: the body uses a tensor from outside the region")
        return ("imm", float(v))

    if all(i == "parallel" for i in iters) and all(ident(mp) for mp in maps):
        prob = fusion.problem(list(dst.shape))
        if prob is None or dst.dtype != torch.float32 or any(t.dtype != torch.float32 or t.shape != dst.shape or not t.is_contiguous() for t in srcs):
            raise MlirTextError("linalg.generic: an elementwise body is run for contiguous f32 tensors of rank 1 or 2 of one shape")
        for a, t in zip(args, srcs + [dst]):
            local[a] = ("leaf", t.view(*prob), "full")
        result = None
        for b in body:
            names = re.findall(r"%[\w.]+", b.text.split(":")[0])
            if b.name == "linalg.yield":
                result = node(names[0])
            elif b.name == "arith.constant":
                v, ty = b.text.rsplit(":", 1)
                local[b.results[0]] = ("imm", _float_literal(v.strip(), ty.strip()))
            elif b.name in _GENERIC_UNARY:
                local[b.results[0]] = ("un", _GENERIC_UNARY[b.name], node(names[0]))
            elif b.name in _GENERIC_BINARY:
                local[b.results[0]] = ("bin", _GENERIC_BINARY[b.name], node(names[0]), node(names[1]))
            else:
                raise MlirTextError(f"linalg.generic: {b.name} in an elementwise body is not supported")
        if result is None:
            raise MlirTextError("linalg.generic: the body does not yield")
        if result[0] == "imm":                               # a fill
            from . import elemwise_binary
            return elemwise_binary("add", torch.zeros_like(dst), result[1], out=dst)
        if not fusion.fits(result):
            raise MlirTextError("linalg.generic: the body is too large for one fused kernel")
        fusion.run([(fusion.Lazy(result, list(dst.shape), prob), dst)], prob)
        return dst
    # last-axis reduction: in (d0, .., dk) -> identity, out drops dk, iterators [.., "reduction"], body = one combiner
    if len(srcs) == 1 and iters and iters[-1] == "reduction" and all(i == "parallel" for i in iters[:-1]) and ident(maps[0]) and \
            [d.strip() for d in maps[1][1].split(",") if d.strip()] == [d.strip() for d in maps[0][0].split(",")][:-1]:
        comb = [b for b in body if b.name != "linalg.yield"]
        if len(comb) != 1 or comb[0].name not in _REDUCE_COMBINERS:
            raise MlirTextError("linalg.generic: a reduction body of one combiner op is supported")
        used = set(re.findall(r"%[\w.]+", comb[0].text.split(":")[0]))
        if used != set(args):
            raise MlirTextError("linalg.generic: the combiner must take the input element and the accumulator")
        src = srcs[0]
        rows = src.numel() // max(src.shape[-1], 1)
        out = reduce_op(_REDUCE_COMBINERS[comb[0].name], src.reshape(rows, src.shape[-1]), dim=1)
        from . import copy as copy_op
        copy_op(out.view(-1), out=dst.view(-1))               # a rank-0 result is one element
        return dst
    raise MlirTextError("linalg.generic: only identity-map elementwise bodies and last-axis reductions are supported")


Function._generic = _generic


def parse(text: str) -> Dict[str, Function]:
    """All `func.func`s of a module, by name."""
    text = _strip_comments(text)
    fns: Dict[str, Function] = {}
    for m in re.finditer(r"func\.func\s+(?:private\s+)?@([\w.]+)\s*\(", text):
        args_end = _balanced(text, m.end() - 1, "(", ")")
        arg_text = text[m.end():args_end - 1]
        args, arg_attrs = [], []
        for a in _split_top(arg_text):
            if not a:
                continue
            nm, ty = a.split(":", 1)
            am = re.search(r"\{[^}]*\}\s*$", ty)
            arg_attrs.append(am.group(0).strip() if am else "")       # e.g. {hacc.arg_type = #hacc.arg_type<output>}
            args.append((nm.strip(), re.sub(r"\{[^}]*\}\s*$", "", ty).strip()))
        brace = text.find("{", args_end)
        # skip `attributes {...}` dictionaries: the body is the last brace group that follows the signature
        fn_attrs = ""
        while True:
            head = text[args_end:brace]
            end = _balanced(text, brace, "{", "}")
            if re.search(r"attributes\s*$", head):
                fn_attrs = text[brace:end]
                args_end = end
                brace = text.find("{", end)
                if brace < 0:
                    break
                continue
            break
        if brace < 0:
            continue                                   # a declaration
        body = text[brace + 1:end - 1]
        fn = Function(m.group(1), args, _statements(body))
        fn.arg_attrs, fn.attrs = arg_attrs, fn_attrs
        fns[m.group(1)] = fn
    if not fns:
        raise MlirTextError("no func.func found")
    return fns
