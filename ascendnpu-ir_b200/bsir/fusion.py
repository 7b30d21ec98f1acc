"""Lazy f32 elementwise expressions and their lowering to one fused kernel.

The reference's op fusion outlines a connected group of elementwise / broadcast ops into one function and
compiles that into one device kernel (PURE_ELEMWISE / ANY_PB fusion kinds,
bishengir/lib/Dialect/HFusion/Transforms/OpFusion/FusibleHelper.cpp:52-72).  The front end does the same at run
time: an elementwise op on f32 tensors does not launch anything, it returns a ``Lazy`` that records the
expression; when a value is needed in memory (a reduction reads it, the function returns it, a rounding cast
stores it) the whole expression tree becomes one ``FusedChain`` -- a tape for the accumulator machine of
``bsir_fused_elementwise`` -- and runs as one kernel.

Only f32 arithmetic is fused: an op on f16 / bf16 tensors rounds its result to that type, so fusing two of them
would change the bits.  The casts around an f32 region fold into the chain instead: a widening cast becomes an
operand read in its storage type, a final rounding cast becomes the output type (the shape LegalizeBF16 gives
16-bit elementwise code, bishengir/lib/Dialect/HFusion/Transforms/LegalizeBF16.cpp:243-275).

A node is a tuple: ("leaf", tensor, kind) | ("imm", value) | ("un", fn, node) | ("bin", fn, left, right).
"""
from typing import List, Optional

import torch

UNARY = {"relu", "sqrt", "rsqrt", "rec", "tanh", "exp", "log", "abs", "ceil", "floor", "negf", "round", "square", "erf",
         "sin", "cos", "exp2", "log2", "reciprocal"}
BINARY = {"add", "sub", "mul", "div", "maxf", "minf", "maxnumf", "minnumf", "powf", "divfhp"}
MAX_INSTR, MAX_OPERANDS, MAX_TEMPS = 24, 8, 4


class Overflow(Exception):
    """The expression does not fit one tape (instructions, operands or temporaries)."""


class Lazy:
    """An f32 elementwise expression of ``shape`` that has not been launched; ``dst`` is the buffer the op named
    as its destination (used when the value is materialised as it is)."""

    def __init__(self, node, shape: List[int], dst: Optional[torch.Tensor]):
        self.node, self.shape, self.dst = node, list(shape), dst


def problem(shape: List[int]):
    """[rows, cols] of a chain over a tensor of this shape (rank 1 or 2), or None."""
    if len(shape) == 1:
        return 1, shape[0]
    if len(shape) == 2:
        return shape[0], shape[1]
    return None


def _is_leaf(n) -> bool:
    return n[0] in ("leaf", "imm")


def _weight(n) -> int:
    """Temporaries an evaluation of n needs (Sethi-Ullman numbering for an accumulator machine)."""
    if _is_leaf(n):
        return 0
    if n[0] == "un":
        return _weight(n[2])
    a, b = n[2], n[3]
    if _is_leaf(a) or _is_leaf(b):
        return max(_weight(a), _weight(b))
    wa, wb = _weight(a), _weight(b)
    return max(wa, wb) if wa != wb else wa + 1


def build(node):
    """The FusedChain that leaves the value of ``node`` in the accumulator."""
    from . import FusedChain
    ch = FusedChain()
    handles = {}
    free = list(range(MAX_TEMPS - 1, -1, -1))

    def src(n):
        if n[0] == "imm":
            return float(n[1])
        key = (n[1].data_ptr(), tuple(n[1].shape), tuple(n[1].stride()), n[1].dtype, n[2])
        if key not in handles:
            if len(handles) == MAX_OPERANDS:
                raise Overflow("operands")
            handles[key] = ch.operand(n[1], n[2])
        return ch.op(handles[key])

    def gen(n):
        if _is_leaf(n):
            ch.load(src(n))
        elif n[0] == "un":
            gen(n[2])
            ch.unary(n[1])
        else:
            fn, a, b = n[1], n[2], n[3]
            if _is_leaf(b):
                gen(a)
                ch.binary(fn, src(b))
            elif _is_leaf(a):
                gen(b)
                ch.rbinary(fn, src(a))
            else:
                if not free:
                    raise Overflow("temporaries")
                # the side that needs more temporaries goes first, while all of them are free
                first, second, emit = (b, a, ch.binary) if _weight(b) >= _weight(a) else (a, b, ch.rbinary)
                gen(first)
                t = free.pop()
                ch.save(t)
                gen(second)
                emit(fn, ("tmp", t))
                free.append(t)
        if len(ch._tape) > MAX_INSTR:
            raise Overflow("instructions")

    gen(node)
    return ch


def fits(node) -> bool:
    try:
        build(node)
        return True
    except Overflow:
        return False


def materialise(lazy: Lazy, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Runs the expression as one kernel into ``out`` (any float type: the single rounding), else into the op's own
    destination, else into a new f32 tensor."""
    rows, cols = problem(lazy.shape)
    dst = out if out is not None else lazy.dst
    if dst is None or list(dst.shape) != lazy.shape or (dst.dim() > 1 and dst.stride(-1) != 1):
        dev = next((n.device for n in _leaves(lazy.node)), torch.device("cuda"))
        dst = torch.empty(lazy.shape, dtype=torch.float32 if out is None else out.dtype, device=dev)
    build(lazy.node).run(rows, cols, outs=[(dst.view(rows, cols) if dst.dim() != 2 else dst, -1)])
    return dst


def _leaves(n):
    if n[0] == "leaf":
        yield n[1]
    elif n[0] == "un":
        yield from _leaves(n[2])
    elif n[0] == "bin":
        yield from _leaves(n[2])
        yield from _leaves(n[3])
