"""Lazy f32 elementwise / last-axis-reduce expressions and their lowering to fused kernels.

The reference's op fusion outlines a connected group of elementwise, broadcast and last-axis reduce ops into
one function and compiles that into one device kernel (fusion kinds PURE_ELEMWISE / ANY_PB / LAST_AXIS_PBR,
bishengir/lib/Dialect/HFusion/Transforms/OpFusion/FusibleHelper.cpp:52-72).  The front end does the same at run
time: such an op on f32 tensors does not launch anything, it returns a ``Lazy`` that records the expression;
values that must exist in memory (a function result, the destination of a rounding cast, the operand of an op
that is not fusible) are collected as requests and served together: all requests over the same [rows, cols]
problem become ONE ``FusedChain`` -- a tape for the accumulator machine of ``bsir_fused_elementwise`` with up to
four outputs -- in which a sub-expression with several users is computed once and kept in a temporary.

Only f32 arithmetic is fused: an op on f16 / bf16 tensors rounds its result to that type, so fusing two of them
would change the bits.  The casts around an f32 region fold into the chain instead: a widening cast becomes an
operand read in its storage type, a final rounding cast becomes the output type (the shape LegalizeBF16 gives
16-bit elementwise code, bishengir/lib/Dialect/HFusion/Transforms/LegalizeBF16.cpp:243-275).  Elementwise
regions keep the bits of op-by-op execution; a fused row sum associates as a tree.

A node is a tuple: ("leaf", tensor, kind) | ("imm", value) | ("un", fn, node) | ("bin", fn, left, right) |
("red", kind, node) -- the reduction of node over each row, as a value that is uniform along the row.
"""
from typing import Dict, List, Optional, Tuple

import torch

UNARY = {"relu", "sqrt", "rsqrt", "rec", "tanh", "exp", "log", "abs", "ceil", "floor", "negf", "round", "square", "erf",
         "sin", "cos", "exp2", "log2", "reciprocal"}
BINARY = {"add", "sub", "mul", "div", "maxf", "minf", "maxnumf", "minnumf", "powf", "divfhp"}
REDUCE = {"sum", "prod", "max", "min"}
MAX_INSTR, MAX_OPERANDS, MAX_TEMPS, MAX_OUTPUTS = 24, 8, 4, 4


class Overflow(Exception):
    """The expressions do not fit one tape (instructions, operands, temporaries or outputs)."""


class Lazy:
    """An f32 expression that has not been launched.  ``prob`` is the [rows, cols] problem it is evaluated in;
    ``per_row`` values have shape [rows] (a row reduction and what is computed from it).  ``dst`` is a buffer the
    value may be written to when it is wanted as it is (f32)."""

    def __init__(self, node, shape: List[int], prob: Tuple[int, int], per_row: bool = False, dst: Optional[torch.Tensor] = None):
        self.node, self.shape, self.prob, self.per_row, self.dst = node, list(shape), tuple(prob), per_row, dst


def problem(shape: List[int]):
    """[rows, cols] of an elementwise chain over a tensor of this shape (rank 1 or 2), or None."""
    if len(shape) == 1:
        return 1, shape[0]
    if len(shape) == 2:
        return shape[0], shape[1]
    return None


def _is_leaf(n) -> bool:
    return n[0] in ("leaf", "imm")


def _children(n):
    return (n[2],) if n[0] in ("un", "red") else (n[2], n[3]) if n[0] == "bin" else ()


def _walk(n, seen=None):
    seen = set() if seen is None else seen
    if id(n) in seen:
        return
    seen.add(id(n))
    yield n
    for c in _children(n):
        yield from _walk(c, seen)


def has_reduction(n) -> bool:
    return any(m[0] == "red" for m in _walk(n))


def build(requests):
    """One FusedChain for ``requests`` = [(node, per_row)], and the temporary (or -1: the accumulator) each value
    ends in.  A node that several users share is computed once."""
    from . import FusedChain
    if len(requests) > MAX_OUTPUTS:
        raise Overflow("outputs")
    ch = FusedChain()
    handles: Dict[tuple, int] = {}
    free = list(range(MAX_TEMPS - 1, -1, -1))
    uses: Dict[int, int] = {}

    def count(n):                                   # users of every node, over all requests
        uses[id(n)] = uses.get(id(n), 0) + 1
        if uses[id(n)] == 1:
            for c in _children(n):
                count(c)

    for n, _ in requests:
        count(n)
    kept: Dict[int, int] = {}                       # shared node -> the temporary that keeps it
    weight_memo: Dict[int, int] = {}

    def weight(n) -> int:
        """Scratch temporaries an evaluation of n needs (Sethi-Ullman numbering for an accumulator machine)."""
        if id(n) in weight_memo:
            return weight_memo[id(n)]
        if _is_leaf(n) or id(n) in kept:
            w = 0
        elif n[0] in ("un", "red"):
            w = weight(n[2])
        else:
            a, b = n[2], n[3]
            if direct(a) or direct(b):
                w = max(weight(a), weight(b))
            else:
                wa, wb = weight(a), weight(b)
                w = max(wa, wb) if wa != wb else wa + 1
        weight_memo[id(n)] = w
        return w

    def direct(n) -> bool:                          # usable as the source of an instruction as it is
        return _is_leaf(n) or id(n) in kept

    def src(n):
        if id(n) in kept:
            return ("tmp", kept[id(n)])
        if n[0] == "imm":
            return float(n[1])
        t, kind = n[1], n[2]
        key = (t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.dtype, kind)
        if key not in handles:
            if len(handles) == MAX_OPERANDS:
                raise Overflow("operands")
            handles[key] = ch.operand(t, kind)
        return ch.op(handles[key])

    def take_temp() -> int:
        if not free:
            raise Overflow("temporaries")
        return free.pop()

    def gen(n):
        """Leaves the value of n in the accumulator."""
        if direct(n):
            ch.load(src(n))
        elif n[0] == "un":
            gen(n[2])
            ch.unary(n[1])
        elif n[0] == "red":
            gen(n[2])
            ch.reduce(n[1])
        else:
            fn, a, b = n[1], n[2], n[3]
            if direct(b):
                gen(a)
                ch.binary(fn, src(b))
            elif direct(a):
                gen(b)
                ch.rbinary(fn, src(a))
            else:
                # the side that needs more scratch goes first, while it is all free
                first, second, emit = (b, a, ch.binary) if weight(b) >= weight(a) else (a, b, ch.rbinary)
                gen(first)
                if id(first) in kept:               # gen kept it because it is shared
                    t, scratch = kept[id(first)], False
                else:
                    t, scratch = take_temp(), True
                    ch.save(t)
                gen(second)
                emit(fn, ("tmp", t))
                if scratch:
                    free.append(t)
        if uses.get(id(n), 0) > 1 and not _is_leaf(n) and id(n) not in kept:
            kept[id(n)] = take_temp()               # several users: keep it (never released: users may come late)
            ch.save(kept[id(n)])
            weight_memo.clear()
        if len(ch._tape) > MAX_INSTR:
            raise Overflow("instructions")

    where = []
    for i, (n, _) in enumerate(requests):
        last = i == len(requests) - 1
        if id(n) in kept:                           # computed on the way to an earlier output
            where.append(kept[id(n)])
            continue
        gen(n)
        if last:
            where.append(-1)
        elif id(n) in kept:
            where.append(kept[id(n)])
        else:
            t = take_temp()                         # an output that is not the last one waits in a temporary
            ch.save(t)
            kept[id(n)] = t
            where.append(t)
    return ch, where


def fits(node) -> bool:
    try:
        build([(node, False)])
        return True
    except Overflow:
        return False


def run(requests, prob) -> None:
    """requests = [(Lazy, destination tensor)] over the problem ``prob``: one kernel where the tape holds them all,
    else one kernel each; chains the library cannot run as they are (a row too long for a block, ragged rows with
    a reduction) are evaluated op by op."""
    from . import BsirError
    rows, cols = prob
    try:
        ch, where = build([(lz.node, lz.per_row) for lz, _ in requests])
        outs = []
        for (lz, dst), tmp in zip(requests, where):
            outs.append((dst.reshape(rows) if lz.per_row else dst.view(rows, cols) if dst.dim() != 2 else dst, tmp))
        try:
            ch.run(rows, cols, outs=outs)
        except BsirError:
            if not any(has_reduction(lz.node) for lz, _ in requests):
                raise
            for lz, dst in requests:
                _store(lz, dst, evaluate(lz.node, prob))
    except Overflow:
        if len(requests) == 1:
            _store(requests[0][0], requests[0][1], evaluate(requests[0][0].node, prob))
        else:
            for r in requests:
                run([r], prob)


def _store(lz: Lazy, dst: torch.Tensor, value: torch.Tensor) -> None:
    """An op-by-op result (f32 [rows, cols]) into its destination: one rounding when the destination is narrower."""
    from . import cast, copy
    v = value[:, 0].contiguous() if lz.per_row else value
    v = v.reshape(dst.shape)
    if dst.dtype == torch.float32:
        copy(v, out=dst)
    else:
        cast(v, dst.dtype, out=dst)


def evaluate(n, prob) -> torch.Tensor:
    """The value of a node as an f32 [rows, cols] tensor, one library call per op (the fallback of ``run``)."""
    from . import cast, elemwise_binary, elemwise_unary, reduce
    rows, cols = prob
    if n[0] == "imm":
        return torch.full((rows, cols), float(n[1]), dtype=torch.float32, device="cuda")
    if n[0] == "leaf":
        t = n[1] if n[1].dtype == torch.float32 else cast(n[1], torch.float32)
        if n[2] == "row_vector":
            return t.reshape(1, cols).expand(rows, cols).contiguous()
        if n[2] == "col_vector":
            return t.reshape(rows, 1).expand(rows, cols).contiguous()
        if n[2] == "scalar":
            return t.reshape(1, 1).expand(rows, cols).contiguous()
        return t.reshape(rows, cols)
    if n[0] == "un":
        return elemwise_unary(n[1], evaluate(n[2], prob))
    if n[0] == "red":
        return reduce(n[1], evaluate(n[2], prob), dim=1).reshape(rows, 1).expand(rows, cols).contiguous()
    return elemwise_binary(n[1], evaluate(n[2], prob), evaluate(n[3], prob))
