"""bsir -- host-side mirror of the HFusion / HIVM operator surface on top of the C ABI.

The functions keep the reference's op names and attribute spellings
(``hfusion.elemwise_binary {fun = ...}``, ``hfusion.cast {round_mode = ..., enable_saturate}``,
``hfusion.reduce_with_index {tie_break_left}``, ...) and take CUDA tensors; each one is a thin
call into ``libbsir_b200.so`` (``include/bsir_b200.h``).  There is no fallback: if the library
has not been built, importing :func:`lib` raises.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libbsir_b200.so")

# ---------------------------------------------------------------------------- enums (bsir_b200.h)
F32, F16, BF16, I8, I16, I32, I64, U8, U16, U32, U64, BOOL = range(12)
_TORCH2DT = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int8: I8, torch.int16: I16,
             torch.int32: I32, torch.int64: I64, torch.uint8: U8, torch.bool: BOOL}
for _n, _c in (("uint16", U16), ("uint32", U32), ("uint64", U64)):
    if hasattr(torch, _n):
        _TORCH2DT[getattr(torch, _n)] = _c
_DT2TORCH = {v: k for k, v in _TORCH2DT.items()}
DTYPE_NAMES = {"f32": F32, "f16": F16, "bf16": BF16, "i8": I8, "i16": I16, "i32": I32, "i64": I64, "u8": U8,
               "u16": U16, "u32": U32, "u64": U64, "i1": BOOL, "bool": BOOL}

ROUND_MODE = {"rint": 0, "round": 1, "floor": 2, "ceil": 3, "trunc": 4, "odd": 5, "truncwithoverflow": 6}
OVERFLOW_MODE = {"wrap": 0, "saturate": 1, "ascend_saturate_trunc_via_f16": 2, "ascend_double_round_via_f16": 3}
UNARY_FN = {"relu": 0, "sqrt": 1, "rsqrt": 2, "rec": 3, "vnot": 4, "tanh": 5, "sin": 6, "cos": 7, "atan": 8, "tan": 9,
            "absi": 10, "erf": 11, "log2": 12, "log10": 13, "log1p": 14, "exp2": 15, "expm1": 16, "ilogb": 17,
            "asin": 18, "acos": 19, "asinh": 20, "acosh": 21, "atanh": 22, "sinh": 23, "lgamma": 24, "cosh": 25,
            "nearbyint": 26, "exp": 100, "log": 101, "abs": 102, "ceil": 103, "floor": 104, "negf": 105,
            "reciprocal": 106, "round": 107, "square": 110}
BINARY_FN = {"vor": 0, "vand": 1, "vxor": 2, "minf": 3, "maxf": 4, "powf": 5, "mod": 6, "modui": 7, "shli": 8,
             "shrsi": 9, "shrui": 10, "ldexp": 11, "ceildivsi": 12, "ceildivui": 13, "floordivsi": 14, "powi": 15,
             "minnumf": 16, "maxnumf": 17, "atan2": 18, "divfhp": 19, "copysign": 20, "add": 100, "sub": 101,
             "mul": 102, "div": 103, "div_unsigned": 104, "max_signed": 105, "min_signed": 106,
             "max_unsigned": 107, "min_unsigned": 108}
COMPARE_FN = {"veq": 0, "vne": 1, "vle": 2, "vlt": 3, "vge": 4, "vgt": 5, "vule": 6, "vult": 7, "vuge": 8, "vugt": 9}
REDUCE_KIND = {"sum": 0, "prod": 1, "max": 2, "min": 3, "any": 4, "all": 5, "xori": 6, "ori": 7, "andi": 8}
RWI_KIND = {"min": 0, "max": 1, "minui": 2, "maxui": 3}
KERNEL_KIND = {"elemwise_binary": 0, "elemwise_unary": 1, "cast": 2, "rms_norm": 3, "softmax": 4,
               "quant_per_token": 5, "reduce_with_index": 6, "reduce": 7, "matmul_w8a8": 8, "matmul_w4a16": 9}


class BsirError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"bsir status {status}: {text}")
        self.status = status


class Operand(C.Structure):
    _fields_ = [("data", C.c_void_p), ("strides", C.c_int64 * 3), ("scalar_bits", C.c_uint64)]


class KernelDesc(C.Structure):
    _fields_ = [("kind", C.c_int32), ("fn", C.c_int32), ("dtype", C.c_int32), ("dst_dtype", C.c_int32),
                ("round_mode", C.c_int32), ("overflow_mode", C.c_int32), ("flags", C.c_int32), ("rank", C.c_int32),
                ("sizes", C.c_int64 * 4), ("eps", C.c_float)]


def memref_type(rank: int):
    class MemRef(C.Structure):
        _fields_ = [("allocated", C.c_void_p), ("aligned", C.c_void_p), ("offset", C.c_int64),
                    ("sizes", C.c_int64 * rank), ("strides", C.c_int64 * rank)]
    return MemRef


_MEMREF = {r: memref_type(r) for r in (1, 2, 3)}


def memref(t: torch.Tensor, rank: Optional[int] = None):
    """MLIR memref descriptor of a tensor (base = aligned + offset, strides in elements)."""
    rank = t.dim() if rank is None else rank
    m = _MEMREF[rank]()
    base = t.untyped_storage().data_ptr() if t.numel() else 0
    m.allocated = base
    m.aligned = base
    m.offset = t.storage_offset()
    for i in range(rank):
        m.sizes[i] = t.shape[i]
        m.strides[i] = t.stride(i)
    return m


_lib = None


def lib() -> C.CDLL:
    """Loads the C-ABI library.  Raises if it was not built: there is no other compute path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise BsirError(-100, f"{LIB_PATH} is missing: build it with `python ascendnpu-ir_b200/build.py`")
        L = C.CDLL(LIB_PATH)
        L.bsir_last_error.restype = C.c_char_p
        L.bsir_status_string.restype = C.c_char_p
        L.bsir_version.restype = C.c_char_p
        L.bsir_get_stream.restype = C.c_void_p
        L.bsir_launch_count.restype = C.c_int64
        L.bsir_reduce_with_index_workspace_bytes.restype = C.c_int64
        L.bsir_matmul_w8a8_workspace_bytes.restype = C.c_int64
        L.bsir_fused_elementwise_source.restype = C.c_int64
        _lib = L
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise BsirError(rc, lib().bsir_last_error().decode() or lib().bsir_status_string(rc).decode())


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t: torch.Tensor) -> int:
    try:
        return _TORCH2DT[t.dtype]
    except KeyError:
        raise BsirError(-4, f"unsupported tensor dtype {t.dtype}") from None


def _i64arr(v: Sequence[int], n: int = 3):
    a = (C.c_int64 * n)()
    for i, x in enumerate(v):
        a[i] = int(x)
    return a


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(t.data_ptr() if t is not None else 0)


def _scalar_bits(v, dtype: torch.dtype) -> int:
    t = torch.tensor([v], dtype=dtype)
    nbytes = t.element_size()
    raw = t.view(torch.uint8).numpy().tobytes() + b"\0" * (8 - nbytes)
    return int.from_bytes(raw, "little")


def _operand(x, shape: Sequence[int], dtype: torch.dtype) -> Operand:
    o = Operand()
    if isinstance(x, torch.Tensor):
        if x.dtype != dtype:
            raise BsirError(-4, f"operand dtype {x.dtype} != {dtype}")
        if x.dim() != len(shape):
            raise BsirError(-2, f"operand rank {x.dim()} != {len(shape)}")
        o.data = x.data_ptr()
        for i in range(len(shape)):
            if x.shape[i] == shape[i]:
                o.strides[i] = x.stride(i)
            elif x.shape[i] == 1:
                o.strides[i] = 0  # inline broadcast
            else:
                raise BsirError(-2, f"operand shape {tuple(x.shape)} does not broadcast to {tuple(shape)}")
    else:
        o.data = None
        o.scalar_bits = _scalar_bits(x, dtype)
    return o


def _result_shape(*xs) -> Sequence[int]:
    ts = [x for x in xs if isinstance(x, torch.Tensor)]
    if not ts:
        raise BsirError(-1, "at least one operand must be a tensor")
    return list(torch.broadcast_shapes(*[t.shape for t in ts]))


def _first_tensor(*xs) -> torch.Tensor:
    return next(x for x in xs if isinstance(x, torch.Tensor))


# ---------------------------------------------------------------------------- elementwise
def elemwise_unary(fun: str, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hfusion.elemwise_unary`` / ``linalg.elemwise_unary`` {fun}."""
    shape = list(x.shape)
    out = torch.empty_like(x, memory_format=torch.contiguous_format) if out is None else out
    op = _operand(x, shape, x.dtype)
    _check(lib().bsir_elemwise_unary(UNARY_FN[fun], _dt(x), len(shape), _i64arr(shape), C.byref(op), _ptr(out),
                                     _i64arr(out.stride()), _stream()))
    return out


def elemwise_binary(fun: str, a, b, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hfusion.elemwise_binary`` / ``linalg.elemwise_binary`` {fun}; a or b may be a Python scalar."""
    ref = _first_tensor(a, b)
    shape = _result_shape(a, b)
    out = torch.empty(shape, dtype=ref.dtype, device=ref.device) if out is None else out
    oa, ob = _operand(a, shape, ref.dtype), _operand(b, shape, ref.dtype)
    _check(lib().bsir_elemwise_binary(BINARY_FN[fun], _dt(ref), len(shape), _i64arr(shape), C.byref(oa), C.byref(ob),
                                      _ptr(out), _i64arr(out.stride()), _stream()))
    return out


def elemwise_ternary(fun: str, a, b, c, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hfusion.elemwise_ternary`` {fun = fma}: a * b + c with one rounding; any operand may be a Python scalar."""
    if fun != "fma":
        raise BsirError(-5, "elemwise_ternary: fun must be 'fma' (select is bsir.select)")
    ref = _first_tensor(a, b, c)
    shape = _result_shape(a, b, c)
    out = torch.empty(shape, dtype=ref.dtype, device=ref.device) if out is None else out
    oa, ob, oc = (_operand(x, shape, ref.dtype) for x in (a, b, c))
    _check(lib().bsir_elemwise_ternary(1, _dt(ref), len(shape), _i64arr(shape), C.byref(oa), C.byref(ob), C.byref(oc),
                                       _ptr(out), _i64arr(out.stride()), _stream()))
    return out


def vadd(a, b, out=None):
    """``hivm.hir.vadd``."""
    return elemwise_binary("add", a, b, out)


def vsub(a, b, out=None):
    return elemwise_binary("sub", a, b, out)


def vmul(a, b, out=None):
    return elemwise_binary("mul", a, b, out)


def vdiv(a, b, out=None):
    return elemwise_binary("div", a, b, out)


def compare(compare_fn: str, a, b) -> torch.Tensor:
    """``hfusion.compare`` {compare_fn}; returns a bool tensor."""
    ref = _first_tensor(a, b)
    shape = _result_shape(a, b)
    out = torch.empty(shape, dtype=torch.bool, device=ref.device)
    oa, ob = _operand(a, shape, ref.dtype), _operand(b, shape, ref.dtype)
    _check(lib().bsir_compare(COMPARE_FN[compare_fn], _dt(ref), len(shape), _i64arr(shape), C.byref(oa), C.byref(ob),
                              _ptr(out), _i64arr(out.stride()), _stream()))
    return out


def select(cond: torch.Tensor, a, b) -> torch.Tensor:
    """``hfusion.select``: cond ? a : b."""
    ref = _first_tensor(a, b)
    shape = _result_shape(cond, a, b)
    out = torch.empty(shape, dtype=ref.dtype, device=ref.device)
    oc = _operand(cond, shape, torch.bool)
    oa, ob = _operand(a, shape, ref.dtype), _operand(b, shape, ref.dtype)
    _check(lib().bsir_select(_dt(ref), len(shape), _i64arr(shape), C.byref(oc), C.byref(oa), C.byref(ob), _ptr(out),
                             _i64arr(out.stride()), _stream()))
    return out


def default_round_mode(src: torch.dtype, dst: torch.dtype) -> str:
    """The round mode the reference picks for a conversion that names none (``selectRoundMode``,
    bishengir/include/bishengir/Dialect/Utils/Util.h:180-213): float -> integer truncates, everything else rounds
    to nearest even."""
    if src.is_floating_point and not dst.is_floating_point:
        return "trunc"
    return "rint"


def cast(x: torch.Tensor, dtype: torch.dtype, round_mode: str = "rint", enable_saturate: bool = False,
         overflow_mode: Optional[str] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hfusion.cast`` {round_mode, enable_saturate}; ``overflow_mode`` selects a named variant."""
    ov = OVERFLOW_MODE[overflow_mode] if overflow_mode else (1 if enable_saturate else 0)
    out = torch.empty(x.shape, dtype=dtype, device=x.device) if out is None else out
    shape = list(x.shape)
    _check(lib().bsir_cast(_dt(x), _TORCH2DT[dtype], ROUND_MODE[round_mode], ov, len(shape), _i64arr(shape), _ptr(x),
                           _i64arr(x.stride()), _ptr(out), _i64arr(out.stride()), _stream()))
    return out


def copy(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hivm.hir.load`` / ``store`` / ``copy``."""
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device) if out is None else out
    shape = list(x.shape)
    _check(lib().bsir_copy(_dt(x), len(shape), _i64arr(shape), _ptr(x), _i64arr(x.stride()), _ptr(out),
                           _i64arr(out.stride()), _stream()))
    return out


def transpose(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hivm.hir.vtranspose`` / ``linalg.transpose`` of the last two axes of a 2-D or 3-D tensor (a copy whose source
    is the transposed view: the library runs it with its tiled transposition kernel)."""
    if x.dim() not in (2, 3):
        raise BsirError(-2, "transpose: a 2-D or 3-D tensor")
    return copy(x.transpose(-1, -2), out=out)


PAD_MODE = {"null": 0, "first_elem": 1, "value": 2}
ATOMIC_KIND = {"none": 0, "add": 1, "max": 2, "min": 3, "and": 4, "or": 5, "xor": 6, "cas": 7, "xchg": 8, "umax": 9,
               "umin": 10}


def load(x: torch.Tensor, out: torch.Tensor, pad_mode: str = "null", pad_value=None, left_padding_num: int = -1,
         right_padding_num: int = -1) -> torch.Tensor:
    """``hivm.hir.load`` with ``pad_mode`` / ``pad_value`` / ``left_padding_num`` / ``right_padding_num``:
    pads the last dimension of ``x`` into ``out`` (same leading shape, wider last dimension)."""
    shape = list(x.shape)
    pv = None
    if pad_value is not None:
        pv = torch.tensor([pad_value], dtype=x.dtype).contiguous()     # one element of the dtype, host memory
    _check(lib().bsir_load(_dt(x), len(shape), _i64arr(shape), _ptr(x), _i64arr(x.stride()), _ptr(out),
                           _i64arr(out.stride()), C.c_int64(out.shape[-1]), PAD_MODE[pad_mode],
                           C.c_void_p(pv.data_ptr() if pv is not None else None), C.c_int64(left_padding_num),
                           C.c_int64(right_padding_num), _stream()))
    return out


def store(x: torch.Tensor, out: torch.Tensor, atomic: str = "none") -> torch.Tensor:
    """``hivm.hir.store`` with ``atomic = <kind>``: out = out <kind> x (a copy for "none")."""
    shape = list(x.shape)
    _check(lib().bsir_store(_dt(x), len(shape), _i64arr(shape), _ptr(x), _i64arr(x.stride()), _ptr(out),
                            _i64arr(out.stride()), ATOMIC_KIND[atomic], _stream()))
    return out


# ---------------------------------------------------------------------------- fused elementwise chains
class _ChainOperand(C.Structure):
    _fields_ = [("data", C.c_void_p), ("row_stride", C.c_int64), ("dtype", C.c_int32), ("kind", C.c_int32)]


class _ChainInstr(C.Structure):
    _fields_ = [("op", C.c_int32), ("fn", C.c_int32), ("src_kind", C.c_int32), ("src", C.c_int32), ("imm", C.c_float)]


class _ChainOutput(C.Structure):
    _fields_ = [("data", C.c_void_p), ("row_stride", C.c_int64), ("dtype", C.c_int32), ("tmp", C.c_int32)]


class FusedChain:
    """A chain of elementwise ops over a [rows, cols] problem, run as ONE kernel (``bsir_fused_elementwise``): what
    HFusion's op fusion outlines as a PURE_ELEMWISE / ANY_PB function.  f32 arithmetic, one rounding per output.

        ch = FusedChain()
        x, g, r = ch.operand(x_t), ch.operand(gamma_t), ch.operand(rstd_t)   # [rows,cols], [cols], [rows]
        ch.load(r); ch.binary("mul", x); ch.rbinary("mul", g)               # gamma * (rstd * x)
        y = ch.run(out_dtype=torch.bfloat16)

    An operand's shape decides how it is broadcast: [rows, cols] full, [cols] or [1, cols] the same for every row,
    [rows] (when rows != cols) or [rows, 1] one value per row, a 0-d / 1-element tensor a scalar.  ``src`` of an
    instruction is an operand handle, ``("tmp", k)`` or a Python number (immediate)."""

    def __init__(self):
        self._ops, self._tape, self._shape = [], [], None

    def operand(self, t: torch.Tensor, kind: Optional[str] = None) -> int:
        self._ops.append((t, kind))
        return len(self._ops) - 1

    def _src(self, src):
        if isinstance(src, tuple):
            return 1, int(src[1]), 0.0
        if isinstance(src, (float, int)) and not isinstance(src, bool):
            return 2, 0, float(src)
        raise BsirError(-5, "source must be an operand handle (use .op(handle)), ('tmp', k) or a number")

    def op(self, handle: int):
        """Marks an operand handle as a source (plain ints are immediates)."""
        return ("operand", handle)

    def _emit(self, op, fn, src):
        if isinstance(src, tuple) and src[0] == "operand":
            kind, idx, imm = 0, int(src[1]), 0.0
        elif src is None:
            kind, idx, imm = 0, 0, 0.0
        else:
            kind, idx, imm = self._src(src)
        self._tape.append((op, fn, kind, idx, imm))
        return self

    def load(self, src):
        return self._emit(0, 0, src)

    def unary(self, fun: str):
        return self._emit(1, UNARY_FN[fun], None)

    def binary(self, fun: str, src):
        """acc = fun(acc, src)"""
        return self._emit(2, BINARY_FN[fun], src)

    def rbinary(self, fun: str, src):
        """acc = fun(src, acc)"""
        return self._emit(3, BINARY_FN[fun], src)

    def save(self, tmp: int):
        self._tape.append((4, 0, 1, int(tmp), 0.0))
        return self

    def reduce(self, kind: str):
        """acc = reduce of acc over the row (sum / prod / max / min), broadcast back to every element of the row.
        A chain with reductions is a LAST_AXIS_PBR function: it runs only as a compiled kernel that keeps the row in
        registers.  An output given as a [rows] (or [rows, 1]) tensor takes the row's value."""
        self._tape.append((5, REDUCE_KIND[kind], 0, 0, 0.0))
        return self

    def run(self, rows: Optional[int] = None, cols: Optional[int] = None, out_dtype: Optional[torch.dtype] = None,
            outs: Optional[Sequence] = None):
        """Runs the tape.  ``outs``: list of (tensor-or-dtype, tmp) with tmp = -1 for the accumulator; default one
        output taking the accumulator.  Returns the output tensor(s)."""
        full = next((t for t, k in self._ops if t.dim() == 2 and (k in (None, "full")) and t.shape[0] > 1 and t.shape[1] > 1), None)
        if rows is None or cols is None:
            if full is None:
                raise BsirError(-2, "rows / cols are needed when no operand is a full [rows, cols] tensor")
            rows, cols = full.shape
        dev = self._ops[0][0].device if self._ops else torch.device("cuda")
        ins = (_ChainOperand * max(1, len(self._ops)))()
        for i, (t, kind) in enumerate(self._ops):
            if kind is None:
                if t.numel() == 1:
                    kind = "scalar"
                elif t.dim() == 2 and tuple(t.shape) == (rows, cols):
                    kind = "full"
                elif (t.dim() == 1 and t.shape[0] == cols and cols != rows) or (t.dim() == 2 and tuple(t.shape) == (1, cols)):
                    kind = "row_vector"
                elif (t.dim() == 1 and t.shape[0] == rows) or (t.dim() == 2 and tuple(t.shape) == (rows, 1)):
                    kind = "col_vector"
                else:
                    raise BsirError(-2, f"operand {i} of shape {tuple(t.shape)} does not broadcast to [{rows}, {cols}]")
            k = {"full": 0, "row_vector": 1, "col_vector": 2, "scalar": 3}[kind]
            if k == 0 and t.stride(1) != 1 and cols > 1:
                raise BsirError(-3, "innermost dimension must be unit-stride")
            if k in (1, 2) and not t.is_contiguous():
                t = t.contiguous()
                self._ops[i] = (t, kind)
            ins[i] = _ChainOperand(t.data_ptr(), t.stride(0) if k == 0 and rows > 1 else cols, _dt(t), k)
        tape = (_ChainInstr * len(self._tape))(*[_ChainInstr(*t) for t in self._tape])
        spec = outs if outs is not None else [(out_dtype or (full.dtype if full is not None else torch.float32), -1)]
        tensors = []
        carr = (_ChainOutput * len(spec))()
        for i, (o, tmp) in enumerate(spec):
            t = o if isinstance(o, torch.Tensor) else torch.empty((rows, cols), dtype=o, device=dev)
            tensors.append(t)
            per_row = cols != 1 and (t.dim() == 1 and t.shape[0] == rows or t.dim() == 2 and tuple(t.shape) == (rows, 1))
            if per_row and not t.is_contiguous():
                raise BsirError(-3, "a per-row output must be contiguous")
            carr[i] = _ChainOutput(t.data_ptr(), 0 if per_row else t.stride(0) if rows > 1 else cols, _dt(t), int(tmp))
        _check(lib().bsir_fused_elementwise(C.c_int64(rows), C.c_int64(cols), len(self._ops), ins, len(self._tape), tape,
                                            len(spec), carr, _stream()))
        return tensors[0] if len(tensors) == 1 else tuple(tensors)

    @staticmethod
    def last_path() -> str:
        """How this thread's last chain ran: "compiled" (a kernel built for the chain with NVRTC), "interpreted"
        (the tape interpreter kernel) or "none"."""
        return {0: "none", 1: "interpreted", 2: "compiled"}[int(lib().bsir_fused_elementwise_path())]

    def _tables_without_data(self, outs):
        """Operand / tape / output tables carrying dtypes and kinds only (for source() and compile())."""
        ins = (_ChainOperand * max(1, len(self._ops)))()
        for i, (t, kind) in enumerate(self._ops):
            if kind is None:
                kind = "scalar" if t.numel() == 1 else "full" if t.dim() == 2 and min(t.shape) > 1 else None
            if kind is None:
                raise BsirError(-2, f"operand {i}: say kind='row_vector' or 'col_vector' for a vector")
            ins[i] = _ChainOperand(None, 0, _dt(t), {"full": 0, "row_vector": 1, "col_vector": 2, "scalar": 3}[kind])
        tape = (_ChainInstr * len(self._tape))(*[_ChainInstr(*t) for t in self._tape])
        spec = outs if outs is not None else [(torch.float32, -1)]
        carr = (_ChainOutput * len(spec))()
        for i, (o, tmp) in enumerate(spec):
            per_row = isinstance(o, torch.Tensor) and o.dim() == 1          # a [rows] tensor stands for a per-row output
            carr[i] = _ChainOutput(None, 0 if per_row else 1, _dt(o) if isinstance(o, torch.Tensor) else _TORCH2DT[o], int(tmp))
        return ins, tape, carr, len(spec)

    def source(self, outs: Optional[Sequence] = None, contiguous: bool = True, in_place: bool = False,
               row_grid: bool = False, cols: int = 4096) -> str:
        """The CUDA C++ of the kernel that is compiled for this chain (no device needed).  ``cols`` matters for chains
        with reductions only: their thread geometry follows the row length."""
        ins, tape, carr, n_out = self._tables_without_data(outs)
        flags = (1 if contiguous else 0) | (2 if in_place else 0) | (4 if row_grid else 0) | ((cols // 8) << 8)
        need = lib().bsir_fused_elementwise_source(len(self._ops), ins, len(self._tape), tape, n_out, carr, flags, None, C.c_int64(0))
        _check(min(int(need), 0))
        buf = C.create_string_buffer(int(need))
        lib().bsir_fused_elementwise_source(len(self._ops), ins, len(self._tape), tape, n_out, carr, flags, buf, C.c_int64(int(need)))
        return buf.value.decode()

    def compile(self, outs: Optional[Sequence] = None, contiguous: bool = True, in_place: bool = False,
                row_grid: bool = False, cols: int = 4096) -> int:
        """Compiles the chain's kernel for sm_100a with NVRTC (no device needed); returns the size of the image."""
        ins, tape, carr, n_out = self._tables_without_data(outs)
        size = C.c_int64(0)
        _check(lib().bsir_fused_elementwise_compile(len(self._ops), ins, len(self._tape), tape, n_out, carr,
                                                    (1 if contiguous else 0) | (2 if in_place else 0) | (4 if row_grid else 0)
                                                    | ((cols // 8) << 8), C.byref(size)))
        return int(size.value)


# ---------------------------------------------------------------------------- reductions
def _rows(x: torch.Tensor):
    if x.dim() != 2:
        raise BsirError(-2, "expected a 2-D tensor")
    if x.shape[1] > 1 and x.stride(1) != 1:
        raise BsirError(-3, "innermost dimension must be unit-stride")
    return x.shape[0], x.shape[1], (x.stride(0) if x.shape[0] > 1 else max(x.shape[1], 1))


def reduce(kind: str, x: torch.Tensor, dim: int = 1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``linalg.reduce`` / ``hivm.hir.vreduce <kind>`` over dim 0 or 1 of a 2-D tensor."""
    rows, cols, rs = _rows(x)
    if dim in (1, -1):
        out = torch.empty(rows, dtype=x.dtype, device=x.device) if out is None else out
        _check(lib().bsir_reduce_last_axis(REDUCE_KIND[kind], _dt(x), C.c_int64(rows), C.c_int64(cols), _ptr(x),
                                           C.c_int64(rs), _ptr(out), _stream()))
    else:
        out = torch.empty(cols, dtype=x.dtype, device=x.device) if out is None else out
        _check(lib().bsir_reduce_first_axis(REDUCE_KIND[kind], _dt(x), C.c_int64(rows), C.c_int64(cols), _ptr(x),
                                            C.c_int64(rs), _ptr(out), _stream()))
    return out


def gather(x: torch.Tensor, index: torch.Tensor, dim: int = -1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hivm.hir.vgather`` {gather_axis = dim}: out[.., j, ..] = x[.., index[.., j, ..], ..] (torch.gather's rule;
    index and out have x's shape but for the gather axis).  index: int16 / int32 / int64."""
    dim = dim % x.dim()
    x, index = x.contiguous(), index.contiguous()
    if index.dim() != x.dim() or any(index.shape[d] != x.shape[d] for d in range(x.dim()) if d != dim):
        raise BsirError(-2, f"gather: index {tuple(index.shape)} does not match {tuple(x.shape)} outside axis {dim}")
    out = torch.empty(index.shape, dtype=x.dtype, device=x.device) if out is None else out
    if not out.is_contiguous() or out.shape != index.shape or out.dtype != x.dtype:
        raise BsirError(-3, "gather: out must be a contiguous tensor of the index's shape and the source's type")
    outer = inner = 1
    for d in range(dim):
        outer *= x.shape[d]
    for d in range(dim + 1, x.dim()):
        inner *= x.shape[d]
    _check(lib().bsir_gather(_dt(x), _dt(index), C.c_int64(outer), C.c_int64(x.shape[dim]), C.c_int64(index.shape[dim]),
                             C.c_int64(inner), _ptr(x), _ptr(index), _ptr(out), _stream()))
    return out


def arange(shape: Sequence[int], strides: Sequence[int], offset: int = 0, dtype: torch.dtype = torch.int32,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hivm.hir.varange offset[o] strides[s..]``: out[i0, i1, ..] = o + sum_d i_d * s_d."""
    shape = list(shape)
    out = torch.empty(shape, dtype=dtype, device="cuda") if out is None else out
    _check(lib().bsir_arange(_dt(out), len(shape), _i64arr(shape), C.c_int64(int(offset)), _i64arr(list(strides)), _ptr(out),
                             _i64arr(out.stride()), _stream()))
    return out


def interleave(srcs: Sequence[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hivm.hir.vinterleave`` of N tensors of one shape along their last axis: out[.., N * i + ch] = srcs[ch][.., i]."""
    srcs = [s.contiguous() for s in srcs]
    n, cols = len(srcs), srcs[0].shape[-1]
    rows = srcs[0].numel() // max(cols, 1)
    if any(s.shape != srcs[0].shape or s.dtype != srcs[0].dtype for s in srcs):
        raise BsirError(-2, "interleave: the sources must have one shape and type")
    out = torch.empty(list(srcs[0].shape[:-1]) + [n * cols], dtype=srcs[0].dtype, device=srcs[0].device) if out is None else out
    if not out.is_contiguous():
        raise BsirError(-3, "interleave: out must be contiguous")
    arr = (C.c_void_p * n)(*[s.data_ptr() for s in srcs])
    _check(lib().bsir_interleave(_dt(srcs[0]), n, C.c_int64(rows), C.c_int64(cols), arr, _ptr(out), _stream()))
    return out


def deinterleave(x: torch.Tensor, channels: int = 2, keep: Optional[Sequence[int]] = None):
    """``hivm.hir.vdeinterleave {channel_num}``: N tensors with out[ch][.., i] = x[.., N * i + ch]; ``keep`` lists the
    channels wanted (the others are not written and come back as None)."""
    x = x.contiguous()
    if x.shape[-1] % channels:
        raise BsirError(-2, "deinterleave: the last axis must be a multiple of the channel count")
    cols = x.shape[-1] // channels
    rows = x.numel() // max(x.shape[-1], 1)
    outs = [torch.empty(list(x.shape[:-1]) + [cols], dtype=x.dtype, device=x.device) if keep is None or ch in keep else None
            for ch in range(channels)]
    arr = (C.c_void_p * channels)(*[(o.data_ptr() if o is not None else None) for o in outs])
    _check(lib().bsir_deinterleave(_dt(x), channels, C.c_int64(rows), C.c_int64(cols), _ptr(x), arr, _stream()))
    return outs


def sort(x: torch.Tensor, descending: bool = False, out_val: Optional[torch.Tensor] = None, out_idx: Optional[torch.Tensor] = None):
    """``hivm.hir.vsort {descending}`` over the last axis of a 1-D or 2-D tensor -> (values, int32 indices); stable."""
    two_d = x if x.dim() == 2 else x.reshape(1, -1)
    rows, cols, rs = _rows(two_d)
    val = torch.empty((rows, cols), dtype=x.dtype, device=x.device) if out_val is None else out_val
    idx = torch.empty((rows, cols), dtype=torch.int32, device=x.device) if out_idx is None else out_idx
    _check(lib().bsir_sort(_dt(x), int(bool(descending)), C.c_int64(rows), C.c_int64(cols), _ptr(two_d), C.c_int64(rs), _ptr(val),
                           C.c_int64(max(cols, 1)), _ptr(idx), C.c_int64(max(cols, 1)), _stream()))
    return val.reshape(x.shape), idx.reshape(x.shape)


CUM_KIND = {"sum": 0, "prod": 1, "max": 2, "min": 3}


def cumulative(kind: str, x: torch.Tensor, dim: int = 1, reverse: bool = False, propagate_nan: bool = True,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hivm.hir.vcumsum`` / ``vcumprod`` / ``vcummax`` / ``vcummin`` {cum_dims = [dim], reverse} of a 2-D tensor."""
    rows, cols, rs = _rows(x)
    out = torch.empty((rows, cols), dtype=x.dtype, device=x.device) if out is None else out
    _check(lib().bsir_cumulative(CUM_KIND[kind], _dt(x), int(dim % 2), int(bool(reverse)), int(bool(propagate_nan)),
                                 C.c_int64(rows), C.c_int64(cols), _ptr(x), C.c_int64(rs), _ptr(out),
                                 C.c_int64(out.stride(0) if rows > 1 else max(cols, 1)), _stream()))
    return out


def reduce_with_index(kind: str, x: torch.Tensor, tie_break_left: bool = True, nan_mode: str = "region",
                      workspace: Optional[torch.Tensor] = None, out_val: Optional[torch.Tensor] = None,
                      out_idx: Optional[torch.Tensor] = None):
    """``hfusion.reduce_with_index <max|min|maxui|minui> {tie_break_left}`` over the last axis -> (values, int32 indices)."""
    rows, cols, rs = _rows(x)
    val = torch.empty(rows, dtype=x.dtype, device=x.device) if out_val is None else out_val
    idx = torch.empty(rows, dtype=torch.int32, device=x.device) if out_idx is None else out_idx
    ws_ptr = _ptr(workspace) if workspace is not None else C.c_void_p(0)
    ws_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    _check(lib().bsir_reduce_with_index(RWI_KIND[kind], _dt(x), int(bool(tie_break_left)),
                                        {"region": 0, "nan_first": 1}[nan_mode], C.c_int64(rows), C.c_int64(cols),
                                        _ptr(x), C.c_int64(rs), _ptr(val), _ptr(idx), ws_ptr, C.c_int64(ws_bytes),
                                        _stream()))
    return val, idx


# ---------------------------------------------------------------------------- fused row patterns
def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float, want_rstd: bool = False,
             out: Optional[torch.Tensor] = None):
    rows, cols, rs = _rows(x)
    y = torch.empty((rows, cols), dtype=x.dtype, device=x.device) if out is None else out
    rstd = torch.empty(rows, dtype=x.dtype, device=x.device) if want_rstd else None
    _check(lib().bsir_rms_norm(_dt(x), C.c_int64(rows), C.c_int64(cols), _ptr(x), C.c_int64(rs), _ptr(gamma),
                               C.c_float(eps), _ptr(y), C.c_int64(y.stride(0) if rows > 1 else max(cols, 1)),
                               _ptr(rstd) if want_rstd else C.c_void_p(0), _stream()))
    return (y, rstd) if want_rstd else y


def softmax(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    rows, cols, rs = _rows(x)
    y = torch.empty((rows, cols), dtype=x.dtype, device=x.device) if out is None else out
    _check(lib().bsir_softmax(_dt(x), C.c_int64(rows), C.c_int64(cols), _ptr(x), C.c_int64(rs), _ptr(y),
                              C.c_int64(y.stride(0) if rows > 1 else max(cols, 1)), _stream()))
    return y


def quant_per_token_i8(x: torch.Tensor, round_mode: str = "rint", q: Optional[torch.Tensor] = None,
                       scale: Optional[torch.Tensor] = None):
    rows, cols, rs = _rows(x)
    q = torch.empty((rows, cols), dtype=torch.int8, device=x.device) if q is None else q
    scale = torch.empty(rows, dtype=torch.float32, device=x.device) if scale is None else scale
    _check(lib().bsir_quant_per_token_i8(_dt(x), ROUND_MODE[round_mode], C.c_int64(rows), C.c_int64(cols), _ptr(x),
                                         C.c_int64(rs), _ptr(q), C.c_int64(q.stride(0) if rows > 1 else max(cols, 1)),
                                         _ptr(scale), _stream()))
    return q, scale


# ---------------------------------------------------------------------------- GEMMs
def matmul_w8a8(a: torch.Tensor, b: torch.Tensor, scale_a: Optional[torch.Tensor] = None,
                scale_b: Optional[torch.Tensor] = None, transpose_b: bool = False,
                out_dtype: torch.dtype = torch.bfloat16, want_acc: bool = False,
                out: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None):
    """``linalg.matmul`` i8 x i8 -> i32 plus the dequant suffix; b is [k, n] or (transpose_b) [n, k]."""
    m, k = a.shape
    n = b.shape[0] if transpose_b else b.shape[1]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    acc = torch.empty((m, n), dtype=torch.int32, device=a.device) if want_acc else None
    ws_ptr = _ptr(workspace) if workspace is not None else C.c_void_p(0)
    ws_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    _check(lib().bsir_matmul_w8a8(C.c_int64(m), C.c_int64(n), C.c_int64(k), _ptr(a), C.c_int64(a.stride(0)), _ptr(b),
                                  C.c_int64(b.stride(0)), int(bool(transpose_b)),
                                  _ptr(scale_a) if scale_a is not None else C.c_void_p(0),
                                  _ptr(scale_b) if scale_b is not None else C.c_void_p(0), _TORCH2DT[out_dtype],
                                  _ptr(out), C.c_int64(out.stride(0)), _ptr(acc) if want_acc else C.c_void_p(0),
                                  ws_ptr, C.c_int64(ws_bytes), _stream()))
    return (out, acc) if want_acc else out


class MatmulDesc(C.Structure):
    _fields_ = [("in_dtype", C.c_int32), ("out_dtype", C.c_int32), ("transpose_a", C.c_int32), ("transpose_b", C.c_int32),
                ("descale_mode", C.c_int32), ("relu", C.c_int32), ("bias_dtype", C.c_int32), ("descale_dtype", C.c_int32),
                ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64), ("batch", C.c_int64),
                ("a", C.c_void_p), ("lda", C.c_int64), ("batch_stride_a", C.c_int64),
                ("b", C.c_void_p), ("ldb", C.c_int64), ("batch_stride_b", C.c_int64),
                ("bias", C.c_void_p), ("descale", C.c_void_p), ("scale_a", C.c_void_p),
                ("out", C.c_void_p), ("ldo", C.c_int64), ("batch_stride_out", C.c_int64),
                ("n_peers", C.c_int32), ("peer_out", C.POINTER(C.c_void_p))]


DESCALE_MODE = {"DescaleNull": 0, "DescalePerChannel": 1, "DescalePerTensor": 2, None: 0}


def matmul(a: torch.Tensor, b: torch.Tensor, *, transpose_a: bool = False, transpose_b: bool = False,
           bias: Optional[torch.Tensor] = None, descale: Optional[torch.Tensor] = None, descale_mode: Optional[str] = None,
           scale_a: Optional[torch.Tensor] = None, relu: bool = False, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None, peer_out: Optional[Sequence[int]] = None, ldo: Optional[int] = None):
    """``hivm.hir.matmul`` / ``linalg.matmul`` (2-D) or ``batch_matmul`` (3-D operands):
    ``C = cast(relu(descale * (A @ B + bias) * scale_a))``.  Operands int8 (int32 accumulation), f16 or bf16 (f32
    accumulation); ``a_transpose`` / ``b_transpose`` as the op's unit attributes; ``descale_mode`` with the reference's
    spellings (``DescaleNull`` | ``DescalePerChannel`` | ``DescalePerTensor``; inferred from the descale's size when
    omitted); ``out_dtype`` f16 / bf16 / f32 / int8 (fixpipe ``S322I8``) / int32 (raw accumulators of an int8 product)."""
    batched = a.dim() == 3
    a3 = a if batched else a.unsqueeze(0)
    b3 = b if b.dim() == 3 else b.unsqueeze(0)
    if (a3.shape[-1] > 1 and a3.stride(-1) != 1) or (b3.shape[-1] > 1 and b3.stride(-1) != 1):
        raise BsirError(-3, "matmul: the last axis of each operand must be contiguous")
    batch = a3.shape[0]
    m, k = (a3.shape[2], a3.shape[1]) if transpose_a else (a3.shape[1], a3.shape[2])
    n = b3.shape[1] if transpose_b else b3.shape[2]
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else (torch.float16 if a.dtype == torch.int8 else a.dtype)
    if peer_out is not None:
        # one-sided N-sharding: device addresses of this rank's block in every rank's output buffer, row pitch ldo
        if batched or ldo is None:
            raise BsirError(-9, "matmul: peer_out needs 2-D operands and the row pitch ldo of the peers' buffers")
        o3 = None
    else:
        if out is None:
            out = torch.empty((batch, m, n) if batched else (m, n), dtype=out_dtype, device=a.device)
        o3 = out if out.dim() == 3 else out.unsqueeze(0)
    if descale is not None and descale_mode is None:
        descale_mode = "DescalePerTensor" if descale.numel() == 1 else "DescalePerChannel"
    d = MatmulDesc()
    d.in_dtype, d.out_dtype = _dt(a), _TORCH2DT[out_dtype]
    d.transpose_a, d.transpose_b = int(transpose_a), int(transpose_b)
    d.descale_mode = DESCALE_MODE[descale_mode] if descale is not None else 0
    d.relu = int(relu)
    d.bias_dtype = _dt(bias) if bias is not None else F32
    d.descale_dtype = _dt(descale) if descale is not None else F32
    d.m, d.n, d.k, d.batch = m, n, k, batch
    # a row pitch only means something with more than one row; a lone row reports its length
    d.a, d.lda, d.batch_stride_a = a3.data_ptr(), (a3.stride(1) if a3.shape[1] > 1 else a3.shape[2]), (a3.stride(0) if batch > 1 else 0)
    d.b, d.ldb, d.batch_stride_b = b3.data_ptr(), (b3.stride(1) if b3.shape[1] > 1 else b3.shape[2]), (b3.stride(0) if b3.shape[0] > 1 else 0)
    d.bias = bias.data_ptr() if bias is not None else None
    d.descale = descale.data_ptr() if descale is not None else None
    d.scale_a = scale_a.data_ptr() if scale_a is not None else None
    if o3 is not None:
        d.out, d.ldo, d.batch_stride_out = o3.data_ptr(), (o3.stride(1) if o3.shape[1] > 1 else o3.shape[2]), (o3.stride(0) if batch > 1 else 0)
    else:
        arr = (C.c_void_p * len(peer_out))(*[int(q) for q in peer_out])
        d.out, d.ldo, d.batch_stride_out, d.n_peers, d.peer_out = None, int(ldo), 0, len(peer_out), arr
    _check(lib().bsir_matmul(C.byref(d), _stream()))
    return out


def matmul_w4a16(a: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                 group: int = 128, out: Optional[torch.Tensor] = None, peer_out: Optional[Sequence[int]] = None,
                 ldo: Optional[int] = None):
    m, k = a.shape
    n = qweight.shape[1]
    if peer_out is not None:      # one-sided N-sharding: this rank's block of every rank's output buffer
        arr = (C.c_void_p * len(peer_out))(*[int(q) for q in peer_out])
        _check(lib().bsir_matmul_w4a16_peers(C.c_int64(m), C.c_int64(n), C.c_int64(k), C.c_int64(group), _ptr(a),
                                             C.c_int64(a.stride(0)), _ptr(qweight), _ptr(scales), _ptr(zeros), C.c_int32(len(peer_out)),
                                             arr, C.c_int64(int(ldo)), _stream()))
        return None
    out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device) if out is None else out
    _check(lib().bsir_matmul_w4a16(C.c_int64(m), C.c_int64(n), C.c_int64(k), C.c_int64(group), _ptr(a),
                                   C.c_int64(a.stride(0)), _ptr(qweight), _ptr(scales), _ptr(zeros), _ptr(out),
                                   C.c_int64(out.stride(0)), _stream()))
    return out


# ---------------------------------------------------------------------------- compiled-kernel ABI
def register_kernel(name: str, kind: str, *, fn: int = 0, dtype: int = F32, dst_dtype: int = F32,
                    round_mode: str = "rint", overflow_mode: str = "wrap", flags: int = 0,
                    sizes: Sequence[int] = (), eps: float = 0.0) -> None:
    d = KernelDesc()
    d.kind = KERNEL_KIND[kind]
    d.fn, d.dtype, d.dst_dtype = fn, dtype, dst_dtype
    d.round_mode, d.overflow_mode, d.flags = ROUND_MODE[round_mode], OVERFLOW_MODE[overflow_mode], flags
    d.rank = len(sizes)
    for i, s in enumerate(sizes):
        d.sizes[i] = int(s)
    d.eps = eps
    _check(lib().bsir_kernel_register(name.encode(), C.byref(d)))


def launch(name: str, args: Sequence[Optional[torch.Tensor]], block_dim: int = 1) -> None:
    """``rtKernelLaunch`` analogue: one bare pointer per memref argument, inputs then outputs."""
    arr = (C.c_void_p * len(args))(*[(t.data_ptr() if t is not None else None) for t in args])
    _check(lib().bsir_launch(name.encode(), C.c_uint32(block_dim), arr, C.c_size_t(C.sizeof(arr)), _stream()))


def device_error() -> int:
    return int(lib().bsir_device_error())


def launch_count() -> int:
    return int(lib().bsir_launch_count())
