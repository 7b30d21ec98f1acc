"""ctypes front end of the CPU oracle (oracle/hfusion_oracle.c).

TEST INFRASTRUCTURE ONLY.  Importable from tests/, the smoke check and the
CPU-baseline leg of the bench; the product package never imports it.

Arrays are numpy, C-contiguous.  f16 / bf16 tensors travel as ``np.uint16`` bit
patterns together with a dtype code (``F16`` / ``BF16``); everything else uses the
natural numpy dtype.  The functions mirror the reference op they restate; the
C file carries the reference file:line citations.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

F32, F16, BF16, I8, I16, I32, I64, U8, U16, U32, U64, BOOL = range(12)
DTYPE_NAMES = {"f32": F32, "f16": F16, "bf16": BF16, "i8": I8, "i16": I16, "i32": I32, "i64": I64,
               "u8": U8, "u16": U16, "u32": U32, "u64": U64, "bool": BOOL, "i1": BOOL}
_NP = {F32: np.float32, F16: np.uint16, BF16: np.uint16, I8: np.int8, I16: np.int16, I32: np.int32,
       I64: np.int64, U8: np.uint8, U16: np.uint16, U32: np.uint32, U64: np.uint64, BOOL: np.uint8}

ROUND = {"rint": 0, "round": 1, "floor": 2, "ceil": 3, "trunc": 4, "odd": 5, "truncwithoverflow": 6}
OVERFLOW = {"wrap": 0, "saturate": 1, "ascend_saturate_trunc_via_f16": 2, "ascend_double_round_via_f16": 3}
UNARY = {"relu": 0, "sqrt": 1, "rsqrt": 2, "rec": 3, "vnot": 4, "tanh": 5, "sin": 6, "cos": 7, "atan": 8,
         "tan": 9, "absi": 10, "erf": 11, "log2": 12, "log10": 13, "log1p": 14, "exp2": 15, "expm1": 16,
         "ilogb": 17, "asin": 18, "acos": 19, "asinh": 20, "acosh": 21, "atanh": 22, "sinh": 23,
         "lgamma": 24, "cosh": 25, "nearbyint": 26, "exp": 100, "log": 101, "abs": 102, "ceil": 103,
         "floor": 104, "negf": 105, "reciprocal": 106, "round": 107, "square": 110}
BINARY = {"vor": 0, "vand": 1, "vxor": 2, "minf": 3, "maxf": 4, "powf": 5, "mod": 6, "modui": 7, "shli": 8,
          "shrsi": 9, "shrui": 10, "ldexp": 11, "ceildivsi": 12, "ceildivui": 13, "floordivsi": 14,
          "powi": 15, "minnumf": 16, "maxnumf": 17, "atan2": 18, "divfhp": 19, "copysign": 20,
          "add": 100, "sub": 101, "mul": 102, "div": 103, "div_unsigned": 104, "max_signed": 105,
          "min_signed": 106, "max_unsigned": 107, "min_unsigned": 108}
COMPARE = {"veq": 0, "vne": 1, "vle": 2, "vlt": 3, "vge": 4, "vgt": 5, "vule": 6, "vult": 7, "vuge": 8, "vugt": 9}
REDUCE = {"sum": 0, "prod": 1, "max": 2, "min": 3, "any": 4, "all": 5, "xori": 6, "ori": 7, "andi": 8}


def build(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile beside this file (gcc); returns its path."""
    if force or not os.path.exists(_LIB_PATH) or \
            os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "hfusion_oracle.c")):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_bf16_to_f32.restype = C.c_float
        _lib.orc_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_bf16.restype = C.c_uint16
        _lib.orc_f32_to_bf16.argtypes = [C.c_float]
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_f32_to_f16_rz.restype = C.c_uint16
        _lib.orc_f32_to_f16_rz.argtypes = [C.c_float]
        _lib.orc_selftest_f16.restype = C.c_int64
        _lib.orc_selftest_f16.argtypes = [C.c_int64]
        _lib.orc_check_recip_division.restype = C.c_int64
        _lib.orc_check_recip_division.argtypes = [C.c_float, C.c_int]
        _lib.orc_check_recip_division_f16.restype = C.c_int64
        _lib.orc_check_recip_division_f16.argtypes = [C.c_float, C.c_int]
    return _lib


def set_threads(n: int) -> None:
    lib().orc_set_threads(C.c_int(int(n)))


def max_threads() -> int:
    return int(lib().orc_get_max_threads())


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dt) -> np.ndarray:
    a = np.ascontiguousarray(a)
    if a.dtype != _NP[dt]:
        if a.dtype == np.bool_ and dt == BOOL:
            a = a.view(np.uint8)
        else:
            raise TypeError(f"array dtype {a.dtype} does not match dtype code {dt} ({_NP[dt]})")
    return a


def _i64(v):
    return C.c_int64(int(v))


def _chk(rc, what):
    if rc != 0:
        raise RuntimeError(f"oracle {what} failed with code {rc}")


# ---------------------------------------------------------------- conversions
def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    out = np.empty(x.shape, np.uint16)
    cast(F32, BF16, np.ascontiguousarray(x, np.float32), out=out)
    return out


def f16_to_f32(bits: np.ndarray) -> np.ndarray:
    return bits.view(np.float16).astype(np.float32)


# ------------------------------------------------------------------------ ops
def elemwise_unary(fn, dt, x):
    fn = UNARY[fn] if isinstance(fn, str) else fn
    x = _c(x, dt)
    out = np.empty_like(x)
    _chk(lib().orc_elemwise_unary(fn, dt, _p(x), _p(out), _i64(x.size)), "elemwise_unary")
    return out


def elemwise_binary(fn, dt, a, b):
    """a / b: arrays of the same shape, or 1-element arrays (scalar operand, stride 0)."""
    fn = BINARY[fn] if isinstance(fn, str) else fn
    a, b = _c(a, dt), _c(b, dt)
    n = max(a.size, b.size)
    shape = a.shape if a.size == n else b.shape
    sa = 1 if a.size == n else 0
    sb = 1 if b.size == n else 0
    out = np.empty(shape, _NP[dt])
    _chk(lib().orc_elemwise_binary(fn, dt, _p(a), _i64(sa), _p(b), _i64(sb), _p(out), _i64(n)), "elemwise_binary")
    return out


def elemwise_fma(dt, a, b, c):
    """hfusion.elemwise_ternary {fma}: a * b + c with one rounding; operands of one shape or 1-element (scalar)."""
    a, b, c = _c(a, dt), _c(b, dt), _c(c, dt)
    n = max(a.size, b.size, c.size)
    shape = next(x.shape for x in (a, b, c) if x.size == n)
    out = np.empty(shape, _NP[dt])
    _chk(lib().orc_elemwise_fma(dt, _p(a), _i64(1 if a.size == n else 0), _p(b), _i64(1 if b.size == n else 0), _p(c),
                                _i64(1 if c.size == n else 0), _p(out), _i64(n)), "elemwise_fma")
    return out


def compare(fn, dt, a, b):
    fn = COMPARE[fn] if isinstance(fn, str) else fn
    a, b = _c(a, dt), _c(b, dt)
    n = max(a.size, b.size)
    shape = a.shape if a.size == n else b.shape
    out = np.empty(shape, np.uint8)
    _chk(lib().orc_compare(fn, dt, _p(a), _i64(1 if a.size == n else 0), _p(b), _i64(1 if b.size == n else 0),
                           _p(out), _i64(n)), "compare")
    return out


def select(dt, cond, a, b):
    cond = np.ascontiguousarray(cond).view(np.uint8)
    a, b = _c(a, dt), _c(b, dt)
    n = max(cond.size, a.size, b.size)
    shape = cond.shape if cond.size == n else (a.shape if a.size == n else b.shape)
    out = np.empty(shape, _NP[dt])
    _chk(lib().orc_select(dt, _p(cond), _i64(1 if cond.size == n else 0), _p(a), _i64(1 if a.size == n else 0),
                          _p(b), _i64(1 if b.size == n else 0), _p(out), _i64(n)), "select")
    return out


def load_pad(dt, src, dst, pad_mode, pad_value=None, left=-1, right=-1):
    """hivm.hir.load with padding; ``src`` [rows, n], ``dst`` [rows, dst_last] (initial contents, returned updated)."""
    src, dst = _c(src, dt), _c(dst, dt).copy()
    rows, n = (1, src.shape[0]) if src.ndim == 1 else (int(np.prod(src.shape[:-1])), src.shape[-1])
    pv = _c(np.asarray([0 if pad_value is None else pad_value]).astype(_NP[dt]) if not isinstance(pad_value, np.ndarray) else pad_value, dt)
    mode = {"first_elem": 1, "value": 2}[pad_mode]
    _chk(lib().orc_load_pad(dt, _p(src), _i64(rows), _i64(n), _p(dst), _i64(dst.shape[-1]), mode, _p(pv), _i64(left),
                            _i64(right)), "load_pad")
    return dst


def store_atomic(dt, kind, src, dst):
    """hivm.hir.store atomic = <kind>: the destination after one store."""
    kinds = {"add": 1, "max": 2, "min": 3, "and": 4, "or": 5, "xor": 6, "umax": 9, "umin": 10}
    src, dst = _c(src, dt), _c(dst, dt).copy()
    _chk(lib().orc_store_atomic(dt, kinds[kind], _p(src), _p(dst), _i64(src.size)), "store_atomic")
    return dst


def cast(src_dt, dst_dt, src, round_mode="rint", overflow="wrap", out=None):
    rm = ROUND[round_mode] if isinstance(round_mode, str) else round_mode
    ov = OVERFLOW[overflow] if isinstance(overflow, str) else overflow
    src = _c(src, src_dt)
    if out is None:
        out = np.empty(src.shape, _NP[dst_dt])
    _chk(lib().orc_cast(src_dt, dst_dt, rm, ov, _p(src), _p(out), _i64(src.size)), "cast")
    return out


def reduce_last_axis(kind, dt, src):
    kind = REDUCE[kind] if isinstance(kind, str) else kind
    src = _c(src, dt)
    rows, cols = src.shape
    out = np.empty(rows, _NP[dt])
    _chk(lib().orc_reduce_last_axis(kind, dt, _p(src), _i64(rows), _i64(cols), _i64(cols), _p(out)), "reduce")
    return out


def reduce_first_axis(kind, dt, src):
    kind = REDUCE[kind] if isinstance(kind, str) else kind
    src = _c(src, dt)
    rows, cols = src.shape
    out = np.empty(cols, _NP[dt])
    _chk(lib().orc_reduce_first_axis(kind, dt, _p(src), _i64(rows), _i64(cols), _i64(cols), _p(out)), "reduce")
    return out


def cumulative(kind, dt, src, axis=1, reverse=False, propagate_nan=True):
    """kind: 'sum' | 'prod' | 'max' | 'min' along axis 0 or 1 of a 2-D array."""
    k = {"sum": 0, "prod": 1, "max": 2, "min": 3}[kind]
    src = _c(src, dt)
    rows, cols = src.shape
    out = np.empty_like(src)
    _chk(lib().orc_cumulative(k, dt, int(axis), int(bool(reverse)), int(bool(propagate_nan)), _p(src), _i64(rows), _i64(cols),
                              _i64(cols), _p(out), _i64(cols)), "cumulative")
    return out


def interleave(srcs):
    """hfusion.interleave / hivm.hir.vinterleave: out[.., N*i + ch] = srcs[ch][.., i] -- the loop nest of scalar inserts the
    reference decomposes it into (bishengir/lib/Dialect/HFusion/Transforms/DecomposeOpInterfaceImpl.cpp:439-560; runner
    golden test/Dialect/HFusion/test_interleave.mlir:16-18).  A move of bits, so any numpy dtype."""
    n = len(srcs)
    out = np.empty(srcs[0].shape[:-1] + (n * srcs[0].shape[-1],), dtype=srcs[0].dtype)
    for ch, s in enumerate(srcs):
        out[..., ch::n] = s
    return out


def deinterleave(src, channel, channels=2):
    """hfusion.deinterleave channel<c>: out[.., i] = src[.., N*i + c] (runner golden test_deinterleave.mlir:83-85)."""
    return np.ascontiguousarray(src[..., channel::channels])


def sort_last_axis_loops(dt, src, descending=False):
    """hfusion.sort / hivm.hir.vsort exactly as the reference lowers it: n-1 bubble passes of n-1 compare-and-swaps
    on `cmpf ugt` / `ult` (DecomposeOpInterfaceImpl.cpp:742-838).  O(n^2) per row: small rows only."""
    src = _c(src, dt)
    cols = src.shape[-1]
    flat = src.reshape(-1, cols)
    val = np.empty_like(flat)
    idx = np.empty(flat.shape, dtype=np.int32)
    _chk(lib().orc_sort_last_axis(dt, int(bool(descending)), _p(flat), _i64(flat.shape[0]), _i64(cols), _p(val), _p(idx)),
         "sort_last_axis")
    return val.reshape(src.shape), idx.reshape(src.shape)


def sort_last_axis(dt, src, descending=False):
    """The closed form of `sort_last_axis_loops` (tests check the two against each other): (sorted values in src's
    storage type, int32 source indices).  Equal keys keep their source order and -0 = +0 (the strict comparison
    never swaps them); a NaN that starts at position p of its row ends at (p + 1) mod n in either direction (every
    pair holding a NaN swaps under the unordered predicates, which moves each NaN one place left per pass and
    carries the one at the front to the end); the other elements fill the remaining places in stable order."""
    src = _c(src, dt)
    n = src.shape[-1]
    if dt in (F32, F16, BF16):
        f = src.astype(np.float32) if dt == F32 else (f16_to_f32(src) if dt == F16 else bf16_to_f32(src))
        bits = f.view(np.uint32).copy()
        bits[bits == 0x80000000] = 0
        order = np.where(bits & 0x80000000, ~bits, bits | np.uint32(0x80000000)).astype(np.uint32)
        nan = np.isnan(f)
    else:
        order = (src.astype(np.int64) + 2 ** 31).astype(np.uint32)
        nan = np.zeros(src.shape, dtype=bool)
    if descending:
        order = ~order
    key = (order.astype(np.uint64) << np.uint64(32)) | np.arange(n, dtype=np.uint64)
    key[nan] = np.uint64(0xFFFFFFFF00000000) | np.broadcast_to(np.arange(n, dtype=np.uint64), src.shape)[nan]
    by_key = np.argsort(key, axis=-1, kind="stable")                  # numbers in order, then the NaNs by position
    if nan.any():
        flat_nan = nan.reshape(-1, n)
        flat_by_key = by_key.reshape(-1, n)
        idx = np.empty_like(flat_by_key)
        for r in range(flat_nan.shape[0]):
            p = np.flatnonzero(flat_nan[r])
            if p.size == 0:
                idx[r] = flat_by_key[r]
                continue
            taken = np.zeros(n, dtype=bool)
            taken[(p + 1) % n] = True
            idx[r, (p + 1) % n] = p
            idx[r, ~taken] = flat_by_key[r, :n - p.size]
        idx = idx.reshape(src.shape)
    else:
        idx = by_key
    idx = idx.astype(np.int32)
    return np.take_along_axis(src, idx.astype(np.int64), axis=-1), idx


def reduce_with_index(kind, dt, src, tie_break_left=True, nan_mode="region"):
    """kind: 'max' | 'min' | 'maxui' | 'minui' (the unsigned kinds: integer inputs).  Returns (values, int32 indices)."""
    k = {"min": 0, "max": 1, "minui": 2, "maxui": 3}[kind]
    nm = {"region": 0, "nan_first": 1}[nan_mode]
    src = _c(src, dt)
    rows, cols = src.shape
    val = np.empty(rows, _NP[dt])
    idx = np.empty(rows, np.int32)
    _chk(lib().orc_reduce_with_index(k, dt, int(bool(tie_break_left)), nm, _p(src), _i64(rows), _i64(cols),
                                     _i64(cols), _p(val), _p(idx)), "reduce_with_index")
    return val, idx


def rms_norm(dt, x, gamma, eps, want_rstd=False):
    x, gamma = _c(x, dt), _c(gamma, dt)
    rows, cols = x.shape
    y = np.empty_like(x)
    rstd = np.empty(rows, _NP[dt]) if want_rstd else None
    _chk(lib().orc_rms_norm(dt, _p(x), _p(gamma), C.c_float(eps), _i64(rows), _i64(cols), _i64(cols), _p(y),
                            _i64(cols), _p(rstd) if want_rstd else None), "rms_norm")
    return (y, rstd) if want_rstd else y


def softmax(dt, x):
    x = _c(x, dt)
    rows, cols = x.shape
    y = np.empty_like(x)
    _chk(lib().orc_softmax(dt, _p(x), _i64(rows), _i64(cols), _i64(cols), _p(y), _i64(cols)), "softmax")
    return y


def quant_per_token_i8(dt, x, round_mode="rint", overflow="saturate"):
    rm = ROUND[round_mode] if isinstance(round_mode, str) else round_mode
    ov = OVERFLOW[overflow] if isinstance(overflow, str) else overflow
    x = _c(x, dt)
    rows, cols = x.shape
    q = np.empty((rows, cols), np.int8)
    scale = np.empty(rows, np.float32)
    _chk(lib().orc_quant_per_token_i8(dt, rm, ov, _p(x), _i64(rows), _i64(cols), _i64(cols), _p(q), _i64(cols),
                                      _p(scale)), "quant_per_token_i8")
    return q, scale


def matmul_w8a8(a, b, sa=None, sw=None, transpose_b=False, out_dt=BF16, want_acc=False):
    a = _c(a, I8)
    b = _c(b, I8)
    m, k = a.shape
    n = b.shape[0] if transpose_b else b.shape[1]
    assert (b.shape[1] if transpose_b else b.shape[0]) == k
    out = np.empty((m, n), np.uint16)
    acc = np.empty((m, n), np.int32) if want_acc else None
    sa_ = _c(sa, F32) if sa is not None else None
    sw_ = _c(sw, F32) if sw is not None else None
    _chk(lib().orc_matmul_w8a8(_i64(m), _i64(n), _i64(k), _p(a), _i64(k), _p(b), _i64(b.shape[1]),
                               int(bool(transpose_b)), _p(sa_) if sa_ is not None else None,
                               _p(sw_) if sw_ is not None else None, out_dt, _p(out), _i64(n),
                               _p(acc) if want_acc else None, _i64(n)), "matmul_w8a8")
    return (out, acc) if want_acc else out


def matmul(in_dt, a, b, out_dt, transpose_a=False, transpose_b=False, bias=None, bias_dt=None, descale=None,
           descale_dt=F32, descale_mode=0, scale_a=None, relu=False):
    """hivm.hir.matmul + fixpipe (see orc_matmul).  a: [m,k] ([k,m] with transpose_a), b: [k,n] ([n,k] with
    transpose_b), in the storage of in_dt (int8, or uint16 bit patterns for f16 / bf16); bias / descale in the
    storage of their dtypes.  Returns C in the storage of out_dt."""
    a, b = _c(a, in_dt), _c(b, in_dt)
    m, k = (a.shape[1], a.shape[0]) if transpose_a else a.shape
    n = b.shape[0] if transpose_b else b.shape[1]
    out = np.empty((m, n), _NP[out_dt])
    if bias is not None:
        bias_dt = bias_dt if bias_dt is not None else (I32 if in_dt == I8 else F32)
        bias = _c(bias, bias_dt)
    if descale is not None:
        descale = _c(descale, descale_dt)
    sa = None if scale_a is None else np.ascontiguousarray(scale_a, dtype=np.float32)
    _chk(lib().orc_matmul(in_dt, out_dt, int(bool(transpose_a)), int(bool(transpose_b)), int(descale_mode), int(bool(relu)),
                          int(bias_dt if bias_dt is not None else F32), int(descale_dt), _i64(m), _i64(n), _i64(k), _p(a),
                          _i64(a.shape[1]), _p(b), _i64(b.shape[1]), _p(bias) if bias is not None else None,
                          _p(descale) if descale is not None else None, _p(sa) if sa is not None else None, _p(out), _i64(n)),
         "matmul")
    return out


def matmul_w4a16(a_bits, qweight, scales_bits, zeros, group=128):
    a = _c(a_bits, BF16)
    qw = _c(qweight, I32)
    sc = _c(scales_bits, BF16)
    zp = _c(zeros, I32)
    m, k = a.shape
    n = qw.shape[1]
    out = np.empty((m, n), np.uint16)
    _chk(lib().orc_matmul_w4a16(_i64(m), _i64(n), _i64(k), _i64(group), _p(a), _i64(k), _p(qw), _p(sc), _p(zp),
                                _p(out), _i64(n)), "matmul_w4a16")
    return out
