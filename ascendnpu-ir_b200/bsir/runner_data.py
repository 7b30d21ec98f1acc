"""The seeded inputs and the dump format of the reference's CPU runner, restated
(bishengir/lib/ExecutionEngine/BiShengIRRunnerUtils.cpp:63-125), so that a run of this backend on a reference test file
can be diffed against a run of the reference's own `mlir-cpu-runner` pipeline made elsewhere.

Inputs.  `getData<Distribution>(memref)` fills a buffer element by element from `static std::mt19937 generator(1)` --
one generator per element type (the static lives in a function template), advancing from call to call -- through
    bf16, f16   std::uniform_real_distribution<float>(-100, 100), converted to the 16-bit type (round to nearest even)
    f32         std::uniform_real_distribution<float>(-1000, 1000)
    i1          std::uniform_int_distribution<uint8_t>(0, 1)
    i8 / i16 / i32 / i64   std::uniform_int_distribution over [-100, 100] / [-1000, 1000] / [-10000, 10000] / [-100000, 100000]
The distributions are libstdc++'s (the reference builds on Linux): `generate_canonical<float, 24>` takes one 32-bit
draw, converts it to float, divides by 2^32 and clamps a result of 1 to the float below it; the integer distribution is
Lemire's multiply-and-reject on 32-bit draws (libstdc++ 11 and later).  The Mersenne Twister itself is numpy's, seeded
the classic way (`init_genrand(1)`), which is what `std::mt19937(1)` does.

Dump.  `printData`: the rank, a line with the sizes, a line with the elements in row-major order separated by blanks;
integers in decimal, floats as `%.9e`.  (The reference streams int8 through `raw_ostream << signed char`, i.e. as raw
characters; here int8 is written in decimal like the other integers.)
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np

_REAL = {"bf16": (-100.0, 100.0), "f16": (-100.0, 100.0), "f32": (-1000.0, 1000.0)}
_INT = {"i1": (0, 1), "i8": (-100, 100), "i16": (-1000, 1000), "i32": (-10000, 10000), "i64": (-100000, 100000)}
_NP = {"f32": np.float32, "i1": np.bool_, "i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64}


class RunnerData:
    """The generators of one runner process: one mt19937(1) per element type."""

    def __init__(self):
        self._gen: Dict[str, np.random.MT19937] = {}

    def _raw(self, elem: str, n: int) -> np.ndarray:
        g = self._gen.get(elem)
        if g is None:
            g = np.random.MT19937()
            g._legacy_seeding(1)                      # init_genrand(1) == std::mt19937(1)
            self._gen[elem] = g
        return g.random_raw(n).astype(np.uint64)

    def get_data(self, elem: str, shape: Sequence[int]) -> np.ndarray:
        """An array of `shape` filled the way getData<..> fills it.  bf16 / f16 come back as uint16 bit patterns."""
        n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        if elem in _REAL:
            a, b = _REAL[elem]
            u = self._raw(elem, n).astype(np.float32)                      # uint32 -> float, round to nearest even
            u = u / np.float32(4294967296.0)
            u = np.where(u >= np.float32(1.0), np.nextafter(np.float32(1.0), np.float32(0.0)), u).astype(np.float32)
            v = (u * np.float32(b - a) + np.float32(a)).astype(np.float32)
            if elem == "f32":
                return v.reshape(shape)
            if elem == "f16":
                return v.astype(np.float16).view(np.uint16).reshape(shape)
            bits = v.view(np.uint32)
            nan = np.isnan(v)
            r = ((bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
            r[nan] = 0x7FC0
            return r.reshape(shape)
        if elem in _INT:
            lo, hi = _INT[elem]
            rng = np.uint64(hi - lo + 1)
            threshold = np.uint64((4294967296 - int(rng)) % int(rng))
            out = np.empty(0, dtype=np.uint64)
            while out.size < n:                                            # a rejected draw is consumed, then the next one is tried
                prod = self._raw(elem, n - out.size) * rng
                keep = (prod & np.uint64(0xFFFFFFFF)) >= threshold
                out = np.concatenate([out, (prod >> np.uint64(32))[keep]])
            return (out.astype(np.int64) + lo).astype(_NP[elem]).reshape(shape)
        raise ValueError(f"runner data: element type {elem}")


def _floats(elem: str, a: np.ndarray) -> np.ndarray:
    if elem == "bf16":
        return (a.astype(np.uint32) << np.uint32(16)).view(np.float32)
    if elem == "f16":
        return a.view(np.float16).astype(np.float32)
    return a.astype(np.float32)


def print_data(elem: str, a: np.ndarray) -> str:
    """One tensor in printData's format (bf16 / f16 given as uint16 bit patterns)."""
    a = np.ascontiguousarray(a)
    head = f"{a.ndim}\n" + " ".join(str(int(s)) for s in a.shape)
    if elem in _REAL:
        body = " ".join("%.9e" % float(v) for v in _floats(elem, a).reshape(-1))
    else:
        body = " ".join(str(int(v)) for v in a.reshape(-1))
    return head + "\n" + body + "\n"


def read_data(text: str) -> List[Tuple[List[int], List[str]]]:
    """Parses a dump file back into (sizes, element tokens) per tensor, in file order."""
    lines = text.split("\n")
    out, i = [], 0
    while i < len(lines) and lines[i].strip():
        rank = int(lines[i])
        sizes = [int(t) for t in lines[i + 1].split()] if rank else []
        out.append((sizes, lines[i + 2].split()))
        i += 3
    return out
