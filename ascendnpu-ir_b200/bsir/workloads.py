"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark
configurations (there is no external dataset behind them: the shapes are LLM-like -- hidden 4096,
FFN 14336, vocabulary 152064 -- and the generators below are the whole definition)."""
from __future__ import annotations

import torch


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def vecadd(n: int = 1 << 24, dtype=torch.float32, seed: int = 0, device="cuda"):
    """a, b ~ U[-1, 1), rounded to `dtype`."""
    g = _gen(seed, device)
    a = (torch.rand(n, generator=g, device=device) * 2 - 1).to(dtype)
    b = (torch.rand(n, generator=g, device=device) * 2 - 1).to(dtype)
    return a, b


def quant_input(rows: int = 16384, cols: int = 4096, seed: int = 0, device="cuda", dtype=torch.bfloat16):
    """x ~ N(0,1) with 0.1 % of the elements scaled x20 (outliers), rounded to bf16."""
    g = _gen(seed, device)
    x = torch.randn(rows, cols, generator=g, device=device)
    mask = torch.rand(rows, cols, generator=g, device=device) < 1e-3
    x = torch.where(mask, x * 20.0, x)
    return x.to(dtype)


def rmsnorm_input(rows: int = 32768, cols: int = 4096, seed: int = 0, device="cuda", dtype=torch.bfloat16):
    g = _gen(seed, device)
    x = torch.randn(rows, cols, generator=g, device=device).to(dtype)
    w = (1.0 + 0.02 * torch.randn(cols, generator=g, device=device)).to(dtype)
    return x, w


def softmax_input(rows: int = 4096, cols: int = 32768, seed: int = 0, device="cuda", dtype=torch.bfloat16):
    g = _gen(seed, device)
    return (3.0 * torch.randn(rows, cols, generator=g, device=device)).to(dtype)


def argmax_input(rows: int = 256, cols: int = 152064, seed: int = 0, device="cuda", dtype=torch.bfloat16):
    g = _gen(seed, device)
    return torch.randn(rows, cols, generator=g, device=device).to(dtype)


def w8a8_input(m: int, n: int = 14336, k: int = 4096, seed: int = 0, device="cuda"):
    """A, W ~ U{-127..127}; per-token scales ~ U(1e-3, 1e-2), per-channel scales ~ U(1e-3, 1e-2)."""
    g = _gen(seed, device)
    a = torch.randint(-127, 128, (m, k), generator=g, device=device, dtype=torch.int8)
    w = torch.randint(-127, 128, (k, n), generator=g, device=device, dtype=torch.int8)
    sa = torch.rand(m, generator=g, device=device) * 9e-3 + 1e-3
    sw = torch.rand(n, generator=g, device=device) * 9e-3 + 1e-3
    return a, sa, w, sw


def w4a16_input(m: int, n: int = 14336, k: int = 4096, group: int = 128, seed: int = 0, device="cuda"):
    """bf16 activations ~ N(0,1); int4 weights / zero points ~ U{0..15} packed 8 per int32; bf16
    group scales ~ U(1e-3, 1e-2).  Packing: qweight[r, c] nibble t = q[8r+t, c]; zeros[g, c] nibble t =
    z[g, 8c+t]."""
    g = _gen(seed, device)
    a = torch.randn(m, k, generator=g, device=device).to(torch.bfloat16)
    q = torch.randint(0, 16, (k, n), generator=g, device=device, dtype=torch.int32)
    z = torch.randint(0, 16, (k // group, n), generator=g, device=device, dtype=torch.int32)
    s = (torch.rand(k // group, n, generator=g, device=device) * 9e-3 + 1e-3).to(torch.bfloat16)
    shifts = (torch.arange(8, device=device, dtype=torch.int32) * 4)
    qw = (q.view(k // 8, 8, n) << shifts.view(1, 8, 1)).sum(dim=1, dtype=torch.int64)
    zw = (z.view(k // group, n // 8, 8) << shifts.view(1, 1, 8)).sum(dim=2, dtype=torch.int64)
    to_i32 = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
    return a, to_i32(qw), s, to_i32(zw)
