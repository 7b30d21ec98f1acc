"""Multi-GPU partitioning of the operator set: one process per GPU, `torch.distributed` for plumbing.

Row-wise ops (elementwise, cast, per-token quantisation, RMSNorm, softmax, argmax) are independent per
row, so rank r simply owns rows [lo, hi) and no collective runs on the data path.  GEMMs are sharded
by output column: rank r holds W[:, lo:hi] (and scale_b[lo:hi], or the matching qweight / scales /
zeros columns) with A replicated; an all-gather reassembles [M, N] only where a consumer needs it.
The reference has no counterpart (a single-kernel compiler; its cross-device layer is a thin wrapper
over aclshmem put/get, bishengir/lib/Template/lib/Shmem/Shmem.cpp:27-120).
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def even_split(total: int, parts: int, multiple: int = 1) -> List[Tuple[int, int]]:
    """Contiguous [lo, hi) ranges covering [0, total): sizes differ by at most `multiple`, every boundary is
    a multiple of `multiple` (8 for W4A16 columns, so zero-point words stay whole)."""
    if parts <= 0 or total < 0 or multiple <= 0:
        raise ValueError("even_split: bad arguments")
    if total % multiple:
        raise ValueError(f"even_split: {total} is not a multiple of {multiple}")
    units = total // multiple
    base, extra = divmod(units, parts)
    out, lo = [], 0
    for r in range(parts):
        n = (base + (1 if r < extra else 0)) * multiple
        out.append((lo, lo + n))
        lo += n
    return out


def my_rows(rows: int, rank: int, world: int) -> Tuple[int, int]:
    return even_split(rows, world)[rank]


def my_columns(n: int, rank: int, world: int, multiple: int = 8) -> Tuple[int, int]:
    return even_split(n, world, multiple)[rank]


def shard_w8a8_weights(w: torch.Tensor, scale_b: torch.Tensor, rank: int, world: int):
    """W [K, N], scale_b [N] -> this rank's contiguous column block."""
    lo, hi = my_columns(w.shape[1], rank, world, 16)
    return w[:, lo:hi].contiguous(), scale_b[lo:hi].contiguous(), (lo, hi)


def shard_w4a16_weights(qweight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, rank: int, world: int):
    """qweight [K/8, N], scales [K/g, N], zeros [K/g, N/8] -> this rank's column block (multiple of 8 columns)."""
    lo, hi = my_columns(qweight.shape[1], rank, world, 8)
    return (qweight[:, lo:hi].contiguous(), scales[:, lo:hi].contiguous(), zeros[:, lo // 8:hi // 8].contiguous(),
            (lo, hi))


def gather_columns(local: torch.Tensor, n_total: int, group=None, multiple: int = 8) -> torch.Tensor:
    """All-gather of N-sharded [M, n_r] blocks into [M, n_total] (uneven blocks allowed).  `multiple` must be
    the one the weights were split with (16 for W8A8, 8 for W4A16)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    ranges = even_split(n_total, world, multiple if n_total % multiple == 0 else 1)
    if n_total % world == 0 and all(hi - lo == n_total // world for lo, hi in ranges):
        # equal blocks: one all_gather_into_tensor on a [world, M, n/world] buffer, then a view shuffle
        m, nr = local.shape
        buf = torch.empty((world * m, nr), dtype=local.dtype, device=local.device)   # rank blocks stacked on dim 0
        dist.all_gather_into_tensor(buf, local.contiguous(), group=group)
        return buf.view(world, m, nr).permute(1, 0, 2).reshape(m, n_total)
    # uneven blocks: collectives want equal sizes, so pad every block to the widest and trim afterwards
    widest = max(hi - lo for lo, hi in ranges)
    m = local.shape[0]
    padded = torch.zeros((m, widest), dtype=local.dtype, device=local.device)
    padded[:, : local.shape[1]] = local
    parts = [torch.empty((m, widest), dtype=local.dtype, device=local.device) for _ in ranges]
    dist.all_gather(parts, padded, group=group)
    assert ranges[rank][1] - ranges[rank][0] == local.shape[1]
    return torch.cat([p[:, : hi - lo] for p, (lo, hi) in zip(parts, ranges)], dim=1)


def gather_rows(local: torch.Tensor, rows_total: int, group=None) -> torch.Tensor:
    """All-gather of row-sharded results (only when a consumer wants the whole tensor)."""
    world = dist.get_world_size(group)
    ranges = even_split(rows_total, world)
    tallest = max(hi - lo for lo, hi in ranges)
    padded = torch.zeros((tallest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in ranges]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[: hi - lo] for p, (lo, hi) in zip(parts, ranges)], dim=0)


# ----------------------------------------------------------------------------------------- N-sharded GEMM steps
def w8a8_allgather_step(bsir, a, w_local, scale_a, scale_b_local, local_out, gathered, group=None):
    """One step of the N-sharded W8A8 GEMM the plain way: local GEMM into [M, N/G], NCCL all-gather into
    [G, M, N/G].  `gathered` is that buffer; `gathered.permute(1, 0, 2).reshape(M, N)` is C."""
    bsir.matmul_w8a8(a, w_local, scale_a, scale_b_local, out=local_out)
    dist.all_gather_into_tensor(gathered.view(-1, local_out.shape[1]), local_out, group=group)
    return gathered


ONESIDED_FUSED_MAX_ROWS = 256   # up to here the GEMM's epilogue stores into the peers itself


def w8a8_onesided_step(bsir, a, w_local, scale_a, scale_b_local, buf, n_total, col0):
    """The same step one-sided, C assembled in every rank's [M, N] buffer (`buf`, a bsir.peer.PeerBuffer).  Few rows:
    the GEMM's epilogue stores this rank's column block straight into every rank's buffer.  Many rows: the GEMM writes
    its block of its own buffer through TMA at full speed and `buf.push` copies it to the peers in a pass of its own.
    Either way one flag exchange closes the step."""
    import torch
    m, nl = a.shape[0], w_local.shape[1]
    if m <= ONESIDED_FUSED_MAX_ROWS:
        bsir.matmul(a, w_local, scale_a=scale_a, descale=scale_b_local, descale_mode="DescalePerChannel",
                    out_dtype=torch.bfloat16, peer_out=buf.block_ptrs(col0 * 2), ldo=n_total)
    else:
        mine = buf.tensor((m, n_total), torch.bfloat16)[:, col0:col0 + nl]
        bsir.matmul_w8a8(a, w_local, scale_a, scale_b_local, out=mine)
        buf.push(col0 * 2, m, nl * 2, n_total * 2)
    buf.signal_wait()


def w4a16_onesided_step(bsir, a, qw_local, scales_local, zeros_local, buf, n_total, col0, group_size=128):
    bsir.matmul_w4a16(a, qw_local, scales_local, zeros_local, group=group_size, peer_out=buf.block_ptrs(col0 * 2), ldo=n_total)
    buf.signal_wait()
