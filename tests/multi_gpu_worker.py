"""One rank of the multi-GPU parity checks (started by tests/test_gpu_multi.py, one process per GPU).

N-sharded W8A8 and W4A16 GEMMs, reassembled (a) by an NCCL all-gather and (b) one-sidedly -- the epilogue stores
each rank's column block into every rank's output buffer, a flag exchange closes the step -- against the CPU oracle;
row-sharded per-token quantisation; and the bounded wait of the flag exchange when a peer never signals."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "ascendnpu-ir_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

import numpy as np
import torch
import torch.distributed as dist

import bsir
import oracle as O
from bsir import peer, shard
from bsir import workloads as W
from conftest import to_bits


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    bsir.lib()
    O.set_threads(4)
    dev = "cuda"

    # ---- row-sharded per-token quantisation: no collective on the data path
    x = W.quant_input(64, 512, seed=3)
    lo, hi = shard.my_rows(64, rank, world)
    q, s = bsir.quant_per_token_i8(x[lo:hi].contiguous())
    wq, ws = O.quant_per_token_i8(O.BF16, to_bits(x))
    assert np.array_equal(q.cpu().numpy(), wq[lo:hi]) and np.array_equal(s.cpu().numpy(), ws[lo:hi])

    # ---- W8A8, N-sharded (same seeded data on every rank)
    for m, n, k in ((16, 1024, 512), (130, 768, 640), (300, 512, 256)):      # the last one takes the TMA + push form
        g = torch.Generator(device=dev).manual_seed(m)
        a = torch.randint(-127, 128, (m, k), generator=g, device=dev, dtype=torch.int8)
        w = torch.randint(-127, 128, (k, n), generator=g, device=dev, dtype=torch.int8)
        sa = torch.rand(m, generator=g, device=dev) * 9e-3 + 1e-3
        sw = torch.rand(n, generator=g, device=dev) * 9e-3 + 1e-3
        want = O.matmul_w8a8(to_bits(a), to_bits(w), to_bits(sa), to_bits(sw))
        wl, swl, (c0, c1) = shard.shard_w8a8_weights(w, sw, rank, world)
        # (a) NCCL all-gather of the [M, N/G] blocks
        out_l = bsir.matmul_w8a8(a, wl, sa, swl)
        full = shard.gather_columns(out_l, n, multiple=16)
        assert np.array_equal(to_bits(full), want), f"W8A8 all-gather ({m},{n},{k}) differs on rank {rank}"
        # (b) one-sided: two steps in a row on the same buffers
        buf = peer.PeerBuffer(m * n * 2)
        for step in range(2):
            shard.w8a8_onesided_step(bsir, a, wl, sa, swl, buf, n, c0)
            torch.cuda.synchronize()
            got = buf.tensor((m, n), torch.bfloat16)
            assert np.array_equal(to_bits(got), want), f"W8A8 one-sided ({m},{n},{k}) step {step} differs on rank {rank}"
            dist.barrier()                      # nobody starts overwriting before everybody has compared
        assert bsir.device_error() == 0
        buf.close()

    # ---- W4A16, N-sharded
    for m in (1, 16):
        n, k = 1024, 512
        a, qw, sc, zp = W.w4a16_input(m, n, k, seed=20 + m)
        want = O.matmul_w4a16(to_bits(a), to_bits(qw), to_bits(sc), to_bits(zp))
        wf = O.bf16_to_f32(want)
        ql, scl, zl, (c0, c1) = shard.shard_w4a16_weights(qw, sc, zp, rank, world)
        full = shard.gather_columns(bsir.matmul_w4a16(a, ql, scl, zl), n, multiple=8)
        assert np.allclose(full.float().cpu().numpy(), wf, rtol=2e-2, atol=1e-3), f"W4A16 all-gather m={m} rank {rank}"
        buf = peer.PeerBuffer(m * n * 2)
        shard.w4a16_onesided_step(bsir, a, ql, scl, zl, buf, n, c0)
        torch.cuda.synchronize()
        got = buf.tensor((m, n), torch.bfloat16)
        assert np.allclose(got.float().cpu().numpy(), wf, rtol=2e-2, atol=1e-3), f"W4A16 one-sided m={m} rank {rank}"
        assert torch.equal(got[:, c0:c1], full[:, c0:c1])
        dist.barrier()
        buf.close()

    # ---- a peer that never signals: the wait gives up, reports through the device error word, and the context lives on
    buf = peer.PeerBuffer(256)
    if rank == 0:
        buf.signal_wait()                        # rank 1 does not take part
        torch.cuda.synchronize()
        assert bsir.device_error() == 0x200, "the bounded wait should have reported BSIR_DEVERR_PEER_WAIT"
        y = bsir.vadd(torch.ones(1024, device=dev), torch.ones(1024, device=dev))
        assert float(y.sum()) == 2048.0          # the GPU still answers
    dist.barrier()
    buf.close()
    dist.barrier()
    dist.destroy_process_group()
    print(f"multi-gpu worker ok rank {rank}/{world}")


if __name__ == "__main__":
    main()
