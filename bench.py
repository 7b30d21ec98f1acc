#!/usr/bin/env python
"""Benchmark of the hot path: per-token dynamic int8 quantisation of bf16 [16384, 4096]
(fused elementwise + cast, the configuration the headline HBM GB/s metric is quoted on), with
the other operator configurations reported beside it in `ops`.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-ops]

One JSON line on stdout (rank 0).  A step = one pass of the fused quantisation kernel over one
batch of seeded synthetic input resident in HBM.  N > 1 (launched by torchrun, one rank per GPU):
rows are independent, so every rank quantises its own batch with no data-path collective
(`scaling: weak`); `value` = bytes all ranks processed / the slowest rank's device time.
`--impl reference` times the CPU restatement of the reference's scalar-loop lowering on the host
cores instead (rank 0 only).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _sub in ("ascendnpu-ir_b200", "oracle"):
    _p = os.path.join(ROOT, _sub)
    if _p not in sys.path:
        sys.path.insert(0, _p)

ROWS, COLS = 16384, 4096
ALGO_BYTES = ROWS * COLS * 2 + ROWS * COLS + ROWS * 4   # read bf16 + write int8 + write f32 scales
# dram__bytes_read.sum + dram__bytes_write.sum of one captured launch of the quantiser on this workload
# (Nsight Compute, summary in profiles/quant_rows_kernel__bf16_16384x4096.txt): 134,288,896 read + 10,988,288 written.
NCU_TRAFFIC_BYTES = 145_277_184
NCU_TRAFFIC_NOTE = ("reads equal the input exactly; 56 MB of the 67 MB output was still dirty in the 126 MB L2 when the "
                    "captured launch ended, so steady-state traffic per launch is 134.3 + 67.2 = 201.5 MB")
METRIC = "per_token_int8_quant_hbm_gbps"
NBUF = 4                                                # input/output sets rotated between steps


def measured_peaks():
    """(HBM GB/s, bf16 TFLOP/s burst, label): the pool's measured numbers, else the stated fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([f.strip() for f in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline_quant(threads: int, sample_rows: int, reps: int = 3):
    """Times the oracle (port of the reference's CPU lowering) on `sample_rows` rows of the workload."""
    import numpy as np
    import oracle as O
    rng = np.random.default_rng(0)
    x = rng.standard_normal((sample_rows, COLS)).astype(np.float32)
    x[rng.random((sample_rows, COLS)) < 1e-3] *= 20.0
    xb = O.f32_to_bf16(x)
    O.set_threads(threads)
    O.quant_per_token_i8(O.BF16, xb[:64])               # warm-up
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        O.quant_per_token_i8(O.BF16, xb)
        best = min(best, time.perf_counter() - t0)
    O.set_threads(1)
    bytes_ = sample_rows * COLS * 3 + sample_rows * 4
    return bytes_ / best / 1e9, best


def run_reference(args):
    """`--impl reference`: the reference's CPU path (oracle port; the MLIR pipeline itself cannot be
    built here) on all host threads, same metric / unit / config.  Each step is a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle as O
    threads = O.max_threads()
    sample_rows = 1024
    for _ in range(max(args.warmup, 1)):
        cpu_baseline_quant(threads, 64, reps=1)
    t_total, n = 0.0, 0
    for _ in range(args.steps):
        gbs, t = cpu_baseline_quant(threads, sample_rows, reps=1)
        t_total += t
        n += 1
    bytes_step = sample_rows * COLS * 3 + sample_rows * 4
    value = bytes_step * n / t_total / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_total / n * 1e3 * (ROWS / sample_rows),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32->i8", "data": "synthetic",
        "config": {"workload": "per-token int8 quant bf16 [16384,4096]", "rows": ROWS, "cols": COLS,
                   "sample": f"each step runs {sample_rows} of the {ROWS} rows; value is bytes of the sample / its time, ms_per_step is scaled to the full batch"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{sample_rows} of {ROWS} rows per step; ms_per_step scaled to the full batch"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def time_op(torch, fn, iters: int, warm: int = 3):
    """Average device time (ms) of one fn(i) launch: `iters` launches captured in a CUDA graph and
    replayed, timed with CUDA events on the launching stream (host launch cost stays out of it)."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i)
    g.replay()                          # untimed replay: graph upload, caches
    torch.cuda.synchronize()
    best, tot, reps = float("inf"), 0.0, 3
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        t = a.elapsed_time(b) / iters
        best, tot = min(best, t), tot + t
    return tot / reps, best


def sustained_bf16_peak():
    """bf16 TFLOP/s of a seconds-long cuBLAS loop under the power cap (the pool's measurement), else the stated fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p)).get("bf16_tflops_sustained", 0.0)) or None
    return 1400.0


def sharded_gemm_ops(torch, dist, bsir, W, rank, world, iters):
    """N-sharded GEMMs on `world` GPUs (configurations 4 and 5): every rank holds W[:, n0:n1] and the whole of A, and C
    [M, 14336] is reassembled on every rank (a) by an NCCL all-gather of the [M, N/G] blocks plus the copy that puts
    them side by side, (b) one-sidedly: the GEMM's epilogue stores its block into every rank's C, a flag exchange
    closes the step.  Each variant is one CUDA graph of `iters` steps timed with CUDA events, max over ranks; weight
    sets are rotated so that a step does not find its weights in L2.  `t1_ms` is the same GEMM with all 14336
    columns on one GPU, timed in the same run; efficiency = t1 / (G x t)."""
    from bsir import peer, shard
    res = {}
    N, K = 14336, 4096

    def timed(fn, reps=3):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        dist.barrier()
        st = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for i in range(iters):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        best = None
        for _ in range(reps):
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            best = float(t) if best is None else min(best, float(t))
        del g
        return best

    def run(name, m, flops, make_full, shard_fn, gemm_local, gemm_full, gemm_peers, multiple):
        try:
            c0, c1 = shard.my_columns(N, rank, world, multiple)
            nl = c1 - c0
            full_sets = [make_full(s) for s in range(2)]
            shard_bytes = max(1, K * nl // (2 if "w4a16" in name else 1))
            nsets = int(min(24, max(3, (256 << 20) // shard_bytes)))
            locs = []
            for s_ in range(nsets):
                full = full_sets[s_ % 2] if s_ < 2 else make_full(s_)
                locs.append(shard_fn(full))
                if s_ >= 2:
                    del full
            a_ref = full_sets[0][0]
            out_full = [torch.empty(m, N, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
            t1 = timed(lambda i: gemm_full(full_sets[i % 2], out_full[i % 2]))
            out_l = [torch.empty(m, nl, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
            t_local = timed(lambda i: gemm_local(locs[i % nsets], out_l[i % 2]))
            equal = N % world == 0 and nl == N // world
            gathered = torch.empty(world, m, nl, dtype=torch.bfloat16, device="cuda")
            c_full = torch.empty(m, N, dtype=torch.bfloat16, device="cuda")

            def step_nccl(i):
                gemm_local(locs[i % nsets], out_l[i % 2])
                dist.all_gather_into_tensor(gathered.view(world * m, nl), out_l[i % 2])
                c_full.view(m, world, nl).copy_(gathered.permute(1, 0, 2))

            t_nccl = timed(step_nccl) if equal else None
            buf = peer.PeerBuffer(m * N * 2)
            ptrs = buf.block_ptrs(c0 * 2)

            def step_peer(i):
                l = locs[i % nsets]
                if gemm_peers is None:      # W8A8: fused epilogue stores for few rows, TMA + push pass for many
                    shard.w8a8_onesided_step(bsir, l[0], l[2], l[1], l[3], buf, N, c0)
                else:
                    gemm_peers(l, ptrs)
                    buf.signal_wait()

            t_peer = timed(step_peer)
            torch.cuda.synchronize()
            same = bool(torch.equal(buf.tensor((m, N), torch.bfloat16)[:, c0:c1], out_l[(iters - 1) % 2])) if True else None
            buf.close()
            r = {"t1_ms": t1, "local_gemm_ms": t_local, "allgather_step_ms": t_nccl, "onesided_step_ms": t_peer,
                 "allgather_share_of_step": None if t_nccl is None else max(0.0, 1.0 - t_local / t_nccl),
                 "speedup_allgather": None if t_nccl is None else t1 / t_nccl, "speedup_onesided": t1 / t_peer,
                 "efficiency_allgather": None if t_nccl is None else t1 / t_nccl / world, "efficiency_onesided": t1 / t_peer / world,
                 "tops_allgather": None if t_nccl is None else flops / t_nccl / 1e9, "tops_onesided": flops / t_peer / 1e9,
                 "onesided_block_matches_local": same, "weight_sets_rotated": nsets, "columns_per_rank": nl}
            res[name] = r
            del locs, full_sets, out_full, out_l, gathered, c_full
            torch.cuda.empty_cache()
        except Exception as e:   # one failing variant must not hide the others
            res[name] = {"error": repr(e)[:300]}
            try:
                dist.barrier()
            except Exception:
                pass

    for m in (16, 128, 4096):
        run(f"w8a8_m{m}_nshard", m, 2 * m * K * N,
            lambda s, m=m: W.w8a8_input(m, seed=s),                                   # (a, sa, w, sw)
            lambda f: (f[0], f[1]) + shard.shard_w8a8_weights(f[2], f[3], rank, world)[:2],
            lambda l, o: bsir.matmul_w8a8(l[0], l[2], l[1], l[3], out=o),
            lambda f, o: bsir.matmul_w8a8(f[0], f[2], f[1], f[3], out=o),
            None, 16)
    for m in (1, 8, 16):
        run(f"w4a16_m{m}_nshard", m, 2 * m * K * N,
            lambda s, m=m: W.w4a16_input(m, seed=s),                                   # (a, qw, scales, zeros)
            lambda f: (f[0],) + shard.shard_w4a16_weights(f[1], f[2], f[3], rank, world)[:3],
            lambda l, o: bsir.matmul_w4a16(l[0], l[1], l[2], l[3], out=o),
            lambda f, o: bsir.matmul_w4a16(f[0], f[1], f[2], f[3], out=o),
            lambda l, ptrs: bsir.matmul_w4a16(l[0], l[1], l[2], l[3], peer_out=ptrs, ldo=N),
            8)
    return res


def other_ops(torch, bsir, W, hbm_peak, tensor_peak, iters, only=None):
    """The remaining configurations, each with inputs larger than L2 or rotated buffers."""
    res = {}
    bf16_sustained = sustained_bf16_peak()

    def rec(name, algo_bytes, fn, flops=None, note=None):
        if only and name != only:
            return
        try:
            avg, best = time_op(torch, fn, iters)
        except Exception as e:  # an op that is not built yet must not hide the others
            res[name] = {"error": str(e)[:200]}
            return
        r = {"ms": avg, "ms_min": best, "gbps": algo_bytes / avg / 1e6, "frac_hbm": algo_bytes / avg / 1e6 / hbm_peak,
             "algo_bytes": algo_bytes}
        if flops:
            r["tops"] = flops / avg / 1e9
            r["frac_int8_peak_2x_bf16"] = flops / avg / 1e9 / (2 * tensor_peak)
        if note:
            r["note"] = note
        res[name] = r

    def want(name):
        return not only or name == only

    n = 1 << 24
    for dt, nm in ((torch.float32, "vecadd_f32"), (torch.float16, "vecadd_f16")):
        if not want(nm):
            continue
        bufs = [W.vecadd(n, dt, seed=s) for s in range(3)]
        outs = [torch.empty_like(b[0]) for b in bufs]
        rec(nm, 3 * n * bufs[0][0].element_size(), lambda i: bsir.vadd(*bufs[i % 3], out=outs[i % 3]))
        del bufs, outs
    if want("bias_add_bf16_32768x4096") or want("row_scale_bf16_32768x4096") or want("slice_mul_bf16_32768x4096"):
        # hivm's inline broadcast (a per-column bias, a per-row scale) and row-strided views of wider tensors
        xs = [W.rmsnorm_input(32768, 4096, seed=s) for s in range(2)]                 # (x bf16 [32768, 4096], w bf16 [4096])
        ys = [torch.empty_like(x[0]) for x in xs]
        scale = (torch.rand(32768, 1, device="cuda") + 0.5).to(torch.bfloat16)
        wide = [torch.randn(32768, 4608, device="cuda").to(torch.bfloat16) for _ in range(2)]
        if want("bias_add_bf16_32768x4096"):
            rec("bias_add_bf16_32768x4096", 2 * 32768 * 4096 * 2 + 8192,
                lambda i: bsir.elemwise_binary("add", xs[i % 2][0], xs[i % 2][1].view(1, -1).expand(32768, 4096), out=ys[i % 2]))
        if want("row_scale_bf16_32768x4096"):
            rec("row_scale_bf16_32768x4096", 2 * 32768 * 4096 * 2 + 65536,
                lambda i: bsir.elemwise_binary("mul", xs[i % 2][0], scale.expand(32768, 4096), out=ys[i % 2]))
        if want("slice_mul_bf16_32768x4096"):
            rec("slice_mul_bf16_32768x4096", 3 * 32768 * 4096 * 2,
                lambda i: bsir.elemwise_binary("mul", xs[i % 2][0], wide[i % 2][:, 256:4352], out=ys[i % 2]))
        del xs, ys, scale, wide
    if want("rmsnorm_bf16_32768x4096"):
        xs = [W.rmsnorm_input(32768, 4096, seed=s) for s in range(2)]
        ys = [torch.empty_like(x[0]) for x in xs]
        rec("rmsnorm_bf16_32768x4096", 2 * 32768 * 4096 * 2 + 8192,
            lambda i: bsir.rms_norm(xs[i % 2][0], xs[i % 2][1], 1e-6, out=ys[i % 2]))
        del xs, ys
    if want("softmax_bf16_4096x32768"):
        xs = [W.softmax_input(4096, 32768, seed=s) for s in range(2)]
        ys = [torch.empty_like(x) for x in xs]
        rec("softmax_bf16_4096x32768", 2 * 4096 * 32768 * 2, lambda i: bsir.softmax(xs[i % 2], out=ys[i % 2]))
        del xs, ys
    if want("argmax_bf16_256x152064"):
        xs = [W.argmax_input(256, 152064, seed=s) for s in range(4)]
        rec("argmax_bf16_256x152064", 256 * 152064 * 2 + 256 * 6, lambda i: bsir.reduce_with_index("max", xs[i % 4]))
        del xs
    if want("chain_rmstail_bf16_32768x4096") or want("chain_gelu_bf16_32768x4096"):
        # fused elementwise chains (one kernel compiled per chain): gamma * (rstd * x), and tanh-GELU in ten ops
        rows, cols = 32768, 4096
        xs = [W.rmsnorm_input(rows, cols, seed=s) for s in range(2)]
        ys = [torch.empty_like(x[0]) for x in xs]
        rstd = torch.rand(rows, 1, device="cuda") + 0.5

        def rms_tail(i):
            ch = bsir.FusedChain()
            hx, hg, hr = ch.operand(xs[i % 2][0]), ch.operand(xs[i % 2][1], "row_vector"), ch.operand(rstd, "col_vector")
            ch.load(ch.op(hr)).binary("mul", ch.op(hx)).rbinary("mul", ch.op(hg))
            ch.run(rows, cols, outs=[(ys[i % 2], -1)])

        def gelu(i):
            ch = bsir.FusedChain()
            hx = ch.op(ch.operand(xs[i % 2][0]))
            (ch.load(hx).unary("square").binary("mul", hx).binary("mul", 0.044715).binary("add", hx).binary("mul", 0.7978845608)
               .unary("tanh").binary("add", 1.0).binary("mul", hx).binary("mul", 0.5))
            ch.run(rows, cols, outs=[(ys[i % 2], -1)])

        rec("chain_rmstail_bf16_32768x4096", 2 * rows * cols * 2 + cols * 2 + rows * 4, rms_tail)
        rec("chain_gelu_bf16_32768x4096", 2 * rows * cols * 2, gelu)
        del xs, ys, rstd
    if want("chain_rmsnorm_bf16_32768x4096"):
        # the same RMSNorm as rmsnorm_bf16_32768x4096, written as a chain with one row reduction (compiled per chain)
        rows, cols = 32768, 4096
        xs = [W.rmsnorm_input(rows, cols, seed=s) for s in range(2)]
        ys = [torch.empty_like(x[0]) for x in xs]

        def rms_chain(i):
            ch = bsir.FusedChain()
            hx, hg = ch.op(ch.operand(xs[i % 2][0])), ch.op(ch.operand(xs[i % 2][1], "row_vector"))
            (ch.load(hx).unary("square").reduce("sum").binary("div", float(cols)).binary("add", 1e-6).unary("sqrt").unary("rec")
               .binary("mul", hx).rbinary("mul", hg))
            ch.run(rows, cols, outs=[(ys[i % 2], -1)])

        rec("chain_rmsnorm_bf16_32768x4096", 2 * rows * cols * 2 + cols * 2, rms_chain)
        del xs, ys
    if want("chain_softmax_bf16_4096x32768"):
        rows, cols = 4096, 32768
        xs = [W.softmax_input(rows, cols, seed=s) for s in range(2)]
        ys = [torch.empty_like(x) for x in xs]

        def softmax_chain(i):
            ch = bsir.FusedChain()
            hx = ch.op(ch.operand(xs[i % 2]))
            (ch.load(hx).reduce("max").save(0).load(hx).binary("sub", ("tmp", 0)).unary("exp").save(1).reduce("sum")
               .rbinary("div", ("tmp", 1)))
            ch.run(rows, cols, outs=[(ys[i % 2], -1)])

        rec("chain_softmax_bf16_4096x32768", 2 * rows * cols * 2, softmax_chain)
        del xs, ys
    # the data-movement / scan ops beside the hot path, same measurement (algorithmic bytes = read + written once)
    if want("transpose_bf16_8192x8192"):
        xs = [torch.randn(8192, 8192, device="cuda").to(torch.bfloat16) for _ in range(2)]
        ys = [torch.empty_like(x) for x in xs]
        rec("transpose_bf16_8192x8192", 2 * 8192 * 8192 * 2, lambda i: bsir.transpose(xs[i % 2], out=ys[i % 2]))
        del xs, ys
    if want("cumsum_f32_32768x4096"):
        xs = [torch.randn(32768, 4096, device="cuda") for _ in range(2)]
        ys = [torch.empty_like(x) for x in xs]
        rec("cumsum_f32_32768x4096", 2 * 32768 * 4096 * 4, lambda i: bsir.cumulative("sum", xs[i % 2], dim=1, out=ys[i % 2]),
            note="sequential along the row, as the reference's loop: exact float sums")
        del xs, ys
    if want("cumsum_f32_32768x4096_axis0"):
        xs = [torch.randn(32768, 4096, device="cuda") for _ in range(2)]
        ys = [torch.empty_like(x) for x in xs]
        rec("cumsum_f32_32768x4096_axis0", 2 * 32768 * 4096 * 4, lambda i: bsir.cumulative("sum", xs[i % 2], dim=0, out=ys[i % 2]),
            note="sequential down the rows: 32768 dependent adds a column, 128 warps in all (one per 128 bytes of columns)")
        del xs, ys
    if want("interleave2_f32_32768x2048"):
        xs = [[torch.randn(32768, 2048, device="cuda") for _ in range(2)] for _ in range(2)]
        ys = [torch.empty(32768, 4096, device="cuda") for _ in range(2)]
        rec("interleave2_f32_32768x2048", 2 * 32768 * 4096 * 4, lambda i: bsir.interleave(xs[i % 2], out=ys[i % 2]))
        del xs, ys
    if want("sort_f32_1024x8192"):
        xs = [torch.randn(1024, 8192, device="cuda") for _ in range(2)]
        rec("sort_f32_1024x8192", 1024 * 8192 * (4 + 4 + 4), lambda i: bsir.sort(xs[i % 2], descending=True),
            note="values + int32 indices; four stable radix passes over keys in device scratch, two tiles a row")
        del xs
    if want("sort_f32_256x152064"):
        xs = [torch.randn(256, 152064, device="cuda") for _ in range(2)]
        rec("sort_f32_256x152064", 256 * 152064 * (4 + 4 + 4), lambda i: bsir.sort(xs[i % 2], descending=True),
            note="values + int32 indices; four stable radix passes over keys in device scratch")
        del xs
    for m in (16, 128, 4096):
        if not want(f"w8a8_m{m}"):
            continue
        try:
            sets = [W.w8a8_input(m, seed=s) for s in range(3 if m < 4096 else 2)]
            outs = [torch.empty(m, 14336, dtype=torch.bfloat16, device="cuda") for _ in sets]
            k = len(sets)
            byts = m * 4096 + 4096 * 14336 + m * 14336 * 2 + m * 4 + 14336 * 4
            rec(f"w8a8_m{m}", byts,
                lambda i: bsir.matmul_w8a8(sets[i % k][0], sets[i % k][2], sets[i % k][1], sets[i % k][3], out=outs[i % k]),
                flops=2 * m * 4096 * 14336)
            del sets, outs
        except Exception as e:
            res[f"w8a8_m{m}"] = {"error": str(e)[:200]}
    # linalg.matmul bf16 x bf16 -> bf16 (f32 accumulation), 4096^3, B as [k, n] and as [n, k]; and hivm.hir.matmul with
    # bias, per-channel descale and relu fused into the way out
    for nm, tb, fused in (("gemm_bf16_4096", False, False), ("gemm_bf16_4096_tb", True, False), ("gemm_bf16_4096_bias_descale_relu", False, True)):
        if not want(nm):
            continue
        try:
            g = torch.Generator(device="cuda").manual_seed(1)
            aa = [torch.randn(4096, 4096, generator=g, device="cuda").to(torch.bfloat16) for _ in range(3)]    # 3 x 96 MB > L2
            bb = [(torch.randn(4096, 4096, generator=g, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(3)]
            oo = [torch.empty(4096, 4096, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
            bias = torch.randn(4096, generator=g, device="cuda").to(torch.bfloat16) if fused else None
            desc = (torch.rand(4096, generator=g, device="cuda") + 0.5).to(torch.bfloat16) if fused else None
            rec(nm, 3 * 4096 * 4096 * 2,
                lambda i: bsir.matmul(aa[i % 3], bb[i % 3], transpose_b=tb, bias=bias, descale=desc, relu=fused, out=oo[i % 3]),
                flops=2 * 4096 ** 3)
            if nm in res and "tops" in res[nm]:
                res[nm]["frac_bf16_sustained"] = res[nm]["tops"] / bf16_sustained if bf16_sustained else None
                res[nm]["frac_bf16_burst"] = res[nm]["tops"] / tensor_peak
                res[nm].pop("frac_int8_peak_2x_bf16", None)
            del aa, bb, oo
        except Exception as e:
            res[nm] = {"error": str(e)[:200]}
    # hivm.hir.matmul bf16 of few rows against [14336, 4096] weights (the decode kernel's form: bound by the 117 MB of weights)
    for m in (1, 16):
        if not want(f"gemm_bf16_m{m}_n14336_k4096"):
            continue
        try:
            g = torch.Generator(device="cuda").manual_seed(2)
            ww = [(torch.randn(14336, 4096, generator=g, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(2)]   # 2 x 117 MB > L2
            aa = torch.randn(m, 4096, generator=g, device="cuda").to(torch.bfloat16)
            oo = torch.empty(m, 14336, dtype=torch.bfloat16, device="cuda")
            rec(f"gemm_bf16_m{m}_n14336_k4096", 14336 * 4096 * 2 + m * 4096 * 2 + m * 14336 * 2,
                lambda i: bsir.matmul(aa, ww[i % 2], transpose_b=True, out=oo), flops=2 * m * 4096 * 14336)
            if f"gemm_bf16_m{m}_n14336_k4096" in res:
                res[f"gemm_bf16_m{m}_n14336_k4096"].pop("frac_int8_peak_2x_bf16", None)
            del ww, aa, oo
        except Exception as e:
            res[f"gemm_bf16_m{m}_n14336_k4096"] = {"error": str(e)[:200]}
    for m in (1, 8, 16):
        if not want(f"w4a16_m{m}"):
            continue
        try:
            sets = [W.w4a16_input(m, seed=s) for s in range(6)]     # 6 x 30 MB of weights > L2
            outs = [torch.empty(m, 14336, dtype=torch.bfloat16, device="cuda") for _ in sets]
            byts = 4096 * 14336 // 2 + 32 * 14336 * 2 + 32 * 14336 // 2 + m * 4096 * 2 + m * 14336 * 2
            rec(f"w4a16_m{m}", byts, lambda i: bsir.matmul_w4a16(*sets[i % 6], out=outs[i % 6]), flops=2 * m * 4096 * 14336)
            del sets, outs
        except Exception as e:
            res[f"w4a16_m{m}"] = {"error": str(e)[:200]}
    torch.cuda.empty_cache()
    return res


def run_ours(args):
    import torch
    import bsir
    from bsir import workloads as W

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    bsir.lib()
    hbm_peak, tensor_peak, peak_kind = measured_peaks()

    # inputs resident in HBM; NBUF distinct sets so no step re-reads lines still in L2
    xs = [W.quant_input(ROWS, COLS, seed=rank * 100 + s) for s in range(NBUF)]
    qs = [torch.empty(ROWS, COLS, dtype=torch.int8, device="cuda") for _ in range(NBUF)]
    ss = [torch.empty(ROWS, dtype=torch.float32, device="cuda") for _ in range(NBUF)]

    def step(i):
        bsir.quant_per_token_i8(xs[i % NBUF], q=qs[i % NBUF], scale=ss[i % NBUF])

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    # the K timed steps are captured once in a CUDA graph: the loop is launch-bound from Python
    # (a 30 us kernel behind a ~10 us ctypes call), and a graph keeps the host out of the timed region
    graph = torch.cuda.CUDAGraph()
    launches0 = bsir.launch_count()
    with torch.cuda.graph(graph):
        for i in range(args.steps):
            step(i)
    launches = bsir.launch_count() - launches0
    graph.replay()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
        torch.cuda.synchronize()
    with ClockSampler(local) as clocks:
        # exactly K steps per measurement; five measurements, the median is reported (one replay lasts well under a
        # millisecond, so a single sample would carry any one-off hiccup of the box: 47 us instead of 32 us per step
        # was seen in one of three 2-GPU runs)
        samples = []
        for _ in range(5):
            if dist:
                dist.barrier()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()               # exactly K steps
            end.record()
            torch.cuda.synchronize()
            samples.append(start.elapsed_time(end))
        total_ms = sorted(samples)[len(samples) // 2]
        t_keep = time.perf_counter()     # keep the GPU under the same load while the sampler reads clocks
        while time.perf_counter() - t_keep < 0.8:
            graph.replay()
            torch.cuda.synchronize()
    kernel_ms = total_ms / args.steps
    if dist:
        t = torch.tensor([total_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
        dist.barrier()
    value = ALGO_BYTES * args.steps * world / (total_ms * 1e-3) / 1e9

    # end to end through the public call with HOST buffers: H2D of the batch, kernel, D2H of q + scales
    hx = torch.empty(ROWS, COLS, dtype=torch.bfloat16).pin_memory()
    hx.copy_(xs[0])
    hq = torch.empty(ROWS, COLS, dtype=torch.int8).pin_memory()
    hs = torch.empty(ROWS, dtype=torch.float32).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    chunks = 8
    rows_c = ROWS // chunks
    streams = [torch.cuda.Stream() for _ in range(2)]

    def e2e_step():
        # row chunks pipelined over two streams so the copies in both directions overlap the kernel
        for c in range(chunks):
            st = streams[c % 2]
            r0, r1 = c * rows_c, (c + 1) * rows_c
            with torch.cuda.stream(st):
                xs[1][r0:r1].copy_(hx[r0:r1], non_blocking=True)
                bsir.quant_per_token_i8(xs[1][r0:r1], q=qs[1][r0:r1], scale=ss[1][r0:r1])
                hq[r0:r1].copy_(qs[1][r0:r1], non_blocking=True)
                hs[r0:r1].copy_(ss[1][r0:r1], non_blocking=True)
        # no host wait here: a chunk always uses the same stream, so step i+1's copies of a chunk queue behind
        # step i's, and the device-to-host tail of one step overlaps the host-to-device head of the next; the
        # timed region ends with a device synchronise, when every step's results are in host memory

    e2e_step()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if dist:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = ALGO_BYTES * world / e2e_s / 1e9
    ok = bool((hq[:8].cuda() == qs[1][:8]).all())

    line = None
    if rank == 0:
        achieved = ALGO_BYTES / (kernel_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32->i8", "data": "synthetic",
            "config": {"workload": "per-token dynamic int8 quantisation, x bf16 [16384,4096] ~ N(0,1) with 0.1% x20 outliers",
                       "rows_per_gpu": ROWS, "cols": COLS, "round_mode": "rint", "saturate": True,
                       "l2": f"{NBUF} input/output sets rotated; one set (201 MB) exceeds the 126 MB L2",
                       "parallelism": f"rows sharded over {world} GPU(s), no collective",
                       "timing": "CUDA events around one graph of exactly K steps, barrier + synchronise on both sides; "
                                 "median of 5 such measurements, max over ranks",
                       "timed_samples_ms": [round(x, 4) for x in samples]},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "traffic": NCU_TRAFFIC_BYTES, "traffic_note": NCU_TRAFFIC_NOTE,
                         "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": ALGO_BYTES, "kernel_ms": kernel_ms,
                         "frac_of_nominal_8000": achieved / 8000.0},
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": ROWS * COLS * 2,
                    "d2h_bytes_per_step": ROWS * COLS + ROWS * 4, "ms_per_step": e2e_s * 1e3,
                    "readback_matches_device": ok},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
        }
        if world == 1:
            g1, _ = cpu_baseline_quant(1, 512)
            import oracle as O
            gN, _ = cpu_baseline_quant(O.max_threads(), 2048)
            line["cpu_baseline"] = {"value": g1, "unit": "GB/s", "cores": 1, "kind": "port",
                                    "sample": "512 of 16384 rows, best of 3 (scalar single-thread loops, as the reference's CPU lowering runs)",
                                    "all_cores": {"value": gN, "cores": O.max_threads(), "sample": "2048 rows, rows in parallel"}}
            if not args.no_ops:
                del xs, qs, ss
                torch.cuda.empty_cache()
                line["ops"] = other_ops(torch, bsir, W, hbm_peak, tensor_peak, iters=max(3, min(args.steps, 20)),
                                        only=args.only_op)
    if dist and world > 1 and not args.no_ops:
        # the N-sharded GEMMs with their exchange step: every rank takes part, rank 0 reports
        del xs, qs, ss
        torch.cuda.empty_cache()
        sharded = sharded_gemm_ops(torch, dist, bsir, W, rank, world, iters=max(3, min(args.steps, 20)))
        if rank == 0:
            line["ops"] = sharded
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-ops", action="store_true", help="skip the per-configuration table")
    ap.add_argument("--only-op", default=None, help="run just this entry of the per-configuration table (for profiling)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
