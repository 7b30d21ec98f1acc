"""CPU (no GPU): the C-ABI library loads, exports every symbol the headers declare, and its host-side
argument validation and kernel registry behave; plus the 2-rank sharding logic over gloo."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")


@pytest.fixture(scope="module")
def L():
    import bsir
    return bsir.lib()


def _declared_symbols():
    """Function names declared in include/*.h, after the C preprocessor expanded the symbol tables."""
    out = subprocess.run(["gcc", "-E", "-P", "-I", INC, os.path.join(INC, "bsir_b200.h")], capture_output=True,
                         text=True, check=True).stdout
    names = set(re.findall(r"\b((?:bsir|_mlir_ciface)_[A-Za-z0-9_]+)\s*\(", out))
    return sorted(names)


def test_headers_compile_as_plain_c():
    src = '#include "bsir_b200.h"\nint main(void){bsir_kernel_desc d; bsir_memref_2d m; (void)d; (void)m; return 0;}\n'
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-I", INC, "-x", "c", "-"],
                       input=src, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_library_exports_every_declared_symbol(L):
    names = _declared_symbols()
    assert len(names) > 590, len(names)
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing[:10]
    for must in ("_mlir_ciface_vadd_1d_float", "_mlir_ciface_vadd_1d_half", "_mlir_ciface_vcast_float_to_int8_t_1d_with_mode",
                 "_mlir_ciface_reduce_max_with_index_left_ar_float", "bsir_launch", "bsir_quant_per_token_i8",
                 "bsir_rms_norm", "bsir_softmax", "bsir_matmul_w8a8", "bsir_matmul_w4a16", "bsir_reduce_with_index_static",
                 "_mlir_ciface_matmul_Xbias_Xdescale_XtransposeA_XtransposeB_TAint8_t_TBint8_t_TChalf"):
        assert must in names


def test_library_does_not_link_the_oracle(L):
    import bsir
    out = subprocess.run(["nm", "-D", bsir.LIB_PATH], capture_output=True, text=True).stdout
    assert "orc_" not in out


def test_status_strings_and_version(L):
    assert b"sm_100a" in L.bsir_version()
    assert L.bsir_status_string(0) == b"ok"
    assert L.bsir_dtype_size(2) == 2 and L.bsir_dtype_size(6) == 8 and L.bsir_dtype_size(99) == 0


def test_registry_and_argument_validation_without_a_gpu(L):
    import bsir
    d = bsir.KernelDesc()
    d.kind, d.fn, d.dtype, d.rank = 0, 100, 0, 1
    d.sizes[0] = 16
    assert L.bsir_kernel_register(b"cpu_add", C.byref(d)) == 0
    assert L.bsir_kernel_num_args(b"cpu_add") == 3
    assert L.bsir_kernel_num_args(b"nope") == -8 and b"nope" in L.bsir_last_error()
    args = (C.c_void_p * 2)(None, None)
    assert L.bsir_launch(b"cpu_add", C.c_uint32(1), args, C.c_size_t(16), None) == -9      # wrong args_size
    assert L.bsir_launch(b"nope", C.c_uint32(1), args, C.c_size_t(16), None) == -8
    d.kind = 77
    assert L.bsir_kernel_register(b"bad", C.byref(d)) == -5
    assert L.bsir_kernel_unregister(b"cpu_add") == 0 and L.bsir_kernel_unregister(b"cpu_add") == -8
    # typed entry points reject bad arguments before touching the device
    i64 = C.c_int64
    assert L.bsir_quant_per_token_i8(5, 0, i64(4), i64(8), None, i64(8), None, i64(8), None, None) == -4   # int dtype
    assert L.bsir_quant_per_token_i8(2, 9, i64(4), i64(8), C.c_void_p(16), i64(8), C.c_void_p(16), i64(8), None, None) == -5
    assert L.bsir_softmax(2, i64(-1), i64(8), None, i64(8), None, i64(8), None) == -2
    assert L.bsir_softmax(2, i64(4), i64(8), None, i64(8), None, i64(8), None) == -1
    assert L.bsir_rms_norm(2, i64(4), i64(8), C.c_void_p(16), i64(4), C.c_void_p(16), C.c_float(1e-6), C.c_void_p(16), i64(8), None, None) == -3
    assert L.bsir_reduce_with_index(1, 5, 1, 0, i64(1), i64(8), None, i64(8), None, None, None, i64(0), None) == -4
    assert L.bsir_reduce_with_index_static(1, 2, 1, 0, i64(5000), i64(8), C.c_void_p(16), i64(8), C.c_void_p(16), C.c_void_p(16), None) == -10
    assert L.bsir_matmul_w4a16(i64(1), i64(12), i64(128), i64(128), None, i64(128), None, None, None, None, i64(12), None) == -2
    assert L.bsir_matmul_w8a8(i64(4), i64(8), i64(16), C.c_void_p(16), i64(8), C.c_void_p(16), i64(8), 0, None, None, 2, C.c_void_p(16), i64(8), None, None, i64(0), None) == -3
    assert L.bsir_cast(0, 3, 0, 9, 1, (i64 * 3)(4, 0, 0), None, None, None, None, None) == -5
    # empty problems are fine and need no pointers
    assert L.bsir_softmax(2, i64(0), i64(8), None, i64(8), None, i64(8), None) == 0
    assert L.bsir_matmul_w8a8(i64(0), i64(8), i64(16), None, i64(16), None, i64(8), 0, None, None, 2, None, i64(8), None, None, i64(0), None) == 0


def test_even_split_properties():
    from bsir import shard
    for total, parts, mult in ((16384, 8, 1), (14336, 8, 8), (14336, 3, 16), (7, 4, 1), (256, 8, 1), (0, 2, 1), (152, 5, 8)):
        r = shard.even_split(total, parts, mult)
        assert r[0][0] == 0 and r[-1][1] == total and all(a[1] == b[0] for a, b in zip(r, r[1:]))
        sizes = [hi - lo for lo, hi in r]
        assert all(s % mult == 0 for s in sizes) and max(sizes) - min(sizes) <= mult
    with pytest.raises(ValueError):
        shard.even_split(10, 2, 8)


_WORKER = r'''
import os, sys
sys.path.insert(0, os.path.join(sys.argv[1], "ascendnpu-ir_b200")); sys.path.insert(0, os.path.join(sys.argv[1], "oracle"))
import numpy as np, torch, torch.distributed as dist
import oracle as O
from bsir import shard
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[2], rank=int(sys.argv[3]), world_size=2)
rank, world = dist.get_rank(), 2
rng = np.random.default_rng(0)                      # same data on both ranks
# row-sharded op: per-token quantisation of the rank's rows, reassembled only for the check
x = O.f32_to_bf16(rng.standard_normal((10, 64)).astype(np.float32))
lo, hi = shard.my_rows(10, rank, world)
q, s = O.quant_per_token_i8(O.BF16, x[lo:hi])        # the oracle stands in for the GPU kernel on CPU ranks
q_all = shard.gather_rows(torch.from_numpy(q), 10)
wq, ws = O.quant_per_token_i8(O.BF16, x)
assert np.array_equal(q_all.numpy(), wq)
# N-sharded GEMM: rank holds W[:, lo:hi]; outputs all-gathered to [M, N]
a = rng.integers(-127, 128, (5, 96), dtype=np.int8); w = rng.integers(-127, 128, (96, 48), dtype=np.int8)
sa = rng.uniform(1e-3, 1e-2, 5).astype(np.float32); sw = rng.uniform(1e-3, 1e-2, 48).astype(np.float32)
wl, swl, (c0, c1) = shard.shard_w8a8_weights(torch.from_numpy(w), torch.from_numpy(sw), rank, world)
out_l = O.matmul_w8a8(a, wl.numpy(), sa, swl.numpy())
out = shard.gather_columns(torch.from_numpy(out_l.astype(np.int32)), 48, multiple=16)   # gloo has no 16-bit integer type
want = O.matmul_w8a8(a, w, sa, sw)
assert np.array_equal(out.numpy().astype(np.uint16), want), "gathered GEMM differs"
# uneven column blocks (n = 40 over 2 ranks in multiples of 8 -> 24 + 16)
blocks = shard.even_split(40, 2, 8); mine = blocks[rank]
loc = torch.arange(40).repeat(3, 1)[:, mine[0]:mine[1]].contiguous()
assert torch.equal(shard.gather_columns(loc, 40), torch.arange(40).repeat(3, 1))
dist.barrier(); dist.destroy_process_group()
print("ok", rank)
'''


def test_two_rank_sharding_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    port = str(29500 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, port, str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"ok {r}" in o, o[-2000:]
