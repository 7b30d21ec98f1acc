"""GPU: the `_mlir_ciface_*` library symbols and the compiled-kernel launch ABI."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O
from conftest import assert_bits_equal, assert_close, to_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bsir():
    import bsir as B
    B.lib()
    return B


def test_vadd_ciface_symbols(bsir):
    L = bsir.lib()
    L.bsir_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    a = torch.randn(1000, device="cuda")
    b = torch.randn(1000, device="cuda")
    out = torch.empty_like(a)
    ma, mb, mo = bsir.memref(a), bsir.memref(b), bsir.memref(out)
    assert L._mlir_ciface_vadd_1d_float(C.byref(ma), C.byref(mb), C.byref(mo), None) == 0
    assert_bits_equal(out, O.elemwise_binary("add", O.F32, to_bits(a), to_bits(b)), "vadd_1d_float")
    # descriptor with a non-zero offset and a row stride
    big = torch.randn(64, 80, device="cuda").half()
    va, vb = big[3:35, 8:72], big[10:42, 0:64]
    o2 = torch.empty(32, 64, device="cuda", dtype=torch.float16)
    assert L._mlir_ciface_vadd_2d_half(C.byref(bsir.memref(va)), C.byref(bsir.memref(vb)), C.byref(bsir.memref(o2)), None) == 0
    assert_bits_equal(o2, O.elemwise_binary("add", O.F16, to_bits(va.contiguous()), to_bits(vb.contiguous())), "vadd_2d_half")
    # vector-scalar and scalar-vector forms
    L._mlir_ciface_vmuls_vs_1d_float.argtypes = [C.c_void_p, C.c_float, C.c_void_p, C.c_void_p]
    assert L._mlir_ciface_vmuls_vs_1d_float(C.byref(ma), C.c_float(3.0), C.byref(mo), None) == 0
    assert_bits_equal(out, O.elemwise_binary("mul", O.F32, to_bits(a), np.array([3.0], np.float32)), "vmuls")
    L._mlir_ciface_vsub_sv_1d_float.argtypes = [C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]
    assert L._mlir_ciface_vsub_sv_1d_float(C.c_float(1.0), C.byref(ma), C.byref(mo), None) == 0
    assert_bits_equal(out, O.elemwise_binary("sub", O.F32, np.array([1.0], np.float32), to_bits(a)), "vsub_sv")


def test_vcast_and_reduce_ciface(bsir):
    L = bsir.lib()
    L.bsir_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    x = (torch.randn(4096, device="cuda") * 50)
    out = torch.empty(4096, device="cuda", dtype=torch.int8)
    assert L._mlir_ciface_vcast_float_to_int8_t_1d_with_mode(C.byref(bsir.memref(x)), C.byref(bsir.memref(out)), C.c_uint32(0)) == 0
    assert_bits_equal(out, O.cast(O.F32, O.I8, to_bits(x), "rint", "saturate"), "vcast f32->i8 R")
    m = torch.randn(37, 501, device="cuda")
    dv = torch.empty(37, 1, device="cuda")
    di = torch.empty(37, 1, device="cuda", dtype=torch.int32)
    f = L._mlir_ciface_reduce_max_with_index_left_ar_float
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float]
    assert f(C.byref(bsir.memref(m)), C.byref(bsir.memref(dv)), C.byref(bsir.memref(di)), None, C.c_float(-np.inf)) == 0
    wv, wi = O.reduce_with_index("max", O.F32, to_bits(m), nan_mode="nan_first")
    assert np.array_equal(di.cpu().numpy()[:, 0], wi)
    g = L._mlir_ciface_reduce_sum_ar_float
    g.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float]
    assert g(C.byref(bsir.memref(m)), C.byref(bsir.memref(dv)), None, C.c_float(0.0)) == 0
    assert_close(dv[:, 0].contiguous(), O.reduce_last_axis("sum", O.F32, to_bits(m)), 1e-4, 1e-4, "reduce_sum_ar")


def test_launch_abi_vecadd_like_reference_host(bsir):
    # the reference host: args = {in0, in1, out}; rtKernelLaunch("add", blockDim, args, sizeof(args), ...)
    n = 1 << 20
    bsir.register_kernel("add", "elemwise_binary", fn=bsir.BINARY_FN["add"], dtype=bsir.F32, sizes=[n])
    a, b = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    out = torch.empty_like(a)
    bsir.launch("add", [a, b, out], block_dim=1)
    assert_bits_equal(out, O.elemwise_binary("add", O.F32, to_bits(a), to_bits(b)), "launch add")
    assert bsir.lib().bsir_kernel_num_args(b"add") == 3
    with pytest.raises(bsir.BsirError):
        bsir.launch("add", [a, b])                     # wrong args_size
    with pytest.raises(bsir.BsirError):
        bsir.launch("no_such_kernel", [a, b, out])


def test_launch_abi_fused_kernels(bsir):
    from bsir import workloads as W
    x, w = W.rmsnorm_input(64, 4096, seed=1)
    bsir.register_kernel("rms_norm_bf16", "rms_norm", dtype=bsir.BF16, sizes=[64, 4096], eps=1e-6)
    y = torch.empty_like(x)
    rstd = torch.empty(64, device="cuda", dtype=torch.bfloat16)
    bsir.launch("rms_norm_bf16", [x, w, y, rstd])
    wy, wr = O.rms_norm(O.BF16, to_bits(x), to_bits(w), 1e-6, want_rstd=True)
    assert_close(y, wy, 1e-2, 1e-3, "launch rms_norm")
    xq = W.quant_input(64, 4096, seed=2)
    bsir.register_kernel("quant", "quant_per_token", dtype=bsir.BF16, sizes=[64, 4096])
    q = torch.empty(64, 4096, device="cuda", dtype=torch.int8)
    s = torch.empty(64, device="cuda")
    bsir.launch("quant", [xq, q, s])
    wq, ws = O.quant_per_token_i8(O.BF16, to_bits(xq))
    assert_bits_equal(q, wq, "launch quant")


def test_errors_do_not_abort(bsir):
    a = torch.randn(16, device="cuda")
    with pytest.raises(bsir.BsirError):
        bsir.elemwise_unary("absi", a)               # integer-only function on a float tensor
    with pytest.raises(bsir.BsirError):
        bsir.cast(a.to(torch.int32), torch.int8, overflow_mode="ascend_saturate_trunc_via_f16")
    with pytest.raises(bsir.BsirError):
        bsir.reduce("xori", a.view(4, 4))            # bitwise reduction of floats
    out = bsir.vadd(a, a)                            # the context is still usable
    assert torch.equal(out, a + a)
    assert bsir.device_error() == 0
