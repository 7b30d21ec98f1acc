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


def test_further_vector_op_library_symbols(bsir):
    """cumsum / cumprod, sort, interleave / deinterleave, arange, transpose, gather under the reference's symbol names."""
    L = bsir.lib()
    L.bsir_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    mr = lambda t: C.byref(bsir.memref(t))
    g = torch.Generator(device="cuda").manual_seed(4)
    # cumsum along the first axis of [r, a]; reverse; the middle axis of [a, r, a]
    x = torch.randn(37, 96, generator=g, device="cuda")
    y = torch.empty_like(x)
    assert L._mlir_ciface_cumsum_ra_float(mr(x), mr(y)) == 0
    assert np.array_equal(y.cpu().numpy(), O.cumulative("sum", O.F32, x.cpu().numpy(), axis=0))
    assert L._mlir_ciface_cumsum_ra_reverse_float(mr(x), mr(y)) == 0
    assert np.array_equal(y.cpu().numpy(), O.cumulative("sum", O.F32, x.cpu().numpy(), axis=0, reverse=True))
    xi = torch.randint(-3, 4, (5, 11, 64), generator=g, device="cuda", dtype=torch.int32)
    yi = torch.empty_like(xi)
    assert L._mlir_ciface_cumprod_ara_int32_t(mr(xi), mr(yi)) == 0
    for a0 in range(5):
        assert np.array_equal(yi[a0].cpu().numpy(), O.cumulative("prod", O.I32, xi[a0].cpu().numpy(), axis=0))
    assert L._mlir_ciface_cumsum_ara_reverse_int32_t(mr(xi), mr(yi)) == 0
    assert np.array_equal(yi[2].cpu().numpy(), O.cumulative("sum", O.I32, xi[2].cpu().numpy(), axis=0, reverse=True))
    # sort with index, NaN included
    s = torch.randn(1000, generator=g, device="cuda")
    s[[5, 999]] = float("nan")
    sv, si, tmp = torch.empty_like(s), torch.empty(1000, dtype=torch.int32, device="cuda"), torch.empty(1, device="cuda")
    L._mlir_ciface_sort_with_index_1d_float.argtypes = [C.c_void_p] * 4 + [C.c_bool]
    assert L._mlir_ciface_sort_with_index_1d_float(mr(s), mr(sv), mr(si), mr(tmp), True) == 0
    wv, wi = O.sort_last_axis(O.F32, s.cpu().numpy()[None, :], descending=True)
    assert np.array_equal(si.cpu().numpy(), wi[0]) and np.array_equal(sv.cpu().numpy().view(np.uint32), wv[0].view(np.uint32))
    L._mlir_ciface_sort_1d_half.argtypes = [C.c_void_p] * 3 + [C.c_bool]
    h = torch.randn(333, generator=g, device="cuda").half()
    hv = torch.empty_like(h)
    assert L._mlir_ciface_sort_1d_half(mr(h), mr(hv), mr(tmp.half()), False) == 0
    assert torch.equal(hv, torch.sort(h).values)
    # interleave / deinterleave
    a, b = torch.randn(640, generator=g, device="cuda").to(torch.bfloat16), torch.randn(640, generator=g, device="cuda").to(torch.bfloat16)
    ab = torch.empty(1280, dtype=torch.bfloat16, device="cuda")
    assert L._mlir_ciface_interleave_1d_bfloat16_t(mr(a), mr(b), mr(ab), mr(ab)) == 0
    assert torch.equal(ab[0::2], a) and torch.equal(ab[1::2], b)
    back = torch.empty_like(a)
    assert L._mlir_ciface_deinterleave_channel_1_from_2_channels_1d_bfloat16_t(mr(ab), mr(back)) == 0
    assert torch.equal(back, b)
    m4 = torch.arange(6 * 32, device="cuda", dtype=torch.int32).reshape(6, 32)
    c0 = torch.empty(6, 8, dtype=torch.int32, device="cuda")
    assert L._mlir_ciface_deinterleave_channel_0_from_n_channels_2d_int32_t(mr(m4), mr(c0)) == 0
    assert torch.equal(c0, m4[:, 0::4])
    # arange
    ar = torch.empty(7, 9, dtype=torch.int32, device="cuda")
    L._mlir_ciface_arange_2d_int32_t.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int64]
    assert L._mlir_ciface_arange_2d_int32_t(mr(ar), 5, 100, -2) == 0
    want = 5 + 100 * torch.arange(7, device="cuda")[:, None] - 2 * torch.arange(9, device="cuda")[None, :]
    assert torch.equal(ar.long(), want)
    # transposes
    t2 = torch.randn(50, 70, generator=g, device="cuda").half()
    o2 = torch.empty(70, 50, dtype=torch.float16, device="cuda")
    assert L._mlir_ciface_transpose_2d_with_last_axis_half(mr(t2), mr(o2)) == 0
    assert torch.equal(o2, t2.t())
    t3 = torch.randint(-100, 100, (4, 6, 40), generator=g, device="cuda", dtype=torch.int32)
    o3 = torch.empty(6, 4, 40, dtype=torch.int32, device="cuda")
    assert L._mlir_ciface_transpose_3d_without_last_axis_int32_t(mr(t3), mr(o3)) == 0
    assert torch.equal(o3, t3.permute(1, 0, 2))
    o3b = torch.empty(40, 6, 4, dtype=torch.int32, device="cuda")
    assert L._mlir_ciface_transpose_3d_with_last_axis_int32_t(mr(t3), mr(o3b)) == 0
    assert torch.equal(o3b, t3.permute(2, 1, 0))
    # gather
    src = torch.randn(500, generator=g, device="cuda")
    idx = torch.randint(0, 500, (333,), generator=g, device="cuda", dtype=torch.int32)
    dst = torch.empty(333, device="cuda")
    assert L._mlir_ciface_gather_1d_float(mr(src), mr(idx), mr(dst), mr(idx)) == 0
    assert torch.equal(dst, src[idx.long()])
    torch.cuda.synchronize()
    assert bsir.device_error() == 0
