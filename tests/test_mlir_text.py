"""The MLIR-assembly front end (bsir/mlir_text.py): parsing on CPU, execution through the CUDA library on GPU.
The IR below is written for these tests in the reference's syntax (generic `ins(...) outs(...)` form, attribute
spellings of HFusionNamedStructuredOps.yaml / HIVMDMAOps.td)."""
import os

import numpy as np
import pytest

import oracle as O

QUANT_IR = """
// per-token int8 quantisation as the composition of hot-path ops
module {
func.func @quant(%x: tensor<64x512xbf16>, %q_out: tensor<64x512xi8>, %scale_out: tensor<64xf32>)
    -> (tensor<64x512xi8>, tensor<64xf32>) attributes {hacc.entry} {
  %e0 = tensor.empty() : tensor<64x512xf32>
  %x32 = hfusion.cast {round_mode = #hfusion.round_mode<rint>} ins(%x : tensor<64x512xbf16>) outs(%e0 : tensor<64x512xf32>) -> tensor<64x512xf32>
  %e1 = tensor.empty() : tensor<64x512xf32>
  %ax = linalg.elemwise_unary {fun = #linalg.unary_fn<abs>} ins(%x32 : tensor<64x512xf32>) outs(%e1 : tensor<64x512xf32>) -> tensor<64x512xf32>
  %amax = linalg.reduce { arith.maximumf } ins(%ax : tensor<64x512xf32>) outs(%scale_out : tensor<64xf32>) dimensions = [1]
  %c127 = arith.constant 1.270000e+02 : f32
  %e2 = tensor.empty() : tensor<64xf32>
  %scale = linalg.elemwise_binary {fun = #linalg.binary_fn<div>} ins(%amax, %c127 : tensor<64xf32>, f32) outs(%e2 : tensor<64xf32>) -> tensor<64xf32>
  %e3 = tensor.empty() : tensor<64x512xf32>
  %brc = linalg.broadcast ins(%scale : tensor<64xf32>) outs(%e3 : tensor<64x512xf32>) dimensions = [1]
  %e4 = tensor.empty() : tensor<64x512xf32>
  %y = linalg.elemwise_binary {fun = #linalg.binary_fn<div>} ins(%x32, %brc : tensor<64x512xf32>, tensor<64x512xf32>)
         outs(%e4 : tensor<64x512xf32>) -> tensor<64x512xf32>
  %q = hfusion.cast {round_mode = #hfusion.round_mode<rint>, enable_saturate = true}
         ins(%y : tensor<64x512xf32>) outs(%q_out : tensor<64x512xi8>) -> tensor<64x512xi8>
  return %q, %scale : tensor<64x512xi8>, tensor<64xf32>
}
}
"""

VEC_IR = """
func.func @axpy(%a: memref<1000xf32, #hivm.address_space<gm>>, %b: memref<1000xf32, #hivm.address_space<gm>>,
                %out: memref<1024xf32, #hivm.address_space<gm>>) attributes {hacc.entry, hacc.function_kind = #hacc.function_kind<DEVICE>} {
  %ua = memref.alloc() : memref<1000xf32, #hivm.address_space<ub>>
  hivm.hir.load ins(%a : memref<1000xf32, #hivm.address_space<gm>>) outs(%ua : memref<1000xf32, #hivm.address_space<ub>>)
  %ub = memref.alloc() : memref<1000xf32, #hivm.address_space<ub>>
  hivm.hir.load ins(%b : memref<1000xf32, #hivm.address_space<gm>>) outs(%ub : memref<1000xf32, #hivm.address_space<ub>>)
  %t = memref.alloc() : memref<1000xf32, #hivm.address_space<ub>>
  hivm.hir.vmul ins(%ua, %ub : memref<1000xf32, #hivm.address_space<ub>>, memref<1000xf32, #hivm.address_space<ub>>) outs(%t : memref<1000xf32, #hivm.address_space<ub>>)
  %s = memref.alloc() : memref<1000xf32, #hivm.address_space<ub>>
  hivm.hir.vadd ins(%t, %ua : memref<1000xf32, #hivm.address_space<ub>>, memref<1000xf32, #hivm.address_space<ub>>) outs(%s : memref<1000xf32, #hivm.address_space<ub>>)
  %pad = arith.constant 7.500000e+00 : f32
  %c8 = arith.constant 8 : index
  %p = memref.alloc() : memref<1024xf32, #hivm.address_space<ub>>
  hivm.hir.load ins(%s : memref<1000xf32, #hivm.address_space<ub>>) outs(%p : memref<1024xf32, #hivm.address_space<ub>>)
      pad_mode = #hivm.padmode<PadValue> pad_value = %pad : f32 left_padding_num = %c8 : index
  hivm.hir.store ins(%p : memref<1024xf32, #hivm.address_space<ub>>) outs(%out : memref<1024xf32, #hivm.address_space<gm>>) atomic = <add>
  return
}
"""

ARGMAX_IR = """
func.func @pick(%x: tensor<8x4096xf32>, %v0: tensor<8xf32>, %i0: tensor<8xi32>, %lo: tensor<8x4096xf32>) -> (tensor<8xf32>, tensor<8xi32>, tensor<8x4096xf32>) {
  %v, %i = hfusion.reduce_with_index {tie_break_left = true} <max> ins(%x : tensor<8x4096xf32>) outs(%v0, %i0 : tensor<8xf32>, tensor<8xi32>) dimensions = [1] -> tensor<8xf32>, tensor<8xi32>
  %zero = arith.constant 0.000000e+00 : f32
  %m0 = tensor.empty() : tensor<8x4096xi1>
  %mask = hfusion.compare {compare_fn = #hfusion.compare_fn<vlt>} ins(%x, %zero : tensor<8x4096xf32>, f32) outs(%m0 : tensor<8x4096xi1>) -> tensor<8x4096xi1>
  %r = hfusion.select ins(%mask, %zero, %x : tensor<8x4096xi1>, f32, tensor<8x4096xf32>) outs(%lo : tensor<8x4096xf32>) -> tensor<8x4096xf32>
  return %v, %i, %r : tensor<8xf32>, tensor<8xi32>, tensor<8x4096xf32>
}
"""


RMS_IR = """
func.func @rms(%x: tensor<40x512xf16>, %gamma: tensor<512xf16>, %out0: tensor<40x512xf16>, %out1: tensor<40xf16>)
      -> (tensor<40x512xf16>, tensor<40xf16>) attributes {hfusion.fusion_kind = #hfusion.fusion_kind<LAST_AXIS_PBR>} {
  %c1 = arith.constant 1 : index
  %t0 = tensor.empty() : tensor<40x512xf32>
  %x32 = hfusion.cast {round_mode = #hfusion.round_mode<rint>} ins(%x : tensor<40x512xf16>) outs(%t0 : tensor<40x512xf32>) -> tensor<40x512xf32>
  %t1 = tensor.empty() : tensor<512xf32>
  %g32 = hfusion.cast {round_mode = #hfusion.round_mode<rint>} ins(%gamma : tensor<512xf16>) outs(%t1 : tensor<512xf32>) -> tensor<512xf32>
  %d = tensor.dim %x32, %c1 : tensor<40x512xf32>
  %eps = arith.constant 1.000000e-06 : f32
  %t2 = tensor.empty() : tensor<40x512xf32>
  %sq = linalg.elemwise_binary {fun = #linalg.binary_fn<mul>} ins(%x32, %x32 : tensor<40x512xf32>, tensor<40x512xf32>) outs(%t2 : tensor<40x512xf32>) -> tensor<40x512xf32>
  %t3 = tensor.empty() : tensor<40xf32>
  %ss = linalg.reduce { arith.addf } ins(%sq : tensor<40x512xf32>) outs(%t3 : tensor<40xf32>) dimensions = [1]
  %one = arith.constant 1.0 : f32
  %di = arith.index_castui %d : index to i32
  %df = arith.uitofp %di : i32 to f32
  %inv = arith.divf %one, %df : f32
  %t4 = tensor.empty() : tensor<40xf32>
  %mean = linalg.elemwise_binary {fun = #linalg.binary_fn<mul>} ins(%ss, %inv : tensor<40xf32>, f32) outs(%t4 : tensor<40xf32>) -> tensor<40xf32>
  %t5 = tensor.empty() : tensor<40xf32>
  %v = linalg.elemwise_binary {fun = #linalg.binary_fn<add>} ins(%mean, %eps : tensor<40xf32>, f32) outs(%t5 : tensor<40xf32>) -> tensor<40xf32>
  %t6 = tensor.empty() : tensor<40xf32>
  %sd = hfusion.elemwise_unary {fun = #hfusion.unary_fn<sqrt>} ins(%v : tensor<40xf32>) outs(%t6 : tensor<40xf32>) -> tensor<40xf32>
  %t7 = tensor.empty() : tensor<40xf32>
  %r = hfusion.elemwise_unary {fun = #hfusion.unary_fn<rec>} ins(%sd : tensor<40xf32>) outs(%t7 : tensor<40xf32>) -> tensor<40xf32>
  %t8 = tensor.empty() : tensor<40x512xf32>
  %rb = linalg.broadcast ins(%r : tensor<40xf32>) outs(%t8 : tensor<40x512xf32>) dimensions = [1]
  %t9 = tensor.empty() : tensor<40x512xf32>
  %xn = linalg.elemwise_binary {fun = #linalg.binary_fn<mul>} ins(%rb, %x32 : tensor<40x512xf32>, tensor<40x512xf32>) outs(%t9 : tensor<40x512xf32>) -> tensor<40x512xf32>
  %t10 = tensor.empty() : tensor<40x512xf32>
  %gb = linalg.broadcast ins(%g32 : tensor<512xf32>) outs(%t10 : tensor<40x512xf32>) dimensions = [0]
  %t11 = tensor.empty() : tensor<40x512xf32>
  %y32 = linalg.elemwise_binary {fun = #linalg.binary_fn<mul>} ins(%gb, %xn : tensor<40x512xf32>, tensor<40x512xf32>) outs(%t11 : tensor<40x512xf32>) -> tensor<40x512xf32>
  %y = hfusion.cast {round_mode = #hfusion.round_mode<rint>} ins(%y32 : tensor<40x512xf32>) outs(%out0 : tensor<40x512xf16>) -> tensor<40x512xf16>
  %rs = hfusion.cast {round_mode = #hfusion.round_mode<rint>} ins(%r : tensor<40xf32>) outs(%out1 : tensor<40xf16>) -> tensor<40xf16>
  return %y, %rs : tensor<40x512xf16>, tensor<40xf16>
}
"""


def _mlir_text():
    import importlib.util
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "..", "ascendnpu-ir_b200", "bsir", "mlir_text.py")
    spec = importlib.util.spec_from_file_location("bsir_mlir_text_standalone", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_parser_splits_ops_and_attributes():
    M = _mlir_text()
    fn = M.parse(QUANT_IR)["quant"]
    assert [a[0] for a in fn.args] == ["%x", "%q_out", "%scale_out"]
    assert fn.op_names() == ["tensor.empty", "hfusion.cast", "tensor.empty", "linalg.elemwise_unary", "linalg.reduce",
                             "arith.constant", "tensor.empty", "linalg.elemwise_binary", "tensor.empty", "linalg.broadcast",
                             "tensor.empty", "linalg.elemwise_binary", "hfusion.cast", "return"]
    last_cast = fn.ops[-2]
    assert last_cast.attr("round_mode") == "rint" and last_cast.attr("enable_saturate") is True
    assert fn.ops[4].int_list("dimensions") == [1]
    ins, types = fn.ops[7].group("ins")
    assert ins == ["%amax", "%c127"] and types == ["tensor<64xf32>", "f32"]
    vec = M.parse(VEC_IR)["axpy"]
    assert vec.op_names().count("hivm.hir.load") == 3 and vec.ops[-2].name == "hivm.hir.store"
    assert vec.ops[-3].attr("pad_mode") == "PadValue"
    with pytest.raises(M.MlirTextError):
        M.parse("module {}")


@pytest.mark.skipif(not os.environ.get("BSIR_REFERENCE_DIR"), reason="needs a checkout of the reference (BSIR_REFERENCE_DIR)")
def test_reference_files_parse_unchanged():
    M = _mlir_text()
    ref = os.environ["BSIR_REFERENCE_DIR"]
    for rel, fn_name in (("bishengir/test/Integration/HIVM/VecAdd/add.mlir", "add"),
                         ("bishengir/test/bishengir-compile/hfusion/compile-rms-norm-fp16-split-n.mlir", "rms_norm_f16")):
        with open(os.path.join(ref, rel), encoding="utf-8") as f:
            fn = M.parse(f.read())[fn_name]
        assert fn.op_names()[-1] == "return" and len(fn.ops) >= 8
    # every function of the reference's HFusion compile tests must at least split into ops; most use only ops
    # this front end executes
    import glob
    files = glob.glob(os.path.join(ref, "bishengir/test/bishengir-compile/hfusion/*.mlir"))
    assert len(files) >= 20
    nfuncs = sum(len(M.parse(open(f, encoding="utf-8").read())) for f in files)
    assert nfuncs >= len(files)


# ------------------------------------------------------------------------------------------------ GPU
@pytest.fixture(scope="module")
def bsir():
    import bsir as B
    B.lib()
    return B


@pytest.mark.gpu
def test_quant_chain_equals_fused_kernel_and_oracle(bsir):
    import torch
    from bsir import mlir_text
    from conftest import to_bits
    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn(64, 512, generator=g, device="cuda") * 3).to(torch.bfloat16)
    x[3] = 0                                                         # an all-zero row: 0/0 -> NaN -> 0
    fn = mlir_text.parse(QUANT_IR)["quant"]
    q, scale = fn(x, torch.empty(64, 512, dtype=torch.int8, device="cuda"), torch.empty(64, device="cuda"))
    fq, fs = bsir.quant_per_token_i8(x)
    assert torch.equal(q, fq) and torch.equal(scale.view(torch.int32), fs.view(torch.int32))
    wq, ws = O.quant_per_token_i8(O.BF16, to_bits(x))
    assert np.array_equal(q.cpu().numpy(), wq) and np.array_equal(scale.cpu().numpy().view(np.uint32), ws.view(np.uint32))


@pytest.mark.gpu
def test_hivm_vector_program_with_padding_and_atomic_store(bsir):
    import torch
    from bsir import mlir_text
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(1000, generator=g, device="cuda")
    b = torch.randn(1000, generator=g, device="cuda")
    out = torch.ones(1024, device="cuda")
    mlir_text.parse(VEC_IR)["axpy"](a, b, out)
    want = torch.full((1024,), 7.5, device="cuda")
    want[8:1008] = a * b + a
    assert torch.equal(out, want + 1.0)                              # atomic add onto the ones


@pytest.mark.gpu
def test_reduce_with_index_compare_select_program(bsir):
    import torch
    from bsir import mlir_text
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(8, 4096, generator=g, device="cuda")
    x[2, [7, 900]] = 9.0
    v, i, r = mlir_text.parse(ARGMAX_IR)["pick"](x, torch.empty(8, device="cuda"), torch.empty(8, dtype=torch.int32, device="cuda"),
                                                 torch.empty(8, 4096, device="cuda"))
    assert torch.equal(v, x.max(dim=1).values) and i[2].item() == 7
    assert torch.equal(r, torch.where(x < 0, torch.zeros_like(x), x))


@pytest.mark.gpu
def test_unsupported_op_fails_loudly(bsir):
    import torch
    from bsir import mlir_text
    fn = mlir_text.parse("func.func @f(%x: tensor<4xf32>) -> tensor<4xf32> {\n  %y = hfusion.sort %x : tensor<4xf32>\n  return %y : tensor<4xf32>\n}")["f"]
    with pytest.raises(mlir_text.MlirTextError):
        fn(torch.zeros(4, device="cuda"))


@pytest.mark.gpu
def test_rms_norm_program_against_oracle_and_fused_kernel(bsir):
    """The RMSNorm op chain in the order the reference writes it; the fused kernel computes the same ops, only the
    row sums associate differently (tolerance 1e-2 relative, as for the fused kernel)."""
    import torch
    from bsir import mlir_text
    from conftest import assert_close, to_bits
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(40, 512, generator=g, device="cuda").to(torch.float16)
    gamma = (1 + 0.02 * torch.randn(512, generator=g, device="cuda")).to(torch.float16)
    y, rstd = mlir_text.parse(RMS_IR)["rms"](x, gamma, torch.empty_like(x), torch.empty(40, dtype=torch.float16, device="cuda"))
    wy, wr = O.rms_norm(O.F16, to_bits(x), to_bits(gamma), 1e-6, want_rstd=True)
    assert_close(y, wy, 1e-2, 1e-3, "rms-norm program vs oracle")
    assert_close(rstd, wr, 1e-2, 1e-3, "rstd vs oracle")
    fy, fr = bsir.rms_norm(x, gamma, 1e-6, want_rstd=True)
    assert (y.float() - fy.float()).abs().max().item() <= 1e-2 * fy.float().abs().max().item()


VIEW_IR = """
func.func @views(%x: tensor<4x6x8xf32>, %o: tensor<8x24xf32>) -> tensor<8x24xf32> {
  %c = tensor.collapse_shape %x [[0, 1], [2]] : tensor<4x6x8xf32> into tensor<24x8xf32>
  %t = linalg.transpose ins(%c : tensor<24x8xf32>) outs(%o : tensor<8x24xf32>) permutation = [1, 0]
  return %t : tensor<8x24xf32>
}
func.func @slice(%x: tensor<16x32xf32>, %o: tensor<4x8xf32>) -> tensor<4x8xf32> {
  %s = tensor.extract_slice %x[2, 8] [4, 8] [2, 1] : tensor<16x32xf32> to tensor<4x8xf32>
  %e = linalg.elemwise_unary {fun = #linalg.unary_fn<negf>} ins(%s : tensor<4x8xf32>) outs(%o : tensor<4x8xf32>) -> tensor<4x8xf32>
  return %e : tensor<4x8xf32>
}
"""


@pytest.mark.gpu
def test_views_transpose_and_slices(bsir):
    import torch
    from bsir import mlir_text
    fns = mlir_text.parse(VIEW_IR)
    x = torch.arange(4 * 6 * 8, device="cuda", dtype=torch.float32).reshape(4, 6, 8)
    y = fns["views"](x, torch.empty(8, 24, device="cuda"))
    assert torch.equal(y, x.reshape(24, 8).t())
    z = torch.randn(16, 32, device="cuda")
    assert torch.equal(fns["slice"](z, torch.empty(4, 8, device="cuda")), -z[2:10:2, 8:16])


GELU_IR = """
func.func @gelu(%x: tensor<64x1024xbf16>, %out: tensor<64x1024xbf16>) -> tensor<64x1024xbf16> {
  %e0 = tensor.empty() : tensor<64x1024xf32>
  %x32 = hfusion.cast {round_mode = #hfusion.round_mode<rint>} ins(%x : tensor<64x1024xbf16>) outs(%e0 : tensor<64x1024xf32>) -> tensor<64x1024xf32>
  %c0 = arith.constant 4.471500e-02 : f32
  %c1 = arith.constant 0.797884583 : f32
  %one = arith.constant 1.000000e+00 : f32
  %half = arith.constant 5.000000e-01 : f32
  %e1 = tensor.empty() : tensor<64x1024xf32>
  %x2 = linalg.elemwise_unary {fun = #linalg.unary_fn<square>} ins(%x32 : tensor<64x1024xf32>) outs(%e1 : tensor<64x1024xf32>) -> tensor<64x1024xf32>
  %x3 = linalg.elemwise_binary {fun = #linalg.binary_fn<mul>} ins(%x2, %x32 : tensor<64x1024xf32>, tensor<64x1024xf32>) outs(%e1 : tensor<64x1024xf32>) -> tensor<64x1024xf32>
  %a = linalg.elemwise_binary {fun = #linalg.binary_fn<mul>} ins(%x3, %c0 : tensor<64x1024xf32>, f32) outs(%e1 : tensor<64x1024xf32>) -> tensor<64x1024xf32>
  %b = linalg.elemwise_binary {fun = #linalg.binary_fn<add>} ins(%a, %x32 : tensor<64x1024xf32>, tensor<64x1024xf32>) outs(%e1 : tensor<64x1024xf32>) -> tensor<64x1024xf32>
  %c = linalg.elemwise_binary {fun = #linalg.binary_fn<mul>} ins(%b, %c1 : tensor<64x1024xf32>, f32) outs(%e1 : tensor<64x1024xf32>) -> tensor<64x1024xf32>
  %t = linalg.elemwise_unary {fun = #linalg.unary_fn<tanh>} ins(%c : tensor<64x1024xf32>) outs(%e1 : tensor<64x1024xf32>) -> tensor<64x1024xf32>
  %u = linalg.elemwise_binary {fun = #linalg.binary_fn<add>} ins(%t, %one : tensor<64x1024xf32>, f32) outs(%e1 : tensor<64x1024xf32>) -> tensor<64x1024xf32>
  %e2 = tensor.empty() : tensor<64x1024xf32>
  %hx = linalg.elemwise_binary {fun = #linalg.binary_fn<mul>} ins(%x32, %half : tensor<64x1024xf32>, f32) outs(%e2 : tensor<64x1024xf32>) -> tensor<64x1024xf32>
  %y32 = linalg.elemwise_binary {fun = #linalg.binary_fn<mul>} ins(%hx, %u : tensor<64x1024xf32>, tensor<64x1024xf32>) outs(%e1 : tensor<64x1024xf32>) -> tensor<64x1024xf32>
  %y = hfusion.cast {round_mode = #hfusion.round_mode<rint>} ins(%y32 : tensor<64x1024xf32>) outs(%out : tensor<64x1024xbf16>) -> tensor<64x1024xbf16>
  return %y : tensor<64x1024xbf16>
}
"""


def _launches(bsir):
    return int(bsir.lib().bsir_launch_count())


@pytest.mark.gpu
def test_f32_elementwise_region_runs_as_one_kernel(bsir):
    """bf16 -> f32, nine elementwise ops (two sub-expressions meet in the last one), -> bf16: one launch instead of
    eleven, and the same bits as running the ops one by one."""
    import torch
    from bsir import mlir_text
    from conftest import to_bits
    fn = mlir_text.parse(GELU_IR)["gelu"]
    x = torch.randn(64, 1024, device="cuda").to(torch.bfloat16)
    n0 = _launches(bsir)
    y = fn(x, torch.empty_like(x))
    assert _launches(bsir) - n0 == 1
    assert bsir.FusedChain.last_path() == "compiled"
    fn.fuse = False
    n0 = _launches(bsir)
    w = fn(x, torch.empty_like(x))
    assert _launches(bsir) - n0 == 11
    assert np.array_equal(to_bits(y), to_bits(w))


@pytest.mark.gpu
def test_rms_norm_program_runs_as_one_kernel(bsir):
    """The outlined LAST_AXIS_PBR function (casts, square, row sum, scalar tail, broadcasts, two multiplies, two
    results) runs as ONE kernel; against op-by-op execution only the association of the row sum differs."""
    import torch
    from bsir import mlir_text
    from conftest import assert_close, to_bits
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(40, 512, generator=g, device="cuda").to(torch.float16)
    gamma = (1 + 0.02 * torch.randn(512, generator=g, device="cuda")).to(torch.float16)
    fn = mlir_text.parse(RMS_IR)["rms"]
    out = lambda: (torch.empty_like(x), torch.empty(40, dtype=torch.float16, device="cuda"))
    n0 = _launches(bsir)
    y, r = fn(x, gamma, *out())
    fused = _launches(bsir) - n0
    fn.fuse = False
    n0 = _launches(bsir)
    wy, wr = fn(x, gamma, *out())
    eager = _launches(bsir) - n0
    assert fused == 1 and eager >= 14
    assert bsir.FusedChain.last_path() == "compiled"
    assert_close(y, to_bits(wy), 2e-3, 1e-4, "fused vs op-by-op y")
    assert_close(r, to_bits(wr), 2e-3, 1e-4, "fused vs op-by-op rstd")


SOFTMAX_IR = """
func.func @softmax(%x: tensor<64x1000xf32>, %out: tensor<64x1000xf32>) -> tensor<64x1000xf32> {
  %ninf = arith.constant 0xFF800000 : f32
  %zero = arith.constant 0.000000e+00 : f32
  %m0 = tensor.empty() : tensor<64xf32>
  %m1 = linalg.fill ins(%ninf : f32) outs(%m0 : tensor<64xf32>) -> tensor<64xf32>
  %e0 = tensor.empty() : tensor<64x1000xf32>
  %xs = linalg.elemwise_binary {fun = #linalg.binary_fn<mul>} ins(%x, %zero : tensor<64x1000xf32>, f32) outs(%e0 : tensor<64x1000xf32>) -> tensor<64x1000xf32>
  %x1 = linalg.elemwise_binary {fun = #linalg.binary_fn<add>} ins(%xs, %x : tensor<64x1000xf32>, tensor<64x1000xf32>) outs(%e0 : tensor<64x1000xf32>) -> tensor<64x1000xf32>
  %mx = linalg.reduce { arith.maximumf } ins(%x1 : tensor<64x1000xf32>) outs(%m1 : tensor<64xf32>) dimensions = [1]
  %e1 = tensor.empty() : tensor<64x1000xf32>
  %mb = linalg.broadcast ins(%mx : tensor<64xf32>) outs(%e1 : tensor<64x1000xf32>) dimensions = [1]
  %e2 = tensor.empty() : tensor<64x1000xf32>
  %d = linalg.elemwise_binary {fun = #linalg.binary_fn<sub>} ins(%x1, %mb : tensor<64x1000xf32>, tensor<64x1000xf32>) outs(%e2 : tensor<64x1000xf32>) -> tensor<64x1000xf32>
  %e3 = tensor.empty() : tensor<64x1000xf32>
  %ex = linalg.elemwise_unary {fun = #linalg.unary_fn<exp>} ins(%d : tensor<64x1000xf32>) outs(%e3 : tensor<64x1000xf32>) -> tensor<64x1000xf32>
  %s0 = tensor.empty() : tensor<64xf32>
  %sm = linalg.reduce { arith.addf } ins(%ex : tensor<64x1000xf32>) outs(%s0 : tensor<64xf32>) dimensions = [1]
  %e4 = tensor.empty() : tensor<64x1000xf32>
  %sb = linalg.broadcast ins(%sm : tensor<64xf32>) outs(%e4 : tensor<64x1000xf32>) dimensions = [1]
  %y = linalg.elemwise_binary {fun = #linalg.binary_fn<div>} ins(%ex, %sb : tensor<64x1000xf32>, tensor<64x1000xf32>) outs(%out : tensor<64x1000xf32>) -> tensor<64x1000xf32>
  return %y : tensor<64x1000xf32>
}
"""


@pytest.mark.gpu
def test_softmax_program_with_two_reductions_runs_as_one_kernel(bsir):
    """Two row reductions and a sub-expression (the exponentials) with two users: one kernel, one temporary."""
    import torch
    from bsir import mlir_text
    x = 3 * torch.randn(64, 1000, device="cuda")
    fn = mlir_text.parse(SOFTMAX_IR)["softmax"]
    n0 = _launches(bsir)
    y = fn(x, torch.empty_like(x))
    assert _launches(bsir) - n0 == 1
    want = torch.softmax(x.double(), dim=1)
    assert (y.double() - want).abs().max().item() < 1e-6
    fn.fuse = False
    w = fn(x, torch.empty_like(x))
    assert (y - w).abs().max().item() < 1e-6


CUM_IR = """
func.func @vcumsum(%arg0: tensor<64x16xf32>) -> tensor<64x16xf32> {
  %0 = tensor.empty() : tensor<64x16xf32>
  %1 = hivm.hir.vcumsum ins(%arg0 : tensor<64x16xf32>) outs(%0 : tensor<64x16xf32>) cum_dims = [0] reverse = false -> tensor<64x16xf32>
  return %1 : tensor<64x16xf32>
}
func.func @gather(%src: memref<100x7x4xf16>, %idx: memref<100x6x4xi32>, %dst: memref<100x6x4xf16>) {
  hivm.hir.vgather ins(%src : memref<100x7x4xf16>) indices(%idx : memref<100x6x4xi32>) outs(%dst : memref<100x6x4xf16>) gather_axis = 1
  return
}
func.func @sort(%src: memref<8x100xf32>, %v: memref<8x100xf32>, %i: memref<8x100xi32>) {
  hivm.hir.vsort ins(%src : memref<8x100xf32>) outs(%v, %i : memref<8x100xf32>, memref<8x100xi32>) descending = true sort_axis = 1
  return
}
func.func @rev(%arg0: tensor<100xi32>) -> tensor<100xi32> {
  %1 = hfusion.cumsum %arg0 : tensor<100xi32> cum_dims = [0] reverse = true -> tensor<100xi32>
  return %1 : tensor<100xi32>
}
"""


@pytest.mark.gpu
def test_cumulative_ops_in_both_spellings(bsir):
    """The vcumsum function of test/ExecutionEngine/convert-hivm-to-upstream.mlir:417-423, and the value form."""
    import torch
    from bsir import mlir_text
    from conftest import to_bits
    fns = mlir_text.parse(CUM_IR)
    x = torch.randn(64, 16, device="cuda")
    assert np.array_equal(to_bits(fns["vcumsum"](x)), O.cumulative("sum", O.F32, to_bits(x), axis=0))
    v = torch.arange(100, device="cuda", dtype=torch.int32)
    assert torch.equal(fns["rev"](v), torch.flip(torch.cumsum(torch.flip(v, [0]), 0), [0]).to(torch.int32))
    src = torch.randn(100, 7, 4, device="cuda").to(torch.float16)
    idx = torch.randint(0, 7, (100, 6, 4), device="cuda", dtype=torch.int32)
    dst = torch.empty(100, 6, 4, device="cuda", dtype=torch.float16)
    fns["gather"](src, idx, dst)
    assert torch.equal(dst, torch.gather(src, 1, idx.long()))
    s = torch.randn(8, 100, device="cuda")
    sv, si = torch.empty_like(s), torch.empty(8, 100, device="cuda", dtype=torch.int32)
    fns["sort"](s, sv, si)
    want = torch.sort(s, dim=1, descending=True, stable=True)
    assert torch.equal(sv, want.values) and torch.equal(si.long(), want.indices)


MATMUL_IR = """
func.func @single_cube(%a: tensor<48x256xf16>, %w: tensor<384x256xf16>, %c: tensor<48x384xf16> {hacc.arg_type = #hacc.arg_type<output>})
    -> tensor<48x384xf16> attributes {hacc.entry, hfusion.fusion_kind = #hfusion.fusion_kind<SINGLE_CUBE>} {
  %0 = linalg.matmul_transpose_b ins(%a, %w : tensor<48x256xf16>, tensor<384x256xf16>) outs(%c : tensor<48x384xf16>) -> tensor<48x384xf16>
  return %0 : tensor<48x384xf16>
}
func.func @dot_int8(%a: tensor<32x128xi8>, %b: tensor<128x256xi8>) -> tensor<32x256xi32> {
  %e = tensor.empty() : tensor<32x256xi32>
  %0 = linalg.matmul ins(%a, %b : tensor<32x128xi8>, tensor<128x256xi8>) outs(%e : tensor<32x256xi32>) -> tensor<32x256xi32>
  %1 = linalg.matmul ins(%a, %b : tensor<32x128xi8>, tensor<128x256xi8>) outs(%0 : tensor<32x256xi32>) -> tensor<32x256xi32>
  return %1 : tensor<32x256xi32>
}
func.func @batched(%a: tensor<3x16x64xbf16>, %b: tensor<3x64x128xbf16>) -> tensor<3x16x128xf32> {
  %e = tensor.empty() : tensor<3x16x128xf32>
  %0 = linalg.batch_matmul ins(%a, %b : tensor<3x16x64xbf16>, tensor<3x64x128xbf16>) outs(%e : tensor<3x16x128xf32>) -> tensor<3x16x128xf32>
  return %0 : tensor<3x16x128xf32>
}
"""


@pytest.mark.gpu
def test_matmul_forms_accumulate_onto_their_init(bsir):
    """linalg.matmul and its transposed / batched forms run on the tensor core; the op adds to its init, a bare
    tensor.empty counting as zero (the SINGLE_CUBE function of the reference's compile tests has this shape)."""
    import torch
    from bsir import mlir_text
    fns = mlir_text.parse(MATMUL_IR)
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn(48, 256, generator=g, device="cuda").half()
    w = torch.randn(384, 256, generator=g, device="cuda").half()
    c = torch.randn(48, 384, generator=g, device="cuda").half()
    want = (c.float() + a.float() @ w.float().t()).half()
    got = fns["single_cube"](a, w, c.clone())
    assert torch.allclose(got.float(), want.float(), rtol=2e-3, atol=2e-2)
    ai = torch.randint(-127, 128, (32, 128), generator=g, device="cuda", dtype=torch.int8)
    bi = torch.randint(-127, 128, (128, 256), generator=g, device="cuda", dtype=torch.int8)
    prod = (ai.cpu().int() @ bi.cpu().int()).cuda()
    assert torch.equal(fns["dot_int8"](ai, bi), 2 * prod)             # the second matmul accumulates onto the first
    ab = torch.randn(3, 16, 64, generator=g, device="cuda").bfloat16()
    bb = torch.randn(3, 64, 128, generator=g, device="cuda").bfloat16()
    assert torch.allclose(fns["batched"](ab, bb), torch.bmm(ab.float(), bb.float()), rtol=1e-3, atol=1e-2)


SCALAR_IR = """
func.func @pieces(%a: tensor<4x8xf32>, %b: tensor<4x24xf32>) -> (tensor<4x32xf32>, tensor<3xindex>) {
  %c7 = arith.constant 7 : index
  %c2 = arith.constant 2 : index
  %cm7 = arith.constant -7 : index
  %q = arith.divui %c7, %c2 : index
  %r = arith.remsi %cm7, %c2 : index
  %p = arith.cmpi slt, %r, %q : index
  %s = arith.select %p, %q, %r : index
  %t = tensor.from_elements %q, %r, %s : tensor<3xindex>
  %cat = tensor.concat dim(1) %a, %b : (tensor<4x8xf32>, tensor<4x24xf32>) -> tensor<4x32xf32>
  return %cat, %t : tensor<4x32xf32>, tensor<3xindex>
}
"""


@pytest.mark.gpu
def test_scalar_arithmetic_from_elements_and_concat(bsir):
    import torch
    from bsir import mlir_text
    a, b = torch.randn(4, 8, device="cuda"), torch.randn(4, 24, device="cuda")
    cat, t = mlir_text.parse(SCALAR_IR)["pieces"](a, b)
    assert torch.equal(cat, torch.cat([a, b], dim=1))
    assert t.tolist() == [3, -1, 3]                                   # 7 / 2, -7 rem 2 (sign of the dividend), select


HIVM_MORE_IR = """
func.func @vector_ops(%x: tensor<16x64xf32>, %y: tensor<16x64xf32>, %row: tensor<1x64xf32>, %i: tensor<16x64xi32>, %j: tensor<16x64xi32>)
    -> (tensor<16x64xf32>, tensor<16x64xf32>, tensor<64x16xf32>, tensor<16x64xi32>, tensor<16x128xf32>, tensor<16x32xf32>, tensor<16x64xi32>) {
  %e0 = tensor.empty() : tensor<16x64xf32>
  %ex = hivm.hir.vexp ins(%x : tensor<16x64xf32>) outs(%e0 : tensor<16x64xf32>) -> tensor<16x64xf32>
  %e1 = tensor.empty() : tensor<16x64xi1>
  %lt = hivm.hir.vcmp ins(%x, %y : tensor<16x64xf32>, tensor<16x64xf32>) outs(%e1 : tensor<16x64xi1>) compare_mode = <lt> -> tensor<16x64xi1>
  %e2 = tensor.empty() : tensor<16x64xf32>
  %sel = hivm.hir.vsel ins(%lt, %ex, %y : tensor<16x64xi1>, tensor<16x64xf32>, tensor<16x64xf32>) outs(%e2 : tensor<16x64xf32>) -> tensor<16x64xf32>
  %e3 = tensor.empty() : tensor<16x64xf32>
  %b = hivm.hir.vbrc ins(%row : tensor<1x64xf32>) outs(%e3 : tensor<16x64xf32>) broadcast_dims = [0] -> tensor<16x64xf32>
  %e4 = tensor.empty() : tensor<16x64xf32>
  %sum = hivm.hir.vadd ins(%sel, %b : tensor<16x64xf32>, tensor<16x64xf32>) outs(%e4 : tensor<16x64xf32>) -> tensor<16x64xf32>
  %e5 = tensor.empty() : tensor<64x16xf32>
  %t = hivm.hir.vtranspose ins(%sum : tensor<16x64xf32>) outs(%e5 : tensor<64x16xf32>) permutation = [1, 0] -> tensor<64x16xf32>
  %e6 = tensor.empty() : tensor<16x64xi32>
  %a = hivm.hir.vand ins(%i, %j : tensor<16x64xi32>, tensor<16x64xi32>) outs(%e6 : tensor<16x64xi32>) -> tensor<16x64xi32>
  %e7 = tensor.empty() : tensor<16x128xf32>
  %il = hivm.hir.vinterleave ins(%x, %y : tensor<16x64xf32>, tensor<16x64xf32>) outs(%e7 : tensor<16x128xf32>) interleave_channel_nums = 2 -> tensor<16x128xf32>
  %e8 = tensor.empty() : tensor<16x32xf32>
  %odd = hivm.hir.vdeinterleave ins(%x : tensor<16x64xf32>) outs(%e8 : tensor<16x32xf32>) channel_num = 32 index_mode = <CHANNEL_1> -> tensor<16x32xf32>
  %c5 = arith.constant 5 : index
  %c64 = arith.constant 64 : index
  %c1 = arith.constant 1 : index
  %e9 = tensor.empty() : tensor<16x64xi32>
  %ar = hivm.hir.varange offset[%c5] strides[%c64, %c1] outs(%e9 : tensor<16x64xi32>) -> tensor<16x64xi32>
  return %sel, %sum, %t, %a, %il, %odd, %ar : tensor<16x64xf32>, tensor<16x64xf32>, tensor<64x16xf32>, tensor<16x64xi32>, tensor<16x128xf32>, tensor<16x32xf32>, tensor<16x64xi32>
}
"""


@pytest.mark.gpu
def test_more_hivm_vector_ops(bsir):
    import torch
    from bsir import mlir_text
    g = torch.Generator(device="cuda").manual_seed(3)
    x, y = torch.randn(16, 64, generator=g, device="cuda"), torch.randn(16, 64, generator=g, device="cuda")
    row = torch.randn(1, 64, generator=g, device="cuda")
    i = torch.randint(0, 1 << 20, (16, 64), generator=g, device="cuda", dtype=torch.int32)
    j = torch.randint(0, 1 << 20, (16, 64), generator=g, device="cuda", dtype=torch.int32)
    fn = mlir_text.parse(HIVM_MORE_IR)["vector_ops"]
    fn.fuse = False                                     # op by op: every op through its own library call
    sel, total, t, a, il, odd, ar = fn(x, y, row, i, j)
    ex = bsir.elemwise_unary("exp", x)
    want_sel = torch.where(x < y, ex, y)
    assert torch.equal(sel, want_sel) and torch.equal(total, want_sel + row) and torch.equal(t, (want_sel + row).t())
    assert torch.equal(a, i & j)
    assert torch.equal(il, torch.stack([x, y], dim=-1).reshape(16, 128)) and torch.equal(odd, x[:, 1::2])
    assert torch.equal(ar.cpu(), (5 + torch.arange(16 * 64, dtype=torch.int32)).reshape(16, 64))


TERNARY_IR = """
func.func @fma_and_bits(%a: tensor<8x32xf32>, %b: tensor<8x32xf32>, %c: tensor<8x32xf32>) -> (tensor<8x32xf32>, tensor<8x32xi32>) {
  %e = tensor.empty() : tensor<8x32xf32>
  %l = hfusion.load ins(%a : tensor<8x32xf32>) outs(%e : tensor<8x32xf32>) -> tensor<8x32xf32>
  %e1 = tensor.empty() : tensor<8x32xf32>
  %f = hfusion.elemwise_ternary {fun = #hfusion.ternary_fn<fma>} ins(%l, %b, %c : tensor<8x32xf32>, tensor<8x32xf32>, tensor<8x32xf32>) outs(%e1 : tensor<8x32xf32>) -> tensor<8x32xf32>
  %e2 = tensor.empty() : tensor<8x32xi32>
  %bits = hfusion.bitcast ins(%f : tensor<8x32xf32>) outs(%e2 : tensor<8x32xi32>) -> tensor<8x32xi32>
  return %f, %bits : tensor<8x32xf32>, tensor<8x32xi32>
}
"""


@pytest.mark.gpu
def test_ternary_bitcast_load(bsir):
    import torch
    from bsir import mlir_text
    a, b, c = (torch.randn(8, 32, device="cuda") for _ in range(3))
    f, bits = mlir_text.parse(TERNARY_IR)["fma_and_bits"](a, b, c)
    want = torch.from_numpy(np.asarray([float(np.float32(np.float64(x) * np.float64(y) + np.float64(z))) for x, y, z in
                                        zip(a.flatten().tolist(), b.flatten().tolist(), c.flatten().tolist())], dtype=np.float32)).reshape(8, 32)
    assert torch.equal(f.cpu(), want) and torch.equal(bits.cpu(), want.view(torch.int32))


GENERIC_IR = """
func.func @generic_forms(%x: tensor<300x128xf32>, %y: tensor<300x128xf32>, %v: tensor<128xf32>) -> (tensor<300x128xf32>, tensor<300xf32>, tensor<f32>) {
  %half = arith.constant 5.000000e-01 : f32
  %e = tensor.empty() : tensor<300x128xf32>
  %d = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                       iterator_types = ["parallel", "parallel"]} ins(%x, %y : tensor<300x128xf32>, tensor<300x128xf32>) outs(%e : tensor<300x128xf32>) {
  ^bb0(%in: f32, %in_1: f32, %out: f32):
    %0 = arith.subf %in, %in_1 : f32
    %1 = arith.mulf %0, %half : f32
    %2 = math.exp %1 : f32
    linalg.yield %2 : f32
  } -> tensor<300x128xf32>
  %r0 = tensor.empty() : tensor<300xf32>
  %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>], iterator_types = ["parallel", "reduction"]}
       ins(%d : tensor<300x128xf32>) outs(%r0 : tensor<300xf32>) {
  ^bb0(%in: f32, %out: f32):
    %0 = arith.addf %in, %out : f32
    linalg.yield %0 : f32
  } -> tensor<300xf32>
  %s0 = tensor.empty() : tensor<f32>
  %s = linalg.generic {indexing_maps = [affine_map<(d0) -> (d0)>, affine_map<(d0) -> ()>], iterator_types = ["reduction"]} ins(%v : tensor<128xf32>) outs(%s0 : tensor<f32>) {
  ^bb0(%in: f32, %out: f32):
    %0 = arith.maximumf %in, %out : f32
    linalg.yield %0 : f32
  } -> tensor<f32>
  return %d, %r, %s : tensor<300x128xf32>, tensor<300xf32>, tensor<f32>
}
"""


@pytest.mark.gpu
def test_linalg_generic_elementwise_and_reduction_bodies(bsir):
    """The hand-written linalg.generic forms of the reference's tile-reduction tests: an elementwise body runs as one
    fused kernel with the bits of op-by-op execution, a one-combiner body over the last axis as a row reduction."""
    import torch
    from bsir import mlir_text
    g = torch.Generator(device="cuda").manual_seed(8)
    x, y = torch.randn(300, 128, generator=g, device="cuda"), torch.randn(300, 128, generator=g, device="cuda")
    v = torch.randn(128, generator=g, device="cuda")
    d, r, s = mlir_text.parse(GENERIC_IR)["generic_forms"](x, y, v)
    want = bsir.elemwise_unary("exp", bsir.elemwise_binary("mul", bsir.elemwise_binary("sub", x, y), 0.5))
    assert torch.equal(d, want)
    assert torch.allclose(r, want.sum(dim=1), rtol=1e-5, atol=1e-4) and s.item() == v.max().item() and s.dim() == 0
