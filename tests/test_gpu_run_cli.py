"""GPU: `python -m bsir.run` -- a function of an MLIR file runs on the seeded inputs of the reference's runner and its
outputs are dumped in the runner's format (host main built by bishengir/lib/ExecutionEngine/CreateHostMain.cpp; data and
dump format: BiShengIRRunnerUtils.cpp:63-125)."""
import os
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(HERE, "..", "ascendnpu-ir_b200")
sys.path.insert(0, PKG)
sys.path.insert(0, os.path.join(HERE, ".."))

pytestmark = pytest.mark.gpu

KERNEL = """
module {
  func.func @colsums(%a: memref<?x5xf32> {hacc.arg_type = #hacc.arg_type<input>}, %b: memref<?x5xf32> {hacc.arg_type = #hacc.arg_type<input>},
                     %sa: memref<5xf32> {hacc.arg_type = #hacc.arg_type<output>}, %sb: memref<5xf32> {hacc.arg_type = #hacc.arg_type<output>},
                     %s: memref<5xf32> {hacc.arg_type = #hacc.arg_type<output>})
      attributes {hacc.function_kind = #hacc.function_kind<HOST>} {
    %zero = arith.constant 0.0 : f32
    linalg.fill ins(%zero : f32) outs(%sa : memref<5xf32>)
    linalg.reduce {arith.addf} ins(%a : memref<?x5xf32>) outs(%sa : memref<5xf32>) dimensions = [0]
    linalg.fill ins(%zero : f32) outs(%sb : memref<5xf32>)
    linalg.reduce {arith.addf} ins(%b : memref<?x5xf32>) outs(%sb : memref<5xf32>) dimensions = [0]
    linalg.elemwise_binary {fun = #linalg.binary_fn<add>} ins(%sa, %sb : memref<5xf32>, memref<5xf32>) outs(%s : memref<5xf32>)
    func.return
  }
}
"""

TENSOR_FN = """
func.func @scale_cast(%x: tensor<64x96xf16>, %y: tensor<64x96xf16>) -> tensor<64x96xf32> {
  %e = tensor.empty() : tensor<64x96xf16>
  %m = linalg.elemwise_binary {fun = #linalg.binary_fn<mul>} ins(%x, %y : tensor<64x96xf16>, tensor<64x96xf16>) outs(%e : tensor<64x96xf16>) -> tensor<64x96xf16>
  %f = tensor.empty() : tensor<64x96xf32>
  %r = hfusion.cast {round_mode = #hfusion.round_mode<rint>} ins(%m : tensor<64x96xf16>) outs(%f : tensor<64x96xf32>) -> tensor<64x96xf32>
  return %r : tensor<64x96xf32>
}
"""


def _cli(tmp_path, text, *extra):
    src = tmp_path / "k.mlir"
    src.write_text(text)
    fin, fout = tmp_path / "in.txt", tmp_path / "out.txt"
    env = dict(os.environ, PYTHONPATH=PKG + os.pathsep + os.environ.get("PYTHONPATH", ""))
    subprocess.run([sys.executable, "-m", "bsir.run", str(src), "--input-file", str(fin), "--output-file", str(fout), *extra],
                   check=True, env=env, timeout=600)
    from bsir import runner_data
    return runner_data.read_data(fin.read_text()), runner_data.read_data(fout.read_text())


def test_memref_kernel_with_dynamic_rows(tmp_path):
    from bsir import runner_data
    ins, outs = _cli(tmp_path, KERNEL, "--dyn", "7", "7")
    # every argument, outputs included, is filled from the one f32 generator in order and dumped to the input file
    gen = runner_data.RunnerData()
    want = [gen.get_data("f32", s) for s in ([7, 5], [7, 5], [5], [5], [5])]
    assert [s for s, _ in ins] == [[7, 5], [7, 5], [5], [5], [5]]
    for (sizes, toks), w in zip(ins, want):
        assert toks == ["%.9e" % float(v) for v in w.reshape(-1)]
    assert [s for s, _ in outs] == [[5], [5], [5]]
    got = [np.array([float(t) for t in toks], dtype=np.float32) for _, toks in outs]
    sa = want[0].astype(np.float64).sum(0)
    sb = want[1].astype(np.float64).sum(0)
    assert np.allclose(got[0], sa, rtol=1e-5, atol=1e-2) and np.allclose(got[1], sb, rtol=1e-5, atol=1e-2)
    assert np.array_equal(got[2], got[0] + got[1])                    # the dump's 10 significant digits carry an f32 exactly


def test_tensor_function_reports_what_it_returns(tmp_path):
    from bsir import runner_data
    ins, outs = _cli(tmp_path, TENSOR_FN)
    gen = runner_data.RunnerData()
    x = gen.get_data("f16", [64, 96]).view(np.float16)
    y = gen.get_data("f16", [64, 96]).view(np.float16)               # the f16 generator goes on after x
    assert len(ins) == 2 and len(outs) == 1 and outs[0][0] == [64, 96]
    got = np.array([float(t) for t in outs[0][1]], dtype=np.float32).reshape(64, 96)
    want = (x.astype(np.float32) * y.astype(np.float32)).astype(np.float16).astype(np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
