"""Operator surface under the reference's op names (layer B3): torch CUDA tensors in, attribute keywords spelled as
in the reference IR.  Every function here is the library call of the same name in the package root."""
from . import (cast, compare, copy, default_round_mode, elemwise_binary, elemwise_unary, load, matmul_w4a16, matmul_w8a8,
               quant_per_token_i8, reduce, reduce_with_index, rms_norm, select, softmax, store, vadd, vdiv, vmul, vsub)

# hfusion.* / linalg.* / hivm.hir.* spellings
hfusion_cast = cast
hfusion_elemwise_unary = linalg_elemwise_unary = elemwise_unary
hfusion_elemwise_binary = linalg_elemwise_binary = elemwise_binary
hfusion_compare = compare
hfusion_select = select
hfusion_reduce_with_index = reduce_with_index
linalg_reduce = hivm_vreduce = reduce
linalg_copy = hivm_copy = copy
hivm_load = load
hivm_store = store
hivm_vadd, hivm_vsub, hivm_vmul, hivm_vdiv = vadd, vsub, vmul, vdiv

__all__ = [n for n in dir() if not n.startswith("_")]
