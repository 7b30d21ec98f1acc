// chain_jit.h -- run-time compilation of an elementwise chain (chain_jit.cu) for fused_chain.cu.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

#include "bsir_b200.h"

namespace bsir {

// What the generated code depends on: everything about a chain but its sizes and addresses.
struct ChainJitSpec {
  int n_in = 0, n_instr = 0, n_out = 0;
  int in_dtype[8] = {}, in_kind[8] = {};
  bsir_chain_instr tape[24] = {};
  int out_dtype[4] = {}, out_tmp[4] = {};
  bool flat = false;    // every tensor is contiguous and nothing is broadcast along an axis: no row / column arithmetic
  bool alias = false;   // an output overlaps an operand: operands are read with coherent loads
  bool row_grid = false;   // blockIdx.x is the row, blockIdx.y a stretch of it (no division); set by chain_jit_plan
  int unroll = 0;          // groups per thread; 0: chosen from the operands
  // a chain with last-axis reductions (a row program): threads per row and groups per thread; 0: no reductions
  int tpr = 0, vpt = 0;
  bool out_per_row[4] = {};   // the output is a [rows] vector (its value is the same along the row)
  // > 0: the block is persistent and its rows arrive through a ring of this many shared-memory buffers filled by bulk
  // copies (rows so long that one or two blocks fill an SM: without the ring the SM loads, computes and stores in turn)
  int ring = 0;
};

// The kernel's parameter block (the generated source declares the same layout).
struct ChainJitArgs {
  long long gpr, total, rows;   // 8-element groups per row, groups in all, rows
  const void *in[8];
  long long in_stride[8];
  void *out[4];
  long long out_stride[4];
  int *err;   // device error word (a bounded wait that gave up sets a bit in it)
};

int chain_jit_unroll(const ChainJitSpec &s);          // groups per thread
void chain_jit_plan(ChainJitSpec *s, long long groups_per_row);   // picks the thread mapping for rows of this length
std::string chain_jit_source(const ChainJitSpec &s);   // CUDA C++ of the chain's kernel
// NVRTC only (no device needed): 0 and the cubin's size, or -1 and the reason.
int chain_jit_compile_only(const ChainJitSpec &s, size_t *cubin_bytes, std::string *why);
// Compiles (once per distinct source), loads and launches: 0, or -1 and the reason (nothing was enqueued).
int chain_jit_launch(const ChainJitSpec &s, const ChainJitArgs &args, cudaStream_t st, std::string *why);

}  // namespace bsir
