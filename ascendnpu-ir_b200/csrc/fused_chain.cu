// fused_chain.cu -- one kernel for a chain of elementwise ops with broadcast operands.
//
// HFusion outlines chains of elementwise / broadcast ops into one function of fusion kind
// PURE_ELEMWISE or ANY_PB (bishengir/lib/Dialect/HFusion/Transforms/OpFusion/FusibleHelper.cpp:52-72)
// and compiles it into one device kernel; for bf16 / f16 data the whole chain then runs in f32 with a
// single rounding at the end (LegalizeBF16 + SimplifyOps,
// bishengir/lib/Dialect/HFusion/Transforms/LegalizeBF16.cpp:243-275, SimplifyOps.cpp:105-230).
// Here the chain arrives as a short tape and one kernel interprets it per 16-byte group of a row, so
// intermediates never touch memory and every input is read once.
//
// Machine: an accumulator and four temporaries, each holding the group's elements as f32.  An
// instruction names an operation and a source: an input operand (loaded on demand and widened), a
// temporary, or an immediate.  Operands are [rows, cols] tensors, [cols] vectors broadcast over the
// rows, [rows] vectors broadcast over the columns, or scalars.  The switch on the operation sits
// outside the per-element loop, so one uniform branch serves the whole group.
#include <cstdint>
#include <cstring>

#include "common.cuh"

namespace bsir {
namespace {

constexpr int kChainMaxOperands = 8;
constexpr int kChainMaxInstr = 24;
constexpr int kChainMaxOutputs = 4;
constexpr int kGroup = 8;   // elements per thread-step: one 16-byte vector of a 16-bit type, two of f32

struct ChainOperand {
  const void *data;
  int64_t row_stride;   // elements; used by kind FULL
  int32_t dtype;        // BSIR_F32 / F16 / BF16
  int32_t kind;         // bsir_chain_operand_kind
};
struct ChainOutput {
  void *data;
  int64_t row_stride;
  int32_t dtype;
  int32_t tmp;          // -1: the accumulator at the end; 0..3: that temporary
};
struct ChainInstr {
  int32_t op;           // bsir_chain_op
  int32_t fn;           // unary / binary function code (the elementwise enums)
  int32_t src_kind;     // bsir_chain_src
  int32_t src;          // operand index / temporary index
  float imm;
};
struct ChainParams {
  int64_t rows, cols;
  int32_t n_in, n_instr, n_out, pad;
  ChainOperand in[kChainMaxOperands];
  ChainOutput out[kChainMaxOutputs];
  ChainInstr tape[kChainMaxInstr];
};

__device__ __forceinline__ float widen_bits(int dtype, const void *p, int64_t i) {
  if (dtype == BSIR_F32) return static_cast<const float *>(p)[i];
  const uint16_t h = static_cast<const uint16_t *>(p)[i];
  return dtype == BSIR_F16 ? __half2float(__ushort_as_half(h)) : __uint_as_float(static_cast<uint32_t>(h) << 16);
}

// the group's elements of an operand, widened to f32
template <bool VEC>
__device__ __forceinline__ void load_group(const ChainOperand &o, int64_t row, int64_t c0, int n, float (&s)[kGroup]) {
  if (o.kind == BSIR_CHAIN_SCALAR || o.kind == BSIR_CHAIN_COL_VECTOR) {
    const float v = widen_bits(o.dtype, o.data, o.kind == BSIR_CHAIN_SCALAR ? 0 : row);
#pragma unroll
    for (int e = 0; e < kGroup; ++e) s[e] = v;
    return;
  }
  const int64_t base = (o.kind == BSIR_CHAIN_FULL ? row * o.row_stride : 0) + c0;
  if constexpr (VEC) {
    if (o.dtype == BSIR_F32) {
      const float4 a = *reinterpret_cast<const float4 *>(static_cast<const float *>(o.data) + base);
      const float4 b = *reinterpret_cast<const float4 *>(static_cast<const float *>(o.data) + base + 4);
      s[0] = a.x; s[1] = a.y; s[2] = a.z; s[3] = a.w; s[4] = b.x; s[5] = b.y; s[6] = b.z; s[7] = b.w;
    } else {
      const uint4 w = *reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(o.data) + base);
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (o.dtype == BSIR_BF16) FloatTraits<BSIR_BF16>::unpack(ws[k], s + 2 * k);
        else FloatTraits<BSIR_F16>::unpack(ws[k], s + 2 * k);
      }
    }
  } else {
#pragma unroll
    for (int e = 0; e < kGroup; ++e) s[e] = e < n ? widen_bits(o.dtype, o.data, base + e) : 0.0f;
  }
}

template <bool VEC>
__device__ __forceinline__ void store_group(const ChainOutput &o, int64_t row, int64_t c0, int n, const float (&v)[kGroup]) {
  const int64_t base = row * o.row_stride + c0;
  if constexpr (VEC) {
    if (o.dtype == BSIR_F32) {
      float *d = static_cast<float *>(o.data) + base;
      *reinterpret_cast<float4 *>(d) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4 *>(d + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      uint32_t w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        w[k] = o.dtype == BSIR_BF16 ? FloatTraits<BSIR_BF16>::pack(v + 2 * k) : FloatTraits<BSIR_F16>::pack(v + 2 * k);
      *reinterpret_cast<uint4 *>(static_cast<uint16_t *>(o.data) + base) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
    for (int e = 0; e < n; ++e) {
      if (o.dtype == BSIR_F32) static_cast<float *>(o.data)[base + e] = v[e];
      else if (o.dtype == BSIR_F16) static_cast<uint16_t *>(o.data)[base + e] = __half_as_ushort(__float2half_rn(v[e]));
      else static_cast<uint16_t *>(o.data)[base + e] = __bfloat16_as_ushort(__float2bfloat16_rn(v[e]));
    }
  }
}

// The scalar function tables of the elementwise kernels, restated for a group (same expressions:
// hfusion unary / binary fns of bishengir/lib/Dialect/HFusion/IR/HFusionOps.cpp:434-639 that have an f32 form).
__device__ __forceinline__ bool chain_unary(int fn, float (&a)[kGroup]) {
#define U(expr)                                                                    \
  {                                                                                \
    _Pragma("unroll") for (int e = 0; e < kGroup; ++e) { const float v = a[e]; a[e] = (expr); } \
    return true;                                                                   \
  }
  switch (fn) {
    case BSIR_UNARY_RELU: U(maximumf(0.0f, v))
    case BSIR_UNARY_SQRT: case BSIR_UNARY_SQRT_L: U(__fsqrt_rn(v))
    case BSIR_UNARY_RSQRT: case BSIR_UNARY_RSQRT_L: U(__fdiv_rn(1.0f, __fsqrt_rn(v)))
    case BSIR_UNARY_REC: case BSIR_UNARY_RECIPROCAL: U(__fdiv_rn(1.0f, v))
    case BSIR_UNARY_TANH: case BSIR_UNARY_TANH_L: U(tanhf(v))
    case BSIR_UNARY_EXP: U(expf(v))
    case BSIR_UNARY_LOG: U(logf(v))
    case BSIR_UNARY_ABS: U(fabsf(v))
    case BSIR_UNARY_CEIL: U(ceilf(v))
    case BSIR_UNARY_FLOOR: U(floorf(v))
    case BSIR_UNARY_NEGF: U(-v)
    case BSIR_UNARY_ROUND: U(roundf(v))
    case BSIR_UNARY_SQUARE: U(__fmul_rn(v, v))
    case BSIR_UNARY_ERF: case BSIR_UNARY_ERF_L: U(erff(v))
    case BSIR_UNARY_SIN: U(sinf(v))
    case BSIR_UNARY_COS: U(cosf(v))
    case BSIR_UNARY_EXP2: U(exp2f(v))
    case BSIR_UNARY_LOG2: U(log2f(v))
    default: return false;
  }
#undef U
}

// acc = fn(acc, s) (REV = false) or fn(s, acc) (REV = true)
template <bool REV>
__device__ __forceinline__ bool chain_binary(int fn, float (&a)[kGroup], const float (&s)[kGroup]) {
#define B(expr)                                                       \
  {                                                                   \
    _Pragma("unroll") for (int e = 0; e < kGroup; ++e) {              \
      const float x = REV ? s[e] : a[e], y = REV ? a[e] : s[e];       \
      a[e] = (expr);                                                  \
    }                                                                 \
    return true;                                                      \
  }
  switch (fn) {
    case BSIR_BINARY_ADD: B(__fadd_rn(x, y))
    case BSIR_BINARY_SUB: B(__fsub_rn(x, y))
    case BSIR_BINARY_MUL: B(__fmul_rn(x, y))
    case BSIR_BINARY_DIV: case BSIR_BINARY_DIVFHP: B(__fdiv_rn(x, y))
    case BSIR_BINARY_MAXF: B(maximumf(x, y))
    case BSIR_BINARY_MINF: B(minimumf(x, y))
    case BSIR_BINARY_MAXNUMF: B(fmaxf(x, y))
    case BSIR_BINARY_MINNUMF: B(fminf(x, y))
    case BSIR_BINARY_POWF: B(powf(x, y))
    default: return false;
  }
#undef B
}

template <bool VEC>
__global__ void __launch_bounds__(256) fused_chain_kernel(const __grid_constant__ ChainParams p, int *bad) {
  const int64_t groups_per_row = (p.cols + kGroup - 1) / kGroup;
  const int64_t total = p.rows * groups_per_row;
  bool ok = true;
  for (int64_t gi = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gi < total;
       gi += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    // 32-bit division when the problem allows it (a 64-bit one costs as much as a tape instruction)
    const int64_t row = total < 0x7fffffffLL ? static_cast<int64_t>(static_cast<uint32_t>(gi) / static_cast<uint32_t>(groups_per_row))
                                             : gi / groups_per_row;
    const int64_t c0 = (gi - row * groups_per_row) * kGroup;
    const int n = p.cols - c0 < kGroup ? static_cast<int>(p.cols - c0) : kGroup;
    float acc[kGroup], t0[kGroup], t1[kGroup], t2[kGroup], t3[kGroup], s[kGroup];
#pragma unroll
    for (int e = 0; e < kGroup; ++e) acc[e] = t0[e] = t1[e] = t2[e] = t3[e] = 0.0f;
    for (int ip = 0; ip < p.n_instr; ++ip) {
      const ChainInstr ins = p.tape[ip];
      if (ins.op == BSIR_CHAIN_SAVE) {      // temporary <- accumulator
        switch (ins.src) {
          case 0: _Pragma("unroll") for (int e = 0; e < kGroup; ++e) t0[e] = acc[e]; break;
          case 1: _Pragma("unroll") for (int e = 0; e < kGroup; ++e) t1[e] = acc[e]; break;
          case 2: _Pragma("unroll") for (int e = 0; e < kGroup; ++e) t2[e] = acc[e]; break;
          default: _Pragma("unroll") for (int e = 0; e < kGroup; ++e) t3[e] = acc[e]; break;
        }
        continue;
      }
      if (ins.op == BSIR_CHAIN_UNARY) {
        ok = chain_unary(ins.fn, acc) && ok;
        continue;
      }
      // the source of a LOAD / BINARY / RBINARY
      if (ins.src_kind == BSIR_CHAIN_SRC_OPERAND) {
        load_group<VEC>(p.in[ins.src], row, c0, n, s);
      } else if (ins.src_kind == BSIR_CHAIN_SRC_IMM) {
#pragma unroll
        for (int e = 0; e < kGroup; ++e) s[e] = ins.imm;
      } else {
        switch (ins.src) {
          case 0: _Pragma("unroll") for (int e = 0; e < kGroup; ++e) s[e] = t0[e]; break;
          case 1: _Pragma("unroll") for (int e = 0; e < kGroup; ++e) s[e] = t1[e]; break;
          case 2: _Pragma("unroll") for (int e = 0; e < kGroup; ++e) s[e] = t2[e]; break;
          default: _Pragma("unroll") for (int e = 0; e < kGroup; ++e) s[e] = t3[e]; break;
        }
      }
      if (ins.op == BSIR_CHAIN_LOAD) {
#pragma unroll
        for (int e = 0; e < kGroup; ++e) acc[e] = s[e];
      } else {
        ok = (ins.op == BSIR_CHAIN_RBINARY ? chain_binary<true>(ins.fn, acc, s) : chain_binary<false>(ins.fn, acc, s)) && ok;
      }
    }
    for (int io = 0; io < p.n_out; ++io) {
      const ChainOutput &o = p.out[io];
      switch (o.tmp) {
        case 0: store_group<VEC>(o, row, c0, n, t0); break;
        case 1: store_group<VEC>(o, row, c0, n, t1); break;
        case 2: store_group<VEC>(o, row, c0, n, t2); break;
        case 3: store_group<VEC>(o, row, c0, n, t3); break;
        default: store_group<VEC>(o, row, c0, n, acc); break;
      }
    }
  }
  if (!ok && bad) *bad = 1;
}

bool chain_float(int dt) { return dt == BSIR_F32 || dt == BSIR_F16 || dt == BSIR_BF16; }

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" int32_t bsir_fused_elementwise(int64_t rows, int64_t cols, int32_t n_in, const bsir_chain_operand *ins,
                                          int32_t n_instr, const bsir_chain_instr *tape, int32_t n_out,
                                          const bsir_chain_output *outs, void *stream) {
  clear_error();
  if (rows < 0 || cols < 0) return fail(BSIR_ERR_SHAPE, "fused_elementwise: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (n_in < 0 || n_in > kChainMaxOperands || n_instr < 1 || n_instr > kChainMaxInstr || n_out < 1 || n_out > kChainMaxOutputs)
    return fail(BSIR_ERR_SHAPE, "fused_elementwise: %d operands (max %d), %d instructions (1..%d), %d outputs (1..%d)", n_in,
                kChainMaxOperands, n_instr, kChainMaxInstr, n_out, kChainMaxOutputs);
  if ((n_in > 0 && !ins) || !tape || !outs) return fail(BSIR_ERR_NULL, "fused_elementwise: null table");
  ChainParams p{};
  p.rows = rows; p.cols = cols; p.n_in = n_in; p.n_instr = n_instr; p.n_out = n_out;
  bool vec = cols % kGroup == 0;
  for (int i = 0; i < n_in; ++i) {
    const bsir_chain_operand &o = ins[i];
    if (!chain_float(o.dtype)) return fail(BSIR_ERR_DTYPE, "fused_elementwise: operand %d dtype %d (f32, f16, bf16)", i, o.dtype);
    if (o.kind < BSIR_CHAIN_FULL || o.kind > BSIR_CHAIN_SCALAR) return fail(BSIR_ERR_ATTR, "fused_elementwise: operand %d kind %d", i, o.kind);
    if (!o.data && rows * cols > 0) return fail(BSIR_ERR_NULL, "fused_elementwise: operand %d is null", i);
    if (o.kind == BSIR_CHAIN_FULL && o.row_stride < cols) return fail(BSIR_ERR_STRIDE, "fused_elementwise: operand %d row stride", i);
    const int eb = dtype_bytes(o.dtype);
    if (!aligned_to(o.data, eb)) return fail(BSIR_ERR_ALIGN, "fused_elementwise: operand %d misaligned", i);
    if (o.kind == BSIR_CHAIN_FULL || o.kind == BSIR_CHAIN_ROW_VECTOR)
      vec = vec && aligned_to(o.data, 16) && (o.kind != BSIR_CHAIN_FULL || (o.row_stride * eb) % 16 == 0);
    p.in[i] = ChainOperand{o.data, o.row_stride, o.dtype, o.kind};
  }
  for (int i = 0; i < n_out; ++i) {
    const bsir_chain_output &o = outs[i];
    if (!chain_float(o.dtype)) return fail(BSIR_ERR_DTYPE, "fused_elementwise: output %d dtype %d", i, o.dtype);
    if (o.tmp < -1 || o.tmp > 3) return fail(BSIR_ERR_ATTR, "fused_elementwise: output %d takes temporary %d", i, o.tmp);
    if (!o.data && rows * cols > 0) return fail(BSIR_ERR_NULL, "fused_elementwise: output %d is null", i);
    if (o.row_stride < cols) return fail(BSIR_ERR_STRIDE, "fused_elementwise: output %d row stride", i);
    const int eb = dtype_bytes(o.dtype);
    if (!aligned_to(o.data, eb)) return fail(BSIR_ERR_ALIGN, "fused_elementwise: output %d misaligned", i);
    vec = vec && aligned_to(o.data, 16) && (o.row_stride * eb) % 16 == 0;
    p.out[i] = ChainOutput{o.data, o.row_stride, o.dtype, o.tmp};
  }
  for (int i = 0; i < n_instr; ++i) {
    const bsir_chain_instr &t = tape[i];
    if (t.op < BSIR_CHAIN_LOAD || t.op > BSIR_CHAIN_SAVE) return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d op %d", i, t.op);
    if (t.op == BSIR_CHAIN_SAVE) {
      if (t.src < 0 || t.src > 3) return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d saves to temporary %d", i, t.src);
    } else if (t.op != BSIR_CHAIN_UNARY) {
      if (t.src_kind < BSIR_CHAIN_SRC_OPERAND || t.src_kind > BSIR_CHAIN_SRC_IMM)
        return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d source kind %d", i, t.src_kind);
      if (t.src_kind == BSIR_CHAIN_SRC_OPERAND && (t.src < 0 || t.src >= n_in))
        return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d reads operand %d of %d", i, t.src, n_in);
      if (t.src_kind == BSIR_CHAIN_SRC_TMP && (t.src < 0 || t.src > 3))
        return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d reads temporary %d", i, t.src);
    }
    // functions are checked on the host, so that a bad tape never launches
    if (t.op == BSIR_CHAIN_UNARY) {
      switch (t.fn) {
        case BSIR_UNARY_SQRT_L: case BSIR_UNARY_RSQRT_L: case BSIR_UNARY_TANH_L: case BSIR_UNARY_ERF_L:
        case BSIR_UNARY_RELU: case BSIR_UNARY_SQRT: case BSIR_UNARY_RSQRT: case BSIR_UNARY_REC: case BSIR_UNARY_RECIPROCAL:
        case BSIR_UNARY_TANH: case BSIR_UNARY_EXP: case BSIR_UNARY_LOG: case BSIR_UNARY_ABS: case BSIR_UNARY_CEIL:
        case BSIR_UNARY_FLOOR: case BSIR_UNARY_NEGF: case BSIR_UNARY_ROUND: case BSIR_UNARY_SQUARE: case BSIR_UNARY_ERF:
        case BSIR_UNARY_SIN: case BSIR_UNARY_COS: case BSIR_UNARY_EXP2: case BSIR_UNARY_LOG2: break;
        default: return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d unary fn %d", i, t.fn);
      }
    } else if (t.op == BSIR_CHAIN_BINARY || t.op == BSIR_CHAIN_RBINARY) {
      switch (t.fn) {
        case BSIR_BINARY_ADD: case BSIR_BINARY_SUB: case BSIR_BINARY_MUL: case BSIR_BINARY_DIV: case BSIR_BINARY_DIVFHP:
        case BSIR_BINARY_MAXF: case BSIR_BINARY_MINF: case BSIR_BINARY_MAXNUMF: case BSIR_BINARY_MINNUMF: case BSIR_BINARY_POWF: break;
        default: return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d binary fn %d", i, t.fn);
      }
    }
    p.tape[i] = ChainInstr{t.op, t.fn, t.src_kind, t.src, t.imm};
  }
  if (rows == 0 || cols == 0) return BSIR_OK;
  cudaStream_t st = resolve_stream(stream);
  const int64_t groups = rows * ceil_div(cols, kGroup);
  int64_t blocks = ceil_div(groups, 256);
  const int64_t cap = static_cast<int64_t>(device_info().sm_count > 0 ? device_info().sm_count : 148) * 32;
  if (blocks > cap) blocks = cap;   // the kernel strides over what the grid does not cover
  if (vec) fused_chain_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, st>>>(p, nullptr);
  else fused_chain_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, st>>>(p, nullptr);
  count_launch();
  return check_launch("fused_elementwise");
}
