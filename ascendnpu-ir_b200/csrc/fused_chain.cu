// fused_chain.cu -- one kernel for a chain of elementwise ops with broadcast operands.
//
// HFusion outlines chains of elementwise / broadcast ops into one function of fusion kind
// PURE_ELEMWISE or ANY_PB (bishengir/lib/Dialect/HFusion/Transforms/OpFusion/FusibleHelper.cpp:52-72)
// and compiles it into one device kernel; for bf16 / f16 data the whole chain then runs in f32 with a
// single rounding at the end (LegalizeBF16 + SimplifyOps,
// bishengir/lib/Dialect/HFusion/Transforms/LegalizeBF16.cpp:243-275, SimplifyOps.cpp:105-230).
// Here the chain arrives as a short tape and one kernel interprets it, so intermediates never touch
// memory and every input is read once.
//
// Machine: an accumulator and four temporaries holding f32 values.  An instruction names an operation
// and a source: an input operand, a temporary, or an immediate.  Operands are [rows, cols] tensors,
// [cols] vectors broadcast over the rows, [rows] vectors broadcast over the columns, or scalars.
//
// Execution: a thread carries G groups of 8 consecutive elements through the tape.
//   1. staging -- every operand's bytes for the thread's groups go to the thread's own column of shared
//      memory: cp.async (16 bytes each) for tensors and [cols] vectors, so that all of a thread's
//      loads are in flight together, then a plain load for per-row values and scalars;
//   2. the tape -- the host has compiled each instruction to a fetch code (how to read the source's
//      slot) and a dense function code, so two jump tables dispatch it for all 8 G elements at once.
//      Only the accumulator lives in registers; temporaries are shared-memory slots like the operands;
//   3. outputs -- rounded once, 16-byte stores.
// A slot is a plane of 16 bytes (or 4, for a per-row value) per thread, so every shared-memory access
// is conflict free, and no barrier is needed: a thread only reads what it wrote or copied itself.
#include <cstdint>
#include <cstdlib>
#include <cstring>

#include "chain_jit.h"
#include "common.cuh"

namespace bsir {
namespace {

constexpr int kChainMaxOperands = 8;
constexpr int kChainMaxInstr = 24;
constexpr int kChainMaxOutputs = 4;
constexpr int kChainTemps = 4;
constexpr int kGroup = 8;            // elements per group: one 16-byte vector of a 16-bit type, two of f32
constexpr int kChainThreads = 256;
constexpr uint32_t kPlane = kChainThreads * 16;   // bytes of one 16-byte-per-thread plane

// how an instruction reads its source
enum Fetch : uint32_t { F_NONE = 0, F_IMM, F_F32, F_BF16, F_F16, F_BCAST };
// what it does with it (dense, so that the switch is a jump table)
enum Fn : uint32_t {
  FN_LOAD = 0, FN_SAVE,
  FN_ADD, FN_MUL, FN_SUB, FN_DIV, FN_MAXF, FN_MINF, FN_MAXNUMF, FN_MINNUMF, FN_POWF,
  FN_RELU, FN_SQRT, FN_RSQRT, FN_REC, FN_TANH, FN_EXP, FN_LOG, FN_ABS, FN_CEIL, FN_FLOOR, FN_NEG, FN_ROUND,
  FN_SQUARE, FN_ERF, FN_SIN, FN_COS, FN_EXP2, FN_LOG2,
  FN_COUNT
};
// how an operand is staged
enum Stage : uint32_t { S_FULL = 0, S_ROW, S_COL, S_SCALAR };

// bytes of a slot for one group
__host__ __device__ constexpr uint32_t slot_group_bytes(uint32_t fetch) {
  return fetch == F_F32 ? 2 * kPlane : fetch == F_BCAST ? kChainThreads * 4u : kPlane;
}

struct DevOperand {
  const void *data;
  int64_t row_stride;   // elements; S_FULL only
  uint32_t stage;       // Stage | dtype << 8 | fetch << 16
  uint32_t off;         // byte offset of the slot in shared memory
};
struct DevOutput {
  void *data;
  int64_t row_stride;
  int32_t dtype;
  int32_t off;          // < 0: the accumulator; else the temporary's slot
};
struct DevInstr {
  uint32_t code;        // Fetch | Fn << 8 | reversed << 16
  uint32_t off;         // slot of the source (fetch) or of the target (FN_SAVE)
  float imm;
  uint32_t pad;
};
struct ChainParams {
  int64_t rows, cols;
  int32_t n_async, n_in, n_instr, n_out;   // operands [0, n_async) are staged by cp.async, the rest by plain loads
  DevOperand in[kChainMaxOperands];
  DevOutput out[kChainMaxOutputs];
  DevInstr tape[kChainMaxInstr];
};

__device__ __forceinline__ float widen_bits(int dtype, const void *p, int64_t i) {
  if (dtype == BSIR_F32) return static_cast<const float *>(p)[i];
  const uint16_t h = static_cast<const uint16_t *>(p)[i];
  return dtype == BSIR_F16 ? __half2float(__ushort_as_half(h)) : __uint_as_float(static_cast<uint32_t>(h) << 16);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool keep_l1) {
  if (keep_l1) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
  else asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ float4 lds128(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t a, float x, float y, float z, float w) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
__device__ __forceinline__ float lds32(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }

// The scalar function tables of the elementwise kernels, restated for a thread's elements (same
// expressions: hfusion unary / binary fns of bishengir/lib/Dialect/HFusion/IR/HFusionOps.cpp:434-639
// that have an f32 form).
// Every switch below ends in an unreachable default (the host has checked the codes): with a
// pass-through default the compiler copies the whole accumulator at every level of its search tree.
template <int N>
__device__ __forceinline__ void chain_unary(uint32_t fn, float (&a)[N]) {
#define U(expr)                                                                            \
  {                                                                                        \
    _Pragma("unroll") for (int e = 0; e < N; ++e) { const float v = a[e]; a[e] = (expr); } \
    break;                                                                                 \
  }
  switch (fn) {
    case FN_RELU: U(maximumf(0.0f, v))
    case FN_SQRT: U(__fsqrt_rn(v))
    case FN_RSQRT: U(__fdiv_rn(1.0f, __fsqrt_rn(v)))
    case FN_REC: U(__fdiv_rn(1.0f, v))
    case FN_TANH: U(tanhf(v))
    case FN_EXP: U(expf(v))
    case FN_LOG: U(logf(v))
    case FN_ABS: U(fabsf(v))
    case FN_CEIL: U(ceilf(v))
    case FN_FLOOR: U(floorf(v))
    case FN_NEG: U(-v)
    case FN_ROUND: U(roundf(v))
    case FN_SQUARE: U(__fmul_rn(v, v))
    case FN_ERF: U(erff(v))
    case FN_SIN: U(sinf(v))
    case FN_COS: U(cosf(v))
    case FN_EXP2: U(exp2f(v))
    case FN_LOG2: U(log2f(v))
    default: __builtin_unreachable();
  }
#undef U
}

// acc = fn(acc, s), or fn(s, acc) when rev (the commutative functions ignore rev); FN_LOAD: acc = s
template <int N>
__device__ __forceinline__ void chain_binary(uint32_t fn, bool rev, float (&a)[N], const float (&s)[N]) {
#define C(expr)                                                                                       \
  {                                                                                                   \
    _Pragma("unroll") for (int e = 0; e < N; ++e) { const float x = a[e], y = s[e]; a[e] = (expr); }   \
    break;                                                                                            \
  }
#define O(expr)                                                                                                    \
  {                                                                                                                \
    if (rev) { _Pragma("unroll") for (int e = 0; e < N; ++e) { const float x = s[e], y = a[e]; a[e] = (expr); } }   \
    else { _Pragma("unroll") for (int e = 0; e < N; ++e) { const float x = a[e], y = s[e]; a[e] = (expr); } }       \
    break;                                                                                                         \
  }
  switch (fn) {
    case FN_LOAD: C(y)
    case FN_ADD: C(__fadd_rn(x, y))
    case FN_MUL: C(__fmul_rn(x, y))
    case FN_SUB: O(__fsub_rn(x, y))
    case FN_DIV: O(__fdiv_rn(x, y))
    case FN_MAXF: C(maximumf(x, y))
    case FN_MINF: C(minimumf(x, y))
    case FN_MAXNUMF: C(fmaxf(x, y))
    case FN_MINNUMF: C(fminf(x, y))
    case FN_POWF: O(powf(x, y))
    default: __builtin_unreachable();
  }
#undef C
#undef O
}

template <bool VEC, int G>
__global__ void __launch_bounds__(kChainThreads) fused_chain_kernel(const __grid_constant__ ChainParams p) {
  extern __shared__ float4 chain_smem[];
  constexpr int N = kGroup * G;
  const uint32_t sm0 = static_cast<uint32_t>(__cvta_generic_to_shared(chain_smem));
  const uint32_t t16 = sm0 + threadIdx.x * 16, t4 = sm0 + threadIdx.x * 4;
  const int64_t gpr = (p.cols + kGroup - 1) / kGroup;      // groups per row
  const int64_t total = p.rows * gpr;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t step = nthreads * G, row_step = step / gpr, cg_step = step - row_step * gpr;

  // positions of the thread's groups, advanced without a division per iteration
  int64_t u[G], row[G], cg[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    u[g] = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x + g * nthreads;
    row[g] = u[g] / gpr;
    cg[g] = u[g] - row[g] * gpr;
  }

  while (u[0] < total) {
    // a group past the end repeats the thread's first group (valid addresses) and is not stored
    int64_t r[G], c0[G];
    bool live[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      live[g] = u[g] < total;
      r[g] = live[g] ? row[g] : row[0];
      c0[g] = (live[g] ? cg[g] : cg[0]) * kGroup;
    }

    // 1. staging
    for (int i = 0; i < p.n_async; ++i) {
      const DevOperand &o = p.in[i];
      const uint32_t stage = o.stage & 0xff, dt = (o.stage >> 8) & 0xff;
      if constexpr (VEC) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const int64_t base = (stage == S_FULL ? r[g] * o.row_stride : 0) + c0[g];
          if (dt == BSIR_F32) {
            const float *src = static_cast<const float *>(o.data) + base;
            cp_async16(t16 + o.off + g * 2 * kPlane, src, stage == S_ROW);
            cp_async16(t16 + o.off + g * 2 * kPlane + kPlane, src + 4, stage == S_ROW);
          } else {
            cp_async16(t16 + o.off + g * kPlane, static_cast<const uint16_t *>(o.data) + base, stage == S_ROW);
          }
        }
      } else {
        // ragged or unaligned problem: element loads, widened into an f32 slot
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const int64_t base = (stage == S_FULL ? r[g] * o.row_stride : 0) + c0[g];
          const int n = p.cols - c0[g] < kGroup ? static_cast<int>(p.cols - c0[g]) : kGroup;
          float v[kGroup];
#pragma unroll
          for (int e = 0; e < kGroup; ++e) v[e] = e < n ? widen_bits(dt, o.data, base + e) : 0.0f;
          sts128(t16 + o.off + g * 2 * kPlane, v[0], v[1], v[2], v[3]);
          sts128(t16 + o.off + g * 2 * kPlane + kPlane, v[4], v[5], v[6], v[7]);
        }
      }
    }
    for (int i = p.n_async; i < p.n_in; ++i) {
      const DevOperand &o = p.in[i];
      const uint32_t stage = o.stage & 0xff, dt = (o.stage >> 8) & 0xff;
#pragma unroll
      for (int g = 0; g < G; ++g) sts32(t4 + o.off + g * kChainThreads * 4, widen_bits(dt, o.data, stage == S_SCALAR ? 0 : r[g]));
    }
    if constexpr (VEC) cp_async_wait_all();

    // 2. the tape
    float acc[N];
#pragma unroll
    for (int e = 0; e < N; ++e) acc[e] = 0.0f;
    for (int ip = 0; ip < p.n_instr; ++ip) {
      const DevInstr ins = p.tape[ip];
      const uint32_t fetch = ins.code & 0xff, fn = (ins.code >> 8) & 0xff;
      if (fn == FN_SAVE) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          sts128(t16 + ins.off + g * 2 * kPlane, acc[8 * g], acc[8 * g + 1], acc[8 * g + 2], acc[8 * g + 3]);
          sts128(t16 + ins.off + g * 2 * kPlane + kPlane, acc[8 * g + 4], acc[8 * g + 5], acc[8 * g + 6], acc[8 * g + 7]);
        }
        continue;
      }
      if (fn >= FN_RELU) {
        chain_unary<N>(fn, acc);
        continue;
      }
      float s[N];
      switch (fetch) {
        case F_IMM:
#pragma unroll
          for (int e = 0; e < N; ++e) s[e] = ins.imm;
          break;
        case F_F32:
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float4 a = lds128(t16 + ins.off + g * 2 * kPlane), b = lds128(t16 + ins.off + g * 2 * kPlane + kPlane);
            s[8 * g] = a.x; s[8 * g + 1] = a.y; s[8 * g + 2] = a.z; s[8 * g + 3] = a.w;
            s[8 * g + 4] = b.x; s[8 * g + 5] = b.y; s[8 * g + 6] = b.z; s[8 * g + 7] = b.w;
          }
          break;
        case F_BF16:
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float4 a = lds128(t16 + ins.off + g * kPlane);
            const uint32_t ws[4] = {__float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(a.z), __float_as_uint(a.w)};
#pragma unroll
            for (int k = 0; k < 4; ++k) FloatTraits<BSIR_BF16>::unpack(ws[k], s + 8 * g + 2 * k);
          }
          break;
        case F_F16:
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float4 a = lds128(t16 + ins.off + g * kPlane);
            const uint32_t ws[4] = {__float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(a.z), __float_as_uint(a.w)};
#pragma unroll
            for (int k = 0; k < 4; ++k) FloatTraits<BSIR_F16>::unpack(ws[k], s + 8 * g + 2 * k);
          }
          break;
        case F_BCAST:
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float v = lds32(t4 + ins.off + g * kChainThreads * 4);
#pragma unroll
            for (int e = 0; e < kGroup; ++e) s[8 * g + e] = v;
          }
          break;
        default: __builtin_unreachable();
      }
      chain_binary<N>(fn, (ins.code >> 16) & 1, acc, s);
    }

    // 3. outputs
    for (int io = 0; io < p.n_out; ++io) {
      const DevOutput &o = p.out[io];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float v[kGroup];
        if (o.off < 0) {
#pragma unroll
          for (int e = 0; e < kGroup; ++e) v[e] = acc[8 * g + e];
        } else {
          const float4 a = lds128(t16 + o.off + g * 2 * kPlane), b = lds128(t16 + o.off + g * 2 * kPlane + kPlane);
          v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
        if (!live[g]) continue;
        const int64_t base = r[g] * o.row_stride + c0[g];
        if constexpr (VEC) {
          if (o.dtype == BSIR_F32) {
            float *d = static_cast<float *>(o.data) + base;
            *reinterpret_cast<float4 *>(d) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4 *>(d + 4) = make_float4(v[4], v[5], v[6], v[7]);
          } else {
            uint32_t w[4];
            if (o.dtype == BSIR_BF16) {
#pragma unroll
              for (int k = 0; k < 4; ++k) w[k] = FloatTraits<BSIR_BF16>::pack(v + 2 * k);
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k) w[k] = FloatTraits<BSIR_F16>::pack(v + 2 * k);
            }
            *reinterpret_cast<uint4 *>(static_cast<uint16_t *>(o.data) + base) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        } else {
          const int n = p.cols - c0[g] < kGroup ? static_cast<int>(p.cols - c0[g]) : kGroup;
          for (int e = 0; e < n; ++e) {
            if (o.dtype == BSIR_F32) static_cast<float *>(o.data)[base + e] = v[e];
            else if (o.dtype == BSIR_F16) static_cast<uint16_t *>(o.data)[base + e] = __half_as_ushort(__float2half_rn(v[e]));
            else static_cast<uint16_t *>(o.data)[base + e] = __bfloat16_as_ushort(__float2bfloat16_rn(v[e]));
          }
        }
      }
    }

#pragma unroll
    for (int g = 0; g < G; ++g) {
      u[g] += step;
      row[g] += row_step;
      cg[g] += cg_step;
      if (cg[g] >= gpr) { cg[g] -= gpr; ++row[g]; }
    }
  }
}

bool chain_float(int dt) { return dt == BSIR_F32 || dt == BSIR_F16 || dt == BSIR_BF16; }

// dense function code of a unary / binary enum value; FN_COUNT when the chain machine has no such function
uint32_t unary_code(int fn) {
  switch (fn) {
    case BSIR_UNARY_RELU: return FN_RELU;
    case BSIR_UNARY_SQRT: case BSIR_UNARY_SQRT_L: return FN_SQRT;
    case BSIR_UNARY_RSQRT: case BSIR_UNARY_RSQRT_L: return FN_RSQRT;
    case BSIR_UNARY_REC: case BSIR_UNARY_RECIPROCAL: return FN_REC;
    case BSIR_UNARY_TANH: case BSIR_UNARY_TANH_L: return FN_TANH;
    case BSIR_UNARY_EXP: return FN_EXP;
    case BSIR_UNARY_LOG: return FN_LOG;
    case BSIR_UNARY_ABS: return FN_ABS;
    case BSIR_UNARY_CEIL: return FN_CEIL;
    case BSIR_UNARY_FLOOR: return FN_FLOOR;
    case BSIR_UNARY_NEGF: return FN_NEG;
    case BSIR_UNARY_ROUND: return FN_ROUND;
    case BSIR_UNARY_SQUARE: return FN_SQUARE;
    case BSIR_UNARY_ERF: case BSIR_UNARY_ERF_L: return FN_ERF;
    case BSIR_UNARY_SIN: return FN_SIN;
    case BSIR_UNARY_COS: return FN_COS;
    case BSIR_UNARY_EXP2: return FN_EXP2;
    case BSIR_UNARY_LOG2: return FN_LOG2;
    default: return FN_COUNT;
  }
}
uint32_t binary_code(int fn) {
  switch (fn) {
    case BSIR_BINARY_ADD: return FN_ADD;
    case BSIR_BINARY_SUB: return FN_SUB;
    case BSIR_BINARY_MUL: return FN_MUL;
    case BSIR_BINARY_DIV: case BSIR_BINARY_DIVFHP: return FN_DIV;
    case BSIR_BINARY_MAXF: return FN_MAXF;
    case BSIR_BINARY_MINF: return FN_MINF;
    case BSIR_BINARY_MAXNUMF: return FN_MAXNUMF;
    case BSIR_BINARY_MINNUMF: return FN_MINNUMF;
    case BSIR_BINARY_POWF: return FN_POWF;
    default: return FN_COUNT;
  }
}

template <bool VEC, int G>
void launch_chain(const ChainParams &p, unsigned blocks, size_t smem, cudaStream_t st) {
  if (smem > 48 * 1024)   // the attribute is per device: set whenever it is needed, not once per process
    cudaFuncSetAttribute(fused_chain_kernel<VEC, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  fused_chain_kernel<VEC, G><<<blocks, kChainThreads, smem, st>>>(p);
}


thread_local int32_t tl_chain_path = 0;   // of the last call on this thread: 0 none, 1 interpreter, 2 compiled

// the part of a chain that its generated source depends on
ChainJitSpec make_spec(int32_t n_in, const bsir_chain_operand *ins, int32_t n_instr, const bsir_chain_instr *tape, int32_t n_out,
                       const bsir_chain_output *outs, bool flat, bool alias) {
  ChainJitSpec s;
  s.n_in = n_in; s.n_instr = n_instr; s.n_out = n_out; s.flat = flat; s.alias = alias;
  for (int i = 0; i < n_in; ++i) { s.in_dtype[i] = ins[i].dtype; s.in_kind[i] = ins[i].kind; }
  for (int i = 0; i < n_instr; ++i) {
    s.tape[i] = tape[i];
    // fields an instruction does not read must not split the cache
    if (tape[i].op == BSIR_CHAIN_REDUCE) { s.tape[i].src_kind = 0; s.tape[i].src = 0; s.tape[i].imm = 0.0f; continue; }
    if (tape[i].op == BSIR_CHAIN_UNARY || tape[i].op == BSIR_CHAIN_SAVE) { s.tape[i].src_kind = 0; s.tape[i].imm = 0.0f; }
    if (tape[i].op == BSIR_CHAIN_UNARY) s.tape[i].src = 0;
    if (tape[i].op == BSIR_CHAIN_SAVE || tape[i].op == BSIR_CHAIN_LOAD) s.tape[i].fn = 0;
    if (tape[i].op != BSIR_CHAIN_UNARY && tape[i].op != BSIR_CHAIN_SAVE && tape[i].src_kind != BSIR_CHAIN_SRC_IMM) s.tape[i].imm = 0.0f;
    if (tape[i].op != BSIR_CHAIN_UNARY && tape[i].op != BSIR_CHAIN_SAVE && tape[i].src_kind == BSIR_CHAIN_SRC_IMM) s.tape[i].src = 0;
  }
  for (int i = 0; i < n_out; ++i) { s.out_dtype[i] = outs[i].dtype; s.out_tmp[i] = outs[i].tmp; }
  return s;
}

// Checks of a chain that need no sizes (shared by the launch and by the source / compile entry points).
int32_t validate_tape(int32_t n_in, const bsir_chain_operand *ins, int32_t n_instr, const bsir_chain_instr *tape, int32_t n_out,
                      const bsir_chain_output *outs, bool (&tmp_used)[kChainTemps], bool *has_reduce = nullptr) {
  if (n_in < 0 || n_in > kChainMaxOperands || n_instr < 1 || n_instr > kChainMaxInstr || n_out < 1 || n_out > kChainMaxOutputs)
    return fail(BSIR_ERR_SHAPE, "fused_elementwise: %d operands (max %d), %d instructions (1..%d), %d outputs (1..%d)", n_in,
                kChainMaxOperands, n_instr, kChainMaxInstr, n_out, kChainMaxOutputs);
  if ((n_in > 0 && !ins) || !tape || !outs) return fail(BSIR_ERR_NULL, "fused_elementwise: null table");
  for (int i = 0; i < n_in; ++i) {
    if (!chain_float(ins[i].dtype)) return fail(BSIR_ERR_DTYPE, "fused_elementwise: operand %d dtype %d (f32, f16, bf16)", i, ins[i].dtype);
    if (ins[i].kind < BSIR_CHAIN_FULL || ins[i].kind > BSIR_CHAIN_SCALAR) return fail(BSIR_ERR_ATTR, "fused_elementwise: operand %d kind %d", i, ins[i].kind);
  }
  bool tmp_saved[kChainTemps] = {false, false, false, false};
  for (int t = 0; t < kChainTemps; ++t) tmp_used[t] = false;
  for (int i = 0; i < n_instr; ++i) {
    const bsir_chain_instr &t = tape[i];
    if (t.op < BSIR_CHAIN_LOAD || t.op > BSIR_CHAIN_REDUCE) return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d op %d", i, t.op);
    if (t.op == BSIR_CHAIN_REDUCE) {
      if (t.fn != BSIR_REDUCE_SUM && t.fn != BSIR_REDUCE_PROD && t.fn != BSIR_REDUCE_MAX && t.fn != BSIR_REDUCE_MIN)
        return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d reduce kind %d (sum, prod, max, min)", i, t.fn);
      if (has_reduce) *has_reduce = true;
    } else if (t.op == BSIR_CHAIN_SAVE) {
      if (t.src < 0 || t.src >= kChainTemps) return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d saves to temporary %d", i, t.src);
      tmp_used[t.src] = tmp_saved[t.src] = true;
    } else if (t.op == BSIR_CHAIN_UNARY) {
      if (unary_code(t.fn) == FN_COUNT) return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d unary fn %d", i, t.fn);
    } else {
      if (t.src_kind < BSIR_CHAIN_SRC_OPERAND || t.src_kind > BSIR_CHAIN_SRC_IMM)
        return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d source kind %d", i, t.src_kind);
      if (t.src_kind == BSIR_CHAIN_SRC_OPERAND && (t.src < 0 || t.src >= n_in))
        return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d reads operand %d of %d", i, t.src, n_in);
      if (t.src_kind == BSIR_CHAIN_SRC_TMP) {
        if (t.src < 0 || t.src >= kChainTemps) return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d reads temporary %d", i, t.src);
        if (!tmp_saved[t.src]) return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d reads temporary %d before any save", i, t.src);
      }
      if (t.op != BSIR_CHAIN_LOAD && binary_code(t.fn) == FN_COUNT)
        return fail(BSIR_ERR_ATTR, "fused_elementwise: instruction %d binary fn %d", i, t.fn);
    }
  }
  for (int i = 0; i < n_out; ++i) {
    if (!chain_float(outs[i].dtype)) return fail(BSIR_ERR_DTYPE, "fused_elementwise: output %d dtype %d", i, outs[i].dtype);
    if (outs[i].tmp < -1 || outs[i].tmp >= kChainTemps) return fail(BSIR_ERR_ATTR, "fused_elementwise: output %d takes temporary %d", i, outs[i].tmp);
    if (outs[i].tmp >= 0 && !tmp_saved[outs[i].tmp])
      return fail(BSIR_ERR_ATTR, "fused_elementwise: output %d takes temporary %d, which is never saved", i, outs[i].tmp);
  }
  return BSIR_OK;
}

// Threads per row and groups per thread of a chain with reductions: the row stays in registers, so the groups a
// thread holds are bounded by what one group costs in registers.  false: one block cannot hold a row.
bool plan_rows(ChainJitSpec *s, int64_t gpr, const bool (&tmp_used)[kChainTemps]) {
  int regs = 16;   // the accumulator and one unpacked operand
  for (int t = 0; t < kChainTemps; ++t) regs += tmp_used[t] ? 8 : 0;
  for (int i = 0; i < s->n_in; ++i)
    if (s->in_kind[i] == BSIR_CHAIN_FULL || s->in_kind[i] == BSIR_CHAIN_ROW_VECTOR) regs += s->in_dtype[i] == BSIR_F32 ? 8 : 4;
  const int fit = 112 / regs, vmax = fit >= 8 ? 8 : fit >= 4 ? 4 : fit >= 2 ? 2 : 1;
  const int64_t need = ceil_div(gpr, vmax);
  int tpr = 4;
  while (tpr < need && tpr < 1024) tpr *= 2;
  const int64_t vpt = ceil_div(gpr, tpr);
  if (vpt > 8) return false;
  s->tpr = tpr;
  s->vpt = static_cast<int>(vpt);
  // Rows so long that their values fill the register file of an SM (1024 threads with three or more groups each)
  // run one block per SM, which loads, computes and stores in turn.  Such blocks are made persistent, with the rows
  // arriving through a ring of shared-memory buffers two rows ahead of the arithmetic -- unless an output overlaps
  // an operand (a row fetched ahead could then be one that is still to be written).  Shorter rows are better off
  // as they are: two or three blocks per SM in different phases overlap by themselves (measured, softmax chain on
  // 16384 columns: 0.49 of the HBM rate without the ring, 0.40 with it).
  s->ring = 0;
  if (tpr >= 1024 && vpt >= 3 && !s->alias) {
    int64_t row_bytes = 0;
    for (int i = 0; i < s->n_in; ++i)
      if (s->in_kind[i] == BSIR_CHAIN_FULL) row_bytes += gpr * (s->in_dtype[i] == BSIR_F32 ? 32 : 16);
    const int64_t budget = 200 * 1024;
    if (row_bytes > 0 && std::getenv("BSIR_CHAIN_NO_RING") == nullptr)
      s->ring = row_bytes * 3 <= budget ? 3 : row_bytes * 2 <= budget ? 2 : 0;
  }
  return true;
}

// 0: interpreter only; 1: the compiled kernel or an error; 2 (default): compiled when it can be, else the interpreter
int jit_mode() {
  const char *e = std::getenv("BSIR_CHAIN_JIT");
  if (!e || !*e) return 2;
  return e[0] == '0' ? 0 : e[0] == '1' ? 1 : 2;
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" int32_t bsir_fused_elementwise(int64_t rows, int64_t cols, int32_t n_in, const bsir_chain_operand *ins,
                                          int32_t n_instr, const bsir_chain_instr *tape, int32_t n_out,
                                          const bsir_chain_output *outs, void *stream) {
  clear_error();
  tl_chain_path = 0;
  if (rows < 0 || cols < 0) return fail(BSIR_ERR_SHAPE, "fused_elementwise: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  bool tmp_used[kChainTemps], has_reduce = false;
  if (const int32_t rc = validate_tape(n_in, ins, n_instr, tape, n_out, outs, tmp_used, &has_reduce)) return rc;

  // ---- sizes and addresses; decides whether the 16-byte paths apply ----
  bool vec = cols % kGroup == 0, flat = true;
  for (int i = 0; i < n_in; ++i) {
    const bsir_chain_operand &o = ins[i];
    if (!o.data && rows * cols > 0) return fail(BSIR_ERR_NULL, "fused_elementwise: operand %d is null", i);
    if (o.kind == BSIR_CHAIN_FULL && o.row_stride < cols) return fail(BSIR_ERR_STRIDE, "fused_elementwise: operand %d row stride", i);
    const int eb = dtype_bytes(o.dtype);
    if (!aligned_to(o.data, eb)) return fail(BSIR_ERR_ALIGN, "fused_elementwise: operand %d misaligned", i);
    if (o.kind == BSIR_CHAIN_FULL || o.kind == BSIR_CHAIN_ROW_VECTOR)
      vec = vec && aligned_to(o.data, 16) && (o.kind != BSIR_CHAIN_FULL || (o.row_stride * eb) % 16 == 0);
    flat = flat && (o.kind == BSIR_CHAIN_SCALAR || (o.kind == BSIR_CHAIN_FULL && o.row_stride == cols));
  }
  for (int i = 0; i < n_out; ++i) {
    const bsir_chain_output &o = outs[i];
    if (!o.data && rows * cols > 0) return fail(BSIR_ERR_NULL, "fused_elementwise: output %d is null", i);
    const int eb = dtype_bytes(o.dtype);
    if (!aligned_to(o.data, eb)) return fail(BSIR_ERR_ALIGN, "fused_elementwise: output %d misaligned", i);
    if (o.row_stride == 0) {   // a [rows] vector
      if (!has_reduce) return fail(BSIR_ERR_ATTR, "fused_elementwise: output %d is per row, but the chain has no reduction", i);
      continue;
    }
    if (o.row_stride < cols) return fail(BSIR_ERR_STRIDE, "fused_elementwise: output %d row stride", i);
    vec = vec && aligned_to(o.data, 16) && (o.row_stride * eb) % 16 == 0;
    flat = flat && o.row_stride == cols;
  }
  if (rows == 0 || cols == 0) return BSIR_OK;
  cudaStream_t st = resolve_stream(stream);

  // ---- the compiled kernel: one per distinct chain, built on first use ----
  const int mode = jit_mode();
  if (has_reduce && (mode == 0 || !vec))
    return fail(BSIR_ERR_UNSUPPORTED, "fused_elementwise: a chain with reductions runs only as a compiled kernel over 16-byte aligned "
                                      "rows of a multiple of 8 columns");
  if (mode != 0 && !vec && mode == 1) return fail(BSIR_ERR_UNSUPPORTED, "fused_elementwise: the compiled path needs 16-byte aligned rows of a multiple of 8 columns");
  if (mode != 0 && vec) {
    // an output that overlaps an operand (in-place use) makes the operands' loads coherent ones
    bool alias = false;
    for (int i = 0; i < n_in && !alias; ++i) {
      const int64_t n_el = ins[i].kind == BSIR_CHAIN_FULL ? (rows - 1) * ins[i].row_stride + cols
                           : ins[i].kind == BSIR_CHAIN_ROW_VECTOR ? cols : ins[i].kind == BSIR_CHAIN_COL_VECTOR ? rows : 1;
      const char *a0 = static_cast<const char *>(ins[i].data), *a1 = a0 + n_el * dtype_bytes(ins[i].dtype);
      for (int k = 0; k < n_out; ++k) {
        const char *b0 = static_cast<const char *>(outs[k].data);
        const int64_t m_el = outs[k].row_stride == 0 ? rows : (rows - 1) * outs[k].row_stride + cols;
        const char *b1 = b0 + m_el * dtype_bytes(outs[k].dtype);
        if (a0 < b1 && b0 < a1) alias = true;
      }
    }
    ChainJitSpec spec = make_spec(n_in, ins, n_instr, tape, n_out, outs, flat, alias);
    if (has_reduce) {
      for (int i = 0; i < n_out; ++i) spec.out_per_row[i] = outs[i].row_stride == 0;
      if (!plan_rows(&spec, cols / kGroup, tmp_used))
        return fail(BSIR_ERR_UNSUPPORTED, "fused_elementwise: rows of %lld columns do not fit the registers of one block for this chain", (long long)cols);
    } else {
      chain_jit_plan(&spec, cols / kGroup);
    }
    ChainJitArgs args{};
    args.gpr = cols / kGroup;
    args.total = rows * args.gpr;
    args.rows = rows;
    for (int i = 0; i < n_in; ++i) { args.in[i] = ins[i].data; args.in_stride[i] = ins[i].row_stride; }
    for (int i = 0; i < n_out; ++i) { args.out[i] = outs[i].data; args.out_stride[i] = outs[i].row_stride; }
    args.err = spec.ring > 0 ? device_error_word() : nullptr;
    std::string why;
    if (chain_jit_launch(spec, args, st, &why) == 0) {
      tl_chain_path = 2;
      count_launch();
      return check_launch("fused_elementwise");
    }
    if (mode == 1 || has_reduce) return fail(BSIR_ERR_UNSUPPORTED, "fused_elementwise: %s", why.c_str());
  }
  tl_chain_path = 1;

  // ---- slots: bytes per group of every operand and used temporary ----
  uint32_t op_fetch[kChainMaxOperands], op_unit[kChainMaxOperands], tmp_unit[kChainTemps], unit_total = 0;
  for (int i = 0; i < n_in; ++i) {
    const bool bcast = ins[i].kind == BSIR_CHAIN_COL_VECTOR || ins[i].kind == BSIR_CHAIN_SCALAR;
    op_fetch[i] = bcast ? F_BCAST : (!vec || ins[i].dtype == BSIR_F32) ? F_F32 : ins[i].dtype == BSIR_BF16 ? F_BF16 : F_F16;
    op_unit[i] = unit_total;
    unit_total += slot_group_bytes(op_fetch[i]);
  }
  for (int t = 0; t < kChainTemps; ++t) {
    tmp_unit[t] = unit_total;
    if (tmp_used[t]) unit_total += slot_group_bytes(F_F32);
  }

  // ---- groups per thread: more of them amortise the decode of an instruction, within 64 KB of slots ----
  const int64_t groups = rows * ceil_div(cols, kGroup);
  const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
  int g = 1;
  if (vec) {
    while (g < 4 && static_cast<int64_t>(unit_total) * g * 2 <= 64 * 1024 && groups >= static_cast<int64_t>(sms) * 4 * kChainThreads * g * 2) g *= 2;
    if (const char *e = std::getenv("BSIR_CHAIN_G")) {
      const int want = std::atoi(e);
      if ((want == 1 || want == 2 || want == 4) && static_cast<int64_t>(unit_total) * want <= 200 * 1024) g = want;
    }
  }
  const size_t smem = static_cast<size_t>(unit_total) * g;
  if (smem > 200 * 1024) return fail(BSIR_ERR_SHAPE, "fused_elementwise: %zu bytes of slots", smem);

  // ---- the device tables ----
  ChainParams p{};
  p.rows = rows; p.cols = cols; p.n_in = n_in; p.n_instr = n_instr; p.n_out = n_out;
  int slot = 0;
  for (int pass = 0; pass < 2; ++pass) {   // tensors and [cols] vectors first: they are staged by cp.async
    for (int i = 0; i < n_in; ++i) {
      const bool bcast = op_fetch[i] == F_BCAST;
      if (bcast != (pass == 1)) continue;
      const uint32_t stage = ins[i].kind == BSIR_CHAIN_FULL ? S_FULL : ins[i].kind == BSIR_CHAIN_ROW_VECTOR ? S_ROW
                             : ins[i].kind == BSIR_CHAIN_COL_VECTOR ? S_COL : S_SCALAR;
      p.in[slot++] = DevOperand{ins[i].data, ins[i].row_stride, stage | static_cast<uint32_t>(ins[i].dtype) << 8 | op_fetch[i] << 16,
                                op_unit[i] * g};
    }
    if (pass == 0) p.n_async = slot;
  }
  for (int i = 0; i < n_out; ++i)
    p.out[i] = DevOutput{outs[i].data, outs[i].row_stride, outs[i].dtype, outs[i].tmp < 0 ? -1 : static_cast<int32_t>(tmp_unit[outs[i].tmp] * g)};
  for (int i = 0; i < n_instr; ++i) {
    const bsir_chain_instr &t = tape[i];
    DevInstr d{};
    if (t.op == BSIR_CHAIN_SAVE) {
      d.code = F_NONE | FN_SAVE << 8;
      d.off = tmp_unit[t.src] * g;
    } else if (t.op == BSIR_CHAIN_UNARY) {
      d.code = F_NONE | unary_code(t.fn) << 8;
    } else {
      uint32_t fetch = F_IMM;
      if (t.src_kind == BSIR_CHAIN_SRC_OPERAND) { fetch = op_fetch[t.src]; d.off = op_unit[t.src] * g; }
      else if (t.src_kind == BSIR_CHAIN_SRC_TMP) { fetch = F_F32; d.off = tmp_unit[t.src] * g; }
      const uint32_t fn = t.op == BSIR_CHAIN_LOAD ? FN_LOAD : binary_code(t.fn);
      d.code = fetch | fn << 8 | (t.op == BSIR_CHAIN_RBINARY ? 1u << 16 : 0u);
      d.imm = t.imm;
    }
    p.tape[i] = d;
  }

  int64_t blocks = ceil_div(groups, static_cast<int64_t>(kChainThreads) * g);
  const int64_t cap = static_cast<int64_t>(sms) * 8;
  if (blocks > cap) blocks = cap;   // the kernel strides over what the grid does not cover
  if (!vec) launch_chain<false, 1>(p, static_cast<unsigned>(blocks), smem, st);
  else if (g == 1) launch_chain<true, 1>(p, static_cast<unsigned>(blocks), smem, st);
  else if (g == 2) launch_chain<true, 2>(p, static_cast<unsigned>(blocks), smem, st);
  else launch_chain<true, 4>(p, static_cast<unsigned>(blocks), smem, st);
  count_launch();
  return check_launch("fused_elementwise");
}

extern "C" int32_t bsir_fused_elementwise_path(void) { return tl_chain_path; }

extern "C" int64_t bsir_fused_elementwise_source(int32_t n_in, const bsir_chain_operand *ins, int32_t n_instr,
                                                 const bsir_chain_instr *tape, int32_t n_out, const bsir_chain_output *outs,
                                                 int32_t flags, char *buf, int64_t cap) {
  clear_error();
  bool tmp_used[kChainTemps];
  bool has_reduce = false;
  if (const int32_t rc = validate_tape(n_in, ins, n_instr, tape, n_out, outs, tmp_used, &has_reduce)) return rc;
  ChainJitSpec spec = make_spec(n_in, ins, n_instr, tape, n_out, outs, (flags & 1) != 0, (flags & 2) != 0);
  spec.row_grid = (flags & 4) != 0 && !spec.flat;
  if (has_reduce) {
    for (int i = 0; i < n_out; ++i) spec.out_per_row[i] = outs[i].row_stride == 0;
    const int64_t gpr = (flags >> 8) > 0 ? (flags >> 8) : 512;
    if (!plan_rows(&spec, gpr, tmp_used)) return fail(BSIR_ERR_UNSUPPORTED, "fused_elementwise_source: rows of %lld groups do not fit one block", (long long)gpr);
  }
  const std::string src = chain_jit_source(spec);
  if (buf && cap > 0) {
    const size_t n = src.size() < static_cast<size_t>(cap - 1) ? src.size() : static_cast<size_t>(cap - 1);
    memcpy(buf, src.data(), n);
    buf[n] = '\0';
  }
  return static_cast<int64_t>(src.size()) + 1;
}

extern "C" int32_t bsir_fused_elementwise_compile(int32_t n_in, const bsir_chain_operand *ins, int32_t n_instr,
                                                  const bsir_chain_instr *tape, int32_t n_out, const bsir_chain_output *outs,
                                                  int32_t flags, int64_t *cubin_bytes) {
  clear_error();
  bool tmp_used[kChainTemps];
  bool has_reduce = false;
  if (const int32_t rc = validate_tape(n_in, ins, n_instr, tape, n_out, outs, tmp_used, &has_reduce)) return rc;
  size_t sz = 0;
  std::string why;
  ChainJitSpec spec = make_spec(n_in, ins, n_instr, tape, n_out, outs, (flags & 1) != 0, (flags & 2) != 0);
  spec.row_grid = (flags & 4) != 0 && !spec.flat;
  if (has_reduce) {
    for (int i = 0; i < n_out; ++i) spec.out_per_row[i] = outs[i].row_stride == 0;
    const int64_t gpr = (flags >> 8) > 0 ? (flags >> 8) : 512;
    if (!plan_rows(&spec, gpr, tmp_used)) return fail(BSIR_ERR_UNSUPPORTED, "fused_elementwise_compile: rows of %lld groups do not fit one block", (long long)gpr);
  }
  if (chain_jit_compile_only(spec, &sz, &why) != 0)
    return fail(BSIR_ERR_UNSUPPORTED, "fused_elementwise_compile: %s", why.c_str());
  if (cubin_bytes) *cubin_bytes = static_cast<int64_t>(sz);
  return BSIR_OK;
}
