// chain_jit.cu -- a chain of elementwise ops compiled into its own sm_100a kernel at run time.
//
// The reference compiles every fused function into one device kernel ahead of time
// (HFusion outlining: bishengir/lib/Dialect/HFusion/Transforms/OpFusion/FusibleHelper.cpp:52-72).  The
// equivalent here: the tape of bsir_fused_elementwise is turned into CUDA C++ (straight-line code,
// every operand a 16-byte streaming load issued before the arithmetic), compiled once with NVRTC for
// sm_100a, loaded through the runtime's library API and cached by what its text depends on (the tape, the
// operand and output types, the thread mapping).  The arithmetic is
// spelled with the same expressions as the tape interpreter of fused_chain.cu (and --fmad=false), so
// both paths give the same bits.
//
// NVRTC is looked up with dlopen when the first chain arrives, so that the library itself does not
// depend on it; where it is missing the caller falls back to the interpreter kernel.
#include <dlfcn.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "chain_jit.h"
#include "common.cuh"

namespace bsir {
namespace {

// ---------------------------------------------------------------- NVRTC through dlopen
typedef struct _nvrtcProgram *nvrtcProgramT;
struct Nvrtc {
  void *lib = nullptr;
  int (*CreateProgram)(nvrtcProgramT *, const char *, const char *, int, const char *const *, const char *const *) = nullptr;
  int (*CompileProgram)(nvrtcProgramT, int, const char *const *) = nullptr;
  int (*GetCUBINSize)(nvrtcProgramT, size_t *) = nullptr;
  int (*GetCUBIN)(nvrtcProgramT, char *) = nullptr;
  int (*GetProgramLogSize)(nvrtcProgramT, size_t *) = nullptr;
  int (*GetProgramLog)(nvrtcProgramT, char *) = nullptr;
  int (*DestroyProgram)(nvrtcProgramT *) = nullptr;
  std::string why;   // non-empty: not usable
};

const Nvrtc &nvrtc() {
  static Nvrtc n;
  static std::once_flag once;
  std::call_once(once, [] {
    // the toolkit the library itself was built with first, then whatever the process can find
    const char *names[] = {"/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so.12", "libnvrtc.so", "libnvrtc.so.13"};
    if (const char *e = std::getenv("BSIR_NVRTC_PATH")) n.lib = dlopen(e, RTLD_NOW | RTLD_LOCAL);
    for (const char *nm : names) {
      if (n.lib) break;
      n.lib = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
    }
    if (!n.lib) {
      n.why = "libnvrtc not found (set BSIR_NVRTC_PATH)";
      return;
    }
    auto sym = [&](const char *s) { return dlsym(n.lib, s); };
    n.CreateProgram = reinterpret_cast<decltype(n.CreateProgram)>(sym("nvrtcCreateProgram"));
    n.CompileProgram = reinterpret_cast<decltype(n.CompileProgram)>(sym("nvrtcCompileProgram"));
    n.GetCUBINSize = reinterpret_cast<decltype(n.GetCUBINSize)>(sym("nvrtcGetCUBINSize"));
    n.GetCUBIN = reinterpret_cast<decltype(n.GetCUBIN)>(sym("nvrtcGetCUBIN"));
    n.GetProgramLogSize = reinterpret_cast<decltype(n.GetProgramLogSize)>(sym("nvrtcGetProgramLogSize"));
    n.GetProgramLog = reinterpret_cast<decltype(n.GetProgramLog)>(sym("nvrtcGetProgramLog"));
    n.DestroyProgram = reinterpret_cast<decltype(n.DestroyProgram)>(sym("nvrtcDestroyProgram"));
    if (!n.CreateProgram || !n.CompileProgram || !n.GetCUBINSize || !n.GetCUBIN || !n.GetProgramLogSize || !n.GetProgramLog ||
        !n.DestroyProgram)
      n.why = "libnvrtc lacks the cubin entry points";
  });
  return n;
}

// ---------------------------------------------------------------- code generation
const char *kPrelude = R"SRC(
typedef unsigned int u32;
typedef unsigned short u16;
typedef long long i64;
struct V4 { u32 x, y, z, w; };
struct Args {
  i64 gpr, total, rows;
  const void *in[8];
  i64 in_stride[8];
  void *out[4];
  i64 out_stride[4];
  int *err;
};
__device__ __forceinline__ V4 ld_stream(const void *p) {
  V4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ V4 ld_keep(const void *p) {
  V4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ V4 ld_plain(const void *p) {
  V4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_stream(void *p, u32 a, u32 b, u32 c, u32 d) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ float f16_bits(u16 h) {
  float r;
  asm("cvt.f32.f16 %0, %1;" : "=f"(r) : "h"(h));
  return r;
}
__device__ __forceinline__ void un_bf16(const V4 &v, float *o) {
  const u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) { o[2 * k] = __uint_as_float(w[k] << 16); o[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u); }
}
__device__ __forceinline__ void un_f16(const V4 &v, float *o) {
  const u32 w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) { o[2 * k] = f16_bits((u16)(w[k] & 0xffffu)); o[2 * k + 1] = f16_bits((u16)(w[k] >> 16)); }
}
__device__ __forceinline__ void un_f32(const V4 &a, const V4 &b, float *o) {
  o[0] = __uint_as_float(a.x); o[1] = __uint_as_float(a.y); o[2] = __uint_as_float(a.z); o[3] = __uint_as_float(a.w);
  o[4] = __uint_as_float(b.x); o[5] = __uint_as_float(b.y); o[6] = __uint_as_float(b.z); o[7] = __uint_as_float(b.w);
}
__device__ __forceinline__ u32 pk_bf16(float a, float b) {
  u32 r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ u32 pk_f16(float a, float b) {
  u32 r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ float one_f32(const void *p, i64 i) { return ((const float *)p)[i]; }
__device__ __forceinline__ float one_bf16(const void *p, i64 i) { return __uint_as_float((u32)((const u16 *)p)[i] << 16); }
__device__ __forceinline__ float one_f16(const void *p, i64 i) { return f16_bits(((const u16 *)p)[i]); }
__device__ __forceinline__ float maximumf(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float minimumf(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float red_sum(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float red_prod(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float red_max(float a, float b) { return maximumf(a, b); }
__device__ __forceinline__ float red_min(float a, float b) { return minimumf(a, b); }
)SRC";

// Reduction of one value per thread over the TPR threads of a row (TPR a power of two; rows of a block are
// aligned groups of threads): shuffles inside a warp, then one shared-memory word per warp.
const char *kRowReduce = R"SRC(
#define ROW_REDUCE(NAME, COMB)                                                                  \
  __device__ __forceinline__ float NAME(float p, float *red) {                                  \
    _Pragma("unroll") for (int o = (TPR < 32 ? TPR : 32) / 2; o > 0; o >>= 1)                   \
      p = COMB(p, __shfl_xor_sync(0xffffffffu, p, o));                                          \
    if (TPR > 32) {                                                                             \
      const int warp = threadIdx.x >> 5, first = (threadIdx.x / TPR) * (TPR / 32);              \
      __syncthreads();                                                                          \
      if ((threadIdx.x & 31) == 0) red[warp] = p;                                               \
      __syncthreads();                                                                          \
      p = red[first];                                                                           \
      for (int k = 1; k < TPR / 32; ++k) p = COMB(p, red[first + k]);                           \
    }                                                                                           \
    return p;                                                                                   \
  }
ROW_REDUCE(row_sum, red_sum)
ROW_REDUCE(row_prod, red_prod)
ROW_REDUCE(row_max, red_max)
ROW_REDUCE(row_min, red_min)
)SRC";

// Persistent row programs: rows arrive in shared memory through bulk copies that complete on an mbarrier.
const char *kRing = R"SRC(
__device__ __forceinline__ u32 smem_u32(const void *p) { return (u32)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_try(u32 bar, u32 parity) {
  u32 ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// bounded: gives up after about two seconds and raises the device error word
__device__ __forceinline__ bool mbar_wait_bounded(u32 bar, u32 parity, int *err) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (u32 spin = 0;; ++spin) {
    if (mbar_try(bar, parity)) return true;
    if ((spin & 1023u) == 1023u && clock64() - t0 > 4000000000LL) {
      if (err) atomicOr(err, 0x20);
      return false;
    }
  }
}
__device__ __forceinline__ void bulk_row(u32 dst, const void *src, u32 bytes, u32 bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
)SRC";

const char *dtype_tag(int dt) { return dt == BSIR_F32 ? "f32" : dt == BSIR_BF16 ? "bf16" : "f16"; }

// v = the accumulator's element
const char *unary_expr(int fn) {
  switch (fn) {
    case BSIR_UNARY_RELU: return "maximumf(0.0f, v)";
    case BSIR_UNARY_SQRT: case BSIR_UNARY_SQRT_L: return "__fsqrt_rn(v)";
    case BSIR_UNARY_RSQRT: case BSIR_UNARY_RSQRT_L: return "__fdiv_rn(1.0f, __fsqrt_rn(v))";
    case BSIR_UNARY_REC: case BSIR_UNARY_RECIPROCAL: return "__fdiv_rn(1.0f, v)";
    case BSIR_UNARY_TANH: case BSIR_UNARY_TANH_L: return "tanhf(v)";
    case BSIR_UNARY_EXP: return "expf(v)";
    case BSIR_UNARY_LOG: return "logf(v)";
    case BSIR_UNARY_ABS: return "fabsf(v)";
    case BSIR_UNARY_CEIL: return "ceilf(v)";
    case BSIR_UNARY_FLOOR: return "floorf(v)";
    case BSIR_UNARY_NEGF: return "-v";
    case BSIR_UNARY_ROUND: return "roundf(v)";
    case BSIR_UNARY_SQUARE: return "__fmul_rn(v, v)";
    case BSIR_UNARY_ERF: case BSIR_UNARY_ERF_L: return "erff(v)";
    case BSIR_UNARY_SIN: return "sinf(v)";
    case BSIR_UNARY_COS: return "cosf(v)";
    case BSIR_UNARY_EXP2: return "exp2f(v)";
    case BSIR_UNARY_LOG2: return "log2f(v)";
    default: return nullptr;
  }
}
// x = left, y = right
const char *binary_expr(int fn) {
  switch (fn) {
    case BSIR_BINARY_ADD: return "__fadd_rn(x, y)";
    case BSIR_BINARY_SUB: return "__fsub_rn(x, y)";
    case BSIR_BINARY_MUL: return "__fmul_rn(x, y)";
    case BSIR_BINARY_DIV: case BSIR_BINARY_DIVFHP: return "__fdiv_rn(x, y)";
    case BSIR_BINARY_MAXF: return "maximumf(x, y)";
    case BSIR_BINARY_MINF: return "minimumf(x, y)";
    case BSIR_BINARY_MAXNUMF: return "fmaxf(x, y)";
    case BSIR_BINARY_MINNUMF: return "fminf(x, y)";
    case BSIR_BINARY_POWF: return "powf(x, y)";
    default: return nullptr;
  }
}

void appendf(std::string &s, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
void appendf(std::string &s, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  s += buf;
}

struct Compiled {
  cudaKernel_t kernel = nullptr;
  std::string why;   // non-empty: this chain cannot be compiled (remembered, so that it is not retried)
};
std::mutex g_mu;
std::unordered_map<std::string, Compiled> g_cache;

// compiles src to a cubin; empty result + why on failure
std::vector<char> compile_cubin(const std::string &src, std::string *why) {
  std::vector<char> cubin;
  const Nvrtc &n = nvrtc();
  if (!n.why.empty()) {
    *why = n.why;
    return cubin;
  }
  nvrtcProgramT prog = nullptr;
  if (n.CreateProgram(&prog, src.c_str(), "bsir_chain.cu", 0, nullptr, nullptr) != 0) {
    *why = "nvrtcCreateProgram failed";
    return cubin;
  }
  const char *opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "--fmad=false"};
  const int rc = n.CompileProgram(prog, 3, opts);
  if (rc != 0) {
    size_t ls = 0;
    n.GetProgramLogSize(prog, &ls);
    std::string log(ls, '\0');
    if (ls) n.GetProgramLog(prog, log.data());
    *why = "nvrtc: " + log.substr(0, 600);
  } else {
    size_t sz = 0;
    if (n.GetCUBINSize(prog, &sz) == 0 && sz > 0) {
      cubin.resize(sz);
      if (n.GetCUBIN(prog, cubin.data()) != 0) cubin.clear();
    }
    if (cubin.empty()) *why = "nvrtc produced no cubin";
  }
  n.DestroyProgram(&prog);
  return cubin;
}

}  // namespace

int chain_jit_unroll(const ChainJitSpec &s) {
  if (s.unroll == 1 || s.unroll == 2 || s.unroll == 4) return s.unroll;
  // 16-byte loads a group issues; keep about eight in flight per thread
  int vecs = 0;
  for (int i = 0; i < s.n_in; ++i)
    if (s.in_kind[i] == BSIR_CHAIN_FULL) vecs += s.in_dtype[i] == BSIR_F32 ? 2 : 1;
  if (vecs <= 2) return 4;
  if (vecs <= 4) return 2;
  return 1;
}

void chain_jit_plan(ChainJitSpec *s, long long gpr) {
  // One block per stretch of a row needs no division at all; it is used when a row fills whole blocks with at
  // most an eighth of the threads idle.  Fewer groups per thread are tried before giving the mapping up.
  s->row_grid = false;
  s->unroll = 0;
  if (s->flat) return;
  for (int u = chain_jit_unroll(*s); u >= 1; u >>= 1) {
    const long long span = 256LL * u, covered = (gpr + span - 1) / span * span;
    if ((covered - gpr) * 8 <= gpr && covered / span <= 65535) {
      s->row_grid = true;
      s->unroll = u;
      return;
    }
  }
}

namespace {
std::string row_source(const ChainJitSpec &s);
}

std::string chain_jit_source(const ChainJitSpec &s) {
  if (s.tpr > 0) return row_source(s);
  const int U = chain_jit_unroll(s);
  bool need_rc = !s.flat;
  for (int i = 0; i < s.n_in; ++i)
    if (s.in_kind[i] == BSIR_CHAIN_ROW_VECTOR || s.in_kind[i] == BSIR_CHAIN_COL_VECTOR) need_rc = true;
  std::string c = kPrelude;
  appendf(c, "#define U %d\n", U);
  c += "extern \"C\" __global__ void __launch_bounds__(256) bsir_chain(const __grid_constant__ Args a) {\n";
  c += "  const i64 base = (i64)blockIdx.x * (256 * U) + threadIdx.x;\n";
  // per-operand registers
  for (int i = 0; i < s.n_in; ++i) {
    switch (s.in_kind[i]) {
      case BSIR_CHAIN_FULL:
      case BSIR_CHAIN_ROW_VECTOR:
        if (s.in_dtype[i] == BSIR_F32) appendf(c, "  V4 r%da[U], r%db[U];\n", i, i);
        else appendf(c, "  V4 r%d[U];\n", i);
        break;
      case BSIR_CHAIN_COL_VECTOR: appendf(c, "  float b%d[U];\n", i); break;
      default: appendf(c, "  const float b%d = one_%s(a.in[%d], 0);\n", i, dtype_tag(s.in_dtype[i]), i); break;
    }
  }
  // ---- positions of the thread's groups: flat (contiguous tensors only: no rows at all), one block per stretch
  // of a row (no division), or a 32-bit division per group.
  c += "  i64 rowv[U], c0v[U];\n  bool live[U];\n#pragma unroll\n  for (int j = 0; j < U; ++j) {\n";
  if (!need_rc) {
    c += "    const i64 u = base + j * 256;\n    live[j] = u < a.total;\n    rowv[j] = 0;\n    c0v[j] = u * 8;\n";
  } else if (s.row_grid) {
    c += "    const i64 g = (i64)blockIdx.y * (256 * U) + threadIdx.x + j * 256;\n"
         "    live[j] = g < a.gpr;\n    rowv[j] = blockIdx.x;\n    c0v[j] = g * 8;\n";
  } else {
    c += "    const i64 u = base + j * 256;\n    live[j] = u < a.total;\n"
         "    rowv[j] = a.total <= 0x7fffffffLL ? (i64)((u32)u / (u32)a.gpr) : u / a.gpr;\n"
         "    c0v[j] = (u - rowv[j] * a.gpr) * 8;\n";
  }
  c += "  }\n";
  const char *pos = "    const i64 row = rowv[j], c0 = c0v[j];\n";
  // ---- loads, all issued before any arithmetic
  c += "#pragma unroll\n  for (int j = 0; j < U; ++j) {\n    if (!live[j]) continue;\n";
  c += pos;
  for (int i = 0; i < s.n_in; ++i) {
    const int k = s.in_kind[i];
    if (k == BSIR_CHAIN_FULL || k == BSIR_CHAIN_ROW_VECTOR) {
      const char *ld = k == BSIR_CHAIN_ROW_VECTOR ? "ld_keep" : s.alias ? "ld_plain" : "ld_stream";
      std::string off = k == BSIR_CHAIN_ROW_VECTOR ? "c0" : std::string("(row * a.in_stride[") + std::to_string(i) + "] + c0)";
      if (s.in_dtype[i] == BSIR_F32) {
        appendf(c, "    r%da[j] = %s((const float *)a.in[%d] + %s);\n", i, ld, i, off.c_str());
        appendf(c, "    r%db[j] = %s((const float *)a.in[%d] + %s + 4);\n", i, ld, i, off.c_str());
      } else {
        appendf(c, "    r%d[j] = %s((const u16 *)a.in[%d] + %s);\n", i, ld, i, off.c_str());
      }
    } else if (k == BSIR_CHAIN_COL_VECTOR) {
      appendf(c, "    b%d[j] = one_%s(a.in[%d], row);\n", i, dtype_tag(s.in_dtype[i]), i);
    }
  }
  c += "  }\n";
  // ---- arithmetic and stores
  c += "#pragma unroll\n  for (int j = 0; j < U; ++j) {\n    if (!live[j]) continue;\n";
  c += pos;
  bool tmp_used[4] = {false, false, false, false};
  for (int i = 0; i < s.n_instr; ++i)
    if (s.tape[i].op == BSIR_CHAIN_SAVE) tmp_used[s.tape[i].src] = true;
  c += "    float acc[8];\n";
  if (s.tape[0].op != BSIR_CHAIN_LOAD) c += "#pragma unroll\n    for (int e = 0; e < 8; ++e) acc[e] = 0.0f;\n";
  for (int t = 0; t < 4; ++t)
    if (tmp_used[t]) appendf(c, "    float t%d[8];\n", t);
  bool unpacked[8] = {false, false, false, false, false, false, false, false};
  for (int ip = 0; ip < s.n_instr; ++ip) {
    const bsir_chain_instr &t = s.tape[ip];
    if (t.op == BSIR_CHAIN_SAVE) {
      appendf(c, "#pragma unroll\n    for (int e = 0; e < 8; ++e) t%d[e] = acc[e];\n", t.src);
      continue;
    }
    if (t.op == BSIR_CHAIN_UNARY) {
      appendf(c, "#pragma unroll\n    for (int e = 0; e < 8; ++e) { const float v = acc[e]; acc[e] = %s; }\n", unary_expr(t.fn));
      continue;
    }
    // the source, as an expression of e
    std::string src;
    if (t.src_kind == BSIR_CHAIN_SRC_IMM) {
      uint32_t bits;
      memcpy(&bits, &t.imm, 4);
      char lit[48];
      snprintf(lit, sizeof lit, "__uint_as_float(0x%08xu)", bits);
      src = lit;
    } else if (t.src_kind == BSIR_CHAIN_SRC_TMP) {
      src = "t" + std::to_string(t.src) + "[e]";
    } else {
      const int i = t.src, k = s.in_kind[i];
      if (k == BSIR_CHAIN_COL_VECTOR) src = "b" + std::to_string(i) + "[j]";
      else if (k == BSIR_CHAIN_SCALAR) src = "b" + std::to_string(i);
      else {
        if (!unpacked[i]) {
          appendf(c, "    float x%d[8];\n", i);
          if (s.in_dtype[i] == BSIR_F32) appendf(c, "    un_f32(r%da[j], r%db[j], x%d);\n", i, i, i);
          else appendf(c, "    un_%s(r%d[j], x%d);\n", dtype_tag(s.in_dtype[i]), i, i);
          unpacked[i] = true;
        }
        src = "x" + std::to_string(i) + "[e]";
      }
    }
    if (t.op == BSIR_CHAIN_LOAD) {
      appendf(c, "#pragma unroll\n    for (int e = 0; e < 8; ++e) acc[e] = %s;\n", src.c_str());
    } else {
      const bool rev = t.op == BSIR_CHAIN_RBINARY;
      appendf(c, "#pragma unroll\n    for (int e = 0; e < 8; ++e) { const float x = %s, y = %s; acc[e] = %s; }\n",
              rev ? src.c_str() : "acc[e]", rev ? "acc[e]" : src.c_str(), binary_expr(t.fn));
    }
  }
  for (int io = 0; io < s.n_out; ++io) {
    std::string v = s.out_tmp[io] < 0 ? "acc" : "t" + std::to_string(s.out_tmp[io]);
    const char *vn = v.c_str();
    if (s.out_dtype[io] == BSIR_F32) {
      appendf(c, "    { float *d = (float *)a.out[%d] + (row * a.out_stride[%d] + c0);\n", io, io);
      appendf(c, "      st_stream(d, __float_as_uint(%s[0]), __float_as_uint(%s[1]), __float_as_uint(%s[2]), __float_as_uint(%s[3]));\n", vn, vn, vn, vn);
      appendf(c, "      st_stream(d + 4, __float_as_uint(%s[4]), __float_as_uint(%s[5]), __float_as_uint(%s[6]), __float_as_uint(%s[7])); }\n", vn, vn, vn, vn);
    } else {
      const char *pk = s.out_dtype[io] == BSIR_BF16 ? "pk_bf16" : "pk_f16";
      appendf(c, "    st_stream((u16 *)a.out[%d] + (row * a.out_stride[%d] + c0), %s(%s[0], %s[1]), %s(%s[2], %s[3]), %s(%s[4], %s[5]), %s(%s[6], %s[7]));\n",
              io, io, pk, vn, vn, pk, vn, vn, pk, vn, vn, pk, vn, vn);
    }
  }
  c += "  }\n}\n";
  return c;
}

namespace {

const char *reduce_tag(int kind) {
  switch (kind) {
    case BSIR_REDUCE_SUM: return "sum";
    case BSIR_REDUCE_PROD: return "prod";
    case BSIR_REDUCE_MAX: return "max";
    case BSIR_REDUCE_MIN: return "min";
    default: return nullptr;
  }
}
const char *reduce_identity(int kind) {
  switch (kind) {
    case BSIR_REDUCE_SUM: return "0.0f";
    case BSIR_REDUCE_PROD: return "1.0f";
    case BSIR_REDUCE_MAX: return "__uint_as_float(0xff800000u)";   // -inf
    default: return "__uint_as_float(0x7f800000u)";                // +inf
  }
}

// A chain with last-axis reductions: TPR threads hold a row in registers (VPT groups of 8 elements each, group
// g of the row with thread g % TPR), so every operand is read once however many reductions the row needs.
std::string row_source(const ChainJitSpec &s) {
  const int tpr = s.tpr, vpt = s.vpt, bt = tpr > 128 ? tpr : 128;
  std::string c = kPrelude;
  appendf(c, "#define TPR %d\n#define VPT %d\n#define BT %d\n", tpr, vpt, bt);
  c += kRowReduce;
  const bool ring = s.ring > 0;
  if (ring) {
    // one row per block at a time (TPR == BT); row k of this block is row blockIdx.x + k * gridDim.x
    c += kRing;
    appendf(c, "#define NBUF %d\n", s.ring);
    int group_bytes = 0;   // bytes of one 8-element group over all staged operands
    for (int i = 0; i < s.n_in; ++i)
      if (s.in_kind[i] == BSIR_CHAIN_FULL) group_bytes += s.in_dtype[i] == BSIR_F32 ? 32 : 16;
    c += "extern \"C\" __global__ void __launch_bounds__(BT) bsir_chain(const __grid_constant__ Args a) {\n"
         "  extern __shared__ __align__(128) unsigned char ring_mem[];\n"
         "  __shared__ float red[BT / 32];\n"
         "  __shared__ __align__(8) unsigned long long bars[NBUF];\n"
         "  const int lane = threadIdx.x;\n"
         "  bool live[VPT];\n  i64 c0v[VPT];\n"
         "#pragma unroll\n  for (int q = 0; q < VPT; ++q) { const i64 g = lane + q * TPR; live[q] = g < a.gpr; c0v[q] = g * 8; }\n";
    appendf(c, "  const u32 row_bytes = (u32)a.gpr * %du;\n", group_bytes);
    c += "  const i64 my_rows = (a.rows - blockIdx.x + gridDim.x - 1) / gridDim.x;\n"
         "  if (threadIdx.x == 0) {\n"
         "    for (int b = 0; b < NBUF; ++b) asm volatile(\"mbarrier.init.shared::cta.b64 [%0], 1;\" ::\"r\"(smem_u32(&bars[b])) : \"memory\");\n"
         "    asm volatile(\"fence.mbarrier_init.release.cluster;\" ::: \"memory\");\n"
         "  }\n"
         "  __syncthreads();\n"
         "  auto issue = [&](i64 kk) {   // bulk copies of this block's kk-th row into buffer kk % NBUF\n"
         "    const int b = (int)(kk % NBUF);\n"
         "    const i64 r = blockIdx.x + kk * gridDim.x;\n"
         "    const u32 bar = smem_u32(&bars[b]), dst = smem_u32(ring_mem) + (u32)b * row_bytes;\n"
         "    asm volatile(\"mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\" ::\"r\"(bar), \"r\"(row_bytes) : \"memory\");\n";
    int off = 0;
    for (int i = 0; i < s.n_in; ++i) {
      if (s.in_kind[i] != BSIR_CHAIN_FULL) continue;
      const int eb = s.in_dtype[i] == BSIR_F32 ? 4 : 2;
      appendf(c, "    bulk_row(dst + (u32)a.gpr * %du, (const char *)a.in[%d] + r * a.in_stride[%d] * %d, (u32)a.gpr * %du, bar);\n", off, i, i, eb, 8 * eb);
      off += 8 * eb;
    }
    c += "  };\n"
         "  if (threadIdx.x == 0)\n    for (i64 kk = 0; kk < NBUF - 1 && kk < my_rows; ++kk) issue(kk);\n"
         "  bool ok = true;\n"
         "  for (i64 k = 0; k < my_rows; ++k) {\n"
         "  const i64 row = blockIdx.x + k * gridDim.x;\n"
         "  if (ok && !mbar_wait_bounded(smem_u32(&bars[k % NBUF]), (u32)((k / NBUF) & 1), a.err)) ok = false;\n"
         "  const bool row_ok = ok;\n"
         "  const unsigned char *buf = ring_mem + (size_t)(k % NBUF) * row_bytes;\n";
  } else {
  c += "extern \"C\" __global__ void __launch_bounds__(BT) bsir_chain(const __grid_constant__ Args a) {\n"
       "  __shared__ float red[BT / 32];\n"
       "  const int lane = threadIdx.x % TPR;\n"
       "  const i64 row_id = (i64)blockIdx.x * (BT / TPR) + threadIdx.x / TPR;\n"
       "  const bool row_ok = row_id < a.rows;\n"
       "  const i64 row = row_ok ? row_id : 0;          // threads past the last row redo row 0 and store nothing\n"
       "  bool live[VPT];\n  i64 c0v[VPT];\n"
       "#pragma unroll\n  for (int q = 0; q < VPT; ++q) { const i64 g = lane + q * TPR; live[q] = g < a.gpr; c0v[q] = g * 8; }\n";
  }
  for (int i = 0; i < s.n_in; ++i) {
    const char *tag = dtype_tag(s.in_dtype[i]);
    switch (s.in_kind[i]) {
      case BSIR_CHAIN_FULL:
      case BSIR_CHAIN_ROW_VECTOR:
        if (s.in_dtype[i] == BSIR_F32) appendf(c, "  V4 r%da[VPT], r%db[VPT];\n", i, i);
        else appendf(c, "  V4 r%d[VPT];\n", i);
        break;
      case BSIR_CHAIN_COL_VECTOR: appendf(c, "  const float b%d = one_%s(a.in[%d], row);\n", i, tag, i); break;
      default: appendf(c, "  const float b%d = one_%s(a.in[%d], 0);\n", i, tag, i); break;
    }
  }
  c += "#pragma unroll\n  for (int q = 0; q < VPT; ++q) {\n    const i64 c0 = c0v[q];\n";
  int ring_off = 0;
  for (int i = 0; i < s.n_in; ++i) {
    const int k = s.in_kind[i];
    if (k != BSIR_CHAIN_FULL && k != BSIR_CHAIN_ROW_VECTOR) continue;
    if (ring && k == BSIR_CHAIN_FULL) {
      // from this row's buffer: operand i's row starts a.gpr * ring_off bytes in
      const int eb = s.in_dtype[i] == BSIR_F32 ? 4 : 2;
      if (s.in_dtype[i] == BSIR_F32) {
        appendf(c, "    r%da[q] = r%db[q] = V4{0, 0, 0, 0};\n", i, i);
        appendf(c, "    if (live[q]) { const V4 *sp = (const V4 *)(buf + (size_t)a.gpr * %d + c0 * 4); r%da[q] = sp[0]; r%db[q] = sp[1]; }\n", ring_off, i, i);
      } else {
        appendf(c, "    r%d[q] = V4{0, 0, 0, 0};\n    if (live[q]) r%d[q] = *(const V4 *)(buf + (size_t)a.gpr * %d + c0 * 2);\n", i, i, ring_off);
      }
      ring_off += 8 * eb;
      continue;
    }
    const char *ld = k == BSIR_CHAIN_ROW_VECTOR ? "ld_keep" : s.alias ? "ld_plain" : "ld_stream";
    std::string off = k == BSIR_CHAIN_ROW_VECTOR ? "c0" : std::string("(row * a.in_stride[") + std::to_string(i) + "] + c0)";
    if (s.in_dtype[i] == BSIR_F32) {
      appendf(c, "    r%da[q] = r%db[q] = V4{0, 0, 0, 0};\n", i, i);
      appendf(c, "    if (live[q]) { r%da[q] = %s((const float *)a.in[%d] + %s); r%db[q] = %s((const float *)a.in[%d] + %s + 4); }\n", i,
              ld, i, off.c_str(), i, ld, i, off.c_str());
    } else {
      appendf(c, "    r%d[q] = V4{0, 0, 0, 0};\n    if (live[q]) r%d[q] = %s((const u16 *)a.in[%d] + %s);\n", i, i, ld, i, off.c_str());
    }
  }
  c += "  }\n";
  if (ring)
    c += "  // every thread has its part of this row in registers, and the buffer the row before was read from is free:\n"
         "  // start the copy of the row NBUF - 1 ahead into it\n"
         "  __syncthreads();\n"
         "  if (threadIdx.x == 0 && k + NBUF - 1 < my_rows) issue(k + NBUF - 1);\n";
  bool tmp_used[4] = {false, false, false, false};
  for (int i = 0; i < s.n_instr; ++i)
    if (s.tape[i].op == BSIR_CHAIN_SAVE) tmp_used[s.tape[i].src] = true;
  c += "  float acc[VPT][8];\n";
  if (s.tape[0].op != BSIR_CHAIN_LOAD) c += "#pragma unroll\n  for (int q = 0; q < VPT; ++q)\n#pragma unroll\n    for (int e = 0; e < 8; ++e) acc[q][e] = 0.0f;\n";
  for (int t = 0; t < 4; ++t)
    if (tmp_used[t]) appendf(c, "  float t%d[VPT][8];\n", t);
  const char *loop = "#pragma unroll\n  for (int q = 0; q < VPT; ++q)\n#pragma unroll\n    for (int e = 0; e < 8; ++e) ";
  bool unpacked[8] = {false, false, false, false, false, false, false, false};
  for (int ip = 0; ip < s.n_instr; ++ip) {
    const bsir_chain_instr &t = s.tape[ip];
    if (t.op == BSIR_CHAIN_SAVE) {
      c += loop;
      appendf(c, "t%d[q][e] = acc[q][e];\n", t.src);
      continue;
    }
    if (t.op == BSIR_CHAIN_UNARY) {
      c += loop;
      appendf(c, "{ const float v = acc[q][e]; acc[q][e] = %s; }\n", unary_expr(t.fn));
      continue;
    }
    if (t.op == BSIR_CHAIN_REDUCE) {
      // elements past the row's end take the identity; every thread of the row ends with the row's value
      appendf(c, "  {\n    float p = %s;\n", reduce_identity(t.fn));
      appendf(c, "#pragma unroll\n    for (int q = 0; q < VPT; ++q)\n#pragma unroll\n      for (int e = 0; e < 8; ++e) if (live[q]) p = red_%s(p, acc[q][e]);\n",
              reduce_tag(t.fn));
      appendf(c, "    p = row_%s(p, red);\n", reduce_tag(t.fn));
      c += "#pragma unroll\n    for (int q = 0; q < VPT; ++q)\n#pragma unroll\n      for (int e = 0; e < 8; ++e) acc[q][e] = p;\n  }\n";
      continue;
    }
    std::string src;
    if (t.src_kind == BSIR_CHAIN_SRC_IMM) {
      uint32_t bits;
      memcpy(&bits, &t.imm, 4);
      char lit[48];
      snprintf(lit, sizeof lit, "__uint_as_float(0x%08xu)", bits);
      src = lit;
    } else if (t.src_kind == BSIR_CHAIN_SRC_TMP) {
      src = "t" + std::to_string(t.src) + "[q][e]";
    } else {
      const int i = t.src, k = s.in_kind[i];
      if (k == BSIR_CHAIN_COL_VECTOR || k == BSIR_CHAIN_SCALAR) src = "b" + std::to_string(i);
      else {
        if (!unpacked[i]) {
          appendf(c, "  float x%d[VPT][8];\n#pragma unroll\n  for (int q = 0; q < VPT; ++q) ", i);
          if (s.in_dtype[i] == BSIR_F32) appendf(c, "un_f32(r%da[q], r%db[q], x%d[q]);\n", i, i, i);
          else appendf(c, "un_%s(r%d[q], x%d[q]);\n", dtype_tag(s.in_dtype[i]), i, i);
          unpacked[i] = true;
        }
        src = "x" + std::to_string(i) + "[q][e]";
      }
    }
    c += loop;
    if (t.op == BSIR_CHAIN_LOAD) {
      appendf(c, "acc[q][e] = %s;\n", src.c_str());
    } else {
      const bool rev = t.op == BSIR_CHAIN_RBINARY;
      appendf(c, "{ const float x = %s, y = %s; acc[q][e] = %s; }\n", rev ? src.c_str() : "acc[q][e]", rev ? "acc[q][e]" : src.c_str(),
              binary_expr(t.fn));
    }
  }
  for (int io = 0; io < s.n_out; ++io) {
    std::string v = s.out_tmp[io] < 0 ? "acc" : "t" + std::to_string(s.out_tmp[io]);
    const char *vn = v.c_str();
    if (s.out_per_row[io]) {
      // one value per row: the row's threads all hold it; the first one stores it
      const char *val = s.out_dtype[io] == BSIR_F32 ? "" : s.out_dtype[io] == BSIR_BF16 ? "pk_bf16" : "pk_f16";
      if (s.out_dtype[io] == BSIR_F32) appendf(c, "  if (row_ok && lane == 0) ((float *)a.out[%d])[row] = %s[0][0];\n", io, vn);
      else appendf(c, "  if (row_ok && lane == 0) ((u16 *)a.out[%d])[row] = (u16)%s(%s[0][0], 0.0f);\n", io, val, vn);
      continue;
    }
    c += "#pragma unroll\n  for (int q = 0; q < VPT; ++q) {\n    if (!row_ok || !live[q]) continue;\n";
    if (s.out_dtype[io] == BSIR_F32) {
      appendf(c, "    float *d = (float *)a.out[%d] + (row * a.out_stride[%d] + c0v[q]);\n", io, io);
      appendf(c, "    st_stream(d, __float_as_uint(%s[q][0]), __float_as_uint(%s[q][1]), __float_as_uint(%s[q][2]), __float_as_uint(%s[q][3]));\n", vn, vn, vn, vn);
      appendf(c, "    st_stream(d + 4, __float_as_uint(%s[q][4]), __float_as_uint(%s[q][5]), __float_as_uint(%s[q][6]), __float_as_uint(%s[q][7]));\n", vn, vn, vn, vn);
    } else {
      const char *pk = s.out_dtype[io] == BSIR_BF16 ? "pk_bf16" : "pk_f16";
      appendf(c, "    st_stream((u16 *)a.out[%d] + (row * a.out_stride[%d] + c0v[q]), %s(%s[q][0], %s[q][1]), %s(%s[q][2], %s[q][3]), %s(%s[q][4], %s[q][5]), %s(%s[q][6], %s[q][7]));\n",
              io, io, pk, vn, vn, pk, vn, vn, pk, vn, vn, pk, vn, vn);
    }
    c += "  }\n";
  }
  if (ring) c += "  }\n";   // the row loop
  c += "}\n";
  return c;
}

}  // namespace

int chain_jit_compile_only(const ChainJitSpec &s, size_t *cubin_bytes, std::string *why) {
  const std::vector<char> cubin = compile_cubin(chain_jit_source(s), why);
  if (cubin.empty()) return -1;
  if (cubin_bytes) *cubin_bytes = cubin.size();
  return 0;
}

namespace {
// Everything the generated source depends on, as bytes: the cache key (the source itself is only built on a miss).
std::string spec_key(const ChainJitSpec &s) {
  std::string k;
  auto put = [&](int32_t v) { k.append(reinterpret_cast<const char *>(&v), sizeof v); };
  put(s.n_in); put(s.n_instr); put(s.n_out);
  put(s.flat); put(s.alias); put(s.row_grid); put(chain_jit_unroll(s)); put(s.tpr); put(s.vpt); put(s.ring);
  for (int i = 0; i < s.n_in; ++i) { put(s.in_dtype[i]); put(s.in_kind[i]); }
  for (int i = 0; i < s.n_instr; ++i) {
    const bsir_chain_instr &t = s.tape[i];
    int32_t imm;
    memcpy(&imm, &t.imm, 4);
    put(t.op); put(t.fn); put(t.src_kind); put(t.src); put(imm);
  }
  for (int i = 0; i < s.n_out; ++i) { put(s.out_dtype[i]); put(s.out_tmp[i]); put(s.out_per_row[i]); }
  return k;
}
}  // namespace

int chain_jit_launch(const ChainJitSpec &s, const ChainJitArgs &args, cudaStream_t st, std::string *why) {
  const std::string key = spec_key(s);
  cudaKernel_t kernel = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_cache.find(key);
    if (it == g_cache.end()) {
      Compiled cpl;
      const std::string src = chain_jit_source(s);
      const std::vector<char> cubin = compile_cubin(src, &cpl.why);
      if (!cubin.empty()) {
        cudaLibrary_t lib = nullptr;
        cudaError_t e = cudaLibraryLoadData(&lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
        if (e == cudaSuccess) e = cudaLibraryGetKernel(&cpl.kernel, lib, "bsir_chain");
        if (e != cudaSuccess) {
          cpl.kernel = nullptr;
          cpl.why = std::string("loading the compiled chain: ") + cudaGetErrorString(e);
          (void)cudaGetLastError();
        }
      }
      it = g_cache.emplace(key, std::move(cpl)).first;
    }
    if (!it->second.kernel) {
      *why = it->second.why;
      return -1;
    }
    kernel = it->second.kernel;
  }
  if (s.tpr > 0 && s.ring > 0) {
    // persistent blocks, as many as are resident at once; the ring lives in dynamic shared memory
    size_t row_bytes = 0;
    for (int i = 0; i < s.n_in; ++i)
      if (s.in_kind[i] == BSIR_CHAIN_FULL) row_bytes += static_cast<size_t>(args.gpr) * (s.in_dtype[i] == BSIR_F32 ? 32 : 16);
    const size_t smem = row_bytes * s.ring;
    const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
    int64_t nblocks = sms;   // 1024 threads with the registers a row takes: one block per SM
    if (nblocks > args.rows) nblocks = args.rows;
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void *>(kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    ChainJitArgs copy = args;
    void *params[] = {&copy};
    if (e == cudaSuccess)
      e = cudaLaunchKernel(reinterpret_cast<const void *>(kernel), dim3(static_cast<unsigned>(nblocks)), dim3(s.tpr), params, smem, st);
    if (e != cudaSuccess) {
      *why = std::string("launching the compiled chain: ") + cudaGetErrorString(e);
      (void)cudaGetLastError();
      return -1;
    }
    return 0;
  }
  if (s.tpr > 0) {
    const int bt = s.tpr > 128 ? s.tpr : 128;
    const int64_t nblocks = (args.rows + bt / s.tpr - 1) / (bt / s.tpr);
    if (nblocks > 0x7fffffffLL) {
      *why = "grid too large";
      return -1;
    }
    ChainJitArgs copy = args;
    void *params[] = {&copy};
    const cudaError_t e = cudaLaunchKernel(reinterpret_cast<const void *>(kernel), dim3(static_cast<unsigned>(nblocks)), dim3(bt), params, 0, st);
    if (e != cudaSuccess) {
      *why = std::string("launching the compiled chain: ") + cudaGetErrorString(e);
      (void)cudaGetLastError();
      return -1;
    }
    return 0;
  }
  const int U = chain_jit_unroll(s);
  const bool rows_on_x = s.row_grid && !s.flat;
  const int64_t blocks = rows_on_x ? args.total / args.gpr : (args.total + 256 * U - 1) / (256 * U);
  const int64_t blocks_y = rows_on_x ? (args.gpr + 256 * U - 1) / (256 * U) : 1;
  if (blocks > 0x7fffffffLL || blocks_y > 65535) {
    *why = "grid too large";
    return -1;
  }
  ChainJitArgs copy = args;
  void *params[] = {&copy};
  const cudaError_t e = cudaLaunchKernel(reinterpret_cast<const void *>(kernel), dim3(static_cast<unsigned>(blocks), static_cast<unsigned>(blocks_y)), dim3(256), params, 0, st);
  if (e != cudaSuccess) {
    *why = std::string("launching the compiled chain: ") + cudaGetErrorString(e);
    (void)cudaGetLastError();
    return -1;
  }
  return 0;
}

}  // namespace bsir
