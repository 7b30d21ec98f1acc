// elementwise_impl.cuh -- the text of two translation units (elementwise.cu and elementwise_rows_outer.cu, which
// defines BSIR_ELEMENTWISE_PART_OUTER first and then holds only the rows kernel's outer-index instantiations:
// compiled side by side they take half the time of one file).
// hfusion.elemwise_unary / elemwise_binary / compare / select and the
// hivm.hir.v* vector ops that lower to them (vadd, vsub, vmul, ...), plus copy.
//
// Scalar semantics follow the region builders of the reference
// (bishengir/lib/Dialect/HFusion/IR/HFusionOps.cpp:434-743): f16/bf16 operands are widened
// to f32, the op runs in f32, the result is rounded once to nearest even
// (bishengir/lib/Dialect/HFusion/Transforms/LegalizeBF16.cpp:243-275); integer ops wrap.
//
// Two paths.  Contiguous operands (or scalars) with 16-byte aligned bases take the
// streaming path: 128-bit loads with four vectors in flight per thread, no L1 allocation,
// streaming stores.  Everything else (strides, inline broadcast with stride 0, odd
// alignment) takes the indexed path, one element per thread.
#include "common.cuh"

namespace bsir {
namespace {

// ------------------------------------------------------------------ scalar function tables
// The switch sits outside the per-element loops, so one uniform branch serves a whole vector.
template <int N>
__device__ __forceinline__ bool unary_f32(int fn, const float *x, float *r) {
#define U(expr)                                  \
  {                                              \
    _Pragma("unroll") for (int i = 0; i < N; ++i) { const float v = x[i]; r[i] = (expr); } \
    return true;                                 \
  }
  switch (fn) {
    case BSIR_UNARY_RELU: U(maximumf(0.0f, v))
    case BSIR_UNARY_SQRT: case BSIR_UNARY_SQRT_L: U(__fsqrt_rn(v))
    case BSIR_UNARY_RSQRT: case BSIR_UNARY_RSQRT_L: U(__fdiv_rn(1.0f, __fsqrt_rn(v)))
    case BSIR_UNARY_REC: case BSIR_UNARY_RECIPROCAL: U(__fdiv_rn(1.0f, v))
    case BSIR_UNARY_TANH: case BSIR_UNARY_TANH_L: U(tanhf(v))
    case BSIR_UNARY_SIN: U(sinf(v))
    case BSIR_UNARY_COS: U(cosf(v))
    case BSIR_UNARY_ATAN: U(atanf(v))
    case BSIR_UNARY_TAN: U(tanf(v))
    case BSIR_UNARY_ERF: case BSIR_UNARY_ERF_L: U(erff(v))
    case BSIR_UNARY_LOG2: U(log2f(v))
    case BSIR_UNARY_LOG10: U(log10f(v))
    case BSIR_UNARY_LOG1P: U(log1pf(v))
    case BSIR_UNARY_EXP2: U(exp2f(v))
    case BSIR_UNARY_EXPM1: U(expm1f(v))
    case BSIR_UNARY_ILOGB: U(logbf(v))   // floor(log2(|x|)), exactly: the exponent (Normalize.cpp:6782-6830)
    case BSIR_UNARY_ASIN: U(asinf(v))
    case BSIR_UNARY_ACOS: U(acosf(v))
    case BSIR_UNARY_ASINH: U(asinhf(v))
    case BSIR_UNARY_ACOSH: U(acoshf(v))
    case BSIR_UNARY_ATANH: U(atanhf(v))
    case BSIR_UNARY_SINH: U(sinhf(v))
    case BSIR_UNARY_LGAMMA: U(lgammaf(v))
    case BSIR_UNARY_COSH: U(coshf(v))
    case BSIR_UNARY_NEARBYINT: U(rintf(v))
    case BSIR_UNARY_EXP: U(expf(v))
    case BSIR_UNARY_LOG: U(logf(v))
    case BSIR_UNARY_ABS: U(fabsf(v))
    case BSIR_UNARY_CEIL: U(ceilf(v))
    case BSIR_UNARY_FLOOR: U(floorf(v))
    case BSIR_UNARY_NEGF: U(-v)
    case BSIR_UNARY_ROUND: U(roundf(v))
    case BSIR_UNARY_SQUARE: U(__fmul_rn(v, v))
    default: return false;
  }
#undef U
}

template <int N>
__device__ __forceinline__ bool binary_f32(int fn, const float *a, const float *b, float *r) {
#define B(expr)                                  \
  {                                              \
    _Pragma("unroll") for (int i = 0; i < N; ++i) { const float x = a[i], y = b[i]; r[i] = (expr); } \
    return true;                                 \
  }
  switch (fn) {
    case BSIR_BINARY_ADD: B(__fadd_rn(x, y))
    case BSIR_BINARY_SUB: B(__fsub_rn(x, y))
    case BSIR_BINARY_MUL: B(__fmul_rn(x, y))
    case BSIR_BINARY_DIV: case BSIR_BINARY_DIVFHP: B(__fdiv_rn(x, y))
    case BSIR_BINARY_MAXF: case BSIR_BINARY_MAX_SIGNED: case BSIR_BINARY_MAX_UNSIGNED: B(maximumf(x, y))
    case BSIR_BINARY_MINF: case BSIR_BINARY_MIN_SIGNED: case BSIR_BINARY_MIN_UNSIGNED: B(minimumf(x, y))
    case BSIR_BINARY_MAXNUMF: B(fmaxf(x, y))
    case BSIR_BINARY_MINNUMF: B(fminf(x, y))
    case BSIR_BINARY_POWF: case BSIR_BINARY_POWF_L: B(powf(x, y))
    case BSIR_BINARY_MOD: case BSIR_BINARY_MODUI: B(fmodf(x, y))
    case BSIR_BINARY_LDEXP: B(ldexpf(x, static_cast<int>(y)))
    case BSIR_BINARY_ATAN2: B(atan2f(x, y))
    case BSIR_BINARY_COPYSIGN: B(copysignf(x, y))
    default: return false;
  }
#undef B
}

template <typename T> struct Unsigned;
template <> struct Unsigned<int8_t> { using type = uint8_t; };
template <> struct Unsigned<int16_t> { using type = uint16_t; };
template <> struct Unsigned<int32_t> { using type = uint32_t; };
template <> struct Unsigned<int64_t> { using type = uint64_t; };
template <> struct Unsigned<uint8_t> { using type = uint8_t; };
template <> struct Unsigned<uint16_t> { using type = uint16_t; };
template <> struct Unsigned<uint32_t> { using type = uint32_t; };
template <> struct Unsigned<uint64_t> { using type = uint64_t; };
template <typename T> struct Signed;
template <> struct Signed<int8_t> { using type = int8_t; };
template <> struct Signed<int16_t> { using type = int16_t; };
template <> struct Signed<int32_t> { using type = int32_t; };
template <> struct Signed<int64_t> { using type = int64_t; };
template <> struct Signed<uint8_t> { using type = int8_t; };
template <> struct Signed<uint16_t> { using type = int16_t; };
template <> struct Signed<uint32_t> { using type = int32_t; };
template <> struct Signed<uint64_t> { using type = int64_t; };

template <typename T>
__device__ __forceinline__ T ipowi(T b, T e) {
  using UT = typename Unsigned<T>::type;
  using ST = typename Signed<T>::type;
  if (static_cast<ST>(e) < 0 && T(-1) < T(0)) {
    if (b == T(1)) return T(1);
    if (b == T(-1)) return (e & 1) ? T(-1) : T(1);
    return T(0);
  }
  UT r = 1, x = static_cast<UT>(b), n = static_cast<UT>(e);
  while (n) { if (n & 1) r = static_cast<UT>(r * x); x = static_cast<UT>(x * x); n >>= 1; }
  return static_cast<T>(r);
}

template <typename T, int N>
__device__ __forceinline__ bool unary_int(int fn, const T *x, T *r) {
  using UT = typename Unsigned<T>::type;
#define U(expr)                                  \
  {                                              \
    _Pragma("unroll") for (int i = 0; i < N; ++i) { const T v = x[i]; r[i] = static_cast<T>(expr); } \
    return true;                                 \
  }
  switch (fn) {
    case BSIR_UNARY_RELU: U(v > T(0) ? v : T(0))
    case BSIR_UNARY_VNOT: U(~v)
    case BSIR_UNARY_ABSI: case BSIR_UNARY_ABS: U(v < T(0) ? static_cast<T>(UT(0) - static_cast<UT>(v)) : v)
    case BSIR_UNARY_SQUARE: U(static_cast<UT>(v) * static_cast<UT>(v))
    default: return false;
  }
#undef U
}

template <typename T, int N>
__device__ __forceinline__ bool binary_int(int fn, const T *a, const T *b, T *r) {
  using UT = typename Unsigned<T>::type;
  using ST = typename Signed<T>::type;
  constexpr int kBits = 8 * sizeof(T);
  constexpr bool kSigned = T(-1) < T(0);
#define B(expr)                                  \
  {                                              \
    _Pragma("unroll") for (int i = 0; i < N; ++i) { \
      const T x = a[i], y = b[i];                \
      const UT ux = static_cast<UT>(x), uy = static_cast<UT>(y); \
      const ST sx = static_cast<ST>(x), sy = static_cast<ST>(y); \
      (void)ux; (void)uy; (void)sx; (void)sy;    \
      r[i] = static_cast<T>(expr);               \
    }                                            \
    return true;                                 \
  }
  switch (fn) {
    case BSIR_BINARY_VOR: B(x | y)
    case BSIR_BINARY_VAND: B(x & y)
    case BSIR_BINARY_VXOR: B(x ^ y)
    case BSIR_BINARY_ADD: B(UT(ux + uy))
    case BSIR_BINARY_SUB: B(UT(ux - uy))
    case BSIR_BINARY_MUL: B(UT(ux * uy))
    case BSIR_BINARY_DIV: B(y == T(0) ? T(0) : (kSigned && sy == ST(-1)) ? T(UT(0) - ux) : T(x / y))
    case BSIR_BINARY_DIV_UNSIGNED: B(uy == 0 ? UT(0) : UT(ux / uy))
    case BSIR_BINARY_MAX_SIGNED: B(x > y ? x : y)
    case BSIR_BINARY_MIN_SIGNED: B(x < y ? x : y)
    case BSIR_BINARY_MAX_UNSIGNED: B(ux > uy ? x : y)
    case BSIR_BINARY_MIN_UNSIGNED: B(ux < uy ? x : y)
    case BSIR_BINARY_MOD: B(y == T(0) ? T(0) : (kSigned && sy == ST(-1)) ? T(0) : T(x % y))
    case BSIR_BINARY_MODUI: B(uy == 0 ? UT(0) : UT(ux % uy))
    case BSIR_BINARY_SHLI: B(uy >= UT(kBits) ? UT(0) : UT(ux << uy))
    case BSIR_BINARY_SHRSI:
      B(kSigned ? (uy >= UT(kBits) ? ST(sx < 0 ? -1 : 0) : ST(sx >> uy)) : ST(uy >= UT(kBits) ? UT(0) : UT(ux >> uy)))
    case BSIR_BINARY_SHRUI: B(uy >= UT(kBits) ? UT(0) : UT(ux >> uy))
    case BSIR_BINARY_CEILDIVSI:
      B(y == T(0) ? T(0) : T(sx / sy + (((sx % sy) != 0 && ((sx < 0) == (sy < 0))) ? 1 : 0)))
    case BSIR_BINARY_CEILDIVUI: B(uy == 0 ? UT(0) : UT(ux / uy + (ux % uy ? 1 : 0)))
    case BSIR_BINARY_FLOORDIVSI:
      B(y == T(0) ? T(0) : T(sx / sy - (((sx % sy) != 0 && ((sx < 0) != (sy < 0))) ? 1 : 0)))
    case BSIR_BINARY_POWI: B(ipowi<T>(x, y))
    default: return false;
  }
#undef B
}

// ------------------------------------------------------------------ storage access by dtype
template <int DT> struct CType;
template <> struct CType<BSIR_F32> { using type = float; };
template <> struct CType<BSIR_F16> { using type = uint16_t; };
template <> struct CType<BSIR_BF16> { using type = uint16_t; };
template <> struct CType<BSIR_I8> { using type = int8_t; };
template <> struct CType<BSIR_I16> { using type = int16_t; };
template <> struct CType<BSIR_I32> { using type = int32_t; };
template <> struct CType<BSIR_I64> { using type = int64_t; };
template <> struct CType<BSIR_U8> { using type = uint8_t; };
template <> struct CType<BSIR_U16> { using type = uint16_t; };
template <> struct CType<BSIR_U32> { using type = uint32_t; };
template <> struct CType<BSIR_U64> { using type = uint64_t; };
template <> struct CType<BSIR_BOOL> { using type = uint8_t; };

template <int DT> struct IsFloat { static constexpr bool value = DT == BSIR_F32 || DT == BSIR_F16 || DT == BSIR_BF16; };

template <int DT>
__device__ __forceinline__ float widen(typename CType<DT>::type v) {
  if constexpr (DT == BSIR_F32) return v;
  else if constexpr (DT == BSIR_F16) return __half2float(__ushort_as_half(v));
  else return __uint_as_float(static_cast<uint32_t>(v) << 16);
}
template <int DT>
__device__ __forceinline__ typename CType<DT>::type narrow(float v) {
  if constexpr (DT == BSIR_F32) return v;
  else if constexpr (DT == BSIR_F16) return __half_as_ushort(__float2half_rn(v));
  else return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

struct Operand {
  const void *p;
  int64_t s0, s1, s2;
  unsigned long long scalar;  // value bits when p == nullptr
};
struct Shape {
  int64_t n0, n1, n2, total;
};

template <int DT>
__device__ __forceinline__ typename CType<DT>::type fetch(const Operand &o, int64_t i0, int64_t i1, int64_t i2) {
  using T = typename CType<DT>::type;
  if (o.p == nullptr) {
    T v;
    const unsigned long long s = o.scalar;
    memcpy(&v, &s, sizeof(T));
    return v;
  }
  return static_cast<const T *>(o.p)[i0 * o.s0 + i1 * o.s1 + i2 * o.s2];
}

enum { kOpUnary = 0, kOpBinary = 1, kOpCompare = 2, kOpSelect = 3, kOpCopy = 4 };

// ------------------------------------------------------------------ indexed (generic) path
// Any strides (views, broadcast operands with stride 0, rank 3).  block = (columns, rows): threadIdx.x
// runs along the innermost dimension, threadIdx.y over the collapsed outer ones, so there is one
// division per row instead of two per element; a thread takes kIdxUnroll columns (a block apart, so
// that a warp's accesses stay together) through one evaluation of the function switch.
constexpr int kIdxUnroll = 4;

template <int DT>
__device__ __forceinline__ bool compare_elem_idx(int fn, typename CType<DT>::type xa, typename CType<DT>::type ya, bool *ok) {
  using T = typename CType<DT>::type;
  if constexpr (IsFloat<DT>::value) {
    const float x = widen<DT>(xa), y = widen<DT>(ya);
    switch (fn) {
      case BSIR_CMP_VEQ: return x == y;
      case BSIR_CMP_VNE: return !(x == y);  // unordered-or-not-equal
      case BSIR_CMP_VLE: return x <= y;
      case BSIR_CMP_VLT: return x < y;
      case BSIR_CMP_VGE: return x >= y;
      case BSIR_CMP_VGT: return x > y;
      default: *ok = false; return false;
    }
  } else {
    using UT = typename Unsigned<T>::type;
    const UT ux = static_cast<UT>(xa), uy = static_cast<UT>(ya);
    switch (fn) {
      case BSIR_CMP_VEQ: return xa == ya;
      case BSIR_CMP_VNE: return xa != ya;
      case BSIR_CMP_VLE: return xa <= ya;
      case BSIR_CMP_VLT: return xa < ya;
      case BSIR_CMP_VGE: return xa >= ya;
      case BSIR_CMP_VGT: return xa > ya;
      case BSIR_CMP_VULE: return ux <= uy;
      case BSIR_CMP_VULT: return ux < uy;
      case BSIR_CMP_VUGE: return ux >= uy;
      case BSIR_CMP_VUGT: return ux > uy;
      default: *ok = false; return false;
    }
  }
}

template <int DT, int KIND>
__global__ void __launch_bounds__(256) indexed_kernel(int fn, Shape sh, Operand a, Operand b, Operand c, void *out,
                                                      int64_t os0, int64_t os1, int64_t os2, int *bad_fn) {
  using T = typename CType<DT>::type;
  bool ok = true;
  const int64_t nrows = sh.n0 * sh.n1;
  const int64_t col_step = static_cast<int64_t>(gridDim.x) * blockDim.x * kIdxUnroll;
  for (int64_t row = static_cast<int64_t>(blockIdx.y) * blockDim.y + threadIdx.y; row < nrows;
       row += static_cast<int64_t>(gridDim.y) * blockDim.y) {
    const int64_t i0 = row / sh.n1, i1 = row - i0 * sh.n1;
    const int64_t obase = i0 * os0 + i1 * os1;
    for (int64_t c0 = static_cast<int64_t>(blockIdx.x) * blockDim.x * kIdxUnroll + threadIdx.x; c0 < sh.n2; c0 += col_step) {
      int64_t i2[kIdxUnroll];
      bool in[kIdxUnroll];
#pragma unroll
      for (int u = 0; u < kIdxUnroll; ++u) {
        i2[u] = c0 + static_cast<int64_t>(u) * blockDim.x;
        in[u] = i2[u] < sh.n2;
        if (!in[u]) i2[u] = c0;                    // a valid address; the result is not stored
      }
      if constexpr (KIND == kOpCopy) {
        T v[kIdxUnroll];
#pragma unroll
        for (int u = 0; u < kIdxUnroll; ++u) v[u] = fetch<DT>(a, i0, i1, i2[u]);
#pragma unroll
        for (int u = 0; u < kIdxUnroll; ++u)
          if (in[u]) static_cast<T *>(out)[obase + i2[u] * os2] = v[u];
      } else if constexpr (KIND == kOpSelect) {
#pragma unroll
        for (int u = 0; u < kIdxUnroll; ++u) {
          const uint8_t cnd = fetch<BSIR_BOOL>(a, i0, i1, i2[u]);
          const T v = cnd ? fetch<DT>(b, i0, i1, i2[u]) : fetch<DT>(c, i0, i1, i2[u]);
          if (in[u]) static_cast<T *>(out)[obase + i2[u] * os2] = v;
        }
      } else if constexpr (KIND == kOpCompare) {
        T x[kIdxUnroll], y[kIdxUnroll];
#pragma unroll
        for (int u = 0; u < kIdxUnroll; ++u) { x[u] = fetch<DT>(a, i0, i1, i2[u]); y[u] = fetch<DT>(b, i0, i1, i2[u]); }
#pragma unroll
        for (int u = 0; u < kIdxUnroll; ++u) {
          const bool r = compare_elem_idx<DT>(fn, x[u], y[u], &ok);
          if (in[u]) static_cast<uint8_t *>(out)[obase + i2[u] * os2] = r ? 1 : 0;
        }
      } else if constexpr (IsFloat<DT>::value) {
        float x[kIdxUnroll], y[kIdxUnroll], r[kIdxUnroll];
#pragma unroll
        for (int u = 0; u < kIdxUnroll; ++u) {
          x[u] = widen<DT>(fetch<DT>(a, i0, i1, i2[u]));
          if constexpr (KIND == kOpBinary) y[u] = widen<DT>(fetch<DT>(b, i0, i1, i2[u]));
          r[u] = 0.0f;
        }
        if constexpr (KIND == kOpUnary) ok = unary_f32<kIdxUnroll>(fn, x, r) && ok;
        else ok = binary_f32<kIdxUnroll>(fn, x, y, r) && ok;
#pragma unroll
        for (int u = 0; u < kIdxUnroll; ++u)
          if (in[u]) static_cast<T *>(out)[obase + i2[u] * os2] = narrow<DT>(r[u]);
      } else {
        T x[kIdxUnroll], y[kIdxUnroll], r[kIdxUnroll];
#pragma unroll
        for (int u = 0; u < kIdxUnroll; ++u) {
          x[u] = fetch<DT>(a, i0, i1, i2[u]);
          if constexpr (KIND == kOpBinary) y[u] = fetch<DT>(b, i0, i1, i2[u]);
          r[u] = 0;
        }
        if constexpr (KIND == kOpUnary) ok = unary_int<T, kIdxUnroll>(fn, x, r) && ok;
        else ok = binary_int<T, kIdxUnroll>(fn, x, y, r) && ok;
#pragma unroll
        for (int u = 0; u < kIdxUnroll; ++u) {
          if constexpr (DT == BSIR_BOOL) r[u] &= 1;
          if (in[u]) static_cast<T *>(out)[obase + i2[u] * os2] = r[u];
        }
      }
    }
  }
  if (!ok && bad_fn) *bad_fn = 1;
}

// ------------------------------------------------------------------ streaming path
constexpr int kStreamThreads = 256;
constexpr int kStreamUnroll = 4;

// a_mode / b_mode: 0 = tensor (contiguous, 16-byte aligned), 1 = scalar.
template <int DT, int KIND>
__global__ void __launch_bounds__(kStreamThreads)
    stream_kernel(int fn, int64_t n, const void *__restrict__ ap, const void *__restrict__ bp,
                  unsigned long long a_scalar, unsigned long long b_scalar, void *__restrict__ outp) {
  using T = typename CType<DT>::type;
  constexpr int kPerVec = 16 / sizeof(T);
  const int64_t nvec = n / kPerVec;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (kStreamThreads * kStreamUnroll) + threadIdx.x;
  pdl_launch_dependents();   // the next launch may be scheduled while this one runs (launch_pdl) ...
  pdl_wait();                // ... and this one touches global memory only after the kernel ahead has completed

  Vec16 va[kStreamUnroll], vb[kStreamUnroll];
  T sa, sb;
  memcpy(&sa, &a_scalar, sizeof(T));
  memcpy(&sb, &b_scalar, sizeof(T));
#pragma unroll
  for (int u = 0; u < kStreamUnroll; ++u) {
    const int64_t v = base + static_cast<int64_t>(u) * kStreamThreads;
    if (v < nvec) {
      if (ap) va[u] = ld_stream(static_cast<const Vec16 *>(ap) + v);
      if constexpr (KIND == kOpBinary) {
        if (bp) vb[u] = ld_stream(static_cast<const Vec16 *>(bp) + v);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kStreamUnroll; ++u) {
    const int64_t v = base + static_cast<int64_t>(u) * kStreamThreads;
    if (v >= nvec) continue;
    Vec16 vo;
    if constexpr (KIND == kOpCopy) {
      vo = va[u];
    } else if constexpr (IsFloat<DT>::value) {
      constexpr int kPerWord = FloatTraits<DT>::kPerWord;
      float x[4 * kPerWord], y[4 * kPerWord], r[4 * kPerWord];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        if (ap) FloatTraits<DT>::unpack(va[u].w[w], x + w * kPerWord);
        else
          for (int e = 0; e < kPerWord; ++e) x[w * kPerWord + e] = widen<DT>(sa);
        if constexpr (KIND == kOpBinary) {
          if (bp) FloatTraits<DT>::unpack(vb[u].w[w], y + w * kPerWord);
          else
            for (int e = 0; e < kPerWord; ++e) y[w * kPerWord + e] = widen<DT>(sb);
        }
      }
      if constexpr (KIND == kOpUnary) unary_f32<4 * kPerWord>(fn, x, r);
      else binary_f32<4 * kPerWord>(fn, x, y, r);
#pragma unroll
      for (int w = 0; w < 4; ++w) vo.w[w] = FloatTraits<DT>::pack(r + w * kPerWord);
    } else {
      T x[kPerVec], y[kPerVec], r[kPerVec];
      if (ap) memcpy(x, &va[u], 16);
      else
        for (int e = 0; e < kPerVec; ++e) x[e] = sa;
      if constexpr (KIND == kOpBinary) {
        if (bp) memcpy(y, &vb[u], 16);
        else
          for (int e = 0; e < kPerVec; ++e) y[e] = sb;
        binary_int<T, kPerVec>(fn, x, y, r);
      } else {
        unary_int<T, kPerVec>(fn, x, r);
      }
      if constexpr (DT == BSIR_BOOL) {
        for (int e = 0; e < kPerVec; ++e) r[e] &= 1;
      }
      memcpy(&vo, r, 16);
    }
    st_stream(static_cast<Vec16 *>(outp) + v, vo);
  }

  // ragged tail (< one vector): the first threads of block 0, one element each
  const int64_t tail0 = nvec * kPerVec;
  if (blockIdx.x == 0 && tail0 + threadIdx.x < n) {
    const int64_t i = tail0 + threadIdx.x;
    const T xa = ap ? static_cast<const T *>(ap)[i] : sa;
    T ro;
    if constexpr (KIND == kOpCopy) {
      ro = xa;
    } else if constexpr (IsFloat<DT>::value) {
      float x = widen<DT>(xa), r = 0.0f;
      if constexpr (KIND == kOpUnary) unary_f32<1>(fn, &x, &r);
      else {
        float y = widen<DT>(bp ? static_cast<const T *>(bp)[i] : sb);
        binary_f32<1>(fn, &x, &y, &r);
      }
      ro = narrow<DT>(r);
    } else {
      T x = xa, r = 0;
      if constexpr (KIND == kOpUnary) unary_int<T, 1>(fn, &x, &r);
      else {
        T y = bp ? static_cast<const T *>(bp)[i] : sb;
        binary_int<T, 1>(fn, &x, &y, &r);
      }
      if constexpr (DT == BSIR_BOOL) r &= 1;
      ro = r;
    }
    static_cast<T *>(outp)[i] = ro;
  }
}

// ------------------------------------------------------------------ [rows, cols] with broadcast / row-strided operands
// The inline-broadcast forms of hivm.hir.v* (`broadcast = [..]`: a per-column or per-row vector, or a scalar held in
// memory, against a full tensor) and operands that are row-strided views of a wider tensor: a [rows, cols] problem in
// which each operand is one of
//   0  a tensor with its own row stride (rows 16-byte aligned),    1  a row vector [cols], the same for every row
//   2  one value per row (a column vector, dense or strided) or one      (of an outer index, when the problem is
//      value in memory,                                                  [n0, n1, cols] and the vector [n0, 1, cols]),
// each with a stride between rows and one between outer indices (either may be 0: [n0, 1, 1], [1, n1, 1], ...).
// A thread handles kStreamUnroll 16-byte vectors of the flattened [rows x cols / per_vec] space; full operands
// and the result move as streaming 16-byte accesses, row vectors come through the read-only cache (every row reads
// the same bytes), column vectors and scalars are single elements replicated.  Arithmetic is that of stream_kernel.
}  // namespace
struct RowsOperand {
  const void *p;
  int64_t rs;               // elements between the rows of one outer index
  int64_t os;               // elements between outer indices (a [n0, n1, cols] problem has rows = n0 * n1; 0 when unused)
  int kind;
};

namespace {

// The operand kinds are template parameters: with a run-time switch per kind the branches end in register moves, a
// move waits for its load, and a thread's loads then run one after the other (measured 0.50-0.74 of the HBM rate
// against 0.95 with every operand a full tensor; predicated loads into the same registers serialise likewise).
// Phase one is the load alone: a single element (kind 2) comes back in word 0 and is replicated in phase two, after
// every load of the thread has been issued.  (q, r) = (row / n1, row % n1): the outer index and the row within it.
template <int DT, int K>
__device__ __forceinline__ Vec16 rows_load(const RowsOperand &o, int64_t q, int64_t r, int64_t c) {
  using T = typename CType<DT>::type;
  if constexpr (K == 0) {
    return ld_stream(reinterpret_cast<const Vec16 *>(static_cast<const T *>(o.p) + q * o.os + r * o.rs) + c);
  } else if constexpr (K == 1) {
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(static_cast<const T *>(o.p) + q * o.os) + c);   // one vector for all rows of q
    return Vec16{{v.x, v.y, v.z, v.w}};
  } else {
    const T e = __ldg(static_cast<const T *>(o.p) + q * o.os + r * o.rs);      // one value per row (strides may be 0)
    Vec16 v{{0u, 0u, 0u, 0u}};
    memcpy(&v, &e, sizeof(T));
    return v;
  }
}
template <int DT, int K>
__device__ __forceinline__ Vec16 rows_expand(Vec16 v) {
  using T = typename CType<DT>::type;
  constexpr int kPerVec = 16 / sizeof(T);
  if constexpr (K < 2) return v;
  T e;
  memcpy(&e, &v, sizeof(T));
  T tmp[kPerVec];
#pragma unroll
  for (int i = 0; i < kPerVec; ++i) tmp[i] = e;
  memcpy(&v, tmp, 16);
  return v;
}

template <int DT, int KIND, int KA, int KB, bool OUTER>
__global__ void __launch_bounds__(kStreamThreads, 4)
    rows_kernel(int fn, int64_t rows, int64_t n1, int64_t vpr, RowsOperand a, RowsOperand b, void *__restrict__ outp, int64_t out_rs,
                int64_t out_os) {
  using T = typename CType<DT>::type;
  constexpr int kPerVec = 16 / sizeof(T);
  const int64_t total = rows * vpr;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (kStreamThreads * kStreamUnroll) + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  Vec16 va[kStreamUnroll], vb[kStreamUnroll];
  int64_t out_off[kStreamUnroll];      // in elements
#pragma unroll
  for (int u = 0; u < kStreamUnroll; ++u) {
    const int64_t v = base + static_cast<int64_t>(u) * kStreamThreads;
    if (v < total) {
      // 32-bit division when it will do: the 64-bit one is a subroutine of a hundred instructions
      const int64_t row = total <= 0x7fffffff ? static_cast<int64_t>(static_cast<uint32_t>(v) / static_cast<uint32_t>(vpr)) : v / vpr;
      const int64_t col = v - row * vpr;
      int64_t q = 0, r = row;            // without an outer index (a template parameter: the second division costs the
      if constexpr (OUTER) {             // plain forms a tenth of their rate even when a branch skips it)
        q = total <= 0x7fffffff ? static_cast<int64_t>(static_cast<uint32_t>(row) / static_cast<uint32_t>(n1)) : row / n1;
        r = row - q * n1;
      }
      out_off[u] = q * out_os + r * out_rs + col * kPerVec;
      va[u] = rows_load<DT, KA>(a, q, r, col);
      if constexpr (KIND == kOpBinary) vb[u] = rows_load<DT, KB>(b, q, r, col);
    }
  }
#pragma unroll
  for (int u = 0; u < kStreamUnroll; ++u) {
    const int64_t v = base + static_cast<int64_t>(u) * kStreamThreads;
    if (v >= total) continue;
    const Vec16 xa = rows_expand<DT, KA>(va[u]);
    Vec16 xb = xa;
    if constexpr (KIND == kOpBinary) xb = rows_expand<DT, KB>(vb[u]);
    Vec16 vo;
    if constexpr (KIND == kOpCopy) {
      vo = xa;
    } else if constexpr (IsFloat<DT>::value) {
      constexpr int kPerWord = FloatTraits<DT>::kPerWord;
      float x[4 * kPerWord], y[4 * kPerWord], r[4 * kPerWord];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        FloatTraits<DT>::unpack(xa.w[w], x + w * kPerWord);
        if constexpr (KIND == kOpBinary) FloatTraits<DT>::unpack(xb.w[w], y + w * kPerWord);
      }
      if constexpr (KIND == kOpUnary) unary_f32<4 * kPerWord>(fn, x, r);
      else binary_f32<4 * kPerWord>(fn, x, y, r);
#pragma unroll
      for (int w = 0; w < 4; ++w) vo.w[w] = FloatTraits<DT>::pack(r + w * kPerWord);
    } else {
      T x[kPerVec], y[kPerVec], r[kPerVec];
      memcpy(x, &xa, 16);
      if constexpr (KIND == kOpBinary) {
        memcpy(y, &xb, 16);
        binary_int<T, kPerVec>(fn, x, y, r);
      } else {
        unary_int<T, kPerVec>(fn, x, r);
      }
      if constexpr (DT == BSIR_BOOL) {
        for (int e = 0; e < kPerVec; ++e) r[e] &= 1;
      }
      memcpy(&vo, r, 16);
    }
    st_stream(static_cast<T *>(outp) + out_off[u], vo);
  }
}

// ------------------------------------------------------------------ streaming compare / select
template <int DT>
__device__ __forceinline__ bool compare_elem(int fn, typename CType<DT>::type xa, typename CType<DT>::type ya) {
  using T = typename CType<DT>::type;
  if constexpr (IsFloat<DT>::value) {
    const float x = widen<DT>(xa), y = widen<DT>(ya);
    switch (fn) {
      case BSIR_CMP_VEQ: return x == y;
      case BSIR_CMP_VNE: return !(x == y);  // unordered-or-not-equal
      case BSIR_CMP_VLE: return x <= y;
      case BSIR_CMP_VLT: return x < y;
      case BSIR_CMP_VGE: return x >= y;
      default: return x > y;
    }
  } else {
    using UT = typename Unsigned<T>::type;
    const UT ux = static_cast<UT>(xa), uy = static_cast<UT>(ya);
    switch (fn) {
      case BSIR_CMP_VEQ: return xa == ya;
      case BSIR_CMP_VNE: return xa != ya;
      case BSIR_CMP_VLE: return xa <= ya;
      case BSIR_CMP_VLT: return xa < ya;
      case BSIR_CMP_VGE: return xa >= ya;
      case BSIR_CMP_VGT: return xa > ya;
      case BSIR_CMP_VULE: return ux <= uy;
      case BSIR_CMP_VULT: return ux < uy;
      case BSIR_CMP_VUGE: return ux >= uy;
      default: return ux > uy;
    }
  }
}

// Contiguous, aligned operands: a thread handles 16-byte vectors of the value type; compare writes the
// vector's results as one store of 16 / sizeof(T) bool bytes, select reads its condition bytes the same way.
// KIND = kOpCompare: out(bool) = a <fn> b.  KIND = kOpSelect: out = cond ? a : b (cond in `cp`).
template <int DT, int KIND>
__global__ void __launch_bounds__(kStreamThreads)
    cmpsel_stream_kernel(int fn, int64_t n, const void *__restrict__ ap, const void *__restrict__ bp,
                         const void *__restrict__ cp, unsigned long long a_scalar, unsigned long long b_scalar,
                         void *__restrict__ outp) {
  using T = typename CType<DT>::type;
  constexpr int kPerVec = 16 / sizeof(T);
  struct alignas(kPerVec) Flags { uint8_t f[kPerVec]; };
  const int64_t nvec = n / kPerVec;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (kStreamThreads * kStreamUnroll) + threadIdx.x;
  T sa, sb;
  memcpy(&sa, &a_scalar, sizeof(T));
  memcpy(&sb, &b_scalar, sizeof(T));
  Vec16 va[kStreamUnroll], vb[kStreamUnroll];
  Flags fc[kStreamUnroll];
#pragma unroll
  for (int u = 0; u < kStreamUnroll; ++u) {
    const int64_t v = base + static_cast<int64_t>(u) * kStreamThreads;
    if (v < nvec) {
      if (ap) va[u] = ld_stream(static_cast<const Vec16 *>(ap) + v);
      if (bp) vb[u] = ld_stream(static_cast<const Vec16 *>(bp) + v);
      if constexpr (KIND == kOpSelect) fc[u] = static_cast<const Flags *>(cp)[v];
    }
  }
  // the predicate is chosen once, outside the loops: inside them it is a constant and the comparison one instruction
  auto all_vectors = [&](auto fn_tag) {
#pragma unroll
    for (int u = 0; u < kStreamUnroll; ++u) {
      const int64_t v = base + static_cast<int64_t>(u) * kStreamThreads;
      if (v >= nvec) continue;
      T x[kPerVec], y[kPerVec];
      if (ap) memcpy(x, &va[u], 16);
      else
        for (int e = 0; e < kPerVec; ++e) x[e] = sa;
      if (bp) memcpy(y, &vb[u], 16);
      else
        for (int e = 0; e < kPerVec; ++e) y[e] = sb;
      if constexpr (KIND == kOpCompare) {
        // the vector's bool bytes are put together in registers and leave as one store of their whole width
        if constexpr (kPerVec == 2) {
          const uint32_t w = (compare_elem<DT>(decltype(fn_tag)::value, x[0], y[0]) ? 1u : 0u) |
                             (compare_elem<DT>(decltype(fn_tag)::value, x[1], y[1]) ? 0x100u : 0u);
          static_cast<uint16_t *>(outp)[v] = static_cast<uint16_t>(w);
        } else {
          uint32_t w[kPerVec / 4];
#pragma unroll
          for (int q = 0; q < kPerVec / 4; ++q) {
            w[q] = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) w[q] |= (compare_elem<DT>(decltype(fn_tag)::value, x[4 * q + e], y[4 * q + e]) ? 1u : 0u) << (8 * e);
          }
          if constexpr (kPerVec == 4) static_cast<uint32_t *>(outp)[v] = w[0];
          else if constexpr (kPerVec == 8) static_cast<uint2 *>(outp)[v] = make_uint2(w[0], w[1]);
          else static_cast<uint4 *>(outp)[v] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
        T r[kPerVec];
#pragma unroll
        for (int e = 0; e < kPerVec; ++e) r[e] = fc[u].f[e] ? x[e] : y[e];
        Vec16 vo;
        memcpy(&vo, r, 16);
        st_stream(static_cast<Vec16 *>(outp) + v, vo);
      }
    }
  };
  if constexpr (KIND == kOpCompare) {
    switch (fn) {
      case BSIR_CMP_VEQ: all_vectors(std::integral_constant<int, BSIR_CMP_VEQ>{}); break;
      case BSIR_CMP_VNE: all_vectors(std::integral_constant<int, BSIR_CMP_VNE>{}); break;
      case BSIR_CMP_VLE: all_vectors(std::integral_constant<int, BSIR_CMP_VLE>{}); break;
      case BSIR_CMP_VLT: all_vectors(std::integral_constant<int, BSIR_CMP_VLT>{}); break;
      case BSIR_CMP_VGE: all_vectors(std::integral_constant<int, BSIR_CMP_VGE>{}); break;
      case BSIR_CMP_VGT: all_vectors(std::integral_constant<int, BSIR_CMP_VGT>{}); break;
      case BSIR_CMP_VULE: all_vectors(std::integral_constant<int, BSIR_CMP_VULE>{}); break;
      case BSIR_CMP_VULT: all_vectors(std::integral_constant<int, BSIR_CMP_VULT>{}); break;
      case BSIR_CMP_VUGE: all_vectors(std::integral_constant<int, BSIR_CMP_VUGE>{}); break;
      default: all_vectors(std::integral_constant<int, BSIR_CMP_VUGT>{}); break;
    }
  } else {
    all_vectors(std::integral_constant<int, 0>{});
  }
  // ragged tail (< one vector): the first threads of block 0, one element each
  const int64_t i = nvec * kPerVec + threadIdx.x;
  if (blockIdx.x == 0 && i < n) {
    const T xa = ap ? static_cast<const T *>(ap)[i] : sa;
    const T ya = bp ? static_cast<const T *>(bp)[i] : sb;
    if constexpr (KIND == kOpCompare) static_cast<uint8_t *>(outp)[i] = compare_elem<DT>(fn, xa, ya) ? 1 : 0;
    else static_cast<T *>(outp)[i] = static_cast<const uint8_t *>(cp)[i] ? xa : ya;
  }
}

// ------------------------------------------------------------------ host dispatch
bool fn_is_valid(int kind, int fn, int dt) {
  const bool f = dtype_is_float(dt);
  if (kind == kOpUnary) {
    if (f) {
      switch (fn) {
        case BSIR_UNARY_VNOT: case BSIR_UNARY_ABSI: return false;
        default: return (fn >= 0 && fn <= 26) || (fn >= 100 && fn <= 112);
      }
    }
    return fn == BSIR_UNARY_RELU || fn == BSIR_UNARY_VNOT || fn == BSIR_UNARY_ABSI || fn == BSIR_UNARY_ABS ||
           fn == BSIR_UNARY_SQUARE;
  }
  if (kind == kOpBinary) {
    if (f) {
      switch (fn) {
        case BSIR_BINARY_ADD: case BSIR_BINARY_SUB: case BSIR_BINARY_MUL: case BSIR_BINARY_DIV:
        case BSIR_BINARY_DIVFHP: case BSIR_BINARY_MAXF: case BSIR_BINARY_MINF: case BSIR_BINARY_MAXNUMF:
        case BSIR_BINARY_MINNUMF: case BSIR_BINARY_POWF: case BSIR_BINARY_POWF_L: case BSIR_BINARY_MOD:
        case BSIR_BINARY_MODUI: case BSIR_BINARY_LDEXP: case BSIR_BINARY_ATAN2: case BSIR_BINARY_COPYSIGN:
        case BSIR_BINARY_MAX_SIGNED: case BSIR_BINARY_MIN_SIGNED: case BSIR_BINARY_MAX_UNSIGNED:
        case BSIR_BINARY_MIN_UNSIGNED:
          return true;
        default: return false;
      }
    }
    switch (fn) {
      case BSIR_BINARY_VOR: case BSIR_BINARY_VAND: case BSIR_BINARY_VXOR: case BSIR_BINARY_ADD:
      case BSIR_BINARY_SUB: case BSIR_BINARY_MUL: case BSIR_BINARY_DIV: case BSIR_BINARY_DIV_UNSIGNED:
      case BSIR_BINARY_MAX_SIGNED: case BSIR_BINARY_MIN_SIGNED: case BSIR_BINARY_MAX_UNSIGNED:
      case BSIR_BINARY_MIN_UNSIGNED: case BSIR_BINARY_MOD: case BSIR_BINARY_MODUI: case BSIR_BINARY_SHLI:
      case BSIR_BINARY_SHRSI: case BSIR_BINARY_SHRUI: case BSIR_BINARY_CEILDIVSI: case BSIR_BINARY_CEILDIVUI:
      case BSIR_BINARY_FLOORDIVSI: case BSIR_BINARY_POWI:
        return true;
      default: return false;
    }
  }
  if (kind == kOpCompare) return f ? (fn >= BSIR_CMP_VEQ && fn <= BSIR_CMP_VGT) : (fn >= BSIR_CMP_VEQ && fn <= BSIR_CMP_VUGT);
  return true;
}

struct Prepared {
  Shape sh;
  int64_t os[3];
  bool out_contig;
};

int32_t prepare(const char *what, int32_t rank, const int64_t *sizes, const int64_t *out_strides, Prepared *p) {
  if (rank < 1 || rank > 3) return fail(BSIR_ERR_SHAPE, "%s: rank %d (1..3 supported)", what, rank);
  if (!sizes) return fail(BSIR_ERR_NULL, "%s: sizes is null", what);
  int64_t n[3] = {1, 1, 1};
  int64_t os[3] = {0, 0, 0};
  for (int i = 0; i < rank; ++i) {
    if (sizes[i] < 0) return fail(BSIR_ERR_SHAPE, "%s: sizes[%d] = %lld", what, i, (long long)sizes[i]);
    n[3 - rank + i] = sizes[i];
  }
  int64_t cs = 1;
  bool contig = true;
  for (int i = rank - 1; i >= 0; --i) {
    const int64_t s = out_strides ? out_strides[i] : cs;
    os[3 - rank + i] = s;
    if (sizes[i] != 1 && s != cs) contig = false;
    cs *= sizes[i];
  }
  p->sh = Shape{n[0], n[1], n[2], n[0] * n[1] * n[2]};
  p->os[0] = os[0]; p->os[1] = os[1]; p->os[2] = os[2];
  p->out_contig = contig;
  return BSIR_OK;
}

// Right-aligns an operand's strides to rank 3; reports whether it is contiguous over `sizes`.
Operand make_operand(const bsir_operand *o, int32_t rank, const int64_t *sizes, bool *contig) {
  Operand r{o->data, 0, 0, 0, o->scalar_bits};
  int64_t s[3] = {0, 0, 0};
  int64_t cs = 1;
  bool c = true;
  for (int i = rank - 1; i >= 0; --i) {
    s[3 - rank + i] = o->strides[i];
    if (sizes[i] != 1 && o->strides[i] != cs) c = false;
    cs *= sizes[i];
  }
  r.s0 = s[0]; r.s1 = s[1]; r.s2 = s[2];
  *contig = c || o->data == nullptr;
  return r;
}

template <int KIND, int DT>
int32_t launch_typed(const char *what, int fn, const Prepared &p, const Operand &a, bool a_c, const Operand &b,
                     bool b_c, const Operand &c, void *out, cudaStream_t st) {
  using T = typename CType<DT>::type;
  const int64_t n = p.sh.total;
  if (n == 0) return BSIR_OK;
  const bool can_stream = (KIND == kOpUnary || KIND == kOpBinary || KIND == kOpCopy) && p.out_contig && a_c &&
                          (KIND != kOpBinary || b_c) && aligned_to(out, 16) && (!a.p || aligned_to(a.p, 16)) &&
                          (KIND != kOpBinary || !b.p || aligned_to(b.p, 16)) &&
                          !(KIND == kOpBinary && !a.p && !b.p) && !(KIND != kOpBinary && !a.p);
  if constexpr (KIND == kOpUnary || KIND == kOpBinary || KIND == kOpCopy) {
    if (can_stream) {
      constexpr int kPerVec = 16 / sizeof(T);
      const int64_t nvec = n / kPerVec;
      int64_t blocks = ceil_div(nvec, kStreamThreads * kStreamUnroll);
      if (blocks < 1) blocks = 1;
      launch_pdl(stream_kernel<DT, KIND>, dim3(static_cast<unsigned>(blocks)), dim3(kStreamThreads), 0, st, fn, n, a.p,
                 KIND == kOpBinary ? b.p : nullptr, a.scalar, b.scalar, out);
      count_launch();
      return check_launch(what);
    }
  }
  if constexpr (KIND == kOpCompare || KIND == kOpSelect) {
    // compare: a, b are the values; select: a is the condition (bool bytes), b and c the values
    constexpr int kPerVec = 16 / sizeof(T);
    auto dense = [&](const Operand &o) {
      if (!o.p) return true;
      return (p.sh.n2 == 1 || o.s2 == 1) && (p.sh.n1 == 1 || o.s1 == p.sh.n2) && (p.sh.n0 == 1 || o.s0 == p.sh.n1 * p.sh.n2);
    };
    const Operand &x = KIND == kOpCompare ? a : b;
    const Operand &y = KIND == kOpCompare ? b : c;
    const bool ok = p.out_contig && dense(x) && dense(y) && (x.p || y.p) && (!x.p || aligned_to(x.p, 16)) &&
                    (!y.p || aligned_to(y.p, 16)) &&
                    (KIND == kOpCompare ? aligned_to(out, kPerVec)
                                        : (a.p && dense(a) && aligned_to(a.p, kPerVec) && aligned_to(out, 16)));
    if (ok) {
      int64_t blocks = ceil_div(n / kPerVec, kStreamThreads * kStreamUnroll);
      if (blocks < 1) blocks = 1;
      cmpsel_stream_kernel<DT, KIND><<<static_cast<unsigned>(blocks), kStreamThreads, 0, st>>>(
          fn, n, x.p, y.p, KIND == kOpSelect ? a.p : nullptr, x.scalar, y.scalar, out);
      count_launch();
      return check_launch(what);
    }
  }
  int bx = 256;                                  // threads along the innermost dimension
  while (bx > 1 && bx / 2 >= p.sh.n2) bx >>= 1;
  const int by = 256 / bx;
  int64_t gx = ceil_div(p.sh.n2, static_cast<int64_t>(bx) * kIdxUnroll), gy = ceil_div(p.sh.n0 * p.sh.n1, by);
  if (gx > 0x7fffffffLL) gx = 0x7fffffffLL;     // the kernel loops over what the grid does not cover
  if (gy > 65535) gy = 65535;
  indexed_kernel<DT, KIND><<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy)), dim3(bx, by), 0, st>>>(
      fn, p.sh, a, b, c, out, p.os[0], p.os[1], p.os[2], nullptr);
  count_launch();
  return check_launch(what);
}

template <int KIND>
int32_t launch_by_dtype(const char *what, int fn, int dt, const Prepared &p, const Operand &a, bool a_c,
                        const Operand &b, bool b_c, const Operand &c, void *out, cudaStream_t st) {
#define D(code) \
  case code: return launch_typed<KIND, code>(what, fn, p, a, a_c, b, b_c, c, out, st);
  switch (dt) {
    D(BSIR_F32) D(BSIR_F16) D(BSIR_BF16) D(BSIR_I8) D(BSIR_I16) D(BSIR_I32) D(BSIR_I64) D(BSIR_U8) D(BSIR_U16)
    D(BSIR_U32) D(BSIR_U64) D(BSIR_BOOL)
    default: return fail(BSIR_ERR_DTYPE, "%s: dtype %d", what, dt);
  }
#undef D
}

// Bitwise ops on float storage act on the raw bits (as the device library's vnot/vand/vor do:
// bishengir/lib/Template/lib/Vector/Elementwise/EltWise1D.cpp:1300-1316).
int bits_dtype(int dt) { return dt == BSIR_F32 ? BSIR_U32 : (dt == BSIR_F16 || dt == BSIR_BF16) ? BSIR_U16 : dt; }

bool check_align(const void *p, int dt) { return p == nullptr || aligned_to(p, static_cast<size_t>(dtype_bytes(dt))); }

}  // namespace
}  // namespace bsir

namespace bsir {
// rows_kernel with an outer index (problems [n0, n1, cols] whose operands do not collapse to [n0 * n1, cols]): defined in
// elementwise_rows_outer.cu.  kind: kOpUnary / kOpBinary / kOpCopy; ka, kb: the operand kinds.
int32_t launch_rows_outer(int kind, int ka, int kb, int fn, int dt, int64_t rows, int64_t n1, int64_t vpr, const RowsOperand &a,
                          const RowsOperand &b, void *out, int64_t out_rs, int64_t out_os, cudaStream_t st);
}

#ifdef BSIR_ELEMENTWISE_PART_OUTER
namespace bsir {
namespace {
template <int KIND, int KA, int KB>
int32_t launch_rows_outer_t(int fn, int dt, int64_t rows, int64_t n1, int64_t vpr, const RowsOperand &a, const RowsOperand &b, void *out,
                            int64_t out_rs, int64_t out_os, cudaStream_t st) {
  const int64_t total = rows * vpr;
  const unsigned grid = static_cast<unsigned>(ceil_div(total, static_cast<int64_t>(kStreamThreads) * kStreamUnroll));
#define D(code) \
  case code: launch_pdl(rows_kernel<code, KIND, KA, KB, true>, dim3(grid), dim3(kStreamThreads), 0, st, fn, rows, n1, vpr, a, b, out, out_rs, out_os); break;
  if constexpr (KIND == kOpCopy) {
    switch (dt) {
      D(BSIR_U8) D(BSIR_U16) D(BSIR_U32) D(BSIR_U64)
      default: return fail(BSIR_ERR_DTYPE, "copy: dtype %d", dt);
    }
  } else {
    switch (dt) {
      D(BSIR_F32) D(BSIR_F16) D(BSIR_BF16) D(BSIR_I8) D(BSIR_I16) D(BSIR_I32) D(BSIR_I64) D(BSIR_U8) D(BSIR_U16)
      D(BSIR_U32) D(BSIR_U64) D(BSIR_BOOL)
      default: return fail(BSIR_ERR_DTYPE, "elemwise: dtype %d", dt);
    }
  }
#undef D
  count_launch();
  return check_launch("elemwise (rows)");
}
}  // namespace

int32_t launch_rows_outer(int kind, int ka, int kb, int fn, int dt, int64_t rows, int64_t n1, int64_t vpr, const RowsOperand &a,
                          const RowsOperand &b, void *out, int64_t out_rs, int64_t out_os, cudaStream_t st) {
#define R(K, A, B) return launch_rows_outer_t<K, A, B>(fn, dt, rows, n1, vpr, a, b, out, out_rs, out_os, st)
  if (kind == kOpCopy) { if (ka == 0) R(kOpCopy, 0, 0); if (ka == 1) R(kOpCopy, 1, 0); R(kOpCopy, 2, 0); }
  if (kind == kOpUnary) { if (ka == 0) R(kOpUnary, 0, 0); if (ka == 1) R(kOpUnary, 1, 0); R(kOpUnary, 2, 0); }
  if (ka == 0 && kb == 0) R(kOpBinary, 0, 0);
  if (ka == 0 && kb == 1) R(kOpBinary, 0, 1);
  if (ka == 0 && kb == 2) R(kOpBinary, 0, 2);
  if (ka == 1 && kb == 2) R(kOpBinary, 1, 2);
  if (ka == 2 && kb == 1) R(kOpBinary, 2, 1);
  if (ka == 1) R(kOpBinary, 1, 0);
  R(kOpBinary, 2, 0);
#undef R
}
}  // namespace bsir
#else

namespace bsir {
bool launch_transpose(int elem_bytes, const void *src, void *dst, int64_t batch, int64_t rows, int64_t cols, int64_t src_row,
                      int64_t dst_row, int64_t src_batch, int64_t dst_batch, cudaStream_t st);
}
using namespace bsir;

extern "C" {

namespace {
bool try_rows_route(int kind, int fn, int dtype, const Prepared &p, const Operand &a, const Operand &b, void *out, void *stream,
                    int32_t *rc);
}

int32_t bsir_elemwise_unary(int32_t fn, int32_t dtype, int32_t rank, const int64_t *sizes, const bsir_operand *x,
                            void *out, const int64_t *out_strides, void *stream) {
  clear_error();
  if (!x) return fail(BSIR_ERR_NULL, "elemwise_unary: null operand");
  if (dtype_bytes(dtype) == 0) return fail(BSIR_ERR_DTYPE, "elemwise_unary: dtype %d", dtype);
  if (fn == BSIR_UNARY_VNOT) dtype = bits_dtype(dtype);
  if (!fn_is_valid(kOpUnary, fn, dtype))
    return fail(BSIR_ERR_ATTR, "elemwise_unary: fn %d is not defined for dtype %d", fn, dtype);
  if (!check_align(x->data, dtype) || !check_align(out, dtype)) return fail(BSIR_ERR_ALIGN, "elemwise_unary: misaligned");
  Prepared p;
  if (int32_t rc = prepare("elemwise_unary", rank, sizes, out_strides, &p)) return rc;
  if (p.sh.total == 0) return BSIR_OK;
  if (!out || !x->data) return fail(BSIR_ERR_NULL, "elemwise_unary: null operand");
  bool ac;
  Operand a = make_operand(x, rank, sizes, &ac), none{nullptr, 0, 0, 0, 0};
  int32_t rc = BSIR_OK;
  if (!(ac && p.out_contig) && try_rows_route(kOpUnary, fn, dtype, p, a, none, out, stream, &rc)) return rc;
  return launch_by_dtype<kOpUnary>("elemwise_unary", fn, dtype, p, a, ac, none, true, none, out, resolve_stream(stream));
}

namespace {

// Unary / binary ops whose operands are row-strided views, or per-column / per-row vectors (bias add, per-row
// scale, slices of a wider tensor): rows_kernel moves 16-byte vectors where the indexed kernel moves elements.
// false: not such a pattern (the caller goes on with the indexed kernel).
extern "C++" {
template <int KIND, int KA, int KB>
int32_t launch_rows(int fn, int dt, int64_t rows, int64_t n1, int64_t vpr, const RowsOperand &a, const RowsOperand &b, void *out,
                    int64_t out_rs, int64_t out_os, cudaStream_t st) {
  if (n1 < rows) return launch_rows_outer(KIND, KA, KB, fn, dt, rows, n1, vpr, a, b, out, out_rs, out_os, st);   // the other translation unit
  const int64_t total = rows * vpr;
  const unsigned grid = static_cast<unsigned>(ceil_div(total, static_cast<int64_t>(kStreamThreads) * kStreamUnroll));
#define D(code) \
  case code: launch_pdl(rows_kernel<code, KIND, KA, KB, false>, dim3(grid), dim3(kStreamThreads), 0, st, fn, rows, n1, vpr, a, b, out, out_rs, out_os); break;
  if constexpr (KIND == kOpCopy) {        // a copy moves bits: the callers pass the unsigned type of the element's width
    switch (dt) {
      D(BSIR_U8) D(BSIR_U16) D(BSIR_U32) D(BSIR_U64)
      default: return fail(BSIR_ERR_DTYPE, "copy: dtype %d", dt);
    }
  } else {
    switch (dt) {
      D(BSIR_F32) D(BSIR_F16) D(BSIR_BF16) D(BSIR_I8) D(BSIR_I16) D(BSIR_I32) D(BSIR_I64) D(BSIR_U8) D(BSIR_U16)
      D(BSIR_U32) D(BSIR_U64) D(BSIR_BOOL)
      default: return fail(BSIR_ERR_DTYPE, "elemwise: dtype %d", dt);
    }
  }
#undef D
  count_launch();
  return check_launch("elemwise (rows)");
}
}  // extern "C++"

bool try_rows_route(int kind, int fn, int dtype, const Prepared &p, const Operand &a, const Operand &b, void *out, void *stream,
                    int32_t *rc) {
  const bool binary = kind == kOpBinary;
  // [n0, n1, cols] with rows = n0 * n1; a problem without a middle axis is [1, n0, cols]
  int64_t n0 = p.sh.n0, n1 = p.sh.n1;
  const int64_t cols = p.sh.n2, rows = n0 * n1;
  const bool fold = n1 == 1;                                           // then every operand's s1 is its s0
  if (fold) { n1 = n0; n0 = 1; }
  const int eb = dtype_bytes(dtype);
  const int per_vec = 16 / eb;
  if (rows < 2 || cols < per_vec || cols % per_vec || rows * (cols / per_vec) >= (int64_t(1) << 40)) return false;   // ragged rows keep the indexed kernel
  struct View { int kind; int64_t rs, os; };
  // strides between rows (of one outer index) and between outer indices, 0 where the axis has one element
  auto strides = [&](int64_t s0, int64_t s1, int64_t *rs, int64_t *os) {
    *rs = n1 == 1 ? 0 : (fold ? s0 : s1);
    *os = n0 == 1 ? 0 : s0;
  };
  auto vector_rows = [&](const void *ptr, int64_t rs, int64_t os) {     // every row starts on a 16-byte boundary
    return aligned_to(ptr, 16) && (rs * eb) % 16 == 0 && (os * eb) % 16 == 0;
  };
  // 0 full, 1 one vector for the rows of an outer index, 2 one value per row, -1 none of these
  auto classify = [&](const Operand &o) -> View {
    if (!o.p) return {-1, 0, 0};                                        // an immediate: the indexed kernel
    int64_t rs, os;
    strides(o.s0, o.s1, &rs, &os);
    if (o.s2 == 0) return {2, rs, os};
    if (o.s2 != 1 || !vector_rows(o.p, rs, os)) return {-1, 0, 0};
    if (rs == 0 && n1 > 1) return {1, 0, os};
    if (rs < cols && n1 > 1) return {-1, 0, 0};                          // overlapping rows: not a tensor view
    return {0, rs, os};
  };
  int64_t out_rs, out_os;
  strides(p.os[0], p.os[1], &out_rs, &out_os);
  if (p.os[2] != 1 || !vector_rows(out, out_rs, out_os) || (n1 > 1 && out_rs < cols) || (n0 > 1 && out_os < n1 * out_rs)) return false;
  const View va = classify(a), vb = binary ? classify(b) : View{0, 0, 0};
  const int ka = va.kind, kb = vb.kind;
  if (ka < 0 || kb < 0) return false;
  if (ka != 0 && kb != 0 && !(ka + kb == 3)) return false;             // two broadcast operands: a row vector against values per row (an outer sum)
  // the outer index matters only to an operand (or a result) whose outer stride is not n1 row strides
  auto collapses = [&](int64_t rs, int64_t os) { return n0 == 1 || os == n1 * rs; };
  const bool outer = !(collapses(out_rs, out_os) && collapses(va.rs, va.os) && (!binary || collapses(vb.rs, vb.os)));
  const int64_t n1k = outer ? n1 : rows;
  const RowsOperand oa{a.p, va.rs, outer ? va.os : 0, ka}, ob{b.p, vb.rs, outer ? vb.os : 0, kb};
  if (!outer) out_os = 0;
  cudaStream_t st = resolve_stream(stream);
  const int64_t vpr = cols / per_vec;
  if (kind == kOpCopy) {
    if (ka == 0) *rc = launch_rows<kOpCopy, 0, 0>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
    else if (ka == 1) *rc = launch_rows<kOpCopy, 1, 0>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
    else *rc = launch_rows<kOpCopy, 2, 0>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
  } else if (!binary) {
    if (ka == 0) *rc = launch_rows<kOpUnary, 0, 0>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
    else if (ka == 1) *rc = launch_rows<kOpUnary, 1, 0>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
    else *rc = launch_rows<kOpUnary, 2, 0>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
  } else if (ka == 0 && kb == 0) *rc = launch_rows<kOpBinary, 0, 0>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
  else if (ka == 0 && kb == 1) *rc = launch_rows<kOpBinary, 0, 1>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
  else if (ka == 0 && kb == 2) *rc = launch_rows<kOpBinary, 0, 2>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
  else if (ka == 1 && kb == 2) *rc = launch_rows<kOpBinary, 1, 2>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
  else if (ka == 2 && kb == 1) *rc = launch_rows<kOpBinary, 2, 1>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
  else if (ka == 1) *rc = launch_rows<kOpBinary, 1, 0>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
  else *rc = launch_rows<kOpBinary, 2, 0>(fn, dtype, rows, n1k, vpr, oa, ob, out, out_rs, out_os, st);
  return true;
}

}  // namespace

int32_t bsir_elemwise_binary(int32_t fn, int32_t dtype, int32_t rank, const int64_t *sizes, const bsir_operand *a,
                             const bsir_operand *b, void *out, const int64_t *out_strides, void *stream) {
  clear_error();
  if (!a || !b) return fail(BSIR_ERR_NULL, "elemwise_binary: null operand");
  if (dtype_bytes(dtype) == 0) return fail(BSIR_ERR_DTYPE, "elemwise_binary: dtype %d", dtype);
  if (fn == BSIR_BINARY_VAND || fn == BSIR_BINARY_VOR || fn == BSIR_BINARY_VXOR) dtype = bits_dtype(dtype);
  if (!fn_is_valid(kOpBinary, fn, dtype))
    return fail(BSIR_ERR_ATTR, "elemwise_binary: fn %d is not defined for dtype %d", fn, dtype);
  if (!check_align(a->data, dtype) || !check_align(b->data, dtype) || !check_align(out, dtype))
    return fail(BSIR_ERR_ALIGN, "elemwise_binary: misaligned");
  Prepared p;
  if (int32_t rc = prepare("elemwise_binary", rank, sizes, out_strides, &p)) return rc;
  if (p.sh.total == 0) return BSIR_OK;
  if (!out) return fail(BSIR_ERR_NULL, "elemwise_binary: null result");
  bool ac, bc;
  Operand oa = make_operand(a, rank, sizes, &ac), ob = make_operand(b, rank, sizes, &bc), none{nullptr, 0, 0, 0, 0};
  int32_t rc = BSIR_OK;
  if (!(ac && bc && p.out_contig) && try_rows_route(kOpBinary, fn, dtype, p, oa, ob, out, stream, &rc)) return rc;
  return launch_by_dtype<kOpBinary>("elemwise_binary", fn, dtype, p, oa, ac, ob, bc, none, out, resolve_stream(stream));
}

int32_t bsir_compare(int32_t fn, int32_t dtype, int32_t rank, const int64_t *sizes, const bsir_operand *a,
                     const bsir_operand *b, void *out, const int64_t *out_strides, void *stream) {
  clear_error();
  if (!a || !b) return fail(BSIR_ERR_NULL, "compare: null operand");
  if (dtype_bytes(dtype) == 0) return fail(BSIR_ERR_DTYPE, "compare: dtype %d", dtype);
  if (!fn_is_valid(kOpCompare, fn, dtype)) return fail(BSIR_ERR_ATTR, "compare: fn %d for dtype %d", fn, dtype);
  if (!check_align(a->data, dtype) || !check_align(b->data, dtype)) return fail(BSIR_ERR_ALIGN, "compare: misaligned");
  Prepared p;
  if (int32_t rc = prepare("compare", rank, sizes, out_strides, &p)) return rc;
  if (p.sh.total == 0) return BSIR_OK;
  if (!out) return fail(BSIR_ERR_NULL, "compare: null result");
  bool ac, bc;
  Operand oa = make_operand(a, rank, sizes, &ac), ob = make_operand(b, rank, sizes, &bc), none{nullptr, 0, 0, 0, 0};
  return launch_by_dtype<kOpCompare>("compare", fn, dtype, p, oa, ac, ob, bc, none, out, resolve_stream(stream));
}

int32_t bsir_select(int32_t dtype, int32_t rank, const int64_t *sizes, const bsir_operand *cond, const bsir_operand *a,
                    const bsir_operand *b, void *out, const int64_t *out_strides, void *stream) {
  clear_error();
  if (!cond || !a || !b) return fail(BSIR_ERR_NULL, "select: null operand");
  if (dtype_bytes(dtype) == 0) return fail(BSIR_ERR_DTYPE, "select: dtype %d", dtype);
  if (!check_align(a->data, dtype) || !check_align(b->data, dtype) || !check_align(out, dtype))
    return fail(BSIR_ERR_ALIGN, "select: misaligned");
  Prepared p;
  if (int32_t rc = prepare("select", rank, sizes, out_strides, &p)) return rc;
  if (p.sh.total == 0) return BSIR_OK;
  if (!out || !cond->data) return fail(BSIR_ERR_NULL, "select: null pointer");
  bool cc, ac, bc;
  Operand oc = make_operand(cond, rank, sizes, &cc), oa = make_operand(a, rank, sizes, &ac),
          ob = make_operand(b, rank, sizes, &bc);
  // select moves bits: use the same-size unsigned type
  const int dt = dtype_bytes(dtype) == 8 ? BSIR_U64 : dtype_bytes(dtype) == 4 ? BSIR_U32 : dtype_bytes(dtype) == 2 ? BSIR_U16 : BSIR_U8;
  return launch_by_dtype<kOpSelect>("select", 0, dt, p, oc, cc, oa, ac, ob, out, resolve_stream(stream));
}

int32_t bsir_copy(int32_t dtype, int32_t rank, const int64_t *sizes, const void *src, const int64_t *src_strides,
                  void *dst, const int64_t *dst_strides, void *stream) {
  clear_error();
  if (dtype_bytes(dtype) == 0) return fail(BSIR_ERR_DTYPE, "copy: dtype %d", dtype);
  if (!check_align(src, dtype) || !check_align(dst, dtype)) return fail(BSIR_ERR_ALIGN, "copy: misaligned");
  Prepared p;
  if (int32_t rc = prepare("copy", rank, sizes, dst_strides, &p)) return rc;
  if (p.sh.total == 0) return BSIR_OK;
  if (!src || !dst) return fail(BSIR_ERR_NULL, "copy: null pointer");
  bsir_operand s{src, {0, 0, 0}, 0};
  int64_t cs = 1;
  for (int i = rank - 1; i >= 0; --i) { s.strides[i] = src_strides ? src_strides[i] : cs; cs *= sizes[i]; }
  if (rank >= 2) {
    // A source that is a transposed view of the last two axes (hivm.hir.vtranspose / linalg.transpose arrive
    // like this): the tiled kernel instead of an element-wise strided copy.
    const int64_t ni = sizes[rank - 2], nj = sizes[rank - 1], nb = rank == 3 ? sizes[0] : 1;
    const int64_t dj = p.os[2], di = p.os[1], db = rank == 3 ? p.os[0] : 0;
    const int64_t si = s.strides[rank - 2], sj = s.strides[rank - 1], sb = rank == 3 ? s.strides[0] : 0;
    if (ni > 1 && nj > 1 && dj == 1 && si == 1 && sj >= ni && di >= nj &&
        launch_transpose(dtype_bytes(dtype), src, dst, nb, /*rows=*/nj, /*cols=*/ni, sj, di, sb, db, resolve_stream(stream))) {
      count_launch();
      return check_launch("copy");
    }
  }
  bool ac;
  Operand oa = make_operand(&s, rank, sizes, &ac), none{nullptr, 0, 0, 0, 0};
  const int dt = dtype_bytes(dtype) == 8 ? BSIR_U64 : dtype_bytes(dtype) == 4 ? BSIR_U32 : dtype_bytes(dtype) == 2 ? BSIR_U16 : BSIR_U8;
  // row-strided views (slices of a wider tensor, a destination with padded rows) and broadcasts of a row, a column or
  // one element (hivm.hir.vbrc arrives as a copy from a stride-0 view): 16-byte vectors through rows_kernel
  int32_t rc = BSIR_OK;
  if (!(ac && p.out_contig) && try_rows_route(kOpCopy, 0, dt, p, oa, none, dst, stream, &rc)) return rc;
  return launch_by_dtype<kOpCopy>("copy", 0, dt, p, oa, ac, none, true, none, dst, resolve_stream(stream));
}

}  // extern "C"

#endif  // BSIR_ELEMENTWISE_PART_OUTER
