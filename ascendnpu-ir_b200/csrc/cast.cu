// cast.cu -- hfusion.cast / hivm.hir.vcast: element type conversion under a round_mode with
// optional saturation (bishengir/include/bishengir/Dialect/HFusion/IR/HFusionNamedStructuredOps.yaml:373-432;
// round modes bishengir/include/bishengir/Dialect/HFusion/IR/HFusionEnums.td:122-141; the host
// constant folder gives the exact per-mode results, bishengir/lib/Dialect/HFusion/IR/HFusionOps.cpp:1951-1994).
//
// Every element goes source type -> (f32 | i64) -> destination type with a single rounding:
//   float -> float : narrowing rounds by mode; widening is exact; same type rounds to an integral value
//   float -> int   : round by mode in f32, then saturate (NaN -> 0) or keep the low bits
//   int   -> float : one rounding from the exact integer
//   int   -> int   : saturate or wrap
// The contiguous path moves 16-byte vectors of the wider of the two types.
#include <climits>
#include <type_traits>

#include "common.cuh"

namespace bsir {
namespace {

template <int DT> struct CT;
template <> struct CT<BSIR_F32> { using type = float; };
template <> struct CT<BSIR_F16> { using type = uint16_t; };
template <> struct CT<BSIR_BF16> { using type = uint16_t; };
template <> struct CT<BSIR_I8> { using type = int8_t; };
template <> struct CT<BSIR_I16> { using type = int16_t; };
template <> struct CT<BSIR_I32> { using type = int32_t; };
template <> struct CT<BSIR_I64> { using type = int64_t; };
template <> struct CT<BSIR_U8> { using type = uint8_t; };
template <> struct CT<BSIR_U16> { using type = uint16_t; };
template <> struct CT<BSIR_U32> { using type = uint32_t; };
template <> struct CT<BSIR_U64> { using type = uint64_t; };
template <> struct CT<BSIR_BOOL> { using type = uint8_t; };

template <int DT> constexpr bool is_f() { return DT == BSIR_F32 || DT == BSIR_F16 || DT == BSIR_BF16; }
template <int DT> constexpr bool is_u() { return DT >= BSIR_U8; }
template <int DT> constexpr int bits_of() { return DT == BSIR_BOOL ? 1 : 8 * static_cast<int>(sizeof(typename CT<DT>::type)); }

__device__ __forceinline__ float round_integral(float x, int mode) {
  switch (mode) {
    case BSIR_ROUND_RINT: return rintf(x);
    case BSIR_ROUND_ROUND: return roundf(x);
    case BSIR_ROUND_FLOOR: return floorf(x);
    case BSIR_ROUND_CEIL: return ceilf(x);
    case BSIR_ROUND_ODD: {
      const float t = truncf(x);
      if (t == x || x != x) return x;
      return (fmodf(t, 2.0f) == 0.0f) ? t + (x > 0.0f ? 1.0f : -1.0f) : t;
    }
    default: return truncf(x);
  }
}

// f32 -> 16-bit float storage under a rounding mode.  HALF selects f16 (else bf16).
template <bool HALF>
__device__ __forceinline__ uint16_t narrow_float(float x, int mode) {
  auto cv = [](float v, int dir) -> uint16_t {  // dir: 0 rn, 1 rz, 2 rd, 3 ru
    if constexpr (HALF) {
      switch (dir) {
        case 0: return __half_as_ushort(__float2half_rn(v));
        case 1: return __half_as_ushort(__float2half_rz(v));
        case 2: return __half_as_ushort(__float2half_rd(v));
        default: return __half_as_ushort(__float2half_ru(v));
      }
    } else {
      switch (dir) {
        case 0: return __bfloat16_as_ushort(__float2bfloat16_rn(v));
        case 1: return __bfloat16_as_ushort(__float2bfloat16_rz(v));
        case 2: return __bfloat16_as_ushort(__float2bfloat16_rd(v));
        default: return __bfloat16_as_ushort(__float2bfloat16_ru(v));
      }
    }
  };
  auto widen = [](uint16_t b) -> float {
    if constexpr (HALF) return __half2float(__ushort_as_half(b));
    else return __uint_as_float(static_cast<uint32_t>(b) << 16);
  };
  switch (mode) {
    case BSIR_ROUND_RINT: return cv(x, 0);
    case BSIR_ROUND_FLOOR: return cv(x, 2);
    case BSIR_ROUND_CEIL: return cv(x, 3);
    case BSIR_ROUND_TRUNC: case BSIR_ROUND_TRUNCWITHOVERFLOW: return cv(x, 1);
    default: break;
  }
  if (x != x) return cv(x, 0);
  const uint16_t lo = cv(x, 2), hi = cv(x, 3);
  if (lo == hi) return lo;
  const float flo = widen(lo), fhi = widen(hi);
  if (mode == BSIR_ROUND_ROUND) {  // nearest, ties away from zero
    // next to the overflow threshold one neighbour is infinity: nearest-even already decides it
    // (the tie at the threshold goes to infinity under both rules)
    if (isinf(flo) || isinf(fhi)) return cv(x, 0);
    const float dl = x - flo, dh = fhi - x;
    if (dl < dh) return lo;
    if (dl > dh) return hi;
    return x > 0.0f ? hi : lo;
  }
  // round to odd: inexact results take the neighbour with an odd last bit
  if (isinf(flo)) return hi;
  if (isinf(fhi)) return lo;
  return (lo & 1u) ? lo : hi;
}

template <int SRC>
__device__ __forceinline__ float src_to_f32(typename CT<SRC>::type v) {
  if constexpr (SRC == BSIR_F32) return v;
  else if constexpr (SRC == BSIR_F16) return __half2float(__ushort_as_half(v));
  else return __uint_as_float(static_cast<uint32_t>(v) << 16);
}

// integral-valued f32 -> low 64 bits of the integer (two's complement), any magnitude
__device__ __forceinline__ unsigned long long f32_integral_to_bits(float r) {
  const float a = fabsf(r);
  if (!(a < 3.4028235e38f)) return 0ull;  // inf / NaN
  if (a < 2.1474836e9f) return static_cast<unsigned long long>(static_cast<long long>(__float2int_rz(r)));  // the common case: one 32-bit convert
  if (a < 9.2233720e18f) return static_cast<unsigned long long>(__float2ll_rz(r));
  const uint32_t u = __float_as_uint(a);
  const int sh = static_cast<int>(u >> 23) - 150;  // value = mant << sh, sh >= 40 here
  const unsigned long long mant = (u & 0x7fffffu) | 0x800000u;
  unsigned long long mag = sh >= 64 ? 0ull : (mant << sh);
  return r < 0.0f ? (0ull - mag) : mag;
}

template <int DST>
__device__ __forceinline__ typename CT<DST>::type float_to_int(float x, int mode, int overflow) {
  using T = typename CT<DST>::type;
  if (x != x) return T(0);
  if (overflow == BSIR_OVERFLOW_ASCEND_SATURATE_TRUNC_VIA_F16 || overflow == BSIR_OVERFLOW_ASCEND_DOUBLE_ROUND_VIA_F16) {
    const int m = overflow == BSIR_OVERFLOW_ASCEND_SATURATE_TRUNC_VIA_F16 ? BSIR_ROUND_TRUNC : mode;
    float h = __half2float(__ushort_as_half(narrow_float<true>(x, m)));
    if (isinf(h)) h = h > 0.0f ? 65504.0f : -65504.0f;
    x = h;
    mode = m;
    overflow = BSIR_OVERFLOW_SATURATE;
  }
  const float r = round_integral(x, mode);
  constexpr int kBits = bits_of<DST>();
  if (overflow == BSIR_OVERFLOW_SATURATE) {
    if constexpr (DST == BSIR_BOOL) return r >= 1.0f ? T(1) : T(0);
    else if constexpr (DST == BSIR_U64) return r <= 0.0f ? T(0) : static_cast<T>(__float2ull_rz(r));
    else if constexpr (DST == BSIR_I64) return static_cast<T>(__float2ll_rz(r));
    else if constexpr (kBits <= 32 && !is_u<DST>()) {
      // cvt.rzi.s32.f32 saturates at the int32 range, which contains every narrower range
      const int v = __float2int_rz(r);
      constexpr int lo = kBits == 32 ? INT_MIN : -(1 << (kBits - 1)), hi = kBits == 32 ? INT_MAX : (1 << (kBits - 1)) - 1;
      return static_cast<T>(v < lo ? lo : v > hi ? hi : v);
    } else if constexpr (kBits <= 32) {
      const unsigned v = __float2uint_rz(r);   // saturates at [0, 2^32 - 1]; negatives give 0
      constexpr unsigned hi = kBits == 32 ? 0xffffffffu : (1u << kBits) - 1u;
      return static_cast<T>(v > hi ? hi : v);
    } else if constexpr (is_u<DST>()) {
      const unsigned long long v = r <= 0.0f ? 0ull : __float2ull_rz(r);
      const unsigned long long hi = (1ull << kBits) - 1ull;
      return static_cast<T>(v > hi ? hi : v);
    } else {
      const long long v = __float2ll_rz(r);
      const long long lo = -(1ll << (kBits - 1)), hi = (1ll << (kBits - 1)) - 1;
      return static_cast<T>(v < lo ? lo : v > hi ? hi : v);
    }
  }
  const unsigned long long bits = f32_integral_to_bits(r);
  if constexpr (DST == BSIR_BOOL) return static_cast<T>(bits & 1ull);
  else return static_cast<T>(bits);
}

template <int SRC, int DST>
__device__ __forceinline__ typename CT<DST>::type convert(typename CT<SRC>::type v, int mode, int overflow) {
  using D = typename CT<DST>::type;
  if constexpr (is_f<SRC>() && is_f<DST>()) {
    const float x = src_to_f32<SRC>(v);
    if constexpr (SRC == DST) {
      const float r = round_integral(x, mode);
      if constexpr (DST == BSIR_F32) return r;
      else if constexpr (DST == BSIR_F16) return narrow_float<true>(r, BSIR_ROUND_RINT);
      else return narrow_float<false>(r, BSIR_ROUND_RINT);
    } else if constexpr (DST == BSIR_F32) {
      return x;
    } else if constexpr (DST == BSIR_F16) {
      return narrow_float<true>(x, mode);
    } else {
      return narrow_float<false>(x, mode);
    }
  } else if constexpr (is_f<SRC>()) {
    return float_to_int<DST>(src_to_f32<SRC>(v), mode, overflow);
  } else if constexpr (is_f<DST>()) {
    // exact integer -> f32 with one rounding; narrower float targets get a sticky bit first
    constexpr bool kU = is_u<SRC>();
    float f;
    if constexpr (DST == BSIR_F32) {
      const long long sv = static_cast<long long>(v);
      const unsigned long long uv = static_cast<unsigned long long>(v);
      switch (mode) {
        case BSIR_ROUND_FLOOR: f = kU ? __ull2float_rd(uv) : __ll2float_rd(sv); break;
        case BSIR_ROUND_CEIL: f = kU ? __ull2float_ru(uv) : __ll2float_ru(sv); break;
        case BSIR_ROUND_TRUNC: case BSIR_ROUND_TRUNCWITHOVERFLOW: f = kU ? __ull2float_rz(uv) : __ll2float_rz(sv); break;
        case BSIR_ROUND_ROUND: {
          const float lo = kU ? __ull2float_rd(uv) : __ll2float_rd(sv), hi = kU ? __ull2float_ru(uv) : __ll2float_ru(sv);
          if (lo == hi) { f = lo; break; }
          const double d = kU ? static_cast<double>(uv) : static_cast<double>(sv);  // exact below 2^53
          const double dl = d - static_cast<double>(lo), dh = static_cast<double>(hi) - d;
          f = dl < dh ? lo : dl > dh ? hi : (d > 0 ? hi : lo);
          break;
        }
        default: f = kU ? __ull2float_rn(uv) : __ll2float_rn(sv); break;
      }
      return f;
    } else {
      const long long sv = static_cast<long long>(v);
      const unsigned long long uv = static_cast<unsigned long long>(v);
      f = kU ? __ull2float_rz(uv) : __ll2float_rz(sv);
      const bool exact = kU ? (__float2ull_rz(f) == uv && f < 1.8446744e19f) : (__float2ll_rz(f) == sv && fabsf(f) < 9.2233720e18f);
      if (!exact) f = __uint_as_float(__float_as_uint(f) | 1u);  // sticky: no double rounding below
      if constexpr (DST == BSIR_F16) return narrow_float<true>(f, mode);
      else return narrow_float<false>(f, mode);
    }
  } else {
    constexpr int kBits = bits_of<DST>();
    if (overflow == BSIR_OVERFLOW_SATURATE) {
      if constexpr (is_u<SRC>()) {
        const unsigned long long uv = static_cast<unsigned long long>(v);
        const unsigned long long hi = is_u<DST>() ? (kBits == 64 ? ~0ull : (1ull << (kBits % 64)) - 1ull)
                                                  : (1ull << (kBits - 1)) - 1ull;
        return static_cast<D>(uv > hi ? hi : uv);
      } else {
        const long long sv = static_cast<long long>(v);
        if constexpr (is_u<DST>()) {
          if (sv < 0) return D(0);
          const unsigned long long hi = kBits == 64 ? ~0ull : (1ull << (kBits % 64)) - 1ull;
          return static_cast<D>(static_cast<unsigned long long>(sv) > hi ? hi : static_cast<unsigned long long>(sv));
        } else {
          const long long lo = kBits == 64 ? LLONG_MIN : -(1ll << (kBits - 1));
          const long long hi = kBits == 64 ? LLONG_MAX : (1ll << (kBits - 1)) - 1;
          return static_cast<D>(sv < lo ? lo : sv > hi ? hi : sv);
        }
      }
    }
    if constexpr (DST == BSIR_BOOL) return static_cast<D>(static_cast<unsigned long long>(v) & 1ull);
    else return static_cast<D>(v);
  }
}

struct CastShape {
  int64_t n0, n1, n2, total;
  int64_t ss0, ss1, ss2, ds0, ds1, ds2;
};

template <int SRC, int DST>
__global__ void __launch_bounds__(256) cast_indexed_kernel(CastShape sh, const void *__restrict__ src,
                                                           void *__restrict__ dst, int mode, int overflow) {
  using S = typename CT<SRC>::type;
  using D = typename CT<DST>::type;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= sh.total) return;
  const int64_t i2 = idx % sh.n2, t = idx / sh.n2, i1 = t % sh.n1, i0 = t / sh.n1;
  const S v = static_cast<const S *>(src)[i0 * sh.ss0 + i1 * sh.ss1 + i2 * sh.ss2];
  static_cast<D *>(dst)[i0 * sh.ds0 + i1 * sh.ds1 + i2 * sh.ds2] = convert<SRC, DST>(v, mode, overflow);
}

// Contiguous path: each thread converts `kElems` consecutive elements, where kElems fills a
// 16-byte vector of the wider type (the narrower side then moves 16 * narrow / wide bytes).
template <int SRC, int DST>
__global__ void __launch_bounds__(256) cast_stream_kernel(int64_t n, const void *__restrict__ src,
                                                          void *__restrict__ dst, int mode, int overflow) {
  using S = typename CT<SRC>::type;
  using D = typename CT<DST>::type;
  constexpr int kWide = sizeof(S) > sizeof(D) ? sizeof(S) : sizeof(D);
  constexpr int kElems = 16 / kWide;
  constexpr int kUnroll = 4;
  const int64_t ngroups = n / kElems;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (256 * kUnroll) + threadIdx.x;
  struct alignas(sizeof(S) * kElems) SV { S e[kElems]; };
  struct alignas(sizeof(D) * kElems) DV { D e[kElems]; };
  SV in[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t gidx = base + static_cast<int64_t>(u) * 256;
    if (gidx < ngroups) in[u] = static_cast<const SV *>(src)[gidx];
  }
  // With the attributes known at compile time the conversion folds to a few instructions; the usual
  // float -> integer combinations get their own copy of the loop, the rest share the general one.
  auto body = [&](auto mode_c, auto overflow_c) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t gidx = base + static_cast<int64_t>(u) * 256;
      if (gidx >= ngroups) continue;
      DV out;
#pragma unroll
      for (int e = 0; e < kElems; ++e) out.e[e] = convert<SRC, DST>(in[u].e[e], mode_c(), overflow_c());
      static_cast<DV *>(dst)[gidx] = out;
    }
  };
  constexpr bool kFloatToInt = (SRC == BSIR_F32 || SRC == BSIR_F16 || SRC == BSIR_BF16) &&
                               !(DST == BSIR_F32 || DST == BSIR_F16 || DST == BSIR_BF16);
  auto fixed = [](auto v) { return [v]() { return decltype(v)::value; }; };
  using std::integral_constant;
  bool done = false;
  if constexpr (kFloatToInt) {
    if (mode == BSIR_ROUND_RINT && overflow == BSIR_OVERFLOW_SATURATE) {
      body(fixed(integral_constant<int, BSIR_ROUND_RINT>{}), fixed(integral_constant<int, BSIR_OVERFLOW_SATURATE>{}));
      done = true;
    } else if (mode == BSIR_ROUND_RINT && overflow == BSIR_OVERFLOW_WRAP) {
      body(fixed(integral_constant<int, BSIR_ROUND_RINT>{}), fixed(integral_constant<int, BSIR_OVERFLOW_WRAP>{}));
      done = true;
    } else if (mode == BSIR_ROUND_TRUNC && overflow == BSIR_OVERFLOW_SATURATE) {
      body(fixed(integral_constant<int, BSIR_ROUND_TRUNC>{}), fixed(integral_constant<int, BSIR_OVERFLOW_SATURATE>{}));
      done = true;
    } else if (mode == BSIR_ROUND_TRUNC && overflow == BSIR_OVERFLOW_WRAP) {
      body(fixed(integral_constant<int, BSIR_ROUND_TRUNC>{}), fixed(integral_constant<int, BSIR_OVERFLOW_WRAP>{}));
      done = true;
    }
  }
  if constexpr (!kFloatToInt) {
    // round-to-nearest-even, the mode conversions between float types and from integers default to: known at
    // compile time the conversion is one instruction per element or pair
    if (mode == BSIR_ROUND_RINT) {
      body(fixed(integral_constant<int, BSIR_ROUND_RINT>{}), [overflow]() { return overflow; });
      done = true;
    }
  }
  if (!done) body([mode]() { return mode; }, [overflow]() { return overflow; });
  const int64_t tail0 = ngroups * kElems;
  if (blockIdx.x == 0 && tail0 + threadIdx.x < n)
    static_cast<D *>(dst)[tail0 + threadIdx.x] = convert<SRC, DST>(static_cast<const S *>(src)[tail0 + threadIdx.x], mode, overflow);
}

template <int SRC, int DST>
int32_t launch_cast(const CastShape &sh, bool contig, const void *src, void *dst, int mode, int overflow, cudaStream_t st) {
  using S = typename CT<SRC>::type;
  using D = typename CT<DST>::type;
  constexpr int kWide = sizeof(S) > sizeof(D) ? sizeof(S) : sizeof(D);
  constexpr int kElems = 16 / kWide;
  if (contig && aligned_to(src, sizeof(S) * kElems) && aligned_to(dst, sizeof(D) * kElems)) {
    int64_t blocks = ceil_div(sh.total / kElems, 256 * 4);
    if (blocks < 1) blocks = 1;
    cast_stream_kernel<SRC, DST><<<static_cast<unsigned>(blocks), 256, 0, st>>>(sh.total, src, dst, mode, overflow);
  } else {
    const int64_t blocks = ceil_div(sh.total, 256);
    if (blocks > 0x7fffffffLL) return fail(BSIR_ERR_SHAPE, "cast: too many elements for the indexed path");
    cast_indexed_kernel<SRC, DST><<<static_cast<unsigned>(blocks), 256, 0, st>>>(sh, src, dst, mode, overflow);
  }
  count_launch();
  return check_launch("cast");
}

}  // namespace
}  // namespace bsir

using namespace bsir;

// Legal (source, destination) pairs: the type table of hivm.hir.vcast
// (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:549-604) plus the pairs the
// library registers (bishengir/lib/Template/lib/Vector/Cast/Cast1D.cpp).
#define BSIR_CAST_PAIRS(X)                                                                                      \
  X(BSIR_F32, BSIR_F32) X(BSIR_F32, BSIR_F16) X(BSIR_F32, BSIR_BF16) X(BSIR_F32, BSIR_I64) X(BSIR_F32, BSIR_I32) \
  X(BSIR_F32, BSIR_I16) X(BSIR_F32, BSIR_I8) X(BSIR_F32, BSIR_U8) X(BSIR_F32, BSIR_BOOL)                         \
  X(BSIR_F16, BSIR_F16) X(BSIR_F16, BSIR_F32) X(BSIR_F16, BSIR_BF16) X(BSIR_F16, BSIR_I32) X(BSIR_F16, BSIR_I16) \
  X(BSIR_F16, BSIR_I8) X(BSIR_F16, BSIR_U8) X(BSIR_F16, BSIR_I64) X(BSIR_F16, BSIR_BOOL)                         \
  X(BSIR_BF16, BSIR_BF16) X(BSIR_BF16, BSIR_F32) X(BSIR_BF16, BSIR_F16) X(BSIR_BF16, BSIR_I32)                   \
  X(BSIR_BF16, BSIR_I16) X(BSIR_BF16, BSIR_I8) X(BSIR_BF16, BSIR_I64) X(BSIR_BF16, BSIR_BOOL)                    \
  X(BSIR_I8, BSIR_F16) X(BSIR_I8, BSIR_F32) X(BSIR_I8, BSIR_BF16) X(BSIR_I8, BSIR_I16) X(BSIR_I8, BSIR_I32)      \
  X(BSIR_I8, BSIR_I64) X(BSIR_I8, BSIR_BOOL)                                                                    \
  X(BSIR_U8, BSIR_F16) X(BSIR_U8, BSIR_F32) X(BSIR_U8, BSIR_BF16) X(BSIR_U8, BSIR_I16) X(BSIR_U8, BSIR_I32)      \
  X(BSIR_U8, BSIR_U16) X(BSIR_U8, BSIR_U32) X(BSIR_U8, BSIR_I64)                                                 \
  X(BSIR_I16, BSIR_F16) X(BSIR_I16, BSIR_F32) X(BSIR_I16, BSIR_BF16) X(BSIR_I16, BSIR_I8) X(BSIR_I16, BSIR_I32)  \
  X(BSIR_I16, BSIR_I64) X(BSIR_I16, BSIR_U8) X(BSIR_I16, BSIR_BOOL)                                              \
  X(BSIR_U16, BSIR_U8) X(BSIR_U16, BSIR_U32) X(BSIR_U16, BSIR_F32)                                               \
  X(BSIR_I32, BSIR_F32) X(BSIR_I32, BSIR_F16) X(BSIR_I32, BSIR_BF16) X(BSIR_I32, BSIR_I64) X(BSIR_I32, BSIR_I16) \
  X(BSIR_I32, BSIR_I8) X(BSIR_I32, BSIR_U8) X(BSIR_I32, BSIR_BOOL)                                               \
  X(BSIR_U32, BSIR_F32) X(BSIR_U32, BSIR_U16) X(BSIR_U32, BSIR_U8) X(BSIR_U32, BSIR_U64)                         \
  X(BSIR_I64, BSIR_I32) X(BSIR_I64, BSIR_I16) X(BSIR_I64, BSIR_I8) X(BSIR_I64, BSIR_F32) X(BSIR_I64, BSIR_F16)   \
  X(BSIR_I64, BSIR_BF16) X(BSIR_I64, BSIR_BOOL)                                                                  \
  X(BSIR_BOOL, BSIR_F16) X(BSIR_BOOL, BSIR_F32) X(BSIR_BOOL, BSIR_BF16) X(BSIR_BOOL, BSIR_I8)                    \
  X(BSIR_BOOL, BSIR_I16) X(BSIR_BOOL, BSIR_I32) X(BSIR_BOOL, BSIR_I64) X(BSIR_BOOL, BSIR_U8)                     \
  X(BSIR_BOOL, BSIR_U16) X(BSIR_BOOL, BSIR_U32)

extern "C" int32_t bsir_cast(int32_t src_dtype, int32_t dst_dtype, int32_t round_mode, int32_t overflow_mode,
                             int32_t rank, const int64_t *sizes, const void *src, const int64_t *src_strides,
                             void *dst, const int64_t *dst_strides, void *stream) {
  clear_error();
  if (dtype_bytes(src_dtype) == 0 || dtype_bytes(dst_dtype) == 0)
    return fail(BSIR_ERR_DTYPE, "cast: dtype %d -> %d", src_dtype, dst_dtype);
  if (round_mode < BSIR_ROUND_RINT || round_mode > BSIR_ROUND_TRUNCWITHOVERFLOW)
    return fail(BSIR_ERR_ATTR, "cast: round_mode %d", round_mode);
  if (overflow_mode < BSIR_OVERFLOW_WRAP || overflow_mode > BSIR_OVERFLOW_ASCEND_DOUBLE_ROUND_VIA_F16)
    return fail(BSIR_ERR_ATTR, "cast: overflow_mode %d", overflow_mode);
  if (overflow_mode >= BSIR_OVERFLOW_ASCEND_SATURATE_TRUNC_VIA_F16 &&
      !((src_dtype == BSIR_F32 || src_dtype == BSIR_F16) && dst_dtype == BSIR_I8))
    return fail(BSIR_ERR_ATTR, "cast: the via-f16 overflow modes apply to f32/f16 -> i8 only");
  if (rank < 1 || rank > 3 || !sizes) return fail(BSIR_ERR_SHAPE, "cast: rank %d (1..3 supported)", rank);
  CastShape sh{1, 1, 1, 1, 0, 0, 0, 0, 0, 0};
  int64_t n[3] = {1, 1, 1}, ss[3] = {0, 0, 0}, ds[3] = {0, 0, 0};
  bool contig = true;
  int64_t cs = 1;
  for (int i = rank - 1; i >= 0; --i) {
    if (sizes[i] < 0) return fail(BSIR_ERR_SHAPE, "cast: sizes[%d] = %lld", i, (long long)sizes[i]);
    n[3 - rank + i] = sizes[i];
    ss[3 - rank + i] = src_strides ? src_strides[i] : cs;
    ds[3 - rank + i] = dst_strides ? dst_strides[i] : cs;
    if (sizes[i] != 1 && (ss[3 - rank + i] != cs || ds[3 - rank + i] != cs)) contig = false;
    cs *= sizes[i];
  }
  sh.n0 = n[0]; sh.n1 = n[1]; sh.n2 = n[2]; sh.total = n[0] * n[1] * n[2];
  sh.ss0 = ss[0]; sh.ss1 = ss[1]; sh.ss2 = ss[2]; sh.ds0 = ds[0]; sh.ds1 = ds[1]; sh.ds2 = ds[2];
  if (sh.total == 0) return BSIR_OK;
  if (!src || !dst) return fail(BSIR_ERR_NULL, "cast: null pointer");
  if (!aligned_to(src, dtype_bytes(src_dtype)) || !aligned_to(dst, dtype_bytes(dst_dtype)))
    return fail(BSIR_ERR_ALIGN, "cast: misaligned");
  cudaStream_t st = resolve_stream(stream);
#define X(S, D) \
  if (src_dtype == S && dst_dtype == D) return launch_cast<S, D>(sh, contig, src, dst, round_mode, overflow_mode, st);
  BSIR_CAST_PAIRS(X)
#undef X
  return fail(BSIR_ERR_DTYPE, "cast: %d -> %d is not a supported pair", src_dtype, dst_dtype);
}
