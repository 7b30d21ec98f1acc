// fused_rows.cu -- the fused last-axis patterns HFusion's op fusion produces (fusion kind
// LAST_AXIS_PBR, bishengir/lib/Dialect/HFusion/Transforms/OpFusion/FusibleHelper.cpp:387-397):
// RMSNorm, softmax and per-token dynamic int8 quantisation.  One pass over HBM: a row is
// read once into registers with 128-bit loads, reduced with warp shuffles (plus one shared
// memory hop when a row spans several warps) and written once.
//
// Row layout: TPR threads share a row (TPR = 32..1024, a power of two, chosen per shape);
// thread t of the row owns the 16-byte vectors t, t + TPR, t + 2 TPR, ... (VPT of them), so
// every load and store instruction of a warp covers 512 contiguous bytes.
//
// Shapes the register path cannot hold (very long rows, rows that are not a whole number of
// 16-byte vectors, unaligned bases) go to the multi-pass kernels at the end of the file, which
// re-read the row from L2 instead.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"

namespace bsir {
namespace {

constexpr int kMaxWarpsPerRow = 32;

struct RowGeom {
  int64_t rows;
  int64_t cols;
  int64_t nvec;  // 16-byte vectors per row
  int tpr;       // threads per row
  int rpc;       // rows per CTA
};

// Cross-thread reduction inside a row group.  `red` points at this row group's slice
// (kMaxWarpsPerRow floats) of a shared array used by this reduction only.
// Rows shorter than a warp's worth of vectors get 4, 8 or 16 lanes (an aligned group of the warp): the
// shuffle steps that would cross into a neighbouring row's lanes are skipped.
template <class Combine, class Shuffle>
__device__ __forceinline__ float row_reduce(float v, int tpr, float *red, float identity, Combine combine,
                                            Shuffle warp_red) {
  v = warp_red(v, tpr < 32 ? tpr : 32);
  if (tpr <= 32) return v;
  const int lane = threadIdx.x & 31;
  const int warp_in_row = (threadIdx.x % tpr) >> 5;
  const int nwarps = tpr >> 5;
  if (lane == 0) red[warp_in_row] = v;
  __syncthreads();
  float p = lane < nwarps ? red[lane] : identity;
  p = warp_red(p, 32);
  (void)combine;
  return p;
}

__device__ __forceinline__ float warp_red_sum(float v, int width = 32) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    if (o < width) v += other;
  }
  return v;
}
__device__ __forceinline__ float warp_red_maxnan(float v, int width = 32) {  // maximumf
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    if (o < width) v = maximumf(v, other);
  }
  return v;
}
__device__ __forceinline__ float warp_red_maxnum(float v, int width = 32) {  // fmaxf: NaN ignored
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    if (o < width) v = fmaxf(v, other);
  }
  return v;
}

// hfusion.round_mode applied to an f32 value (result integral, still f32).
__device__ __forceinline__ float round_by_mode(float x, int mode) {
  switch (mode) {
    case BSIR_ROUND_RINT: return rintf(x);
    case BSIR_ROUND_ROUND: return roundf(x);
    case BSIR_ROUND_FLOOR: return floorf(x);
    case BSIR_ROUND_CEIL: return ceilf(x);
    case BSIR_ROUND_ODD: {
      const float t = truncf(x);
      if (t == x) return x;
      return (fmodf(t, 2.0f) == 0.0f) ? t + (x > 0.0f ? 1.0f : -1.0f) : t;
    }
    default: return truncf(x);
  }
}
// integral f32 -> saturated int8, NaN -> 0
__device__ __forceinline__ int sat_i8(float r) {
  int i = __float2int_rz(r);  // saturates at the int32 range, NaN -> 0
  return max(-128, min(127, i));
}

// ------------------------------------------------------------------ per-token int8 quantisation
// scale = max|x| / 127 (IEEE divide); q = cast{round_mode, saturate}(x / scale).
// Rows whose max|x| is 0, inf or NaN quantise to all zeros: every quotient is then 0/0, x/inf
// or involves a NaN, and NaN saturates to 0.
//
// For bf16 and f16 rows with a scale in [2^-60, 2^60] the per-element divide is replaced by the
// reciprocal r = RN(1/scale) and one correction step, q0 = x r, q = fma(fma(-q0, scale, x), r, q0):
// for every bf16 / f16 x with |x / scale| <= 127.5 this rounds to the same integer as the IEEE
// quotient (checked on the CPU for every scale a row can have -- RN(amax / 127) for each finite amax of the
// type -- against every x with |x| <= amax: 1.5e9 pairs, no mismatch).
// TPR_C != 0: the threads per row are a compile-time constant and the row is exactly TPR_C * VPT vectors, so
// the vector offsets are immediates and no bounds are checked (the usual power-of-two hidden sizes).
template <int DT, int VPT, int TPR_C = 0>
__global__ void __launch_bounds__(VPT >= 16 ? 256 : VPT >= 8 ? 512 : 1024) quant_rows_kernel(RowGeom g, const void *__restrict__ xp, int64_t x_stride,
                                                          int8_t *__restrict__ qp, int64_t q_stride,
                                                          float *__restrict__ scale_out, int round_mode) {
  constexpr int kPerWord = FloatTraits<DT>::kPerWord;
  constexpr int kPerVec = 4 * kPerWord;
  __shared__ float red[kMaxWarpsPerRow * 32];
  const int tpr = TPR_C ? TPR_C : g.tpr;
  constexpr bool kExact = TPR_C != 0;
  pdl_launch_dependents();   // the next launch may be scheduled while this one runs (launch_pdl) ...
  pdl_wait();                // ... and this one touches global memory only after the kernel ahead has completed
  const int sub = threadIdx.x / tpr;
  const int t = threadIdx.x % tpr;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * g.rpc + sub;
  const bool row_ok = row < g.rows;
  using E = typename std::conditional<DT == BSIR_F32, float, uint16_t>::type;
  const E *xrow = static_cast<const E *>(xp) + (row_ok ? row : 0) * x_stride;

  Vec16 v[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int64_t vi = t + static_cast<int64_t>(i) * tpr;
    if (row_ok && (kExact || vi < g.nvec)) v[i] = ld_stream(reinterpret_cast<const Vec16 *>(xrow) + vi);
    else v[i] = Vec16{{0u, 0u, 0u, 0u}};
  }
  // row maximum of |x|, NaN-propagating.  16-bit types stay packed: clear both sign bits, then one
  // max.NaN.{bf16x2,f16x2} per word.
  float amax = 0.0f;
  if constexpr (kPerWord == 2) {
    uint32_t m2 = 0u;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        // abs + max in one asm block so the assembler can fold |.| into the max as an operand modifier
        if constexpr (DT == BSIR_BF16)
          asm("{\n\t.reg .b32 t;\n\tabs.bf16x2 t, %2;\n\tmax.NaN.bf16x2 %0, %1, t;\n\t}" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
        else
          asm("{\n\t.reg .b32 t;\n\tabs.f16x2 t, %2;\n\tmax.NaN.f16x2 %0, %1, t;\n\t}" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
      }
    float e[2];
    FloatTraits<DT>::unpack(m2, e);
    amax = maximumf(e[0], e[1]);
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int w = 0; w < 4; ++w) amax = maximumf(amax, fabsf(__uint_as_float(v[i].w[w])));
  }
  amax = row_reduce(amax, tpr, red + sub * kMaxWarpsPerRow, 0.0f, 0, warp_red_maxnan);
  const float scale = __fdiv_rn(amax, 127.0f);
  if (row_ok && t == 0) scale_out[row] = scale;
  if (!row_ok) return;

  const bool degenerate = !(amax > 0.0f && amax < __int_as_float(0x7f800000));
  const bool fast = (DT == BSIR_BF16 || DT == BSIR_F16) && round_mode == BSIR_ROUND_RINT && scale > 8.6736174e-19f && scale < 1.1529215e18f;
  int8_t *qrow = qp + row * q_stride;

  if (degenerate) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t vi = t + static_cast<int64_t>(i) * tpr;
      if (!kExact && vi >= g.nvec) continue;
      if constexpr (kPerVec == 8) *reinterpret_cast<uint2 *>(qrow + vi * 8) = make_uint2(0u, 0u);
      else *reinterpret_cast<uint32_t *>(qrow + vi * 4) = 0u;
    }
    return;
  }
  if constexpr (DT == BSIR_BF16 || DT == BSIR_F16) {
    if (fast) {
      // two elements per instruction (f32x2): q0 = x r; q = fma(fma(q0, -scale, x), r, q0); then
      // q + 1.5 * 2^23 rounds to nearest even and leaves the integer in the low mantissa byte
      const float rcp = __frcp_rn(scale);
      unsigned long long rcp2, nscale2, magic2;
      asm("mov.b64 %0, {%1, %1};" : "=l"(rcp2) : "f"(rcp));
      asm("mov.b64 %0, {%1, %1};" : "=l"(nscale2) : "f"(-scale));
      asm("mov.b64 %0, {%1, %1};" : "=l"(magic2) : "f"(12582912.0f));
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int64_t vi = t + static_cast<int64_t>(i) * tpr;
        if (!kExact && vi >= g.nvec) continue;
        uint32_t lo8[8];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const uint32_t word = v[i].w[w];
          unsigned long long x2, q0, e2, q1, r2;
          if constexpr (DT == BSIR_BF16) {
            asm("mov.b64 %0, {%1, %2};" : "=l"(x2) : "r"(word << 16), "r"(word & 0xffff0000u));
          } else {
            float e2[2];
            FloatTraits<DT>::unpack(word, e2);
            asm("mov.b64 %0, {%1, %2};" : "=l"(x2) : "f"(e2[0]), "f"(e2[1]));
          }
          asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(q0) : "l"(x2), "l"(rcp2));
          asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(e2) : "l"(q0), "l"(nscale2), "l"(x2));
          asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q1) : "l"(e2), "l"(rcp2), "l"(q0));
          asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r2) : "l"(q1), "l"(magic2));
          asm("mov.b64 {%0, %1}, %2;" : "=r"(lo8[2 * w]), "=r"(lo8[2 * w + 1]) : "l"(r2));
        }
        // byte 0 of each of the eight results -> two packed words
        const uint32_t p01 = __byte_perm(lo8[0], lo8[1], 0x0040), p23 = __byte_perm(lo8[2], lo8[3], 0x0040);
        const uint32_t p45 = __byte_perm(lo8[4], lo8[5], 0x0040), p67 = __byte_perm(lo8[6], lo8[7], 0x0040);
        *reinterpret_cast<uint2 *>(qrow + vi * 8) =
            make_uint2(__byte_perm(p01, p23, 0x5410), __byte_perm(p45, p67, 0x5410));
      }
      return;
    }
  }
  // general path: IEEE divide per element, any round mode, saturating conversion.  The round mode is
  // decided once: rint (the default) is one cvt.rni, which saturates at the int32 range and maps NaN to 0.
  auto run = [&](auto conv) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t vi = t + static_cast<int64_t>(i) * tpr;
      if (!kExact && vi >= g.nvec) continue;
      uint32_t bytes[kPerVec / 4];
#pragma unroll
      for (int w4 = 0; w4 < kPerVec / 4; ++w4) {
        float e[4];
        if constexpr (kPerWord == 2) {
          FloatTraits<DT>::unpack(v[i].w[2 * w4], e);
          FloatTraits<DT>::unpack(v[i].w[2 * w4 + 1], e + 2);
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) e[k] = __uint_as_float(v[i].w[k]);
        }
        uint32_t b[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) b[k] = static_cast<uint32_t>(conv(__fdiv_rn(e[k], scale)));
        bytes[w4] = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
      }
      if constexpr (kPerVec == 8) {
        *reinterpret_cast<uint2 *>(qrow + vi * 8) = make_uint2(bytes[0], bytes[1]);
      } else {
        *reinterpret_cast<uint32_t *>(qrow + vi * 4) = bytes[0];
      }
    }
  };
  if (round_mode == BSIR_ROUND_RINT) run([](float d) { return max(-128, min(127, __float2int_rn(d))); });
  else run([&](float d) { return sat_i8(round_by_mode(d, round_mode)); });
}

// ------------------------------------------------------------------ RMSNorm
// y = cast_rint(gamma32 * (rstd * x32)), rstd = 1 / sqrt(sum(x32^2) * (1/cols) + eps), in the
// op order of the reference IR
// (test/bishengir-compile/hfusion/compile-rms-norm-fp16-split-n.mlir:27-61).
template <int DT, int VPT>
__global__ void __launch_bounds__(VPT >= 16 ? 256 : VPT >= 8 ? 512 : 1024) rmsnorm_rows_kernel(RowGeom g, const void *__restrict__ xp, int64_t x_stride,
                                                            const void *__restrict__ gammap, float eps, float avg,
                                                            void *__restrict__ yp, int64_t y_stride,
                                                            void *__restrict__ rstd_out) {
  constexpr int kPerWord = FloatTraits<DT>::kPerWord;
  __shared__ float red[kMaxWarpsPerRow * 32];
  using E = typename std::conditional<DT == BSIR_F32, float, uint16_t>::type;
  const int sub = threadIdx.x / g.tpr;
  const int t = threadIdx.x % g.tpr;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * g.rpc + sub;
  const bool row_ok = row < g.rows;
  const E *xrow = static_cast<const E *>(xp) + (row_ok ? row : 0) * x_stride;

  Vec16 v[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int64_t vi = t + static_cast<int64_t>(i) * g.tpr;
    if (row_ok && vi < g.nvec) v[i] = ld_stream(reinterpret_cast<const Vec16 *>(xrow) + vi);
    else v[i] = Vec16{{0u, 0u, 0u, 0u}};
  }
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      float e[kPerWord];
      FloatTraits<DT>::unpack(v[i].w[w], e);
#pragma unroll
      for (int k = 0; k < kPerWord; ++k) ss = __fmaf_rn(e[k], e[k], ss);
    }
  }
  ss = row_reduce(ss, g.tpr, red + sub * kMaxWarpsPerRow, 0.0f, 0, warp_red_sum);
  const float mean = __fmul_rn(ss, avg);
  const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
  if (!row_ok) return;
  if (rstd_out && t == 0) {
    float r1[kPerWord];
    r1[0] = rstd;
    if constexpr (kPerWord == 2) r1[1] = 0.0f;
    const uint32_t packed = FloatTraits<DT>::pack(r1);
    if constexpr (DT == BSIR_F32) static_cast<float *>(rstd_out)[row] = rstd;
    else static_cast<uint16_t *>(rstd_out)[row] = static_cast<uint16_t>(packed & 0xffffu);
  }
  E *yrow = static_cast<E *>(yp) + row * y_stride;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int64_t vi = t + static_cast<int64_t>(i) * g.tpr;
    if (vi >= g.nvec) continue;
    const Vec16 gv = *(reinterpret_cast<const Vec16 *>(gammap) + vi);  // gamma stays in L1/L2
    Vec16 o;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      float e[kPerWord], ge[kPerWord], r[kPerWord];
      FloatTraits<DT>::unpack(v[i].w[w], e);
      FloatTraits<DT>::unpack(gv.w[w], ge);
#pragma unroll
      for (int k = 0; k < kPerWord; ++k) r[k] = __fmul_rn(ge[k], __fmul_rn(rstd, e[k]));
      o.w[w] = FloatTraits<DT>::pack(r);
    }
    st_stream(reinterpret_cast<Vec16 *>(yrow) + vi, o);
  }
}

// ------------------------------------------------------------------ softmax
// m = max over non-NaN x; e = exp(x - m); y = cast_rint(e / sum e)
// (test/Dialect/Analysis/VFFusion/MaxParallelKind/softmax_small_shape.mlir:86-117).
// exp runs on the special-function unit: ex2.approx(x log2e - m log2e), relative error below 3e-6
// for the arguments a softmax sees (results below 2^-126 flush to zero).  The arithmetic around it is
// two elements per instruction (f32x2).  16-bit outputs multiply by the reciprocal of the row sum
// (the result is rounded to 8 or 11 bits afterwards); f32 outputs add one correction step so the
// quotient is the IEEE one.
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &a, float &b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

template <int DT, int VPT>
__global__ void __launch_bounds__(VPT * (DT == BSIR_F32 ? 4 : 8) > 32 ? 256 : 1024) softmax_rows_kernel(RowGeom g, const void *__restrict__ xp, int64_t x_stride,
                                                            void *__restrict__ yp, int64_t y_stride) {
  constexpr int kPerWord = FloatTraits<DT>::kPerWord;
  constexpr int kPerVec = 4 * kPerWord;
  constexpr int kPairs = VPT * kPerVec / 2;   // element pairs held by a thread
  __shared__ float red_max[kMaxWarpsPerRow * 32];
  __shared__ float red_sum[kMaxWarpsPerRow * 32];
  using E = typename std::conditional<DT == BSIR_F32, float, uint16_t>::type;
  const int sub = threadIdx.x / g.tpr;
  const int t = threadIdx.x % g.tpr;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * g.rpc + sub;
  const bool row_ok = row < g.rows;
  const E *xrow = static_cast<const E *>(xp) + (row_ok ? row : 0) * x_stride;
  const float ninf = __int_as_float(0xff800000);
  // padding is -inf in the storage type: ignored by the max, exp gives 0
  constexpr uint32_t kPad = DT == BSIR_F32 ? 0xff800000u : DT == BSIR_BF16 ? 0xff80ff80u : 0xfc00fc00u;

  Vec16 v[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int64_t vi = t + static_cast<int64_t>(i) * g.tpr;
    if (row_ok && vi < g.nvec) v[i] = ld_stream(reinterpret_cast<const Vec16 *>(xrow) + vi);
    else v[i] = Vec16{{kPad, kPad, kPad, kPad}};
  }
  // row maximum, NaN ignored (= the NaN -> -inf mask of the reference IR); 16-bit types stay packed
  float m = ninf;
  if constexpr (kPerWord == 2) {
    uint32_t m2 = kPad;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        if constexpr (DT == BSIR_BF16) asm("max.bf16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
        else asm("max.f16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
      }
    float e2[2];
    FloatTraits<DT>::unpack(m2, e2);
    m = fmaxf(e2[0], e2[1]);
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int w = 0; w < 4; ++w) m = fmaxf(m, __uint_as_float(v[i].w[w]));
  }
  m = row_reduce(m, g.tpr, red_max + sub * kMaxWarpsPerRow, ninf, 0, warp_red_maxnum);

  const float kLog2e = 1.4426950408889634f;
  const unsigned long long l2e2 = pack2(kLog2e, kLog2e);
  const float nm = -m * kLog2e;   // -inf * c stays inf of the right sign; NaN cannot occur (m ignores NaN)
  const unsigned long long nm2 = pack2(nm, nm);
  unsigned long long e[kPairs];
  unsigned long long s2 = pack2(0.0f, 0.0f);
#pragma unroll
  for (int pi = 0; pi < kPairs; ++pi) {
    float x0, x1;
    if constexpr (kPerWord == 2) {
      const uint32_t word = v[pi / 4].w[pi % 4];
      float xe[2];
      FloatTraits<DT>::unpack(word, xe);
      x0 = xe[0];
      x1 = xe[1];
    } else {
      x0 = __uint_as_float(v[pi / 2].w[(pi % 2) * 2]);
      x1 = __uint_as_float(v[pi / 2].w[(pi % 2) * 2 + 1]);
    }
    const unsigned long long d = fma2(pack2(x0, x1), l2e2, nm2);
    float d0, d1;
    unpack2(d, d0, d1);
    e[pi] = pack2(ex2_approx(d0), ex2_approx(d1));
    s2 = add2(s2, e[pi]);
  }
  float s0, s1;
  unpack2(s2, s0, s1);
  float s = row_reduce(s0 + s1, g.tpr, red_sum + sub * kMaxWarpsPerRow, 0.0f, 0, warp_red_sum);
  if (!row_ok) return;
  const float rcp = __frcp_rn(s);
  const unsigned long long rcp2 = pack2(rcp, rcp), ns2 = pack2(-s, -s);
  E *yrow = static_cast<E *>(yp) + row * y_stride;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int64_t vi = t + static_cast<int64_t>(i) * g.tpr;
    if (vi >= g.nvec) continue;
    Vec16 o;
    if constexpr (kPerWord == 2) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        float y0, y1;
        unpack2(mul2(e[i * 4 + w], rcp2), y0, y1);
        const float yy[2] = {y0, y1};
        o.w[w] = FloatTraits<DT>::pack(yy);
      }
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const unsigned long long ev = e[i * 2 + h];
        const unsigned long long q0 = mul2(ev, rcp2);
        float y0, y1;
        unpack2(fma2(fma2(q0, ns2, ev), rcp2, q0), y0, y1);
        o.w[2 * h] = __float_as_uint(y0);
        o.w[2 * h + 1] = __float_as_uint(y1);
      }
    }
    st_stream(reinterpret_cast<Vec16 *>(yrow) + vi, o);
  }
}

// ------------------------------------------------------------------ softmax, long rows
// Rows of 32-64 KB leave room for one CTA per SM only, so in the kernel above every thread of the SM
// is in the same phase and HBM idles while the row is reduced.  Here the CTA is persistent and the
// rows stream through shared memory: one thread issues a bulk copy (cp.async.bulk, completion on an
// mbarrier) of the row after next while the 1024 threads work on the current one, so two rows per SM
// are always in flight.  The arithmetic is the same as above.
constexpr int kStreamBufs = 3;
constexpr uint32_t kErrRowWait = 0x20;

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// bounded: gives up after about two seconds and raises the device error word
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int *err) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t spin = 0;; ++spin) {
    if (mbar_try(bar, parity)) return true;
    if ((spin & 1023u) == 1023u && clock64() - t0 > 4000000000LL) {
      if (err) atomicOr(err, static_cast<int>(kErrRowWait));
      return false;
    }
  }
}

template <int DT, int VPT>
__global__ void __launch_bounds__(1024, 1) softmax_stream_kernel(RowGeom g, const void *__restrict__ xp, int64_t x_stride,
                                                                  void *__restrict__ yp, int64_t y_stride, int *err) {
  constexpr int kPerWord = FloatTraits<DT>::kPerWord;
  constexpr int kPerVec = 4 * kPerWord;
  constexpr int kPairs = VPT * kPerVec / 2;
  extern __shared__ __align__(128) uint8_t row_smem[];
  __shared__ float red_max[32];
  __shared__ float red_sum[32];
  __shared__ __align__(8) unsigned long long bars[kStreamBufs];
  using E = typename std::conditional<DT == BSIR_F32, float, uint16_t>::type;
  const int t = threadIdx.x;
  const uint32_t row_bytes = static_cast<uint32_t>(g.nvec) * 16u;
  const float ninf = __int_as_float(0xff800000);
  constexpr uint32_t kPad = DT == BSIR_F32 ? 0xff800000u : DT == BSIR_BF16 ? 0xff80ff80u : 0xfc00fc00u;
  const int64_t my_rows = (g.rows - blockIdx.x + gridDim.x - 1) / gridDim.x;   // rows blockIdx.x, + gridDim.x, ...

  auto issue = [&](int64_t k) {   // bulk copy of this CTA's k-th row into buffer k % kStreamBufs
    const int b = static_cast<int>(k % kStreamBufs);
    const E *src = static_cast<const E *>(xp) + (blockIdx.x + k * gridDim.x) * x_stride;
    const uint32_t bar = smem_addr(&bars[b]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(row_bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(row_smem) + static_cast<uint32_t>(b) * row_bytes),
                 "l"(src), "r"(row_bytes), "r"(bar)
                 : "memory");
  };

  if (t == 0) {
    for (int b = 0; b < kStreamBufs; ++b)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bars[b])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (t == 0)
    for (int64_t k = 0; k < kStreamBufs - 1 && k < my_rows; ++k) issue(k);

  bool ok = true;
  for (int64_t k = 0; k < my_rows; ++k) {
    const int b = static_cast<int>(k % kStreamBufs);
    const uint32_t parity = static_cast<uint32_t>((k / kStreamBufs) & 1);
    if (ok && !mbar_wait_bounded(smem_addr(&bars[b]), parity, err)) ok = false;
    const Vec16 *buf = reinterpret_cast<const Vec16 *>(row_smem + static_cast<size_t>(b) * row_bytes);
    Vec16 v[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t vi = t + static_cast<int64_t>(i) * 1024;
      v[i] = (ok && vi < g.nvec) ? buf[vi] : Vec16{{kPad, kPad, kPad, kPad}};
    }
    float m = ninf;
    if constexpr (kPerWord == 2) {
      uint32_t m2 = kPad;
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          if constexpr (DT == BSIR_BF16) asm("max.bf16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
          else asm("max.f16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
        }
      float e2[2];
      FloatTraits<DT>::unpack(m2, e2);
      m = fmaxf(e2[0], e2[1]);
    } else {
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, __uint_as_float(v[i].w[w]));
    }
    m = row_reduce(m, 1024, red_max, ninf, 0, warp_red_maxnum);
    // every thread has its part of buffer b in registers (the barrier inside row_reduce is behind us),
    // and buffer (k + 2) % 3 was released one row ago: start the copy of the row after next
    if (t == 0 && k + kStreamBufs - 1 < my_rows) issue(k + kStreamBufs - 1);

    const float kLog2e = 1.4426950408889634f;
    const unsigned long long l2e2 = pack2(kLog2e, kLog2e);
    const float nm = -m * kLog2e;
    const unsigned long long nm2 = pack2(nm, nm);
    unsigned long long e[kPairs];
    unsigned long long s2 = pack2(0.0f, 0.0f);
#pragma unroll
    for (int pi = 0; pi < kPairs; ++pi) {
      float x0, x1;
      if constexpr (kPerWord == 2) {
        float xe[2];
        FloatTraits<DT>::unpack(v[pi / 4].w[pi % 4], xe);
        x0 = xe[0];
        x1 = xe[1];
      } else {
        x0 = __uint_as_float(v[pi / 2].w[(pi % 2) * 2]);
        x1 = __uint_as_float(v[pi / 2].w[(pi % 2) * 2 + 1]);
      }
      float d0, d1;
      unpack2(fma2(pack2(x0, x1), l2e2, nm2), d0, d1);
      e[pi] = pack2(ex2_approx(d0), ex2_approx(d1));
      s2 = add2(s2, e[pi]);
    }
    float s0, s1;
    unpack2(s2, s0, s1);
    const float s = row_reduce(s0 + s1, 1024, red_sum, 0.0f, 0, warp_red_sum);
    const float rcp = __frcp_rn(s);
    const unsigned long long rcp2 = pack2(rcp, rcp), ns2 = pack2(-s, -s);
    E *yrow = static_cast<E *>(yp) + (blockIdx.x + k * gridDim.x) * y_stride;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t vi = t + static_cast<int64_t>(i) * 1024;
      if (vi >= g.nvec || !ok) continue;
      Vec16 o;
      if constexpr (kPerWord == 2) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          float y0, y1;
          unpack2(mul2(e[i * 4 + w], rcp2), y0, y1);
          const float yy[2] = {y0, y1};
          o.w[w] = FloatTraits<DT>::pack(yy);
        }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const unsigned long long ev = e[i * 2 + h];
          const unsigned long long q0 = mul2(ev, rcp2);
          float y0, y1;
          unpack2(fma2(fma2(q0, ns2, ev), rcp2, q0), y0, y1);
          o.w[2 * h] = __float_as_uint(y0);
          o.w[2 * h + 1] = __float_as_uint(y1);
        }
      }
      st_stream(reinterpret_cast<Vec16 *>(yrow) + vi, o);
    }
  }
}

// ------------------------------------------------------------------ multi-pass fallbacks
// One CTA per row, any cols / stride / alignment; the row is re-read from L2 on each pass.
template <int DT>
__device__ __forceinline__ float load_elem(const void *p, int64_t i) {
  if constexpr (DT == BSIR_F32) return static_cast<const float *>(p)[i];
  else if constexpr (DT == BSIR_F16) return __half2float(__ushort_as_half(static_cast<const uint16_t *>(p)[i]));
  else return __uint_as_float(static_cast<uint32_t>(static_cast<const uint16_t *>(p)[i]) << 16);
}
template <int DT>
__device__ __forceinline__ void store_elem(void *p, int64_t i, float v) {
  if constexpr (DT == BSIR_F32) static_cast<float *>(p)[i] = v;
  else if constexpr (DT == BSIR_F16) static_cast<uint16_t *>(p)[i] = __half_as_ushort(__float2half_rn(v));
  else static_cast<uint16_t *>(p)[i] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

template <class WarpRed>
__device__ __forceinline__ float block_reduce(float v, float *red, float identity, WarpRed warp_red) {
  v = warp_red(v, 32);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();  // red may still be read from the previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float p = lane < nw ? red[lane] : identity;
  return warp_red(p, 32);
}

enum { kRowQuant = 0, kRowRms = 1, kRowSoftmax = 2 };

template <int DT, int OP>
__global__ void __launch_bounds__(256) rows_multipass_kernel(int64_t rows, int64_t cols, const void *__restrict__ xp,
                                                             int64_t x_stride, const void *__restrict__ gammap,
                                                             float eps, float avg, void *__restrict__ yp,
                                                             int64_t y_stride, void *__restrict__ aux, int round_mode) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  if (row >= rows) return;
  const int64_t xo = row * x_stride, yo = row * y_stride;
  if constexpr (OP == kRowQuant) {
    float amax = 0.0f;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) amax = maximumf(amax, fabsf(load_elem<DT>(xp, xo + j)));
    amax = block_reduce(amax, red, 0.0f, warp_red_maxnan);
    const float scale = __fdiv_rn(amax, 127.0f);
    if (threadIdx.x == 0) static_cast<float *>(aux)[row] = scale;
    const bool degenerate = !(amax > 0.0f && amax < __int_as_float(0x7f800000));
    int8_t *q = static_cast<int8_t *>(yp) + yo;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x)
      q[j] = degenerate ? 0 : static_cast<int8_t>(sat_i8(round_by_mode(__fdiv_rn(load_elem<DT>(xp, xo + j), scale), round_mode)));
  } else if constexpr (OP == kRowRms) {
    float ss = 0.0f;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
      const float v = load_elem<DT>(xp, xo + j);
      ss = __fmaf_rn(v, v, ss);
    }
    ss = block_reduce(ss, red, 0.0f, warp_red_sum);
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(ss, avg), eps)));
    if (aux && threadIdx.x == 0) store_elem<DT>(aux, row, rstd);
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x)
      store_elem<DT>(yp, yo + j, __fmul_rn(load_elem<DT>(gammap, j), __fmul_rn(rstd, load_elem<DT>(xp, xo + j))));
  } else {
    const float ninf = __int_as_float(0xff800000);
    float m = ninf;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, load_elem<DT>(xp, xo + j));
    m = block_reduce(m, red, ninf, warp_red_maxnum);
    float s = 0.0f;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) s += expf(__fsub_rn(load_elem<DT>(xp, xo + j), m));
    s = block_reduce(s, red, 0.0f, warp_red_sum);
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x)
      store_elem<DT>(yp, yo + j, __fdiv_rn(expf(__fsub_rn(load_elem<DT>(xp, xo + j), m)), s));
  }
}

// ------------------------------------------------------------------ rows longer than the on-chip kernels hold
// A row of more than 64 KB (a softmax over a 150k-entry vocabulary, say) does not fit the registers or the
// shared memory of one CTA.  It is cut into parts of 2048 vectors (32 KB, eight vectors per thread of a
// 256-thread CTA).  Pass one leaves one statistic per (row, part) in a scratch array: the part's
// max|x| (quantiser), its sum of squares (RMSNorm), or its maximum and the sum of exp(x - that maximum)
// (softmax).  Pass two combines a row's statistics in part order -- every CTA of the row does it for
// itself, the numbers are few -- and streams its part again, now mostly from L2, to produce the output.
// Element arithmetic is that of the kernels above.
constexpr int kLongPartVecs = 2048;
struct LongStat { float a, b; };

template <int DT>
__device__ __forceinline__ void long_load(const void *xp, int64_t x_stride, int64_t row, int64_t v0, int64_t nvec,
                                          Vec16 (&v)[8], bool (&have)[8]) {
  using E = typename std::conditional<DT == BSIR_F32, float, uint16_t>::type;
  const Vec16 *xv = reinterpret_cast<const Vec16 *>(static_cast<const E *>(xp) + row * x_stride);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t vi = v0 + threadIdx.x + i * 256;
    have[i] = vi < nvec;
    if (have[i]) v[i] = ld_stream(xv + vi);
  }
}

template <int DT, int OP>
__global__ void __launch_bounds__(256) rows_long_stat_kernel(int64_t row0, int64_t nvec, const void *__restrict__ xp,
                                                             int64_t x_stride, LongStat *__restrict__ stats, int nparts) {
  constexpr int kPerWord = FloatTraits<DT>::kPerWord;
  __shared__ float red[32];
  const int64_t row = row0 + blockIdx.y;
  const int part = blockIdx.x;
  Vec16 v[8];
  bool have[8];
  long_load<DT>(xp, x_stride, row, static_cast<int64_t>(part) * kLongPartVecs, nvec, v, have);
  auto for_each = [&](auto f) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (have[i]) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          float e[kPerWord];
          FloatTraits<DT>::unpack(v[i].w[w], e);
#pragma unroll
          for (int k = 0; k < kPerWord; ++k) f(e[k]);
        }
      }
  };
  LongStat st{0.0f, 0.0f};
  if constexpr (OP == kRowQuant) {
    float amax = 0.0f;
    for_each([&](float x) { amax = maximumf(amax, fabsf(x)); });
    st.a = block_reduce(amax, red, 0.0f, warp_red_maxnan);
  } else if constexpr (OP == kRowRms) {
    float ss = 0.0f;
    for_each([&](float x) { ss = __fmaf_rn(x, x, ss); });
    st.a = block_reduce(ss, red, 0.0f, warp_red_sum);
  } else {
    const float ninf = __int_as_float(0xff800000);
    float m = ninf, nans = 0.0f;
    for_each([&](float x) { m = fmaxf(m, x); if (x != x) nans = 1.0f; });
    m = block_reduce(m, red, ninf, warp_red_maxnum);
    nans = block_reduce(nans, red, 0.0f, warp_red_sum);
    const float l2e = 1.4426950408889634f, nm = -m * l2e;
    float s = 0.0f;
    for_each([&](float x) { s += ex2_approx(__fmaf_rn(x, l2e, nm)); });
    s = block_reduce(s, red, 0.0f, warp_red_sum);
    // a part whose maximum is -inf holds no finite value: it adds nothing, unless it holds a NaN
    if (m == ninf) s = nans > 0.0f ? __int_as_float(0x7fc00000) : 0.0f;
    st.a = m;
    st.b = s;
  }
  if (threadIdx.x == 0) stats[static_cast<int64_t>(blockIdx.y) * nparts + part] = st;
}

template <int DT, int OP>
__global__ void __launch_bounds__(256) rows_long_apply_kernel(int64_t row0, int64_t nvec, const void *__restrict__ xp,
                                                              int64_t x_stride, const void *__restrict__ gammap, float eps,
                                                              float avg, void *__restrict__ yp, int64_t y_stride,
                                                              void *__restrict__ aux, int round_mode,
                                                              const LongStat *__restrict__ stats, int nparts) {
  constexpr int kPerWord = FloatTraits<DT>::kPerWord;
  constexpr int kPerVec = 4 * kPerWord;
  using E = typename std::conditional<DT == BSIR_F32, float, uint16_t>::type;
  const int64_t row = row0 + blockIdx.y;
  const int part = blockIdx.x;
  const int64_t v0 = static_cast<int64_t>(part) * kLongPartVecs;
  Vec16 v[8];
  bool have[8];
  long_load<DT>(xp, x_stride, row, v0, nvec, v, have);       // in flight while the statistics are combined
  const LongStat *rs = stats + static_cast<int64_t>(blockIdx.y) * nparts;
  if constexpr (OP == kRowQuant) {
    float amax = 0.0f;
    for (int p = 0; p < nparts; ++p) amax = maximumf(amax, rs[p].a);
    const float scale = __fdiv_rn(amax, 127.0f);
    if (part == 0 && threadIdx.x == 0) static_cast<float *>(aux)[row] = scale;
    const bool degenerate = !(amax > 0.0f && amax < __int_as_float(0x7f800000));
    const bool fast = (DT == BSIR_BF16 || DT == BSIR_F16) && round_mode == BSIR_ROUND_RINT && scale > 8.6736174e-19f &&
                      scale < 1.1529215e18f;
    const float rcp = __frcp_rn(scale);
    int8_t *qrow = static_cast<int8_t *>(yp) + row * y_stride;
    // one loop per case, so that the case is decided once and not per element
    auto run = [&](auto conv) {   // conv(x) -> a word whose low byte is the int8 result
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (!have[i]) continue;
        const int64_t vi = v0 + threadIdx.x + i * 256;
        uint32_t b[kPerVec];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          float e[kPerWord];
          FloatTraits<DT>::unpack(v[i].w[w], e);
#pragma unroll
          for (int k = 0; k < kPerWord; ++k) b[w * kPerWord + k] = conv(e[k]);
        }
        // byte 0 of each result -> packed words
        const uint32_t p01 = __byte_perm(b[0], b[1], 0x0040), p23 = __byte_perm(b[2], b[3], 0x0040);
        if constexpr (kPerVec == 8) {
          const uint32_t p45 = __byte_perm(b[4], b[5], 0x0040), p67 = __byte_perm(b[6], b[7], 0x0040);
          *reinterpret_cast<uint2 *>(qrow + vi * 8) = make_uint2(__byte_perm(p01, p23, 0x5410), __byte_perm(p45, p67, 0x5410));
        } else {
          *reinterpret_cast<uint32_t *>(qrow + vi * 4) = __byte_perm(p01, p23, 0x5410);
        }
      }
    };
    if (degenerate) {
      run([](float) { return 0u; });
    } else if (fast) {
      // the reciprocal form of the register kernel: same operations, one element at a time
      const float nscale = -scale;
      run([&](float x) {
        const float q0 = __fmul_rn(x, rcp);
        return __float_as_uint(__fadd_rn(__fmaf_rn(__fmaf_rn(q0, nscale, x), rcp, q0), 12582912.0f));
      });
    } else {
      run([&](float x) { return static_cast<uint32_t>(sat_i8(round_by_mode(__fdiv_rn(x, scale), round_mode))); });
    }
  } else if constexpr (OP == kRowRms) {
    float ss = 0.0f;
    for (int p = 0; p < nparts; ++p) ss += rs[p].a;
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(ss, avg), eps)));
    if (aux && part == 0 && threadIdx.x == 0) store_elem<DT>(aux, row, rstd);
    E *yrow = static_cast<E *>(yp) + row * y_stride;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (!have[i]) continue;
      const int64_t vi = v0 + threadIdx.x + i * 256;
      const Vec16 gv = *(reinterpret_cast<const Vec16 *>(gammap) + vi);
      Vec16 o;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        float e[kPerWord], ge[kPerWord], r[kPerWord];
        FloatTraits<DT>::unpack(v[i].w[w], e);
        FloatTraits<DT>::unpack(gv.w[w], ge);
#pragma unroll
        for (int k = 0; k < kPerWord; ++k) r[k] = __fmul_rn(ge[k], __fmul_rn(rstd, e[k]));
        o.w[w] = FloatTraits<DT>::pack(r);
      }
      st_stream(reinterpret_cast<Vec16 *>(yrow) + vi, o);
    }
  } else {
    const float ninf = __int_as_float(0xff800000);
    const float l2e = 1.4426950408889634f;
    float m = ninf;
    for (int p = 0; p < nparts; ++p) m = fmaxf(m, rs[p].a);
    float s = 0.0f;
    for (int p = 0; p < nparts; ++p) s += rs[p].b * ex2_approx((rs[p].a - m) * l2e);   // weight 1 for the part that holds m
    const float nm = -m * l2e, rcp = __frcp_rn(s);
    E *yrow = static_cast<E *>(yp) + row * y_stride;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (!have[i]) continue;
      const int64_t vi = v0 + threadIdx.x + i * 256;
      Vec16 o;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        float e[kPerWord], r[kPerWord];
        FloatTraits<DT>::unpack(v[i].w[w], e);
#pragma unroll
        for (int k = 0; k < kPerWord; ++k) {
          const float ex = ex2_approx(__fmaf_rn(e[k], l2e, nm));
          const float q0 = __fmul_rn(ex, rcp);
          r[k] = DT == BSIR_F32 ? __fmaf_rn(__fmaf_rn(q0, -s, ex), rcp, q0) : q0;
        }
        o.w[w] = FloatTraits<DT>::pack(r);
      }
      st_stream(reinterpret_cast<Vec16 *>(yrow) + vi, o);
    }
  }
}

// ------------------------------------------------------------------ host side
int env_int(const char *name, int dflt) {
  const char *s = std::getenv(name);
  return s && *s ? std::atoi(s) : dflt;
}

// Picks threads-per-row (TPR, a power of two in 4..1024) and vectors-per-thread (VPT).  Measured on
// B200: rows spread over enough threads that each holds about `want_vpt` vectors run fastest (4 for
// the 8 KB rows of the benchmark shapes, 8 for the 16-bit quantiser: 64 threads per 4096-element row); `max_vpt` is what the kernel's registers can hold.
// Register budget: 16 vectors per thread only up to 256 threads per CTA, 8 up to 512, 4 at 1024.
// Returns false when the row does not fit.
bool pick_geometry(int64_t rows, int64_t cols, int elem_bytes, int max_vpt, int want_vpt, int forced_tpr, RowGeom *g,
                   int *vpt) {
  const int per_vec = 16 / elem_bytes;
  if (cols <= 0 || cols % per_vec) return false;
  const int64_t nvec = cols / per_vec;
  auto allowed = [&](int tpr) { int a = tpr <= 256 ? 16 : tpr <= 512 ? 8 : 4; return a < max_vpt ? a : max_vpt; };
  int tpr = 4;
  if (forced_tpr >= 4 && forced_tpr <= 1024 && (forced_tpr & (forced_tpr - 1)) == 0) {
    tpr = forced_tpr;
  } else {
    while (tpr < 1024 && ceil_div(nvec, tpr) > want_vpt) tpr <<= 1;
  }
  while (tpr < 1024 && ceil_div(nvec, tpr) > allowed(tpr)) tpr <<= 1;
  const int64_t need = ceil_div(nvec, tpr);
  if (need > allowed(tpr)) return false;
  int v = 1;
  while (v < need) v <<= 1;
  g->rows = rows; g->cols = cols; g->nvec = nvec; g->tpr = tpr;
  const int cta = tpr < 128 ? 128 : tpr;
  g->rpc = cta / tpr;
  *vpt = v;
  return true;
}

bool rows_vector_ok(const void *p, int64_t stride_elems, int elem_bytes) {
  return aligned_to(p, 16) && (stride_elems * elem_bytes) % 16 == 0;
}

#define DISPATCH_VPT(vpt, ...)                         \
  switch (vpt) {                                       \
    case 1: { constexpr int V = 1; __VA_ARGS__; break; }   \
    case 2: { constexpr int V = 2; __VA_ARGS__; break; }   \
    case 4: { constexpr int V = 4; __VA_ARGS__; break; }   \
    case 8: { constexpr int V = 8; __VA_ARGS__; break; }   \
    default: { constexpr int V = 16; __VA_ARGS__; break; } \
  }
#define DISPATCH_VPT_LE8(vpt, ...)                     \
  switch (vpt) {                                       \
    case 1: { constexpr int V = 1; __VA_ARGS__; break; }   \
    case 2: { constexpr int V = 2; __VA_ARGS__; break; }   \
    case 4: { constexpr int V = 4; __VA_ARGS__; break; }   \
    default: { constexpr int V = 8; __VA_ARGS__; break; }  \
  }
#define DISPATCH_FLOAT_DT(dt, ...)                                 \
  switch (dt) {                                                    \
    case BSIR_F32: { constexpr int D = BSIR_F32; __VA_ARGS__; break; }   \
    case BSIR_F16: { constexpr int D = BSIR_F16; __VA_ARGS__; break; }   \
    default: { constexpr int D = BSIR_BF16; __VA_ARGS__; break; }        \
  }

// Both passes of the long-row path; rows beyond a grid dimension go in slabs.
template <int OP>
int32_t launch_long_rows(const char *what, int32_t dtype, int64_t rows, int64_t cols, const void *x, int64_t xs,
                         const void *gamma, float eps, float avg, void *y, int64_t ys, void *aux, int round_mode,
                         cudaStream_t st) {
  const int eb = dtype_bytes(dtype);
  const int64_t nvec = cols / (16 / eb);
  const int nparts = static_cast<int>(ceil_div(nvec, kLongPartVecs));
  const int64_t slab = rows < 65535 ? rows : 65535;
  char *ws = static_cast<char *>(device_workspace(kScratchCounterBytes + static_cast<size_t>(slab) * nparts * sizeof(LongStat), st));
  if (!ws) return BSIR_ERR_WORKSPACE;
  LongStat *stats = reinterpret_cast<LongStat *>(ws + kScratchCounterBytes);
  for (int64_t r0 = 0; r0 < rows; r0 += slab) {
    const int64_t nr = rows - r0 < slab ? rows - r0 : slab;
    const dim3 grid(static_cast<unsigned>(nparts), static_cast<unsigned>(nr));
    DISPATCH_FLOAT_DT(dtype, {
      rows_long_stat_kernel<D, OP><<<grid, 256, 0, st>>>(r0, nvec, x, xs, stats, nparts);
      rows_long_apply_kernel<D, OP><<<grid, 256, 0, st>>>(r0, nvec, x, xs, gamma, eps, avg, y, ys, aux, round_mode, stats, nparts);
    });
    count_launch(2);
  }
  return check_launch(what);
}

int32_t check_rows_args(const char *what, int32_t dtype, int64_t rows, int64_t cols, const void *x, int64_t xs,
                        const void *y, int64_t ys) {
  if (!dtype_is_float(dtype)) return fail(BSIR_ERR_DTYPE, "%s: dtype %d (f32, f16 or bf16 required)", what, dtype);
  if (rows < 0 || cols < 0) return fail(BSIR_ERR_SHAPE, "%s: rows=%lld cols=%lld", what, (long long)rows, (long long)cols);
  if (rows == 0) return BSIR_OK;
  if (!x || !y) return fail(BSIR_ERR_NULL, "%s: null pointer", what);
  if (xs < cols || ys < cols) return fail(BSIR_ERR_STRIDE, "%s: row stride smaller than cols", what);
  if (rows > 0x7fffffffLL) return fail(BSIR_ERR_SHAPE, "%s: too many rows", what);
  return BSIR_OK;
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" {

int32_t bsir_quant_per_token_i8(int32_t dtype, int32_t round_mode, int64_t rows, int64_t cols, const void *x,
                                int64_t x_row_stride, int8_t *q, int64_t q_row_stride, float *scale, void *stream) {
  clear_error();
  if (int32_t rc = check_rows_args("quant_per_token_i8", dtype, rows, cols, x, x_row_stride, q, q_row_stride)) return rc;
  if (round_mode < BSIR_ROUND_RINT || round_mode > BSIR_ROUND_TRUNCWITHOVERFLOW)
    return fail(BSIR_ERR_ATTR, "quant_per_token_i8: round_mode %d", round_mode);
  if (rows == 0) return BSIR_OK;
  if (!scale) return fail(BSIR_ERR_NULL, "quant_per_token_i8: scale is null");
  const int eb = dtype_bytes(dtype);
  if (!aligned_to(x, eb) || !aligned_to(scale, 4)) return fail(BSIR_ERR_ALIGN, "quant_per_token_i8: misaligned");
  cudaStream_t st = resolve_stream(stream);
  RowGeom g;
  int vpt = 0;
  const int per_vec = 16 / eb;
  const bool aligned_ok = cols > 0 && cols % per_vec == 0 && rows_vector_ok(x, x_row_stride, eb) && aligned_to(q, per_vec) &&
                          q_row_stride % per_vec == 0;
  const bool vec_ok = aligned_ok && pick_geometry(rows, cols, eb, 16, eb == 2 ? 8 : 4, env_int("BSIR_QUANT_TPR", 0), &g, &vpt);
  if (aligned_ok && !vec_ok)   // the row does not fit one CTA's registers
    return launch_long_rows<kRowQuant>("quant_per_token_i8", dtype, rows, cols, x, x_row_stride, nullptr, 0.0f, 0.0f, q,
                                       q_row_stride, scale, round_mode, st);
  if (vec_ok) {
    const unsigned blocks = static_cast<unsigned>(ceil_div(rows, g.rpc));
    const unsigned threads = static_cast<unsigned>(g.tpr * g.rpc);
    const bool exact = (vpt == 8 || vpt == 4) && g.nvec == static_cast<int64_t>(g.tpr) * vpt && (dtype == BSIR_BF16 || dtype == BSIR_F16) &&
                       (g.tpr == 32 || g.tpr == 64 || g.tpr == 128) && !env_int("BSIR_QUANT_GENERIC", 0);
    if (exact) {
#define QUANT_EXACT(D, V, T) launch_pdl(quant_rows_kernel<D, V, T>, dim3(blocks), dim3(threads), 0, st, g, x, x_row_stride, q, q_row_stride, scale, round_mode)
#define QUANT_EXACT_T(D, V)                                                                        \
  if (g.tpr == 32) QUANT_EXACT(D, V, 32); else if (g.tpr == 64) QUANT_EXACT(D, V, 64); else QUANT_EXACT(D, V, 128)
      if (dtype == BSIR_BF16) {
        if (vpt == 8) { QUANT_EXACT_T(BSIR_BF16, 8); } else { QUANT_EXACT_T(BSIR_BF16, 4); }
      } else {
        if (vpt == 8) { QUANT_EXACT_T(BSIR_F16, 8); } else { QUANT_EXACT_T(BSIR_F16, 4); }
      }
#undef QUANT_EXACT_T
#undef QUANT_EXACT
    } else {
      DISPATCH_FLOAT_DT(dtype, DISPATCH_VPT(vpt, (launch_pdl(quant_rows_kernel<D, V, 0>, dim3(blocks), dim3(threads), 0, st, g, x,
                                                             x_row_stride, q, q_row_stride, scale, round_mode))));
    }
  } else {
    DISPATCH_FLOAT_DT(dtype, (rows_multipass_kernel<D, kRowQuant><<<static_cast<unsigned>(rows), 256, 0, st>>>(
                                 rows, cols, x, x_row_stride, nullptr, 0.0f, 0.0f, q, q_row_stride, scale, round_mode)));
  }
  count_launch();
  return check_launch("quant_per_token_i8");
}

int32_t bsir_rms_norm(int32_t dtype, int64_t rows, int64_t cols, const void *x, int64_t x_row_stride,
                      const void *gamma, float eps, void *y, int64_t y_row_stride, void *rstd_out, void *stream) {
  clear_error();
  if (int32_t rc = check_rows_args("rms_norm", dtype, rows, cols, x, x_row_stride, y, y_row_stride)) return rc;
  if (rows == 0) return BSIR_OK;
  if (!gamma && cols > 0) return fail(BSIR_ERR_NULL, "rms_norm: gamma is null");
  const int eb = dtype_bytes(dtype);
  if (!aligned_to(x, eb) || !aligned_to(y, eb) || !aligned_to(gamma, eb) || !aligned_to(rstd_out, eb))
    return fail(BSIR_ERR_ALIGN, "rms_norm: misaligned");
  cudaStream_t st = resolve_stream(stream);
  // 1.0 / float(cols), computed in f32 like the arith.divf of the reference IR
  const float avg = 1.0f / static_cast<float>(static_cast<uint32_t>(cols));
  RowGeom g;
  int vpt = 0;
  const bool aligned_ok = cols > 0 && cols % (16 / eb) == 0 && rows_vector_ok(x, x_row_stride, eb) &&
                          rows_vector_ok(y, y_row_stride, eb) && aligned_to(gamma, 16);
  const bool vec_ok = aligned_ok && pick_geometry(rows, cols, eb, 16, 4, env_int("BSIR_RMS_TPR", 0), &g, &vpt);
  if (aligned_ok && !vec_ok)
    return launch_long_rows<kRowRms>("rms_norm", dtype, rows, cols, x, x_row_stride, gamma, eps, avg, y, y_row_stride, rstd_out, 0, st);
  if (vec_ok) {
    const unsigned blocks = static_cast<unsigned>(ceil_div(rows, g.rpc));
    const unsigned threads = static_cast<unsigned>(g.tpr * g.rpc);
    DISPATCH_FLOAT_DT(dtype, DISPATCH_VPT(vpt, (rmsnorm_rows_kernel<D, V><<<blocks, threads, 0, st>>>(
                                                    g, x, x_row_stride, gamma, eps, avg, y, y_row_stride, rstd_out))));
  } else {
    DISPATCH_FLOAT_DT(dtype, (rows_multipass_kernel<D, kRowRms><<<static_cast<unsigned>(rows), 256, 0, st>>>(
                                 rows, cols, x, x_row_stride, gamma, eps, avg, y, y_row_stride, rstd_out, 0)));
  }
  count_launch();
  return check_launch("rms_norm");
}

int32_t bsir_softmax(int32_t dtype, int64_t rows, int64_t cols, const void *x, int64_t x_row_stride, void *y,
                     int64_t y_row_stride, void *stream) {
  clear_error();
  if (int32_t rc = check_rows_args("softmax", dtype, rows, cols, x, x_row_stride, y, y_row_stride)) return rc;
  if (rows == 0 || cols == 0) return BSIR_OK;
  const int eb = dtype_bytes(dtype);
  if (!aligned_to(x, eb) || !aligned_to(y, eb)) return fail(BSIR_ERR_ALIGN, "softmax: misaligned");
  cudaStream_t st = resolve_stream(stream);
  RowGeom g;
  int vpt = 0;
  // exp values live in registers: at most 32 per thread
  const int max_vpt = eb == 4 ? 8 : 4;
  const bool aligned_ok = cols % (16 / eb) == 0 && rows_vector_ok(x, x_row_stride, eb) && rows_vector_ok(y, y_row_stride, eb);
  const bool vec_ok = aligned_ok && pick_geometry(rows, cols, eb, max_vpt, 4, env_int("BSIR_SOFTMAX_TPR", 0), &g, &vpt);
  if (aligned_ok && !vec_ok)
    return launch_long_rows<kRowSoftmax>("softmax", dtype, rows, cols, x, x_row_stride, nullptr, 0.0f, 0.0f, y, y_row_stride, nullptr, 0, st);
  // long rows: persistent CTAs with the rows streamed through shared memory by bulk copies
  const bool want_stream = env_int("BSIR_SOFTMAX_STREAM", 1) != 0;
  if (vec_ok && want_stream && g.tpr == 1024 && g.nvec >= 2048 && g.nvec * 16 <= 65536 && device_info().cc_major >= 9) {
    const size_t smem = static_cast<size_t>(kStreamBufs) * static_cast<size_t>(g.nvec) * 16u;
    int grid = device_info().sm_count > 0 ? device_info().sm_count : 148;
    if (grid > rows) grid = static_cast<int>(rows);
    int *err = device_error_word();
    DISPATCH_FLOAT_DT(dtype, DISPATCH_VPT_LE8(vpt, {
      cudaFuncSetAttribute(softmax_stream_kernel<D, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      softmax_stream_kernel<D, V><<<grid, 1024, smem, st>>>(g, x, x_row_stride, y, y_row_stride, err);
    }));
    count_launch();
    return check_launch("softmax");
  }
  if (vec_ok) {
    const unsigned blocks = static_cast<unsigned>(ceil_div(rows, g.rpc));
    const unsigned threads = static_cast<unsigned>(g.tpr * g.rpc);
    DISPATCH_FLOAT_DT(dtype, DISPATCH_VPT_LE8(vpt, (softmax_rows_kernel<D, V><<<blocks, threads, 0, st>>>(
                                                        g, x, x_row_stride, y, y_row_stride))));
  } else {
    DISPATCH_FLOAT_DT(dtype, (rows_multipass_kernel<D, kRowSoftmax><<<static_cast<unsigned>(rows), 256, 0, st>>>(
                                 rows, cols, x, x_row_stride, nullptr, 0.0f, 0.0f, y, y_row_stride, nullptr, 0)));
  }
  count_launch();
  return check_launch("softmax");
}

}  // extern "C"
