// cumulative.cu -- hivm.hir.vcumsum / vcumprod / vcummax / vcummin over one axis of a [rows, cols] problem
// (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:1937-2220).
//
// Semantics restated from the reference's scalar lowering (test/Dialect/HIVM/hivm-lower-to-loops-op.mlir:1558-1599):
// dst[0] = src[0]; dst[i] = src[i] (op) dst[i-1], in index order (from the last index backwards with
// reverse).  f16 / bf16 run in f32 and round once per output (the cast-up / cast-down normalisation of
// lib/Dialect/HIVM/Transforms/regbase/Normalize/NormalizeTypeConversion.cpp:714-745,818-822); integers
// wrap in their own width.  Float sums are not associative, so the scan along the axis stays sequential
// and the parallelism is across the other axis:
//   * axis 0: a thread owns a column (or the 16 bytes of columns of one vector) and walks down the rows,
//     loads of the next rows in flight while it adds;
//   * axis 1: a warp owns 32 rows; it brings a 32 x 128-byte tile into shared memory with coalesced
//     16-byte cp.async copies (a ring of four tiles in flight per warp), every lane scans its own row of the tile 16 bytes
//     at a time (row pitch 36 words: conflict-free 16-byte accesses), and the tile goes back with coalesced 16-byte stores.
#include <cstdint>
#include <cstring>
#include <type_traits>

#include "common.cuh"

namespace bsir {
namespace {

enum CumKind { kCumSum = 0, kCumProd = 1, kCumMax = 2, kCumMin = 3 };

template <typename T> struct CumAcc { using type = T; };
template <> struct CumAcc<__half> { using type = float; };
template <> struct CumAcc<__nv_bfloat16> { using type = float; };
template <> struct CumAcc<int8_t> { using type = int32_t; };
template <> struct CumAcc<int16_t> { using type = int32_t; };

template <typename T> __device__ __forceinline__ typename CumAcc<T>::type cum_widen(T v) { return static_cast<typename CumAcc<T>::type>(v); }
template <> __device__ __forceinline__ float cum_widen<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float cum_widen<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T cum_narrow(typename CumAcc<T>::type v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ __half cum_narrow<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cum_narrow<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// x (op) acc, the operand order of the reference's loop body
template <int KIND, bool NANP, typename A>
__device__ __forceinline__ A cum_comb(A x, A acc) {
  if constexpr (std::is_same<A, float>::value) {
    if constexpr (KIND == kCumSum) return __fadd_rn(x, acc);
    else if constexpr (KIND == kCumProd) return __fmul_rn(x, acc);
    else if constexpr (KIND == kCumMax) return NANP ? maximumf(x, acc) : fmaxf(x, acc);
    else return NANP ? minimumf(x, acc) : fminf(x, acc);
  } else {
    using U = typename std::make_unsigned<A>::type;
    if constexpr (KIND == kCumSum) return static_cast<A>(static_cast<U>(x) + static_cast<U>(acc));
    else if constexpr (KIND == kCumProd) return static_cast<A>(static_cast<U>(x) * static_cast<U>(acc));
    else if constexpr (KIND == kCumMax) return x > acc ? x : acc;
    else return x < acc ? x : acc;
  }
}

// One step of the scan.  The running value of 16-bit floats stays in f32 (only the stored copy is rounded);
// 8- and 16-bit integers wrap in their own width at every step.
template <typename T, int KIND, bool NANP>
__device__ __forceinline__ typename CumAcc<T>::type cum_step(typename CumAcc<T>::type acc, T x, bool first) {
  using A = typename CumAcc<T>::type;
  if (first) return cum_widen<T>(x);
  const A r = cum_comb<KIND, NANP, A>(cum_widen<T>(x), acc);
  if constexpr (std::is_integral<T>::value && sizeof(T) < 4) return cum_widen<T>(cum_narrow<T>(r));   // wrap in T
  else return r;
}

// ------------------------------------------------------------------ axis 0: a thread per column
template <typename T, int KIND, bool NANP>
__global__ void __launch_bounds__(64) cum_first_seq_kernel(const T *__restrict__ src, T *__restrict__ dst, int64_t rows, int64_t cols,
                                                            int64_t ss, int64_t ds, int reverse) {
  using A = typename CumAcc<T>::type;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  constexpr int kAhead = 16;   // rows requested before the first of them is used
  A acc{};
  for (int64_t r0 = 0; r0 < rows; r0 += kAhead) {
    T v[kAhead];
#pragma unroll
    for (int k = 0; k < kAhead; ++k)
      if (r0 + k < rows) v[k] = src[(reverse ? rows - 1 - (r0 + k) : r0 + k) * ss + c];
#pragma unroll
    for (int k = 0; k < kAhead; ++k) {
      const int64_t r = r0 + k;
      if (r >= rows) break;
      acc = cum_step<T, KIND, NANP>(acc, v[k], r == 0);
      dst[(reverse ? rows - 1 - r : r) * ds + c] = cum_narrow<T>(acc);
    }
  }
}

// ------------------------------------------------------------------ axis 1: a warp per 32 rows, tiles of 128 bytes
constexpr int kCumWarps = 2;   // two warps x four tiles of 4.5 KB: 36 KB of static shared memory
// words per tile row in shared memory: 36, so that every row starts on a 16-byte boundary and the rows of the
// eight lanes that share a 16-byte access phase start in different banks (lane * 36 mod 32 = 4 * lane)
constexpr int kCumPitch = 36;

template <typename T, int KIND, bool NANP>
__global__ void __launch_bounds__(kCumWarps * 32) cum_last_kernel(const T *__restrict__ src, T *__restrict__ dst, int64_t rows,
                                                                   int64_t cols, int64_t ss, int64_t ds, int reverse) {
  using A = typename CumAcc<T>::type;
  constexpr int EPT = 128 / sizeof(T);              // elements of a tile row
  constexpr int EPV = 16 / sizeof(T);               // elements of a 16-byte chunk
  constexpr int kDepth = 4;                          // tiles in flight per warp (cp.async ring)
  __shared__ __align__(16) uint32_t sm[kCumWarps][kDepth][32 * kCumPitch];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row0 = (static_cast<int64_t>(blockIdx.x) * kCumWarps + warp) * 32;
  if (row0 >= rows) return;
  const int64_t ntiles = cols / EPT;                // the host sends only whole tiles here
  const char *sb = reinterpret_cast<const char *>(src);
  char *db = reinterpret_cast<char *>(dst);

  // lane -> (row i*4 + lane/8, 16-byte chunk lane%8) of a tile; one commit group per tile, empty past the end
  auto fetch = [&](int64_t it) {
    if (it < ntiles) {
      const int64_t t = reverse ? ntiles - 1 - it : it;
      uint32_t *tile = sm[warp][it % kDepth];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int64_t r = row0 + i * 4 + lane / 8;
        if (r < rows) {
          const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(tile + (i * 4 + lane / 8) * kCumPitch + (lane % 8) * 4));
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(sb + (r * ss + t * EPT) * sizeof(T) + (lane % 8) * 16) : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  for (int64_t it = 0; it < kDepth - 1; ++it) fetch(it);
  A acc{};
  for (int64_t it = 0; it < ntiles; ++it) {
    const int64_t t = reverse ? ntiles - 1 - it : it;
    uint32_t *tile = sm[warp][it % kDepth];
    fetch(it + kDepth - 1);                           // its buffer was drained in the previous iteration
    asm volatile("cp.async.wait_group %0;" ::"n"(kDepth - 1) : "memory");
    __syncwarp();
    // lane = row: scan the 128 bytes of this row in place, 16 bytes at a time
    if (row0 + lane < rows) {
      uint4 *mine = reinterpret_cast<uint4 *>(tile + lane * kCumPitch);
      auto scan = [&](auto rev_tag) {                 // the direction is a compile-time constant inside
        constexpr bool REV = decltype(rev_tag)::value;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int cc = REV ? 7 - c : c;
          const uint4 raw = mine[cc];
          T x[EPV];
          memcpy(x, &raw, 16);
#pragma unroll
          for (int e = 0; e < EPV; ++e) {
            const int j = REV ? EPV - 1 - e : e;
            acc = cum_step<T, KIND, NANP>(acc, x[j], it == 0 && c == 0 && e == 0);
            x[j] = cum_narrow<T>(acc);
          }
          uint4 res;
          memcpy(&res, x, 16);
          mine[cc] = res;
        }
      };
      if (reverse) scan(std::true_type{});
      else scan(std::false_type{});
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int64_t r = row0 + i * 4 + lane / 8;
      const uint4 w = *reinterpret_cast<const uint4 *>(tile + (i * 4 + lane / 8) * kCumPitch + (lane % 8) * 4);
      Vec16 o;
      o.w[0] = w.x; o.w[1] = w.y; o.w[2] = w.z; o.w[3] = w.w;
      if (r < rows) st_stream(db + (r * ds + t * EPT) * sizeof(T) + (lane % 8) * 16, o);
    }
    __syncwarp();                                     // the buffer may be refilled from the next iteration on
  }
}

// generality path for axis 1: a thread per row (ragged or unaligned rows)
template <typename T, int KIND, bool NANP>
__global__ void __launch_bounds__(128) cum_last_seq_kernel(const T *__restrict__ src, T *__restrict__ dst, int64_t rows, int64_t cols,
                                                           int64_t ss, int64_t ds, int reverse) {
  using A = typename CumAcc<T>::type;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  A acc{};
  for (int64_t e = 0; e < cols; ++e) {
    const int64_t j = reverse ? cols - 1 - e : e;
    acc = cum_step<T, KIND, NANP>(acc, src[r * ss + j], e == 0);
    dst[r * ds + j] = cum_narrow<T>(acc);
  }
}

template <typename T, int KIND, bool NANP>
void launch_cum(int axis, int reverse, int64_t rows, int64_t cols, const void *src, int64_t ss, void *dst, int64_t ds, cudaStream_t st) {
  const T *s = static_cast<const T *>(src);
  T *d = static_cast<T *>(dst);
  if (axis == 0) {
    // small blocks: a tall, narrow problem has few columns, and they should spread over the SMs
    cum_first_seq_kernel<T, KIND, NANP><<<static_cast<unsigned>(ceil_div(cols, 64)), 64, 0, st>>>(s, d, rows, cols, ss, ds, reverse);
    return;
  }
  constexpr int64_t ept = 128 / sizeof(T);
  const bool tiles = cols % ept == 0 && aligned_to(src, 16) && aligned_to(dst, 16) && (ss * sizeof(T)) % 16 == 0 && (ds * sizeof(T)) % 16 == 0;
  if (tiles) cum_last_kernel<T, KIND, NANP><<<static_cast<unsigned>(ceil_div(rows, 32 * kCumWarps)), kCumWarps * 32, 0, st>>>(s, d, rows, cols, ss, ds, reverse);
  else cum_last_seq_kernel<T, KIND, NANP><<<static_cast<unsigned>(ceil_div(rows, 128)), 128, 0, st>>>(s, d, rows, cols, ss, ds, reverse);
}

template <typename T>
void launch_cum_kind(int kind, int nanp, int axis, int reverse, int64_t rows, int64_t cols, const void *src, int64_t ss, void *dst,
                     int64_t ds, cudaStream_t st) {
  switch (kind) {
    case kCumSum: launch_cum<T, kCumSum, false>(axis, reverse, rows, cols, src, ss, dst, ds, st); break;
    case kCumProd: launch_cum<T, kCumProd, false>(axis, reverse, rows, cols, src, ss, dst, ds, st); break;
    case kCumMax:
      if (nanp) launch_cum<T, kCumMax, true>(axis, reverse, rows, cols, src, ss, dst, ds, st);
      else launch_cum<T, kCumMax, false>(axis, reverse, rows, cols, src, ss, dst, ds, st);
      break;
    default:
      if (nanp) launch_cum<T, kCumMin, true>(axis, reverse, rows, cols, src, ss, dst, ds, st);
      else launch_cum<T, kCumMin, false>(axis, reverse, rows, cols, src, ss, dst, ds, st);
      break;
  }
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" int32_t bsir_cumulative(int32_t kind, int32_t dtype, int32_t axis, int32_t reverse, int32_t propagate_nan, int64_t rows,
                                   int64_t cols, const void *src, int64_t src_row_stride, void *dst, int64_t dst_row_stride,
                                   void *stream) {
  clear_error();
  if (kind < BSIR_CUM_SUM || kind > BSIR_CUM_MIN) return fail(BSIR_ERR_ATTR, "cumulative: kind %d", kind);
  if (axis != 0 && axis != 1) return fail(BSIR_ERR_ATTR, "cumulative: axis %d of a [rows, cols] problem", axis);
  if (rows < 0 || cols < 0) return fail(BSIR_ERR_SHAPE, "cumulative: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  const int eb = dtype_bytes(dtype);
  const bool ok_type = dtype == BSIR_F32 || dtype == BSIR_F16 || dtype == BSIR_BF16 || dtype == BSIR_I8 || dtype == BSIR_I16 ||
                       dtype == BSIR_I32 || dtype == BSIR_I64;
  if (!ok_type) return fail(BSIR_ERR_DTYPE, "cumulative: dtype %d (f32, f16, bf16, i8, i16, i32, i64)", dtype);
  if (rows == 0 || cols == 0) return BSIR_OK;
  if (!src || !dst) return fail(BSIR_ERR_NULL, "cumulative: null pointer");
  if (src_row_stride < cols || dst_row_stride < cols) return fail(BSIR_ERR_STRIDE, "cumulative: row stride below the row length");
  if (!aligned_to(src, eb) || !aligned_to(dst, eb)) return fail(BSIR_ERR_ALIGN, "cumulative: misaligned");
  cudaStream_t st = resolve_stream(stream);
  const int nanp = propagate_nan != 0;
  switch (dtype) {
    case BSIR_F32: launch_cum_kind<float>(kind, nanp, axis, reverse != 0, rows, cols, src, src_row_stride, dst, dst_row_stride, st); break;
    case BSIR_F16: launch_cum_kind<__half>(kind, nanp, axis, reverse != 0, rows, cols, src, src_row_stride, dst, dst_row_stride, st); break;
    case BSIR_BF16: launch_cum_kind<__nv_bfloat16>(kind, nanp, axis, reverse != 0, rows, cols, src, src_row_stride, dst, dst_row_stride, st); break;
    case BSIR_I8: launch_cum_kind<int8_t>(kind, 0, axis, reverse != 0, rows, cols, src, src_row_stride, dst, dst_row_stride, st); break;
    case BSIR_I16: launch_cum_kind<int16_t>(kind, 0, axis, reverse != 0, rows, cols, src, src_row_stride, dst, dst_row_stride, st); break;
    case BSIR_I32: launch_cum_kind<int32_t>(kind, 0, axis, reverse != 0, rows, cols, src, src_row_stride, dst, dst_row_stride, st); break;
    default: launch_cum_kind<int64_t>(kind, 0, axis, reverse != 0, rows, cols, src, src_row_stride, dst, dst_row_stride, st); break;
  }
  count_launch();
  return check_launch("cumulative");
}
