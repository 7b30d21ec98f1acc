// cumulative.cu -- hivm.hir.vcumsum / vcumprod / vcummax / vcummin over one axis of a [rows, cols] problem
// (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:1937-2220).
//
// Semantics restated from the reference's scalar lowering (test/Dialect/HIVM/hivm-lower-to-loops-op.mlir:1558-1599):
// dst[0] = src[0]; dst[i] = src[i] (op) dst[i-1], in index order (from the last index backwards with
// reverse).  f16 / bf16 run in f32 and round once per output (the cast-up / cast-down normalisation of
// lib/Dialect/HIVM/Transforms/regbase/Normalize/NormalizeTypeConversion.cpp:714-745,818-822); integers
// wrap in their own width.  Float sums are not associative, so the scan along the axis stays sequential
// and the parallelism is across the other axis:
//   * axis 0: a warp owns 128 bytes of columns and walks down the rows through tiles the copy engine brings and
//     takes back (without a tensor-map encoder, or for short or unaligned problems: a thread per column, the loads
//     of the next 16 rows in flight while it adds);
//   * axis 1: a warp owns 32 rows and every lane scans its own row of a 32-row x 128-byte tile in shared memory,
//     16 bytes at a time.  The tiles come and go through the copy engine (a tensor map over the rows as bytes,
//     128-byte swizzle); without a tensor-map encoder, with coalesced 16-byte cp.async copies into tiles of row
//     pitch 36 words (conflict-free 16-byte accesses) and coalesced 16-byte stores, a ring of six tiles per warp.
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "tc_ptx.cuh"

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

// The same walk down the rows with the copy engine doing the memory side: a warp owns 128 bytes of columns (a lane
// the 4-byte word of one, two or four of them) and gets tiles of 64 or 128 rows x 128 bytes through a 2-D tensor map over the
// rows as bytes, scans them in place in shared memory and hands them back the same way.  What the thread-per-column
// kernel can keep in flight is what fits its registers (16 rows); here it is the ring of tiles -- up to
// 192 KB an SM -- which is what a column-wise walk over rows 16 KB apart needs to keep HBM busy.
constexpr int kCumColMaxDepth = 24;                  // 192 KB of 64-row tiles

// A whole tile that is not the first of its columns: every offset is a constant, so a row costs its load,
// its adds and its store -- with one warp on its scheduler each instruction waits for the one before, and every
// instruction saved shows.
template <typename T, int KIND, bool NANP, bool REV, int kCumColRows>
__device__ __forceinline__ void cum_col_full_tile(uint32_t *col, typename CumAcc<T>::type (&acc)[4 / sizeof(T)]) {
  constexpr int EPW = 4 / sizeof(T);
  constexpr int kGroups = kCumColRows / 8;
  auto at = [](int q) { return (REV ? kCumColRows - 1 - q : q) * 32; };
  uint32_t w[2][8];                                   // the next eight rows are loaded while these eight are added
#pragma unroll
  for (int k = 0; k < 8; ++k) w[0][k] = col[at(k)];
#pragma unroll
  for (int g = 0; g < kGroups; ++g) {
    if (g + 1 < kGroups) {
#pragma unroll
      for (int k = 0; k < 8; ++k) w[(g + 1) & 1][k] = col[at((g + 1) * 8 + k)];
    }
    uint32_t out[8];                                  // the chain of adds first, its eight stores after it
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      T x[EPW];
      memcpy(x, &w[g & 1][k], 4);
#pragma unroll
      for (int e = 0; e < EPW; ++e) {
        acc[e] = cum_step<T, KIND, NANP>(acc[e], x[e], false);
        x[e] = cum_narrow<T>(acc[e]);
      }
      memcpy(&out[k], x, 4);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) col[at(g * 8 + k)] = out[k];
  }
}

template <typename T, int KIND, bool NANP, int kCumColRows>
__global__ void __launch_bounds__(32) cum_first_tma_kernel(const __grid_constant__ CUtensorMap tsrc, const __grid_constant__ CUtensorMap tdst,
                                                           int64_t rows, int reverse, int depth, int *err) {
  using A = typename CumAcc<T>::type;
  constexpr int EPW = 4 / sizeof(T);                 // columns in a lane's word
  constexpr int kCumColTileBytes = kCumColRows * 128;
  extern __shared__ __align__(1024) uint8_t tiles[];   // depth tiles
  __shared__ __align__(8) uint64_t full[kCumColMaxDepth];
  __shared__ int abort_flag;
  const int lane = threadIdx.x;
  const int x0 = static_cast<int>(blockIdx.x) * 128;
  const int64_t ntiles = (rows + kCumColRows - 1) / kCumColRows;
  if (lane == 0) {
    for (int b = 0; b < kCumColMaxDepth; ++b) mbar_init(smem_u32(&full[b]), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tsrc);
    prefetch_tmap(&tdst);
  }
  __syncwarp();
  auto fetch = [&](int64_t it) {                      // lane 0 only
    if (it < ntiles) {
      const int64_t s = reverse ? ntiles - 1 - it : it;
      const int b = static_cast<int>(it % depth);
      mbar_expect_tx(smem_u32(&full[b]), kCumColTileBytes);
      tma_load_2d(smem_u32(tiles + b * kCumColTileBytes), &tsrc, x0, static_cast<int>(s * kCumColRows), smem_u32(&full[b]));
    }
  };
  if (lane == 0)
    for (int64_t it = 0; it < depth - 2; ++it) fetch(it);
  A acc[EPW];
#pragma unroll
  for (int e = 0; e < EPW; ++e) acc[e] = A{};
  for (int64_t it = 0; it < ntiles; ++it) {
    const int64_t s = reverse ? ntiles - 1 - it : it;
    const int b = static_cast<int>(it % depth);
    const int64_t left = rows - s * kCumColRows;
    const int nv = left < kCumColRows ? static_cast<int>(left) : kCumColRows;       // rows of this tile that exist
    if (!mbar_wait(smem_u32(&full[b]), static_cast<uint32_t>(it / depth) & 1u, &abort_flag, err)) break;
    uint32_t *col = reinterpret_cast<uint32_t *>(tiles + b * kCumColTileBytes) + lane;   // 32 words a row
    if (it > 0 && nv == kCumColRows) {
      if (reverse) cum_col_full_tile<T, KIND, NANP, true, kCumColRows>(col, acc);
      else cum_col_full_tile<T, KIND, NANP, false, kCumColRows>(col, acc);
    } else
    for (int q0 = 0; q0 < nv; q0 += 8) {
      uint32_t w[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {                   // all eight loads before the first add
        const int q = q0 + k < nv ? q0 + k : nv - 1;
        w[k] = col[(reverse ? nv - 1 - q : q) * 32];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int q = q0 + k;
        if (q < nv) {
          T x[EPW];
          memcpy(x, &w[k], 4);
#pragma unroll
          for (int e = 0; e < EPW; ++e) {
            acc[e] = cum_step<T, KIND, NANP>(acc[e], x[e], it == 0 && q == 0);
            x[e] = cum_narrow<T>(acc[e]);
          }
          uint32_t out;
          memcpy(&out, x, 4);
          col[(reverse ? nv - 1 - q : q) * 32] = out;
        }
      }
    }
    if (lane == 0) {
      // the buffer of tile it + depth - 2 went out two tiles ago; only the last store may still be reading its own
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      fetch(it + depth - 2);
    }
    fence_proxy_async();                              // the lanes' writes, before the copy engine reads them
    __syncwarp();
    if (lane == 0) {
      asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(reinterpret_cast<uint64_t>(&tdst)),
                   "r"(x0), "r"(static_cast<int>(s * kCumColRows)), "r"(smem_u32(tiles + b * kCumColTileBytes))
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  }
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// ------------------------------------------------------------------ axis 1: a warp per 32 rows, tiles of 128 bytes
constexpr int kCumWarps = 1;   // one warp x six tiles of 4.5 KB: 27 KB of static shared memory (the path without tensor maps)
// words per tile row in shared memory: 36, so that every row starts on a 16-byte boundary and the rows of the
// eight lanes that share a 16-byte access phase start in different banks (lane * 36 mod 32 = 4 * lane)
constexpr int kCumPitch = 36;

template <typename T, int KIND, bool NANP>
__global__ void __launch_bounds__(kCumWarps * 32) cum_last_kernel(const T *__restrict__ src, T *__restrict__ dst, int64_t rows,
                                                                   int64_t cols, int64_t ss, int64_t ds, int reverse) {
  using A = typename CumAcc<T>::type;
  constexpr int EPT = 128 / sizeof(T);              // elements of a tile row
  constexpr int EPV = 16 / sizeof(T);               // elements of a 16-byte chunk
  constexpr int kDepth = 6;                          // tiles in flight per warp (cp.async ring)
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

// The same walk with the tiles moved by the copy engine: a 2-D tensor map over the rows as bytes (box 32 rows x 128
// bytes, 128-byte swizzle, so that the 32 lanes' 16-byte accesses to their own rows fall into different banks) brings
// a tile with one instruction and takes it back with another, which leaves the warp's instruction stream to the
// scan itself -- with one lane a row and two warps a scheduler at best, every instruction it does not issue counts.
// A ring of `depth` steps per warp (as many as the warps that share an SM leave room for); the load that refills a
// buffer is issued a scan after the store that emptied it.  Rows past the end read as zero and are not written.
constexpr int kCumTmaMaxDepth = 11;                  // 44 KB of tiles: within the shared memory a kernel gets unasked
constexpr int kCumTileBytes = 32 * 128;

template <typename T, int KIND, bool NANP, int W>
__global__ void __launch_bounds__(32) cum_last_tma_kernel(const __grid_constant__ CUtensorMap tsrc, const __grid_constant__ CUtensorMap tdst,
                                                          int64_t cols, int reverse, int depth, int *err) {
  // a step is W neighbouring tiles of a row block (W x 128 bytes of each row), fetched together: the wider the
  // stretch of a row that is asked for at once, the fewer times DRAM opens a page for 128 bytes
  using A = typename CumAcc<T>::type;
  constexpr int EPV = 16 / sizeof(T);               // elements of a 16-byte chunk
  constexpr int kStepBytes = W * kCumTileBytes;
  extern __shared__ __align__(1024) uint8_t tiles[];   // depth steps
  __shared__ __align__(8) uint64_t full[kCumTmaMaxDepth];
  __shared__ int abort_flag;
  const int lane = threadIdx.x;
  const int row0 = static_cast<int>(blockIdx.x) * 32;
  const int64_t ntiles = cols * static_cast<int64_t>(sizeof(T)) / 128;
  const int64_t nsteps = (ntiles + W - 1) / W;
  if (lane == 0) {
#pragma unroll
    for (int b = 0; b < kCumTmaMaxDepth; ++b) mbar_init(smem_u32(&full[b]), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tsrc);
    prefetch_tmap(&tdst);
  }
  __syncwarp();
  auto fetch = [&](int64_t it) {                      // lane 0 only
    if (it < nsteps) {
      const int64_t s = reverse ? nsteps - 1 - it : it;
      const int b = static_cast<int>(it % depth);
      const int nb = static_cast<int>(ntiles - s * W < W ? ntiles - s * W : W);
      mbar_expect_tx(smem_u32(&full[b]), static_cast<uint32_t>(nb) * kCumTileBytes);
      for (int j = 0; j < nb; ++j)
        tma_load_2d(smem_u32(tiles + b * kStepBytes + j * kCumTileBytes), &tsrc, static_cast<int>((s * W + j) * 128), row0, smem_u32(&full[b]));
    }
  };
  if (lane == 0)
    for (int64_t it = 0; it < depth - 1; ++it) fetch(it);
  A acc{};
  for (int64_t it = 0; it < nsteps; ++it) {
    const int64_t s = reverse ? nsteps - 1 - it : it;
    const int b = static_cast<int>(it % depth);
    const int nb = static_cast<int>(ntiles - s * W < W ? ntiles - s * W : W);
    if (!mbar_wait(smem_u32(&full[b]), static_cast<uint32_t>(it / depth) & 1u, &abort_flag, err)) break;
#pragma unroll
    for (int jj = 0; jj < W; ++jj) {
      if (jj < nb) {
        const int j = reverse ? nb - 1 - jj : jj;
        // lane = row: chunk c of the row sits at c ^ (row % 8) within the row's 128 bytes
        uint4 *mine = reinterpret_cast<uint4 *>(tiles + b * kStepBytes + j * kCumTileBytes + lane * 128);
        uint4 raw[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) raw[c] = mine[c ^ (lane & 7)];
        auto scan = [&](auto rev_tag) {               // the direction is a compile-time constant inside
          constexpr bool REV = decltype(rev_tag)::value;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const int cc = REV ? 7 - c : c;
            T x[EPV];
            memcpy(x, &raw[cc], 16);
#pragma unroll
            for (int e = 0; e < EPV; ++e) {
              const int k = REV ? EPV - 1 - e : e;
              acc = cum_step<T, KIND, NANP>(acc, x[k], it == 0 && jj == 0 && c == 0 && e == 0);
              x[k] = cum_narrow<T>(acc);
            }
            memcpy(&raw[cc], x, 16);
          }
        };
        if (reverse) scan(std::true_type{});
        else scan(std::false_type{});
#pragma unroll
        for (int c = 0; c < 8; ++c) mine[c ^ (lane & 7)] = raw[c];
      }
    }
    if (lane == 0) {
      // the buffer of step it + depth - 1 went out one step ago, a whole scan back: its store has read it by now
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      fetch(it + depth - 1);
    }
    fence_proxy_async();                              // the lanes' writes, before the copy engine reads them
    __syncwarp();
    if (lane == 0) {
      for (int j = 0; j < nb; ++j)
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(reinterpret_cast<uint64_t>(&tdst)),
                     "r"(static_cast<int>((s * W + j) * 128)), "r"(row0), "r"(smem_u32(tiles + b * kStepBytes + j * kCumTileBytes))
                     : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  }
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
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
    if constexpr (sizeof(T) <= 4) {
      const int64_t row_bytes = cols * static_cast<int64_t>(sizeof(T));
      if (rows >= 256 && rows <= 0x7fffffffLL && row_bytes <= 0x7fffffffLL && aligned_to(src, 16) && aligned_to(dst, 16) &&
          (ss * sizeof(T)) % 16 == 0 && (ds * sizeof(T)) % 16 == 0 && std::getenv("BSIR_CUM_NO_TMA") == nullptr) {
        // the ring as deep as the warps that will share an SM leave room for (about 200 KB among them); tiles of 128
        // rows (half as many waits, fences and copies a row) when that still leaves a ring of four
        const int64_t groups = ceil_div(row_bytes, static_cast<int64_t>(128));
        const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
        int64_t per_sm = ceil_div(groups, static_cast<int64_t>(sms));
        if (per_sm > 16) per_sm = 16;
        const int room = static_cast<int>((200 * 1024 / per_sm - 1024) / (64 * 128));     // 64-row tiles a warp may hold
        const int tile_rows = room >= 8 ? 128 : 64;
        int depth = tile_rows == 128 ? room / 2 : room;
        depth = depth < 3 ? 3 : depth > kCumColMaxDepth * 64 / tile_rows ? kCumColMaxDepth * 64 / tile_rows : depth;   // three at least: in use, going out, coming in
        const size_t smem = static_cast<size_t>(depth) * tile_rows * 128;
        CUtensorMap tsrc, tdst;
        if (make_byte_tmap(&tsrc, src, static_cast<uint64_t>(row_bytes), static_cast<uint64_t>(rows), static_cast<uint64_t>(ss) * sizeof(T), tile_rows, false) &&
            make_byte_tmap(&tdst, dst, static_cast<uint64_t>(row_bytes), static_cast<uint64_t>(rows), static_cast<uint64_t>(ds) * sizeof(T), tile_rows, false)) {
          if (tile_rows == 128) {
            cudaFuncSetAttribute(cum_first_tma_kernel<T, KIND, NANP, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCumColMaxDepth * 64 * 128);
            cum_first_tma_kernel<T, KIND, NANP, 128><<<static_cast<unsigned>(groups), 32, smem, st>>>(tsrc, tdst, rows, reverse, depth, device_error_word());
          } else {
            cudaFuncSetAttribute(cum_first_tma_kernel<T, KIND, NANP, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCumColMaxDepth * 64 * 128);
            cum_first_tma_kernel<T, KIND, NANP, 64><<<static_cast<unsigned>(groups), 32, smem, st>>>(tsrc, tdst, rows, reverse, depth, device_error_word());
          }
          return;
        }
      }
    }
    // small blocks: a tall, narrow problem has few columns, and they should spread over the SMs
    cum_first_seq_kernel<T, KIND, NANP><<<static_cast<unsigned>(ceil_div(cols, 64)), 64, 0, st>>>(s, d, rows, cols, ss, ds, reverse);
    return;
  }
  constexpr int64_t ept = 128 / sizeof(T);
  const bool tiles = cols % ept == 0 && aligned_to(src, 16) && aligned_to(dst, 16) && (ss * sizeof(T)) % 16 == 0 && (ds * sizeof(T)) % 16 == 0;
  if (tiles && rows <= 0x7fffffffLL && cols * static_cast<int64_t>(sizeof(T)) <= 0x7fffffffLL && std::getenv("BSIR_CUM_NO_TMA") == nullptr) {
    CUtensorMap tsrc, tdst;
    if (make_byte_tmap(&tsrc, src, static_cast<uint64_t>(cols) * sizeof(T), static_cast<uint64_t>(rows), static_cast<uint64_t>(ss) * sizeof(T), 32) &&
        make_byte_tmap(&tdst, dst, static_cast<uint64_t>(cols) * sizeof(T), static_cast<uint64_t>(rows), static_cast<uint64_t>(ds) * sizeof(T), 32)) {
      // the ring as deep as the warps that will share an SM leave room for (about 200 KB among them)
      const int64_t blocks = ceil_div(rows, static_cast<int64_t>(32));
      const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
      int64_t per_sm = ceil_div(blocks, static_cast<int64_t>(sms));
      if (per_sm > 16) per_sm = 16;
      const int room = static_cast<int>((200 * 1024 / per_sm - 1024) / kCumTileBytes);      // tiles a warp may hold
      int wide = room >= 6 ? 2 : 1;
      if (const char *e = std::getenv("BSIR_CUM_WIDE")) wide = std::atoi(e) == 2 ? 2 : 1;
      int depth = room / wide;
      depth = depth < 2 ? 2 : depth * wide > kCumTmaMaxDepth ? kCumTmaMaxDepth / wide : depth;
      const size_t smem = static_cast<size_t>(depth) * wide * kCumTileBytes;
      if (wide == 2) cum_last_tma_kernel<T, KIND, NANP, 2><<<static_cast<unsigned>(blocks), 32, smem, st>>>(tsrc, tdst, cols, reverse, depth, device_error_word());
      else cum_last_tma_kernel<T, KIND, NANP, 1><<<static_cast<unsigned>(blocks), 32, smem, st>>>(tsrc, tdst, cols, reverse, depth, device_error_word());
      return;
    }
  }
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
