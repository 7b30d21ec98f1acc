// reduce.cu -- linalg.reduce / hivm.hir.vreduce over one axis of a 2-D view and
// hfusion.reduce_with_index (argmax / argmin) over the last axis.
//
// Combiners are the ones the reference's CPU lowering emits
// (bishengir/lib/ExecutionEngine/ConvertHIVMToUpstream.cpp:573-753): addf/addi, mulf/muli,
// maximumf/minimumf (NaN-propagating) and maxsi/minsi/maxui/minui, xori/ori/andi; dst is
// write-only and starts from the identity (bishengir/lib/Dialect/HIVM/IR/HIVMVectorOps.cpp:571-640).
// Float sums are accumulated in f32 (f16 sums are promoted by the reference too:
// bishengir/lib/Dialect/HFusion/Transforms/Normalize.cpp:7679-7716) in a tree order, so they
// match the sequential CPU order only to rounding; everything else is order-independent.
#include <cstdlib>
#include <climits>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace bsir {
namespace {

// ------------------------------------------------------------------ generic reductions
template <int DT> struct Acc;  // accumulator type per storage type
template <> struct Acc<BSIR_F32> { using type = float; using elem = float; };
template <> struct Acc<BSIR_F16> { using type = float; using elem = uint16_t; };
template <> struct Acc<BSIR_BF16> { using type = float; using elem = uint16_t; };
template <> struct Acc<BSIR_I8> { using type = int32_t; using elem = int8_t; };
template <> struct Acc<BSIR_I16> { using type = int32_t; using elem = int16_t; };
template <> struct Acc<BSIR_I32> { using type = int32_t; using elem = int32_t; };
template <> struct Acc<BSIR_I64> { using type = long long; using elem = int64_t; };
template <> struct Acc<BSIR_U8> { using type = uint32_t; using elem = uint8_t; };
template <> struct Acc<BSIR_U16> { using type = uint32_t; using elem = uint16_t; };
template <> struct Acc<BSIR_U32> { using type = uint32_t; using elem = uint32_t; };
template <> struct Acc<BSIR_U64> { using type = unsigned long long; using elem = uint64_t; };
template <> struct Acc<BSIR_BOOL> { using type = uint32_t; using elem = uint8_t; };

template <int DT>
__device__ __forceinline__ typename Acc<DT>::type load_acc(const void *p, int64_t i) {
  using E = typename Acc<DT>::elem;
  const E v = static_cast<const E *>(p)[i];
  if constexpr (DT == BSIR_F16) return __half2float(__ushort_as_half(v));
  else if constexpr (DT == BSIR_BF16) return __uint_as_float(static_cast<uint32_t>(v) << 16);
  else return static_cast<typename Acc<DT>::type>(v);
}
template <int DT>
__device__ __forceinline__ void store_acc(void *p, int64_t i, typename Acc<DT>::type v) {
  using E = typename Acc<DT>::elem;
  if constexpr (DT == BSIR_F16) static_cast<E *>(p)[i] = __half_as_ushort(__float2half_rn(v));
  else if constexpr (DT == BSIR_BF16) static_cast<E *>(p)[i] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
  else if constexpr (DT == BSIR_BOOL) static_cast<E *>(p)[i] = static_cast<E>(v & 1u);
  else static_cast<E *>(p)[i] = static_cast<E>(v);
}

template <int DT, int KIND>
__device__ __forceinline__ typename Acc<DT>::type identity() {
  using A = typename Acc<DT>::type;
  using E = typename Acc<DT>::elem;
  if constexpr (std::is_same<A, float>::value) {
    if (KIND == BSIR_REDUCE_SUM) return 0.0f;
    if (KIND == BSIR_REDUCE_PROD) return 1.0f;
    if (KIND == BSIR_REDUCE_MAX || KIND == BSIR_REDUCE_ANY) return __int_as_float(0xff800000);
    return __int_as_float(0x7f800000);
  } else {
    constexpr bool kSigned = std::is_signed<E>::value;
    constexpr int kBits = DT == BSIR_BOOL ? 1 : 8 * sizeof(E);
    switch (KIND) {
      case BSIR_REDUCE_SUM: case BSIR_REDUCE_XORI: case BSIR_REDUCE_ORI: return A(0);
      case BSIR_REDUCE_PROD: return A(1);
      case BSIR_REDUCE_MAX: case BSIR_REDUCE_ANY:
        return kSigned ? static_cast<A>(-(static_cast<long long>(1) << (kBits - 1))) : A(0);
      case BSIR_REDUCE_MIN: case BSIR_REDUCE_ALL:
        return kSigned ? static_cast<A>((static_cast<unsigned long long>(1) << (kBits - 1)) - 1)
                       : static_cast<A>(kBits == 64 ? ~0ull : ((1ull << (kBits % 64)) - 1));
      default: return static_cast<A>(~0ull);  // andi
    }
  }
}

template <int KIND, typename A>
__device__ __forceinline__ A combine(A a, A b) {
  if constexpr (std::is_same<A, float>::value) {
    if (KIND == BSIR_REDUCE_SUM) return a + b;
    if (KIND == BSIR_REDUCE_PROD) return a * b;
    if (KIND == BSIR_REDUCE_MAX || KIND == BSIR_REDUCE_ANY) return maximumf(a, b);
    return minimumf(a, b);
  } else {
    using U = typename std::make_unsigned<A>::type;
    switch (KIND) {
      case BSIR_REDUCE_SUM: return static_cast<A>(static_cast<U>(a) + static_cast<U>(b));
      case BSIR_REDUCE_PROD: return static_cast<A>(static_cast<U>(a) * static_cast<U>(b));
      case BSIR_REDUCE_MAX: case BSIR_REDUCE_ANY: return a > b ? a : b;
      case BSIR_REDUCE_MIN: case BSIR_REDUCE_ALL: return a < b ? a : b;
      case BSIR_REDUCE_XORI: return a ^ b;
      case BSIR_REDUCE_ORI: return a | b;
      default: return a & b;
    }
  }
}

template <typename A>
__device__ __forceinline__ A shfl_xor_any(A v, int o) {
  if constexpr (sizeof(A) == 8) {
    unsigned long long u;
    memcpy(&u, &v, 8);
    u = __shfl_xor_sync(0xffffffffu, u, o);
    memcpy(&v, &u, 8);
    return v;
  } else {
    return __shfl_xor_sync(0xffffffffu, v, o);
  }
}

// Last axis: `tpr` threads (power of two, 32..256) cooperate on a row.
template <int DT, int KIND>
__global__ void __launch_bounds__(256) reduce_last_kernel(int64_t rows, int64_t cols, const void *__restrict__ src,
                                                          int64_t row_stride, void *__restrict__ dst, int tpr) {
  using A = typename Acc<DT>::type;
  __shared__ unsigned long long red[8][8];
  const int rpc = 256 / tpr;
  const int sub = threadIdx.x / tpr, t = threadIdx.x % tpr;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * rpc + sub;
  A acc = identity<DT, KIND>();
  if (row < rows) {
    const int64_t base = row * row_stride;
    for (int64_t j = t; j < cols; j += tpr) acc = combine<KIND, A>(load_acc<DT>(src, base + j), acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc = combine<KIND, A>(acc, shfl_xor_any(acc, o));
  if (tpr > 32) {
    const int lane = threadIdx.x & 31, w = t >> 5, nw = tpr >> 5;
    unsigned long long bits = 0;
    memcpy(&bits, &acc, sizeof(A));
    if (lane == 0) red[sub][w] = bits;
    __syncthreads();
    A p = identity<DT, KIND>();
    if (lane < nw) { bits = red[sub][lane]; memcpy(&p, &bits, sizeof(A)); }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) p = combine<KIND, A>(p, shfl_xor_any(p, o));
    acc = p;
  }
  if (row < rows && t == 0) store_acc<DT>(dst, row, acc);
}

// First axis: block = 32 columns x 8 row slices.
template <int DT, int KIND>
__global__ void __launch_bounds__(256) reduce_first_kernel(int64_t rows, int64_t cols, const void *__restrict__ src,
                                                           int64_t row_stride, void *__restrict__ dst) {
  using A = typename Acc<DT>::type;
  __shared__ unsigned long long red[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 32 + cx;
  A acc = identity<DT, KIND>();
  if (c < cols)
    for (int64_t r = ry; r < rows; r += 8) acc = combine<KIND, A>(load_acc<DT>(src, r * row_stride + c), acc);
  unsigned long long bits = 0;
  memcpy(&bits, &acc, sizeof(A));
  red[ry][cx] = bits;
  __syncthreads();
  if (ry == 0 && c < cols) {
#pragma unroll
    for (int k = 1; k < 8; ++k) {
      A p;
      bits = red[k][cx];
      memcpy(&p, &bits, sizeof(A));
      acc = combine<KIND, A>(acc, p);
    }
    store_acc<DT>(dst, c, acc);
  }
}

// ------------------------------------------------------------------ vectorised paths
// Rows (or columns) whose base and pitch are 16-byte aligned are read as 16-byte vectors, several per
// thread in flight.  When a single pass would leave most SMs idle (few long rows; a tall matrix
// reduced over its first axis) the work is cut into parts, every part leaves one partial per output
// in a scratch array, and a second, tiny launch combines the partials in part order -- no atomics, the
// result does not depend on timing.
template <int DT>
__device__ __forceinline__ typename Acc<DT>::type acc_from_vec(const Vec16 &v, int k) {
  using A = typename Acc<DT>::type;
  using E = typename Acc<DT>::elem;
  if constexpr (sizeof(E) == 4) {
    const uint32_t w = v.w[k];
    if constexpr (std::is_same<A, float>::value) return __uint_as_float(w);
    else return static_cast<A>(static_cast<E>(w));
  } else if constexpr (sizeof(E) == 8) {
    const unsigned long long u = static_cast<unsigned long long>(v.w[2 * k]) | (static_cast<unsigned long long>(v.w[2 * k + 1]) << 32);
    return static_cast<A>(static_cast<E>(u));
  } else if constexpr (sizeof(E) == 2) {
    const uint16_t h = static_cast<uint16_t>(v.w[k >> 1] >> (16 * (k & 1)));
    if constexpr (DT == BSIR_F16) return __half2float(__ushort_as_half(h));
    else if constexpr (DT == BSIR_BF16) return __uint_as_float(static_cast<uint32_t>(h) << 16);
    else return static_cast<A>(static_cast<E>(h));
  } else {
    const uint8_t b = static_cast<uint8_t>(v.w[k >> 2] >> (8 * (k & 3)));
    return static_cast<A>(static_cast<E>(b));
  }
}

template <typename A>
__device__ __forceinline__ unsigned long long acc_bits(A a) {
  unsigned long long u = 0;
  memcpy(&u, &a, sizeof(A));
  return u;
}
template <typename A>
__device__ __forceinline__ A acc_of_bits(unsigned long long u) {
  A a;
  memcpy(&a, &u, sizeof(A));
  return a;
}

// Last axis.  grid = (row groups, parts); `tpr` threads (4..256, a power of two) share a row part.
template <int DT, int KIND>
__global__ void __launch_bounds__(256) reduce_last_vec_kernel(int64_t rows, int64_t nvec, int64_t row_stride,
                                                              const void *__restrict__ src, int64_t part_vecs, int nparts,
                                                              int tpr, void *__restrict__ dst, unsigned long long *partials) {
  using A = typename Acc<DT>::type;
  using E = typename Acc<DT>::elem;
  constexpr int kPerVec = 16 / sizeof(E);
  __shared__ unsigned long long red[4][8];     // used only when a row has more than one warp (tpr >= 64)
  pdl_launch_dependents();   // the finishing launch (or the next op) is scheduled while this one runs (launch_pdl) ...
  pdl_wait();                // ... and global memory is touched only after the kernel ahead has completed
  const int rpc = 256 / tpr;
  const int sub = threadIdx.x / tpr, t = threadIdx.x % tpr;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * rpc + sub;
  const int part = blockIdx.y;
  const int64_t v0 = static_cast<int64_t>(part) * part_vecs;
  const int64_t v1 = min(nvec, v0 + part_vecs);
  A acc[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) acc[u] = identity<DT, KIND>();
  if (row < rows) {
    const Vec16 *xv = reinterpret_cast<const Vec16 *>(static_cast<const E *>(src) + row * row_stride);
    for (int64_t j = v0 + t; j < v1; j += 4 * tpr) {
      Vec16 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (j + u * tpr < v1) v[u] = ld_stream(xv + j + u * tpr);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (j + u * tpr < v1) {
#pragma unroll
          for (int k = 0; k < kPerVec; ++k) acc[u] = combine<KIND, A>(acc_from_vec<DT>(v[u], k), acc[u]);
        }
    }
  }
  A a = combine<KIND, A>(combine<KIND, A>(acc[0], acc[1]), combine<KIND, A>(acc[2], acc[3]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    if (o < tpr) a = combine<KIND, A>(a, shfl_xor_any(a, o));
  if (tpr > 32) {
    const int lane = threadIdx.x & 31, w = t >> 5, nw = tpr >> 5;
    if (lane == 0) red[sub][w] = acc_bits(a);
    __syncthreads();
    A p = identity<DT, KIND>();
    if (lane < nw) p = acc_of_bits<A>(red[sub][lane]);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) p = combine<KIND, A>(p, shfl_xor_any(p, o));
    a = p;
  }
  if (row < rows && t == 0) {
    if (nparts == 1) store_acc<DT>(dst, row, a);
    else partials[row * nparts + part] = acc_bits(a);
  }
}

// First axis.  A thread owns CW 16-byte column vectors 512 bytes apart, so a warp reads CW x 512 contiguous bytes of
// a row (rows lie a whole row pitch apart in DRAM: the longer the stretch read from one, the fewer pages are opened
// for it); block = 32 x CW column vectors x 8 row slices; grid = (column groups, row slabs).
template <int DT, int KIND, int CW>
__global__ void __launch_bounds__(256) reduce_first_vec_kernel(int64_t rows, int64_t cvecs, int64_t row_stride,
                                                               const void *__restrict__ src, int64_t slab_rows, int nslabs,
                                                               void *__restrict__ dst, unsigned long long *partials) {
  using A = typename Acc<DT>::type;
  using E = typename Acc<DT>::elem;
  constexpr int kPerVec = 16 / sizeof(E);
  constexpr int kRowsAhead = CW == 1 ? 4 : 2;        // rows a thread asks for before it adds the first
  __shared__ unsigned long long red[7][32][kPerVec < 8 ? kPerVec : 8];
  pdl_launch_dependents();   // the finishing launch (or the next op) is scheduled while this one runs (launch_pdl) ...
  pdl_wait();                // ... and global memory is touched only after the kernel ahead has completed
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int64_t cv0 = static_cast<int64_t>(blockIdx.x) * (32 * CW) + cx;
  const int slab = blockIdx.y;
  const int64_t r0 = static_cast<int64_t>(slab) * slab_rows, r1 = min(rows, r0 + slab_rows);
  A acc[CW][kPerVec];
#pragma unroll
  for (int w = 0; w < CW; ++w)
#pragma unroll
    for (int k = 0; k < kPerVec; ++k) acc[w][k] = identity<DT, KIND>();
  const E *base = static_cast<const E *>(src) + cv0 * kPerVec;
  for (int64_t r = r0 + ry; r < r1; r += 8 * kRowsAhead) {
    Vec16 v[kRowsAhead][CW];
#pragma unroll
    for (int u = 0; u < kRowsAhead; ++u)
#pragma unroll
      for (int w = 0; w < CW; ++w)
        if (r + 8 * u < r1 && cv0 + 32 * w < cvecs)
          v[u][w] = ld_stream(reinterpret_cast<const Vec16 *>(base + (r + 8 * u) * row_stride + 32 * w * kPerVec));
#pragma unroll
    for (int u = 0; u < kRowsAhead; ++u)
#pragma unroll
      for (int w = 0; w < CW; ++w)
        if (r + 8 * u < r1 && cv0 + 32 * w < cvecs) {
#pragma unroll
          for (int k = 0; k < kPerVec; ++k) acc[w][k] = combine<KIND, A>(acc_from_vec<DT>(v[u][w], k), acc[w][k]);
        }
  }
  // the eight row slices meet in shared memory, 8 elements of a vector at a time
  constexpr int kChunk = kPerVec < 8 ? kPerVec : 8;
#pragma unroll
  for (int w = 0; w < CW; ++w) {
    const bool mine = cv0 + 32 * w < cvecs;
#pragma unroll
    for (int c0 = 0; c0 < kPerVec; c0 += kChunk) {
      if (ry > 0) {
#pragma unroll
        for (int k = 0; k < kChunk; ++k) red[ry - 1][cx][k] = acc_bits(acc[w][c0 + k]);
      }
      __syncthreads();
      if (ry == 0 && mine) {
#pragma unroll
        for (int s = 0; s < 7; ++s)
#pragma unroll
          for (int k = 0; k < kChunk; ++k) acc[w][c0 + k] = combine<KIND, A>(acc[w][c0 + k], acc_of_bits<A>(red[s][cx][k]));
      }
      __syncthreads();
    }
    if (ry == 0 && mine) {
#pragma unroll
      for (int k = 0; k < kPerVec; ++k) {
        const int64_t c = (cv0 + 32 * w) * kPerVec + k;
        if (nslabs == 1) store_acc<DT>(dst, c, acc[w][k]);
        else partials[static_cast<int64_t>(slab) * (cvecs * kPerVec) + c] = acc_bits(acc[w][k]);
      }
    }
  }
}

// out[o] = combine over p of partials[o * out_stride + p * part_stride], in part order
template <int DT, int KIND>
__global__ void __launch_bounds__(256) reduce_finish_kernel(int64_t nout, int nparts, int64_t out_stride, int64_t part_stride,
                                                            const unsigned long long *__restrict__ partials, void *__restrict__ dst) {
  using A = typename Acc<DT>::type;
  pdl_launch_dependents();
  pdl_wait();                // the partials of the launch ahead are complete from here on
  const int64_t o = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (o >= nout) return;
  A a = identity<DT, KIND>();
  for (int p = 0; p < nparts; ++p) a = combine<KIND, A>(a, acc_of_bits<A>(partials[o * out_stride + p * part_stride]));
  store_acc<DT>(dst, o, a);
}

bool reduce_kind_valid(int kind, int dt) {
  if (kind < BSIR_REDUCE_SUM || kind > BSIR_REDUCE_ANDI) return false;
  if (dtype_is_float(dt)) return kind <= BSIR_REDUCE_MIN;
  return true;
}

template <int DT, int KIND>
void launch_reduce(bool last, int64_t rows, int64_t cols, const void *src, int64_t rs, void *dst, cudaStream_t st) {
  using E = typename Acc<DT>::elem;
  constexpr int kPerVec = 16 / sizeof(E);
  const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
  const bool vec_ok = rows > 0 && cols > 0 && cols % kPerVec == 0 && rs % kPerVec == 0 && aligned_to(src, 16) &&
                      std::getenv("BSIR_REDUCE_SCALAR") == nullptr;
  if (last && vec_ok) {
    const int64_t nvec = cols / kPerVec;
    int tpr = 4;
    while (tpr < 256 && nvec > tpr * 4) tpr <<= 1;          // about 4 vectors per thread before a row gets more threads
    // with rows enough to fill every SM with warps, a warp a row: the row's sum ends in shuffles, no block-wide barrier
    // ([32768,4096] f32: 89.6 -> 77.1 us; bf16 45.2 -> 41.5 us)
    if (tpr > 32 && rows >= static_cast<int64_t>(sms) * 64) tpr = 32;
    const int rpc = 256 / tpr;
    const int64_t row_groups = ceil_div(rows, rpc);
    // few long rows: cut them so that about 4 CTAs per SM have work, parts of at least 1024 vectors
    int64_t parts = 1;
    if (tpr == 256 && row_groups < 4 * sms) {
      parts = ceil_div(4 * sms, row_groups);
      if (parts > nvec / 1024) parts = nvec / 1024;
      if (parts > 1024) parts = 1024;
      if (parts < 1) parts = 1;
    }
    const int64_t part_vecs = ceil_div(nvec, parts);
    parts = ceil_div(nvec, part_vecs);
    unsigned long long *partials = nullptr;
    if (parts > 1) {
      char *ws = static_cast<char *>(device_workspace(kScratchCounterBytes + static_cast<size_t>(rows) * parts * 8, st));
      if (ws) partials = reinterpret_cast<unsigned long long *>(ws + kScratchCounterBytes);
      else parts = 1;
    }
    const dim3 grid(static_cast<unsigned>(row_groups), static_cast<unsigned>(parts));
    launch_pdl(reduce_last_vec_kernel<DT, KIND>, grid, dim3(256), 0, st, rows, nvec, rs, src, parts > 1 ? part_vecs : nvec,
               static_cast<int>(parts), tpr, dst, partials);
    if (parts > 1) {
      launch_pdl(reduce_finish_kernel<DT, KIND>, dim3(static_cast<unsigned>(ceil_div(rows, 256))), dim3(256), 0, st, rows,
                 static_cast<int>(parts), static_cast<int64_t>(parts), static_cast<int64_t>(1), partials, dst);
      count_launch();
    }
    return;
  }
  if (!last && vec_ok) {
    const int64_t cvecs = cols / kPerVec;
    // four column vectors a thread (2 KB of a row a warp) for 4- and 8-byte elements when the rows are long enough and
    // there are enough of them to cut into slabs that still fill the SMs: [32768,4096] f32 116 -> 105 us
    const int cw = kPerVec <= 4 && cvecs >= 128 && rows >= 512 ? 4 : 1;   // (16-bit elements: 32 accumulators a thread cost more than the longer stretches gain)
    const int64_t col_groups = ceil_div(cvecs, static_cast<int64_t>(32 * cw));
    int64_t slabs = 1;
    if (col_groups < 4 * sms) {
      slabs = ceil_div(4 * sms, col_groups);
      if (slabs > rows / 64) slabs = rows / 64;
      if (slabs > 1024) slabs = 1024;
      if (slabs < 1) slabs = 1;
    }
    const int64_t slab_rows = ceil_div(rows, slabs);
    slabs = ceil_div(rows, slab_rows);
    unsigned long long *partials = nullptr;
    if (slabs > 1) {
      char *ws = static_cast<char *>(device_workspace(kScratchCounterBytes + static_cast<size_t>(cols) * slabs * 8, st));
      if (ws) partials = reinterpret_cast<unsigned long long *>(ws + kScratchCounterBytes);
      else slabs = 1;
    }
    const dim3 grid(static_cast<unsigned>(col_groups), static_cast<unsigned>(slabs));
    if (cw == 4)
      launch_pdl(reduce_first_vec_kernel<DT, KIND, 4>, grid, dim3(256), 0, st, rows, cvecs, rs, src, slabs > 1 ? slab_rows : rows,
                 static_cast<int>(slabs), dst, partials);
    else
      launch_pdl(reduce_first_vec_kernel<DT, KIND, 1>, grid, dim3(256), 0, st, rows, cvecs, rs, src, slabs > 1 ? slab_rows : rows,
                 static_cast<int>(slabs), dst, partials);
    if (slabs > 1) {
      launch_pdl(reduce_finish_kernel<DT, KIND>, dim3(static_cast<unsigned>(ceil_div(cols, 256))), dim3(256), 0, st, cols,
                 static_cast<int>(slabs), static_cast<int64_t>(1), cols, partials, dst);
      count_launch();
    }
    return;
  }
  if (last) {
    int tpr = 32;
    while (tpr < 256 && cols > tpr * 8) tpr <<= 1;
    const int rpc = 256 / tpr;
    reduce_last_kernel<DT, KIND><<<static_cast<unsigned>(ceil_div(rows, rpc)), 256, 0, st>>>(rows, cols, src, rs, dst, tpr);
  } else {
    reduce_first_kernel<DT, KIND><<<static_cast<unsigned>(ceil_div(cols, 32)), 256, 0, st>>>(rows, cols, src, rs, dst);
  }
}

template <int DT>
int32_t dispatch_kind(bool last, int kind, int64_t rows, int64_t cols, const void *src, int64_t rs, void *dst,
                      cudaStream_t st) {
#define K(k) \
  case k: launch_reduce<DT, k>(last, rows, cols, src, rs, dst, st); return BSIR_OK;
  if constexpr (DT == BSIR_F32 || DT == BSIR_F16 || DT == BSIR_BF16) {
    switch (kind) { K(BSIR_REDUCE_SUM) K(BSIR_REDUCE_PROD) K(BSIR_REDUCE_MAX) K(BSIR_REDUCE_MIN) default: break; }
  } else {
    switch (kind) {
      K(BSIR_REDUCE_SUM) K(BSIR_REDUCE_PROD) K(BSIR_REDUCE_MAX) K(BSIR_REDUCE_MIN) K(BSIR_REDUCE_ANY)
      K(BSIR_REDUCE_ALL) K(BSIR_REDUCE_XORI) K(BSIR_REDUCE_ORI) K(BSIR_REDUCE_ANDI)
      default: break;
    }
  }
#undef K
  return fail(BSIR_ERR_ATTR, "reduce: kind %d", kind);
}

int32_t reduce_axis(const char *what, bool last, int32_t kind, int32_t dtype, int64_t rows, int64_t cols,
                    const void *src, int64_t rs, void *dst, void *stream) {
  clear_error();
  if (dtype_bytes(dtype) == 0) return fail(BSIR_ERR_DTYPE, "%s: dtype %d", what, dtype);
  if (!reduce_kind_valid(kind, dtype)) return fail(BSIR_ERR_ATTR, "%s: kind %d for dtype %d", what, kind, dtype);
  if (rows < 0 || cols < 0) return fail(BSIR_ERR_SHAPE, "%s: rows=%lld cols=%lld", what, (long long)rows, (long long)cols);
  const int64_t nout = last ? rows : cols;
  if (nout == 0) return BSIR_OK;
  if (!dst || (!src && rows * cols > 0)) return fail(BSIR_ERR_NULL, "%s: null pointer", what);
  if (rs < cols) return fail(BSIR_ERR_STRIDE, "%s: row stride %lld < cols %lld", what, (long long)rs, (long long)cols);
  if (!aligned_to(src, dtype_bytes(dtype)) || !aligned_to(dst, dtype_bytes(dtype)))
    return fail(BSIR_ERR_ALIGN, "%s: misaligned", what);
  cudaStream_t st = resolve_stream(stream);
  int32_t rc;
#define D(code) \
  case code: rc = dispatch_kind<code>(last, kind, rows, cols, src, rs, dst, st); break;
  switch (dtype) {
    D(BSIR_F32) D(BSIR_F16) D(BSIR_BF16) D(BSIR_I8) D(BSIR_I16) D(BSIR_I32) D(BSIR_I64) D(BSIR_U8) D(BSIR_U16)
    D(BSIR_U32) D(BSIR_U64) D(BSIR_BOOL)
    default: return fail(BSIR_ERR_DTYPE, "%s: dtype %d", what, dtype);
  }
#undef D
  if (rc) return rc;
  count_launch();
  return check_launch(what);
}

// ------------------------------------------------------------------ reduce_with_index
// A row is cut into segments of up to 256 x VPT (VPT <= 8) 16-byte vectors; one CTA per (segment, row)
// keeps its segment in registers, finds the segment extreme with a NaN-propagating
// max/min, then looks for the first (or last) element equal to it.  Partial results go to a
// scratch array; the CTA that finishes a row last (a counter in the same scratch, left at zero
// again afterwards) folds the partials in segment order and writes the outputs.
struct Partial {
  float val;     // extreme of the segment (of its NaN-free prefix when it holds a NaN)
  int32_t idx;   // index of that extreme within the row
  int32_t nan;   // row index of the segment's first NaN, INT_MAX when none
  int32_t pad;
};

struct RwiParams {
  int64_t rows, cols, row_stride;
  int64_t nvec;       // vectors per row
  int64_t seg_vecs;   // vectors per segment
  int nseg;
  int tie_left;
  int nan_first;
};

template <bool IS_MAX>
__device__ __forceinline__ float ext_nan(float a, float b) { return IS_MAX ? maximumf(a, b) : minimumf(a, b); }
template <bool IS_MAX>
__device__ __forceinline__ float ext_num(float a, float b) { return IS_MAX ? fmaxf(a, b) : fminf(a, b); }

template <class F>
__device__ __forceinline__ float cta_reduce_f(float v, float *red, F f) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = f(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float p = red[lane & 7];
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) p = f(p, __shfl_xor_sync(0xffffffffu, p, o));
  return p;
}
template <class F>
__device__ __forceinline__ int cta_reduce_i(int v, int *red, F f) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = f(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  int p = red[lane & 7];
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) p = f(p, __shfl_xor_sync(0xffffffffu, p, o));
  return p;
}

// Writes one row's result.  Under the first-NaN-wins rule the value is the element at the
// reported index itself (its sign of zero and NaN payload included), as the device library's
// scalar loop returns it (bishengir/lib/Template/lib/Vector/Reduction/ReduceR_With_Index.cpp:83-125).
template <int DT>
__device__ __forceinline__ void rwi_write(const RwiParams &p, const void *src, int64_t row, float val, int idx,
                                          void *dst_val, int32_t *dst_idx) {
  if constexpr (DT == BSIR_F32) {
    const float *x = static_cast<const float *>(src) + row * p.row_stride;
    static_cast<float *>(dst_val)[row] = (p.nan_first && p.cols > 0) ? x[idx] : val;
  } else {
    const uint16_t *x = static_cast<const uint16_t *>(src) + row * p.row_stride;
    uint16_t bits;
    if (p.nan_first && p.cols > 0) bits = x[idx];
    else if constexpr (DT == BSIR_F16) bits = __half_as_ushort(__float2half_rn(val));
    else bits = __bfloat16_as_ushort(__float2bfloat16_rn(val));
    static_cast<uint16_t *>(dst_val)[row] = bits;
  }
  dst_idx[row] = idx;
}

// Warp 0 of a (row, segment) CTA publishes the segment's result; the warp that completes the row
// folds the row's `nseg` partials in segment order and writes the outputs.  Called by all 32 lanes.
template <int DT, bool IS_MAX>
__device__ __forceinline__ void rwi_publish_and_fold(const RwiParams &p, const void *src, int64_t row, int seg, int nseg,
                                                     float m, int best, int nanpos, void *dst_val, int32_t *dst_idx,
                                                     unsigned *counters, Partial *partials) {
  const int lane = threadIdx.x & 31;
  const float ident = IS_MAX ? __int_as_float(0xff800000) : __int_as_float(0x7f800000);
  Partial *mine = partials + row * nseg;
  // lane 0 publishes this segment and counts
  unsigned done = 0u;
  if (lane == 0) {
    mine[seg] = Partial{m, best, nanpos, 0};
    __threadfence();
    done = atomicAdd(&counters[row], 1u);
  }
  done = __shfl_sync(0xffffffffu, done, 0);
  if (done != static_cast<unsigned>(nseg - 1)) return;   // not the last segment of this row to finish
  __threadfence();
  // Ordered fold of the row's partials.  The combine below ("strictly better moves the index; on a
  // tie the left rule keeps the earlier segment, the right rule takes the later one; nothing after
  // the first NaN counts") is associative, so each lane folds a contiguous stretch of segments (its
  // loads independent of one another) and the 32 stretches are joined in order by shuffles.
  float val = ident;
  int idx = 0, nan_at = INT_MAX;
  bool have = false, saw_nan = false;
  auto join = [&](float sv, int si, bool sh, bool sn, int sa) {   // state (left) <- state (+) right
    if (saw_nan) return;
    if (sh) {
      const bool better = IS_MAX ? (sv > val) : (sv < val);
      const bool tie = sv == val;
      if (!have || better || (tie && !p.tie_left)) idx = si;
      val = have ? ext_nan<IS_MAX>(val, sv) : sv;
      have = true;
    }
    saw_nan = sn;
    nan_at = sa;
  };
  const int per_lane = (nseg + 31) / 32;
  const int s_begin = min(nseg, lane * per_lane), s_end = min(nseg, s_begin + per_lane);
  for (int s0 = s_begin; s0 < s_end; s0 += 4) {
    float pv[4];
    int pi[4], pn[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      pv[k] = ident; pi[k] = -1; pn[k] = INT_MAX;
      if (s0 + k < s_end) {
        const volatile Partial *q = mine + s0 + k;
        pv[k] = q->val; pi[k] = q->idx; pn[k] = q->nan;
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (s0 + k < s_end) join(pv[k], pi[k], pi[k] >= 0, pn[k] != INT_MAX, pn[k]);
  }
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float sv = __shfl_down_sync(0xffffffffu, val, o);
    const int si = __shfl_down_sync(0xffffffffu, idx, o);
    const int sa = __shfl_down_sync(0xffffffffu, nan_at, o);
    const int flags = __shfl_down_sync(0xffffffffu, (have ? 1 : 0) | (saw_nan ? 2 : 0), o);
    if ((lane & (2 * o - 1)) == 0 && lane + o < 32) join(sv, si, (flags & 1) != 0, (flags & 2) != 0, sa);
  }
  if (saw_nan && p.nan_first) idx = nan_at;
  if (lane != 0) return;
  if (saw_nan) val = __int_as_float(0x7fc00000);
  rwi_write<DT>(p, src, row, val, idx, dst_val, dst_idx);
  counters[row] = 0u;  // scratch is zero again for the next call
}

template <int DT, int VPT, bool IS_MAX>
__global__ void __launch_bounds__(256) rwi_kernel(RwiParams p, const void *__restrict__ src, void *__restrict__ dst_val,
                                                  int32_t *__restrict__ dst_idx, unsigned *__restrict__ counters,
                                                  Partial *__restrict__ partials) {
  constexpr int kPerWord = FloatTraits<DT>::kPerWord;
  constexpr int kPerVec = 4 * kPerWord;
  using E = typename std::conditional<DT == BSIR_F32, float, uint16_t>::type;
  __shared__ float redf[8];
  __shared__ int redi[8];
  const int seg = blockIdx.x;
  const int64_t row = blockIdx.y;
  const E *xrow = static_cast<const E *>(src) + row * p.row_stride;
  const int64_t v0 = static_cast<int64_t>(seg) * p.seg_vecs;
  const int64_t v1 = min(v0 + p.seg_vecs, p.nvec);
  const float ident = IS_MAX ? __int_as_float(0xff800000) : __int_as_float(0x7f800000);

  Vec16 v[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int64_t vi = v0 + threadIdx.x + static_cast<int64_t>(i) * 256;
    if (vi < v1) v[i] = ld_stream(reinterpret_cast<const Vec16 *>(xrow) + vi);
  }
  // pass 1: NaN-propagating extreme; 16-bit types stay packed (one max/min.NaN.x2 per word)
  float m = ident;
  if constexpr (kPerWord == 2) {
    constexpr uint32_t kIdent2 = DT == BSIR_BF16 ? (IS_MAX ? 0xff80ff80u : 0x7f807f80u) : (IS_MAX ? 0xfc00fc00u : 0x7c007c00u);
    uint32_t m2 = kIdent2;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t vi = v0 + threadIdx.x + static_cast<int64_t>(i) * 256;
      if (vi < v1) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          if constexpr (DT == BSIR_BF16) {
            if constexpr (IS_MAX) asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
            else asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
          } else {
            if constexpr (IS_MAX) asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
            else asm("min.NaN.f16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
          }
        }
      }
    }
    float e2[2];
    FloatTraits<DT>::unpack(m2, e2);
    m = ext_nan<IS_MAX>(e2[0], e2[1]);
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t vi = v0 + threadIdx.x + static_cast<int64_t>(i) * 256;
      if (vi < v1) {
#pragma unroll
        for (int w = 0; w < 4; ++w) m = ext_nan<IS_MAX>(m, __uint_as_float(v[i].w[w]));
      }
    }
  }
  const float tm = m;  // this thread's own extreme
  // Common case (no NaN in the segment): the warps agree on the segment extreme through shared
  // memory, then only the warps that hold it (normally one of eight) search their registers for
  // its first (last) position.  Searching in every warp costs ten times the instructions of the
  // reduction itself, which made the kernel issue-bound.
  __shared__ float warp_val[8];
  __shared__ int warp_idx[8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float wm = tm;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wm = ext_nan<IS_MAX>(wm, __shfl_xor_sync(0xffffffffu, wm, o));
  if (lane == 0) warp_val[wid] = wm;
  __syncthreads();
  m = warp_val[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) m = ext_nan<IS_MAX>(m, warp_val[k]);
  int nanpos = INT_MAX;
  int best = p.tie_left ? INT_MAX : -1;
  if (m == m) {
    if (wm == m) {  // warp-uniform
      if (tm == m) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int64_t vi = v0 + threadIdx.x + static_cast<int64_t>(i) * 256;
          if (vi < v1) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              float e[kPerWord];
              FloatTraits<DT>::unpack(v[i].w[w], e);
#pragma unroll
              for (int k = 0; k < kPerWord; ++k) {
                const int gi = static_cast<int>(vi * kPerVec + w * kPerWord + k);
                if (e[k] == m) best = p.tie_left ? min(best, gi) : max(best, gi);
              }
            }
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const int other = __shfl_xor_sync(0xffffffffu, best, o);
        best = p.tie_left ? min(best, other) : max(best, other);
      }
    }
    if (lane == 0) warp_idx[wid] = best;
    __syncthreads();
    best = warp_idx[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) best = p.tie_left ? min(best, warp_idx[k]) : max(best, warp_idx[k]);
  } else {
    // rare: the segment holds a NaN.  Find the first one, redo the extreme on the prefix before it,
    // then look for that extreme's position inside the prefix (whole-CTA reductions, several barriers).
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t vi = v0 + threadIdx.x + static_cast<int64_t>(i) * 256;
      if (vi < v1) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          float e[kPerWord];
          FloatTraits<DT>::unpack(v[i].w[w], e);
#pragma unroll
          for (int k = 0; k < kPerWord; ++k)
            if (e[k] != e[k]) nanpos = min(nanpos, static_cast<int>(vi * kPerVec + w * kPerWord + k));
        }
      }
    }
    nanpos = cta_reduce_i(nanpos, redi, [](int a, int b) { return min(a, b); });
    m = ident;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t vi = v0 + threadIdx.x + static_cast<int64_t>(i) * 256;
      if (vi < v1) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          float e[kPerWord];
          FloatTraits<DT>::unpack(v[i].w[w], e);
#pragma unroll
          for (int k = 0; k < kPerWord; ++k)
            if (static_cast<int>(vi * kPerVec + w * kPerWord + k) < nanpos) m = ext_nan<IS_MAX>(m, e[k]);
        }
      }
    }
    m = cta_reduce_f(m, redf, [](float a, float b) { return ext_nan<IS_MAX>(a, b); });
    best = p.tie_left ? INT_MAX : -1;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t vi = v0 + threadIdx.x + static_cast<int64_t>(i) * 256;
      if (vi < v1) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          float e[kPerWord];
          FloatTraits<DT>::unpack(v[i].w[w], e);
#pragma unroll
          for (int k = 0; k < kPerWord; ++k) {
            const int gi = static_cast<int>(vi * kPerVec + w * kPerWord + k);
            if (e[k] == m && gi < nanpos) best = p.tie_left ? min(best, gi) : max(best, gi);
          }
        }
      }
    }
    if (p.tie_left) best = cta_reduce_i(best, redi, [](int a, int b) { return min(a, b); });
    else best = cta_reduce_i(best, redi, [](int a, int b) { return max(a, b); });
  }
  // a segment whose prefix is empty or all at the identity reports "nothing better than the start"
  if (best == INT_MAX || best < 0) best = -1;

  if (p.nseg == 1) {
    if (threadIdx.x == 0) {
      float val = m;
      int idx = best < 0 ? 0 : best;
      if (nanpos != INT_MAX) {
        val = __int_as_float(0x7fc00000);
        if (p.nan_first) idx = nanpos;
      }
      rwi_write<DT>(p, src, row, val, idx, dst_val, dst_idx);
    }
    return;
  }

  if (threadIdx.x >= 32) return;
  rwi_publish_and_fold<DT, IS_MAX>(p, src, row, seg, p.nseg, m, best, nanpos, dst_val, dst_idx, counters, partials);
}

// Long rows: each row is cut into `nseg` equal parts of `p.seg_vecs` vectors and one CTA streams a
// part through two register buffers of 256 x 4 vectors, so that the loads of tile t+1 are in flight
// while tile t is reduced (a 12 us launch cannot afford CTAs that load, wait, reduce and leave).
// A part that holds a NaN is redone by three scalar sweeps.
template <int DT, bool IS_MAX>
__device__ __noinline__ void rwi_part_with_nan(const RwiParams &p, const void *src, int64_t row, int64_t e0, int64_t e1,
                                               float *redf, int *redi, float *out_val, int *out_idx, int *out_nan) {
  const int64_t base = row * p.row_stride;
  const float ident = IS_MAX ? __int_as_float(0xff800000) : __int_as_float(0x7f800000);
  auto at = [&](int64_t j) -> float {
    if constexpr (DT == BSIR_F32) return static_cast<const float *>(src)[base + j];
    else if constexpr (DT == BSIR_F16) return __half2float(__ushort_as_half(static_cast<const uint16_t *>(src)[base + j]));
    else return __uint_as_float(static_cast<uint32_t>(static_cast<const uint16_t *>(src)[base + j]) << 16);
  };
  int nanpos = INT_MAX;
  for (int64_t j = e0 + threadIdx.x; j < e1; j += 256) {
    const float e = at(j);
    if (e != e) { nanpos = static_cast<int>(j); break; }
  }
  nanpos = cta_reduce_i(nanpos, redi, [](int a, int b) { return min(a, b); });
  const int64_t lim = nanpos == INT_MAX ? e1 : nanpos;
  float m = ident;
  for (int64_t j = e0 + threadIdx.x; j < lim; j += 256) m = ext_nan<IS_MAX>(m, at(j));
  m = cta_reduce_f(m, redf, [](float a, float b) { return ext_nan<IS_MAX>(a, b); });
  int best = p.tie_left ? INT_MAX : -1;
  for (int64_t j = e0 + threadIdx.x; j < lim; j += 256)
    if (at(j) == m) best = p.tie_left ? min(best, static_cast<int>(j)) : max(best, static_cast<int>(j));
  if (p.tie_left) best = cta_reduce_i(best, redi, [](int a, int b) { return min(a, b); });
  else best = cta_reduce_i(best, redi, [](int a, int b) { return max(a, b); });
  *out_val = m;
  *out_idx = (best == INT_MAX || best < 0) ? -1 : best;
  *out_nan = nanpos;
}

// The parts of a row meet either in global scratch (rwi_publish_and_fold) or, when a row has at most eight
// parts, in the shared memory of the first CTA of a thread-block cluster that spans the row: every CTA stores
// its partial there (st.shared::cluster), one cluster barrier orders the stores before the fold, and no
// counter, fence or scratch is involved -- about 1.5 us less tail on a launch of 12 us.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_cluster_u32(void *local_smem, uint32_t rank, uint32_t v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(local_smem))), "r"(rank));
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(v) : "memory");
}

template <int DT, bool IS_MAX>
__global__ void __launch_bounds__(256, 4) rwi_stream_kernel(RwiParams p, const void *__restrict__ src,
                                                            void *__restrict__ dst_val, int32_t *__restrict__ dst_idx,
                                                            unsigned *__restrict__ counters, Partial *__restrict__ partials) {
  constexpr int VPT = 4;
  constexpr int kTileVecs = 256 * VPT;
  constexpr int kPerWord = FloatTraits<DT>::kPerWord;
  constexpr int kPerVec = 4 * kPerWord;
  constexpr uint32_t kIdentWord =
      DT == BSIR_F32 ? (IS_MAX ? 0xff800000u : 0x7f800000u)
                     : DT == BSIR_BF16 ? (IS_MAX ? 0xff80ff80u : 0x7f807f80u) : (IS_MAX ? 0xfc00fc00u : 0x7c007c00u);
  using E = typename std::conditional<DT == BSIR_F32, float, uint16_t>::type;
  __shared__ float redf[8];
  __shared__ int redi[8];
  __shared__ float warp_val[8];
  __shared__ int warp_idx[8];
  __shared__ Partial row_parts[8];   // cluster fold: the row's partials, filled by the cluster's CTAs in the first one
  const bool in_cluster = counters == nullptr;
  if (in_cluster) cluster_arrive_relaxed();   // "this CTA runs": waited for before anyone stores into its shared memory
  pdl_launch_dependents();   // the next launch may be scheduled while this one runs (launch_pdl) ...
  pdl_wait();                // ... and this one touches global memory only after the kernel ahead has completed
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const float ident = IS_MAX ? __int_as_float(0xff800000) : __int_as_float(0x7f800000);
  const int seg = blockIdx.x;
  const int64_t row = blockIdx.y;
  const int64_t a = static_cast<int64_t>(seg) * p.seg_vecs;   // first vector of the part within the row
  const int64_t b = min(p.nvec, a + p.seg_vecs);              // one past its last vector
  const Vec16 *xv = reinterpret_cast<const Vec16 *>(static_cast<const E *>(src) + row * p.row_stride);
  const int ntiles = static_cast<int>((b - a + kTileVecs - 1) / kTileVecs);

  auto load_tile = [&](Vec16 (&buf)[VPT], int t) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t vi = a + static_cast<int64_t>(t) * kTileVecs + i * 256 + threadIdx.x;
      if (vi < b) buf[i] = ld_stream(xv + vi);
      else buf[i] = Vec16{{kIdentWord, kIdentWord, kIdentWord, kIdentWord}};
    }
  };
  // A thread keeps its running extreme, and the vector (index and contents) in which it first (tie_left) or last
  // rose to it: the position then comes out of registers.  The loop is bound by memory, not by these selects.
  float rm = ident;
  Vec16 bv = Vec16{{kIdentWord, kIdentWord, kIdentWord, kIdentWord}};
  int bvi = -1;
  auto reduce_tile = [&](const Vec16 (&buf)[VPT], int t) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t vi = a + static_cast<int64_t>(t) * kTileVecs + i * 256 + threadIdx.x;
      float vm;
      if constexpr (kPerWord == 2) {
        uint32_t x, y;
        if constexpr (DT == BSIR_BF16) {
          if constexpr (IS_MAX) {
            asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(x) : "r"(buf[i].w[0]), "r"(buf[i].w[1]));
            asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(y) : "r"(buf[i].w[2]), "r"(buf[i].w[3]));
            asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(x) : "r"(x), "r"(y));
          } else {
            asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(x) : "r"(buf[i].w[0]), "r"(buf[i].w[1]));
            asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(y) : "r"(buf[i].w[2]), "r"(buf[i].w[3]));
            asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(x) : "r"(x), "r"(y));
          }
        } else {
          if constexpr (IS_MAX) {
            asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(x) : "r"(buf[i].w[0]), "r"(buf[i].w[1]));
            asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(y) : "r"(buf[i].w[2]), "r"(buf[i].w[3]));
            asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(x) : "r"(x), "r"(y));
          } else {
            asm("min.NaN.f16x2 %0, %1, %2;" : "=r"(x) : "r"(buf[i].w[0]), "r"(buf[i].w[1]));
            asm("min.NaN.f16x2 %0, %1, %2;" : "=r"(y) : "r"(buf[i].w[2]), "r"(buf[i].w[3]));
            asm("min.NaN.f16x2 %0, %1, %2;" : "=r"(x) : "r"(x), "r"(y));
          }
        }
        float e2[2];
        FloatTraits<DT>::unpack(x, e2);
        vm = ext_nan<IS_MAX>(e2[0], e2[1]);
      } else {
        vm = ext_nan<IS_MAX>(ext_nan<IS_MAX>(__uint_as_float(buf[i].w[0]), __uint_as_float(buf[i].w[1])),
                             ext_nan<IS_MAX>(__uint_as_float(buf[i].w[2]), __uint_as_float(buf[i].w[3])));
      }
      // a vector past the end of the part (filled with the identity) must not claim the position
      const bool rises = vi < b && (p.tie_left ? (IS_MAX ? vm > rm : vm < rm) : (IS_MAX ? vm >= rm : vm <= rm));
      if (rises) { bv = buf[i]; bvi = static_cast<int>(vi); }
      rm = ext_nan<IS_MAX>(rm, vm);
    }
  };

  Vec16 bufa[VPT], bufb[VPT];
  load_tile(bufa, 0);
  for (int t = 0; t < ntiles; t += 2) {
    if (t + 1 < ntiles) load_tile(bufb, t + 1);
    reduce_tile(bufa, t);
    if (t + 1 >= ntiles) break;
    if (t + 2 < ntiles) load_tile(bufa, t + 2);
    reduce_tile(bufb, t + 1);
  }

  // the part's extreme over the CTA, then its position from the threads that hold it
  float wm = rm;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wm = ext_nan<IS_MAX>(wm, __shfl_xor_sync(0xffffffffu, wm, o));
  if (lane == 0) warp_val[wid] = wm;
  __syncthreads();
  float m = warp_val[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) m = ext_nan<IS_MAX>(m, warp_val[k]);
  int best = p.tie_left ? INT_MAX : -1;
  int nanpos = INT_MAX;
  if (m == m) {
    if (wm == m) {  // warp-uniform: normally one warp in eight
      if (rm == m && bvi >= 0) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          float e[kPerWord];
          FloatTraits<DT>::unpack(bv.w[w], e);
#pragma unroll
          for (int k = 0; k < kPerWord; ++k) {
            const int gi = bvi * kPerVec + w * kPerWord + k;
            if (e[k] == m) best = p.tie_left ? min(best, gi) : max(best, gi);
          }
        }
      }
      // a part made of the identity alone (all -inf under max) never "rises" under the left rule: its first element
      if (p.tie_left && threadIdx.x == 0 && m == ident && b > a) best = min(best, static_cast<int>(a * kPerVec));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const int other = __shfl_xor_sync(0xffffffffu, best, o);
        best = p.tie_left ? min(best, other) : max(best, other);
      }
    }
    if (lane == 0) warp_idx[wid] = best;
    __syncthreads();
    best = warp_idx[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) best = p.tie_left ? min(best, warp_idx[k]) : max(best, warp_idx[k]);
    if (best == INT_MAX || best < 0) best = -1;
  } else {
    rwi_part_with_nan<DT, IS_MAX>(p, src, row, a * kPerVec, b * kPerVec, redf, redi, &m, &best, &nanpos);
  }
  if (!in_cluster) {
    if (threadIdx.x >= 32) return;
    rwi_publish_and_fold<DT, IS_MAX>(p, src, row, seg, p.nseg, m, best, nanpos, dst_val, dst_idx, counters, partials);
    return;
  }
  // cluster fold: all threads of all CTAs of the row pass both barrier phases
  cluster_wait_acquire();                      // every CTA of the cluster has started
  if (threadIdx.x == 0) {
    st_cluster_u32(&row_parts[seg].val, 0u, __float_as_uint(m));
    st_cluster_u32(&row_parts[seg].idx, 0u, static_cast<uint32_t>(best));
    st_cluster_u32(&row_parts[seg].nan, 0u, static_cast<uint32_t>(nanpos));
  }
  cluster_arrive_release();
  cluster_wait_acquire();
  if (seg != 0 || threadIdx.x != 0) return;
  // ordered fold, as in rwi_publish_and_fold: strictly better moves the index; on a tie the left rule keeps the
  // earlier part and the right rule takes the later one; nothing after the first NaN counts
  float val = ident;
  int idx = 0, nan_at = INT_MAX;
  bool have = false, saw_nan = false;
  for (int s = 0; s < p.nseg && !saw_nan; ++s) {
    const float sv = row_parts[s].val;
    const int si = row_parts[s].idx, sa = row_parts[s].nan;
    if (si >= 0) {
      const bool better = IS_MAX ? (sv > val) : (sv < val);
      if (!have || better || (sv == val && !p.tie_left)) idx = si;
      val = have ? ext_nan<IS_MAX>(val, sv) : sv;
      have = true;
    }
    saw_nan = sa != INT_MAX;
    nan_at = sa;
  }
  if (saw_nan && p.nan_first) idx = nan_at;
  if (saw_nan) val = __int_as_float(0x7fc00000);
  rwi_write<DT>(p, src, row, val, idx, dst_val, dst_idx);
}

// Short rows (at most 64 vectors): `gs` lanes (4, 8, 16 or 32) share a row, so a warp holds 32 / gs rows and
// every lane has a load in flight; no shared memory, no barrier; a lane holds up to two vectors.  Same
// result as the kernels above.
template <int DT, bool IS_MAX, int NV>
__global__ void __launch_bounds__(256) rwi_warp_kernel(RwiParams p, int gs, const void *__restrict__ src,
                                                       void *__restrict__ dst_val, int32_t *__restrict__ dst_idx) {
  // gs lanes share a row, each holding up to NV of its 16-byte vectors; no block-wide barrier anywhere.  The common
  // row has no NaN: its extreme comes from packed max / min (16-bit types), the position from a second look at the
  // registers by the lanes that hold the extreme, and nothing else runs.  maximum / minimum propagate NaN, so a NaN
  // anywhere in a row shows in its extreme, and only then is the prefix before the first NaN searched.
  constexpr int kPerWord = FloatTraits<DT>::kPerWord;
  constexpr int kPerVec = 4 * kPerWord;
  using E = typename std::conditional<DT == BSIR_F32, float, uint16_t>::type;
  const int lane = threadIdx.x & 31, sl = lane & (gs - 1);
  const int rows_per_warp = 32 / gs;
  const int64_t warp_id = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int64_t row = warp_id * rows_per_warp + lane / gs;
  const bool row_ok = row < p.rows;                           // lanes of missing rows still take part in the shuffles
  const float ident = IS_MAX ? __int_as_float(0xff800000) : __int_as_float(0x7f800000);
  const Vec16 *xv = reinterpret_cast<const Vec16 *>(static_cast<const E *>(src) + (row_ok ? row : 0) * p.row_stride);
  Vec16 v[NV];
  bool have[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    have[i] = row_ok && sl + gs * i < p.nvec;
    if (have[i]) v[i] = ld_stream(xv + sl + gs * i);
  }
  auto for_each = [&](auto f) {   // f(row index of the element, its value)
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (have[i]) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          float e[kPerWord];
          FloatTraits<DT>::unpack(v[i].w[w], e);
#pragma unroll
          for (int k = 0; k < kPerWord; ++k) f((sl + gs * i) * kPerVec + w * kPerWord + k, e[k]);
        }
      }
  };
  auto group_ext = [&](float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, x, o);
      if (o < gs) x = ext_nan<IS_MAX>(x, other);
    }
    return x;
  };
  auto group_pick = [&](int b) {   // lowest (tie_left) or highest index over the row's lanes
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const int other = __shfl_xor_sync(0xffffffffu, b, o);
      if (o < gs) b = p.tie_left ? min(b, other) : max(b, other);
    }
    return b;
  };
  float tm = ident;
  if constexpr (kPerWord == 2) {   // 16-bit types stay packed: one max / min.NaN.x2 per word
    constexpr uint32_t kIdent2 = DT == BSIR_BF16 ? (IS_MAX ? 0xff80ff80u : 0x7f807f80u) : (IS_MAX ? 0xfc00fc00u : 0x7c007c00u);
    uint32_t m2 = kIdent2;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (have[i]) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          if constexpr (DT == BSIR_BF16) {
            if constexpr (IS_MAX) asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
            else asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
          } else {
            if constexpr (IS_MAX) asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
            else asm("min.NaN.f16x2 %0, %1, %2;" : "=r"(m2) : "r"(m2), "r"(v[i].w[w]));
          }
        }
      }
    float e2[2];
    FloatTraits<DT>::unpack(m2, e2);
    tm = ext_nan<IS_MAX>(e2[0], e2[1]);
  } else {
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (have[i]) {
#pragma unroll
        for (int w = 0; w < 4; ++w) tm = ext_nan<IS_MAX>(tm, __uint_as_float(v[i].w[w]));
      }
  }
  float m = group_ext(tm);
  // rows of one warp may differ in whether they hold a NaN: both searches run for all lanes, each row
  // keeps the one that applies to it
  int best = p.tie_left ? INT_MAX : -1;
  if (m == m && tm == m) for_each([&](int gi, float e) { if (e == m) best = p.tie_left ? min(best, gi) : max(best, gi); });
  best = group_pick(best);
  int nanpos = INT_MAX;
  if (__any_sync(0xffffffffu, m != m)) {
    // some row holds a NaN: its first position, the extreme of the prefix before it and that extreme's position
    for_each([&](int gi, float e) { if (e != e) nanpos = min(nanpos, gi); });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const int other = __shfl_xor_sync(0xffffffffu, nanpos, o);
      if (o < gs) nanpos = min(nanpos, other);
    }
    float tm2 = ident;
    for_each([&](int gi, float e) { if (gi < nanpos) tm2 = ext_nan<IS_MAX>(tm2, e); });
    const float m2 = group_ext(tm2);
    int best2 = p.tie_left ? INT_MAX : -1;
    for_each([&](int gi, float e) { if (gi < nanpos && e == m2) best2 = p.tie_left ? min(best2, gi) : max(best2, gi); });
    best2 = group_pick(best2);
    if (nanpos != INT_MAX) { m = m2; best = best2; }
  }
  if (row_ok && sl == 0) {
    float val = m;
    int idx = (best == INT_MAX || best < 0) ? 0 : best;
    if (nanpos != INT_MAX) {
      val = __int_as_float(0x7fc00000);
      if (p.nan_first) idx = nanpos;
    }
    rwi_write<DT>(p, src, row, val, idx, dst_val, dst_idx);
  }
}

// Scalar fallback: one CTA per row, any stride / alignment / length.
template <int DT, bool IS_MAX>
__global__ void __launch_bounds__(256) rwi_scalar_kernel(RwiParams p, const void *__restrict__ src,
                                                         void *__restrict__ dst_val, int32_t *__restrict__ dst_idx) {
  __shared__ float redf[8];
  __shared__ int redi[8];
  const int64_t row = blockIdx.x;
  const int64_t base = row * p.row_stride;
  const float ident = IS_MAX ? __int_as_float(0xff800000) : __int_as_float(0x7f800000);
  auto at = [&](int64_t j) -> float {
    if constexpr (DT == BSIR_F32) return static_cast<const float *>(src)[base + j];
    else if constexpr (DT == BSIR_F16) return __half2float(__ushort_as_half(static_cast<const uint16_t *>(src)[base + j]));
    else return __uint_as_float(static_cast<uint32_t>(static_cast<const uint16_t *>(src)[base + j]) << 16);
  };
  int nanpos = INT_MAX;
  for (int64_t j = threadIdx.x; j < p.cols; j += 256) {
    const float e = at(j);
    if (e != e) { nanpos = static_cast<int>(j); break; }
  }
  nanpos = cta_reduce_i(nanpos, redi, [](int a, int b) { return min(a, b); });
  const int64_t lim = nanpos == INT_MAX ? p.cols : nanpos;
  float m = ident;
  for (int64_t j = threadIdx.x; j < lim; j += 256) m = ext_nan<IS_MAX>(m, at(j));
  m = cta_reduce_f(m, redf, [](float a, float b) { return ext_nan<IS_MAX>(a, b); });
  int best = p.tie_left ? INT_MAX : -1;
  for (int64_t j = threadIdx.x; j < lim; j += 256)
    if (at(j) == m) best = p.tie_left ? min(best, static_cast<int>(j)) : max(best, static_cast<int>(j));
  if (p.tie_left) best = cta_reduce_i(best, redi, [](int a, int b) { return min(a, b); });
  else best = cta_reduce_i(best, redi, [](int a, int b) { return max(a, b); });
  if (threadIdx.x == 0) {
    int idx = (best == INT_MAX || best < 0) ? 0 : best;
    float val = m;
    if (nanpos != INT_MAX) {
      val = __int_as_float(0x7fc00000);
      if (p.nan_first) idx = nanpos;
    }
    rwi_write<DT>(p, src, row, val, idx, dst_val, dst_idx);
  }
}

// Segment plan: enough CTAs to fill the device, segments of at most 256 x 8 vectors.
void plan_segments(int64_t rows, int64_t nvec, int sm_count, int64_t *seg_vecs, int *nseg, int *vpt) {
  const int64_t target_ctas = static_cast<int64_t>(sm_count > 0 ? sm_count : 148) * 4;
  int64_t want_seg = rows > 0 ? ceil_div(target_ctas, rows) : 1;
  if (want_seg < 1) want_seg = 1;
  int64_t sv = ceil_div(nvec, want_seg);
  int64_t cap = 2048;
  if (const char *e = std::getenv("BSIR_RWI_SEGVECS")) { const long c = std::atol(e); if (c >= 256 && c <= 2048) cap = c; }
  if (sv > cap) sv = cap;
  if (sv < 256) sv = 256;
  int v = 1;
  while (v * 256 < sv) v <<= 1;
  *vpt = v;
  *seg_vecs = static_cast<int64_t>(v) * 256;
  *nseg = static_cast<int>(ceil_div(nvec, *seg_vecs));
  if (*nseg < 1) *nseg = 1;
}

// Streaming plan for long rows: as many equal parts per row as keep the CTA count within what is
// resident at once (4 CTAs of 256 threads per SM), each part at least 2048 vectors (two tiles).
bool plan_stream(int64_t rows, int64_t nvec, int sm_count, int64_t *seg_vecs, int *nseg) {
  const int64_t ctas = static_cast<int64_t>(sm_count > 0 ? sm_count : 148) * 4;
  if (nvec < 4096 || rows > ctas) return false;
  int64_t parts = ctas / rows;
  if (parts > nvec / 2048) parts = nvec / 2048;
  if (parts < 1) return false;
  const int64_t per = ceil_div(nvec, parts);
  *seg_vecs = per;
  *nseg = static_cast<int>(ceil_div(nvec, per));
  return true;
}

// Scratch layout: a fixed region of per-row counters first (so that, whatever shapes follow one
// another, only counters ever live there and "zero between calls" holds), partial results after it.
size_t rwi_scratch_bytes(int64_t rows, int nseg) {
  return kScratchCounterBytes + static_cast<size_t>(rows) * static_cast<size_t>(nseg) * sizeof(Partial);
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" {

int32_t bsir_reduce_last_axis(int32_t kind, int32_t dtype, int64_t rows, int64_t cols, const void *src,
                              int64_t src_row_stride, void *dst, void *stream) {
  return reduce_axis("reduce_last_axis", true, kind, dtype, rows, cols, src, src_row_stride, dst, stream);
}
int32_t bsir_reduce_first_axis(int32_t kind, int32_t dtype, int64_t rows, int64_t cols, const void *src,
                               int64_t src_row_stride, void *dst, void *stream) {
  return reduce_axis("reduce_first_axis", false, kind, dtype, rows, cols, src, src_row_stride, dst, stream);
}

int64_t bsir_reduce_with_index_workspace_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  size_t worst = 0;
  for (int eb = 2; eb <= 4; eb += 2) {
    int64_t sv; int ns, v;
    plan_segments(rows, ceil_div(cols * eb, 16), device_info().sm_count, &sv, &ns, &v);
    if (ns > 1) { const size_t b = rwi_scratch_bytes(rows, ns); if (b > worst) worst = b; }
    // the streaming kernel for long rows
    int64_t sv2; int ns2;
    if (plan_stream(rows < 65535 ? rows : 65535, ceil_div(cols * eb, 16), device_info().sm_count, &sv2, &ns2)) {
      const size_t b = rwi_scratch_bytes(rows < 65535 ? rows : 65535, ns2);
      if (b > worst) worst = b;
    }
  }
  return static_cast<int64_t>(worst);
}

int32_t bsir_reduce_with_index(int32_t kind, int32_t dtype, int32_t tie_break_left, int32_t nan_mode, int64_t rows,
                               int64_t cols, const void *src, int64_t src_row_stride, void *dst_value,
                               int32_t *dst_index, void *workspace, int64_t workspace_bytes, void *stream) {
  clear_error();
  if (kind < BSIR_RWI_MIN || kind > BSIR_RWI_MAXUI) return fail(BSIR_ERR_ATTR, "reduce_with_index: kind %d", kind);
  if (!dtype_is_float(dtype)) {
    if (dtype == BSIR_BOOL || dtype_bytes(dtype) == 0) return fail(BSIR_ERR_DTYPE, "reduce_with_index: dtype %d", dtype);
    return reduce_with_index_int(kind, dtype, tie_break_left, rows, cols, src, src_row_stride, dst_value, dst_index, resolve_stream(stream));
  }
  if (kind != BSIR_RWI_MAX && kind != BSIR_RWI_MIN)
    return fail(BSIR_ERR_ATTR, "reduce_with_index: kind %d (the unsigned kinds take integer inputs)", kind);
  if (nan_mode != BSIR_RWI_NAN_REGION && nan_mode != BSIR_RWI_NAN_FIRST)
    return fail(BSIR_ERR_ATTR, "reduce_with_index: nan_mode %d", nan_mode);
  if (rows < 0 || cols < 0) return fail(BSIR_ERR_SHAPE, "reduce_with_index: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (cols > INT_MAX - 64) return fail(BSIR_ERR_SHAPE, "reduce_with_index: cols exceed the int32 index range");
  // short rows: one warp per row, any number of rows in one launch
  if (rows > 0 && cols > 0 && src && dst_value && dst_index) {
    const int eb0 = dtype_bytes(dtype), pv0 = 16 / eb0;
    // up to two vectors a lane for any number of rows; up to four (a row of 128 vectors: 1024 bf16) when there are rows
    // enough to fill every SM with warps.  Beyond that a block a row wins: every row's warp has to look through its
    // registers for the position of the extreme, which in a block only the one warp that holds it does (measured on
    // bf16 [32768,4096]: 68 us with sixteen vectors a lane against 56 us with a block a row).
    const int sms0 = device_info().sm_count > 0 ? device_info().sm_count : 148;
    const int64_t nvec0 = cols % pv0 == 0 ? cols / pv0 : 0;
    const bool many_rows = rows >= static_cast<int64_t>(sms0) * 64;
    if (nvec0 > 0 && (nvec0 <= 64 || (many_rows && nvec0 <= 128)) && src_row_stride >= cols &&
        aligned_to(src, 16) && (src_row_stride * eb0) % 16 == 0 &&
        aligned_to(dst_value, eb0) && aligned_to(dst_index, 4) && rows <= 0x7fffffffLL * 8) {
      RwiParams q{};
      q.rows = rows; q.cols = cols; q.row_stride = src_row_stride; q.nvec = cols / pv0; q.nseg = 1;
      q.tie_left = tie_break_left ? 1 : 0;
      q.nan_first = nan_mode == BSIR_RWI_NAN_FIRST;
      cudaStream_t st0 = resolve_stream(stream);
      int gs = 4;                                           // lanes per row: each lane holds up to two vectors ...
      while (gs < 32 && q.nvec > 2 * gs) gs <<= 1;
      int nv = 2;                                           // ... or, with a whole warp on the row, up to four
      while (nv < 4 && q.nvec > static_cast<int64_t>(nv) * gs) nv <<= 1;
      const unsigned blocks = static_cast<unsigned>(ceil_div(rows, 8 * (32 / gs)));
      const bool mx = kind == BSIR_RWI_MAX;
#define W2(D, NV)                                                                                       \
  if (mx) rwi_warp_kernel<D, true, NV><<<blocks, 256, 0, st0>>>(q, gs, src, dst_value, dst_index);        \
  else rwi_warp_kernel<D, false, NV><<<blocks, 256, 0, st0>>>(q, gs, src, dst_value, dst_index);
#define W(D) \
  if (nv == 2) { W2(D, 2) } else { W2(D, 4) }
      if (dtype == BSIR_F32) { W(BSIR_F32) } else if (dtype == BSIR_F16) { W(BSIR_F16) } else { W(BSIR_BF16) }
#undef W2
#undef W
      count_launch();
      return check_launch("reduce_with_index");
    }
  }
  if (rows > 65535) {
    // grid.y limit: fold very tall inputs in slabs
    for (int64_t r0 = 0; r0 < rows; r0 += 65535) {
      const int64_t nr = rows - r0 < 65535 ? rows - r0 : 65535;
      const int eb0 = dtype_bytes(dtype);
      int32_t rc = bsir_reduce_with_index(kind, dtype, tie_break_left, nan_mode, nr, cols,
                                          static_cast<const char *>(src) + r0 * src_row_stride * eb0, src_row_stride,
                                          static_cast<char *>(dst_value) + r0 * eb0, dst_index + r0, workspace,
                                          workspace_bytes, stream);
      if (rc) return rc;
    }
    return BSIR_OK;
  }
  if (rows == 0) return BSIR_OK;
  if (!dst_value || !dst_index || (!src && cols > 0)) return fail(BSIR_ERR_NULL, "reduce_with_index: null pointer");
  if (src_row_stride < cols) return fail(BSIR_ERR_STRIDE, "reduce_with_index: row stride < cols");
  const int eb = dtype_bytes(dtype);
  if (!aligned_to(src, eb) || !aligned_to(dst_value, eb) || !aligned_to(dst_index, 4))
    return fail(BSIR_ERR_ALIGN, "reduce_with_index: misaligned");
  cudaStream_t st = resolve_stream(stream);
  RwiParams p{};
  p.rows = rows; p.cols = cols; p.row_stride = src_row_stride;
  p.tie_left = tie_break_left ? 1 : 0;
  p.nan_first = nan_mode == BSIR_RWI_NAN_FIRST;
  const bool is_max = kind == BSIR_RWI_MAX;
  const int per_vec = 16 / eb;
  const bool vec_ok = cols > 0 && cols % per_vec == 0 && aligned_to(src, 16) && (src_row_stride * eb) % 16 == 0;
  if (!vec_ok) {
    p.nseg = 1;
#define S(D) \
  if (is_max) rwi_scalar_kernel<D, true><<<static_cast<unsigned>(rows), 256, 0, st>>>(p, src, dst_value, dst_index); \
  else rwi_scalar_kernel<D, false><<<static_cast<unsigned>(rows), 256, 0, st>>>(p, src, dst_value, dst_index);
    if (dtype == BSIR_F32) { S(BSIR_F32) } else if (dtype == BSIR_F16) { S(BSIR_F16) } else { S(BSIR_BF16) }
#undef S
    count_launch();
    return check_launch("reduce_with_index");
  }
  p.nvec = cols / per_vec;
  // long rows, no more of them than CTAs fit on the device: rows cut into equal parts, streamed
  if (plan_stream(rows, p.nvec, device_info().sm_count, &p.seg_vecs, &p.nseg) &&
      std::getenv("BSIR_RWI_NO_STREAM") == nullptr) {
    const dim3 grid1(static_cast<unsigned>(p.nseg), static_cast<unsigned>(rows));
    if (p.nseg <= 8 && std::getenv("BSIR_RWI_NO_CLUSTER") == nullptr) {
      // a row's parts are one thread-block cluster and meet in shared memory: no scratch, no counters
      unsigned *no_cnt = nullptr;
      Partial *no_parts = nullptr;
#define LC(D)                                                                                                                    \
  if (is_max) launch_pdl_cluster(rwi_stream_kernel<D, true>, grid1, dim3(256), 0, st, p.nseg, p, src, dst_value, dst_index, no_cnt, no_parts); \
  else launch_pdl_cluster(rwi_stream_kernel<D, false>, grid1, dim3(256), 0, st, p.nseg, p, src, dst_value, dst_index, no_cnt, no_parts);
      if (dtype == BSIR_F32) { LC(BSIR_F32) } else if (dtype == BSIR_F16) { LC(BSIR_F16) } else { LC(BSIR_BF16) }
#undef LC
      count_launch();
      return check_launch("reduce_with_index");
    }
    const size_t need = rwi_scratch_bytes(rows, p.nseg);
    char *ws = static_cast<char *>(workspace);
    if (ws && (static_cast<size_t>(workspace_bytes) < need || !aligned_to(ws, 16)))
      return fail(BSIR_ERR_WORKSPACE, "reduce_with_index: the workspace given is %s (need %zu bytes, 16-byte aligned; "
                  "bsir_reduce_with_index_workspace_bytes gives the size)", aligned_to(ws, 16) ? "too small" : "misaligned", need);
    if (!ws) ws = static_cast<char *>(device_workspace(need, st));
    if (!ws) return BSIR_ERR_WORKSPACE;
    unsigned *cnt = reinterpret_cast<unsigned *>(ws);
    Partial *parts = reinterpret_cast<Partial *>(ws + kScratchCounterBytes);
#define LS(D)                                                                                         \
  if (is_max) launch_pdl(rwi_stream_kernel<D, true>, grid1, dim3(256), 0, st, p, src, dst_value, dst_index, cnt, parts); \
  else launch_pdl(rwi_stream_kernel<D, false>, grid1, dim3(256), 0, st, p, src, dst_value, dst_index, cnt, parts);
    if (dtype == BSIR_F32) { LS(BSIR_F32) } else if (dtype == BSIR_F16) { LS(BSIR_F16) } else { LS(BSIR_BF16) }
#undef LS
    count_launch();
    return check_launch("reduce_with_index");
  }
  int vpt = 1;
  plan_segments(rows, p.nvec, device_info().sm_count, &p.seg_vecs, &p.nseg, &vpt);
  unsigned *counters = nullptr;
  Partial *partials = nullptr;
  if (p.nseg > 1) {
    const size_t need = rwi_scratch_bytes(rows, p.nseg);
    char *ws = static_cast<char *>(workspace);
    if (ws && (static_cast<size_t>(workspace_bytes) < need || !aligned_to(ws, 16)))
      return fail(BSIR_ERR_WORKSPACE, "reduce_with_index: the workspace given is %s (need %zu bytes, 16-byte aligned; "
                  "bsir_reduce_with_index_workspace_bytes gives the size)", aligned_to(ws, 16) ? "too small" : "misaligned", need);
    if (!ws) ws = static_cast<char *>(device_workspace(need, st));
    if (!ws) return BSIR_ERR_WORKSPACE;
    counters = reinterpret_cast<unsigned *>(ws);
    partials = reinterpret_cast<Partial *>(ws + kScratchCounterBytes);
  }
  const dim3 grid(static_cast<unsigned>(p.nseg), static_cast<unsigned>(rows));
#define L(D, V)                                                                                             \
  if (is_max) rwi_kernel<D, V, true><<<grid, 256, 0, st>>>(p, src, dst_value, dst_index, counters, partials); \
  else rwi_kernel<D, V, false><<<grid, 256, 0, st>>>(p, src, dst_value, dst_index, counters, partials);
#define LV(D)                      \
  switch (vpt) {                   \
    case 1: L(D, 1) break;         \
    case 2: L(D, 2) break;         \
    case 4: L(D, 4) break;         \
    case 8: L(D, 8) break;         \
    default: L(D, 16) break;       \
  }
  if (dtype == BSIR_F32) { LV(BSIR_F32) } else if (dtype == BSIR_F16) { LV(BSIR_F16) } else { LV(BSIR_BF16) }
#undef LV
#undef L
  count_launch();
  return check_launch("reduce_with_index");
}

}  // extern "C"

// ------------------------------------------------------------------ reduce_with_index without allocation
// Some hosts hand every byte of device memory to their own pool at start-up (an inference server that
// sizes its cache to whatever is left), or call from places where the CUDA allocator must not be
// entered; they cannot let a library call cudaMalloc behind their back, and they may have no pool
// block to spare for a workspace argument either.  For them the scratch of the segmented argmax /
// argmin lives in the library image itself: a fixed array in device memory that every GPU loading the
// library carries until the process exits.
namespace bsir {
namespace {

constexpr int kStaticMaxRows = 4096;                                   // one counter per row
constexpr size_t kStaticCounterBytes = kStaticMaxRows * sizeof(unsigned);
constexpr size_t kStaticScratchBytes = 512 * 1024;                     // counters + partial results
constexpr size_t kStaticMaxPartials = (kStaticScratchBytes - kStaticCounterBytes) / sizeof(Partial);

static __device__ __align__(256) unsigned char g_rwi_static_scratch[kStaticScratchBytes];

// Device address of the array on each device, looked up once per device.  In host code the array's
// name is only a handle for the runtime, not a pointer a kernel could use.
void *g_rwi_static_ptr[64] = {nullptr};
std::mutex g_rwi_static_mu;

int32_t static_scratch(void **out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return fail(BSIR_ERR_WORKSPACE, "reduce_with_index_static: no current CUDA device");
  }
  std::lock_guard<std::mutex> lock(g_rwi_static_mu);
  if (!g_rwi_static_ptr[dev]) {
    void *ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_rwi_static_scratch);
    if (e != cudaSuccess || !ptr) {
      cudaGetLastError();
      return fail(BSIR_ERR_WORKSPACE, "reduce_with_index_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    }
    g_rwi_static_ptr[dev] = ptr;
  }
  *out = g_rwi_static_ptr[dev];
  return BSIR_OK;
}

}  // namespace
}  // namespace bsir

// Same result as bsir_reduce_with_index, with the scratch taken from the fixed in-library array:
// no cudaMalloc, cudaFree or other allocating call, on any path.
//
// Limits: rows <= 4096 and rows x segments <= 31744 partial results (the segment count is what
// bsir_reduce_with_index would choose).  Larger problems are refused with BSIR_ERR_WORKSPACE and
// nothing is enqueued.  Kernels: the same ones bsir_reduce_with_index picks -- the streaming kernel
// for long rows (the 256 x 152064 shape: 2 parts per row), the segmented kernel otherwise, the
// one-CTA-per-row kernel for unaligned rows -- except that rows of at most 64 vectors also take the
// segmented kernel; one small memset ahead of the launch clears the row counters.
//
// The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
// that device current); make that first call before any stream capture begins on the device.
// All calls share the one array, which keeps whatever the previous call left in it: the row
// counters the kernel needs at zero are cleared on `stream` ahead of each launch.  Two calls whose
// kernels may overlap on the GPU (different streams, no ordering between them) race on the array;
// order them, or give one of them bsir_reduce_with_index with a workspace of its own.
extern "C" int32_t bsir_reduce_with_index_static(int32_t kind, int32_t dtype, int32_t tie_break_left, int32_t nan_mode,
                                                 int64_t rows, int64_t cols, const void *src, int64_t src_row_stride,
                                                 void *dst_value, int32_t *dst_index, void *stream) {
  clear_error();
  if (!dtype_is_float(dtype)) return fail(BSIR_ERR_DTYPE, "reduce_with_index_static: dtype %d (f32, f16 or bf16)", dtype);
  if (kind != BSIR_RWI_MAX && kind != BSIR_RWI_MIN) return fail(BSIR_ERR_ATTR, "reduce_with_index_static: kind %d", kind);
  if (nan_mode != BSIR_RWI_NAN_REGION && nan_mode != BSIR_RWI_NAN_FIRST)
    return fail(BSIR_ERR_ATTR, "reduce_with_index_static: nan_mode %d", nan_mode);
  if (rows < 0 || cols < 0) return fail(BSIR_ERR_SHAPE, "reduce_with_index_static: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (cols > INT_MAX - 64) return fail(BSIR_ERR_SHAPE, "reduce_with_index_static: cols exceed the int32 index range");
  if (rows > kStaticMaxRows)
    return fail(BSIR_ERR_WORKSPACE, "reduce_with_index_static: %lld rows exceed the fixed scratch (at most %d rows)",
                (long long)rows, kStaticMaxRows);
  if (rows == 0) return BSIR_OK;
  if (!dst_value || !dst_index || (!src && cols > 0)) return fail(BSIR_ERR_NULL, "reduce_with_index_static: null pointer");
  if (src_row_stride < cols) return fail(BSIR_ERR_STRIDE, "reduce_with_index_static: row stride < cols");
  const int eb = dtype_bytes(dtype);
  if (!aligned_to(src, eb) || !aligned_to(dst_value, eb) || !aligned_to(dst_index, 4))
    return fail(BSIR_ERR_ALIGN, "reduce_with_index_static: misaligned");
  void *scratch = nullptr;
  if (int32_t rc = static_scratch(&scratch)) return rc;
  cudaStream_t st = resolve_stream(stream);
  RwiParams p{};
  p.rows = rows; p.cols = cols; p.row_stride = src_row_stride;
  p.tie_left = tie_break_left ? 1 : 0;
  p.nan_first = nan_mode == BSIR_RWI_NAN_FIRST;
  const bool is_max = kind == BSIR_RWI_MAX;
  const int per_vec = 16 / eb;
  const bool vec_ok = cols > 0 && cols % per_vec == 0 && aligned_to(src, 16) && (src_row_stride * eb) % 16 == 0;
  if (!vec_ok) {
    p.nseg = 1;  // the one-CTA-per-row kernel needs no scratch at all
#define S(D) \
  if (is_max) rwi_scalar_kernel<D, true><<<static_cast<unsigned>(rows), 256, 0, st>>>(p, src, dst_value, dst_index); \
  else rwi_scalar_kernel<D, false><<<static_cast<unsigned>(rows), 256, 0, st>>>(p, src, dst_value, dst_index);
    if (dtype == BSIR_F32) { S(BSIR_F32) } else if (dtype == BSIR_F16) { S(BSIR_F16) } else { S(BSIR_BF16) }
#undef S
    count_launch();
    return check_launch("reduce_with_index_static");
  }
  p.nvec = cols / per_vec;
  unsigned *counters = reinterpret_cast<unsigned *>(scratch);
  Partial *partials = reinterpret_cast<Partial *>(static_cast<unsigned char *>(scratch) + kStaticCounterBytes);
  // long rows: the streaming kernel bsir_reduce_with_index uses for them, whenever its partial results fit the array
  if (plan_stream(rows, p.nvec, device_info().sm_count, &p.seg_vecs, &p.nseg) && std::getenv("BSIR_RWI_NO_STREAM") == nullptr &&
      static_cast<size_t>(rows) * static_cast<size_t>(p.nseg) <= kStaticMaxPartials) {
    if (cudaMemsetAsync(counters, 0, static_cast<size_t>(rows) * sizeof(unsigned), st) != cudaSuccess)
      return check_launch("reduce_with_index_static (clearing the counters)");
    const dim3 grid1(static_cast<unsigned>(p.nseg), static_cast<unsigned>(rows));
#define LS(D)                                                                                                    \
  if (is_max) rwi_stream_kernel<D, true><<<grid1, 256, 0, st>>>(p, src, dst_value, dst_index, counters, partials); \
  else rwi_stream_kernel<D, false><<<grid1, 256, 0, st>>>(p, src, dst_value, dst_index, counters, partials);
    if (dtype == BSIR_F32) { LS(BSIR_F32) } else if (dtype == BSIR_F16) { LS(BSIR_F16) } else { LS(BSIR_BF16) }
#undef LS
    count_launch();
    return check_launch("reduce_with_index_static");
  }
  int vpt = 1;
  plan_segments(rows, p.nvec, device_info().sm_count, &p.seg_vecs, &p.nseg, &vpt);
  if (static_cast<size_t>(rows) * static_cast<size_t>(p.nseg) > kStaticMaxPartials)
    return fail(BSIR_ERR_WORKSPACE,
                "reduce_with_index_static: %lld rows x %d segments exceed the fixed scratch (at most %zu partial results)",
                (long long)rows, p.nseg, kStaticMaxPartials);
  if (p.nseg > 1) {
    // the counters must start at zero whatever an earlier (possibly failed) call left behind
    if (cudaMemsetAsync(counters, 0, static_cast<size_t>(rows) * sizeof(unsigned), st) != cudaSuccess)
      return check_launch("reduce_with_index_static (clearing the counters)");
  }
  const dim3 grid(static_cast<unsigned>(p.nseg), static_cast<unsigned>(rows));
#define L(D, V)                                                                                             \
  if (is_max) rwi_kernel<D, V, true><<<grid, 256, 0, st>>>(p, src, dst_value, dst_index, counters, partials); \
  else rwi_kernel<D, V, false><<<grid, 256, 0, st>>>(p, src, dst_value, dst_index, counters, partials);
#define LV(D)                      \
  switch (vpt) {                   \
    case 1: L(D, 1) break;         \
    case 2: L(D, 2) break;         \
    case 4: L(D, 4) break;         \
    default: L(D, 8) break;        \
  }
  if (dtype == BSIR_F32) { LV(BSIR_F32) } else if (dtype == BSIR_F16) { LV(BSIR_F16) } else { LV(BSIR_BF16) }
#undef LV
#undef L
  count_launch();
  return check_launch("reduce_with_index_static");
}
