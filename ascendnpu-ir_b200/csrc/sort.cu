// sort.cu -- hivm.hir.vsort over the last axis: sorted values and the source index of each
// (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:2222-2283).
//
// The result is the one the reference's lowering of hfusion.sort produces: n-1 bubble passes of n-1 adjacent
// compare-and-swaps on `cmpf ugt` (ascending) / `cmpf ult` (descending), `cmpi sgt` / `slt` for integers
// (bishengir/lib/Dialect/HFusion/Transforms/DecomposeOpInterfaceImpl.cpp:742-838).  In closed form: equal values
// keep their source order (stable; -0 and +0 are equal); a pair holding a NaN always swaps, which moves every NaN
// one place to the left per pass and carries the one at the front to the end, so a NaN that starts at position p
// ends at (p + 1) mod n whatever the direction; the numbers fill the other places in order.
//
// A row becomes 64-bit keys  order(value) << 32 | index  (order() maps the element type to unsigned integers
// that compare like the values; descending complements it; NaN is the largest key in both directions), so one
// integer comparison decides value and tie at once and the bitonic network -- not stable by itself -- gives a
// stable result with the NaNs at the end in source order; the write-out then moves them to their places.  A CTA sorts one row in shared memory
// (rows of up to 8192 elements: 64 KB of keys); longer rows keep their keys in device scratch and run the wide
// steps of the network on global memory.  The values are read back from the source by index, so their bits
// (the sign of a zero, the payload of a NaN) are the source's.
#include <cstdint>

#include "common.cuh"

namespace bsir {
namespace {

constexpr int kSortThreads = 512;
constexpr int kSortMaxLen = 8192;

template <int DT> struct SortElem;
template <> struct SortElem<BSIR_F32> { using type = float; };
template <> struct SortElem<BSIR_F16> { using type = uint16_t; };
template <> struct SortElem<BSIR_BF16> { using type = uint16_t; };
template <> struct SortElem<BSIR_I8> { using type = int8_t; };
template <> struct SortElem<BSIR_I16> { using type = int16_t; };
template <> struct SortElem<BSIR_I32> { using type = int32_t; };

// unsigned integers that compare like the values
template <int DT>
__device__ __forceinline__ uint32_t sort_order(typename SortElem<DT>::type v) {
  if constexpr (DT == BSIR_I8 || DT == BSIR_I16 || DT == BSIR_I32) {
    return static_cast<uint32_t>(static_cast<int32_t>(v)) ^ 0x80000000u;
  } else {
    float f;
    if constexpr (DT == BSIR_F32) f = v;
    else if constexpr (DT == BSIR_F16) f = __half2float(__ushort_as_half(v));
    else f = __uint_as_float(static_cast<uint32_t>(v) << 16);
    if (f != f) return 0xffffffffu;                 // NaN: no number maps here (+inf is 0xff800000)
    uint32_t b = __float_as_uint(f);
    if (b == 0x80000000u) b = 0u;                   // -0 ties with +0
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  }
}

template <int DT> constexpr bool kSortFloat = DT == BSIR_F32 || DT == BSIR_F16 || DT == BSIR_BF16;

template <int DT>
__device__ __forceinline__ unsigned long long sort_key(typename SortElem<DT>::type v, int64_t pos, int descending) {
  uint32_t o = sort_order<DT>(v);
  if (descending && !(kSortFloat<DT> && o == 0xffffffffu)) o = ~o;      // a NaN key stays the largest
  return (static_cast<unsigned long long>(o) << 32) | static_cast<uint32_t>(pos);
}

__device__ __forceinline__ bool sort_key_is_nan(unsigned long long k) { return (k >> 32) == 0xffffffffull && k != ~0ull; }

// Where element i of the sorted keys (numbers first, then the row's `nan` NaNs in source order) goes in a row of
// `cols`.  The NaN from source position p goes to (p + 1) mod cols; number r takes the r-th place no NaN took:
// with the NaN places T[0] < T[1] < ... ascending, that is r + #{j : T[j] - j <= r}.
__device__ __forceinline__ int64_t sort_place(const unsigned long long *keys, int64_t i, int64_t cols, int64_t nan) {
  const int64_t numbers = cols - nan;
  if (i >= numbers) {
    const int64_t p = static_cast<uint32_t>(keys[i]);
    return p + 1 == cols ? 0 : p + 1;
  }
  const bool wrap = static_cast<uint32_t>(keys[cols - 1]) == cols - 1;   // the last NaN sits at the row's end
  int64_t lo = 0, hi = nan;                                             // first j with T[j] - j > i
  while (lo < hi) {
    const int64_t j = (lo + hi) >> 1;
    const int64_t t = wrap ? (j == 0 ? 0 : static_cast<int64_t>(static_cast<uint32_t>(keys[numbers + j - 1])) + 1)
                           : static_cast<int64_t>(static_cast<uint32_t>(keys[numbers + j])) + 1;
    if (t - j <= i) lo = j + 1; else hi = j;
  }
  return i + lo;
}

// number of NaN keys at the end of a sorted row (keys[0 .. cols))
__device__ __forceinline__ int64_t sort_count_nan(const unsigned long long *keys, int64_t cols) {
  if (!sort_key_is_nan(keys[cols - 1])) return 0;
  int64_t lo = 0, hi = cols - 1;                                        // first NaN key
  while (lo < hi) {
    const int64_t m = (lo + hi) >> 1;
    if (sort_key_is_nan(keys[m])) hi = m; else lo = m + 1;
  }
  return cols - lo;
}

template <int DT>
__global__ void __launch_bounds__(kSortThreads) sort_rows_kernel(const typename SortElem<DT>::type *__restrict__ src, int64_t src_stride,
                                                                 typename SortElem<DT>::type *__restrict__ dst_value, int64_t val_stride,
                                                                 int32_t *__restrict__ dst_index, int64_t idx_stride, int64_t cols,
                                                                 int npow2, int descending) {
  extern __shared__ unsigned long long keys[];
  const int64_t row = blockIdx.x;
  const auto *s = src + row * src_stride;
  for (int i = threadIdx.x; i < npow2; i += blockDim.x) {
    unsigned long long k = ~0ull;                   // padding sorts last
    if (i < cols) k = sort_key<DT>(s[i], i, descending);
    keys[i] = k;
  }
  __syncthreads();
  for (int k = 2; k <= npow2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < npow2 / 2; t += blockDim.x) {
        const int lo = ((t & ~(j - 1)) << 1) | (t & (j - 1)), hi = lo | j;   // the pair this step compares
        const bool up = (lo & k) == 0;
        const unsigned long long a = keys[lo], b = keys[hi];
        if ((a > b) == up) {
          keys[lo] = b;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  int64_t nan = 0;
  if constexpr (kSortFloat<DT>) nan = sort_count_nan(keys, cols);
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    const uint32_t idx = static_cast<uint32_t>(keys[i]);
    const int64_t at = nan ? sort_place(keys, i, cols, nan) : i;
    if (dst_value) dst_value[row * val_stride + at] = s[idx];
    if (dst_index) dst_index[row * idx_stride + at] = static_cast<int32_t>(idx);
  }
}

// ------------------------------------------------------------------ rows longer than one CTA's shared memory
// The same network over keys kept in device scratch ([rows][npow2] 64-bit words): one launch sorts every 8192-key
// chunk in shared memory (all steps with k <= 8192, directions taken from the position in the whole row), then
// for k = 16384, 32768, ...: the steps whose partners are 8192 or more apart run on global memory, one launch
// each, and the steps below that again in shared memory, one launch per k.
template <int DT>
__global__ void __launch_bounds__(kSortThreads) sort_chunks_kernel(const typename SortElem<DT>::type *__restrict__ src, int64_t src_stride,
                                                                   unsigned long long *__restrict__ keys_g, int64_t cols, int npow2,
                                                                   int descending, int k_first, int k_last) {
  // k_first == 2: build the keys from the source and run k = 2 .. k_last; otherwise k = k_first only, with the
  // steps j < kSortMaxLen (the wider ones were done on global memory)
  extern __shared__ unsigned long long keys[];
  const int64_t row = blockIdx.y;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kSortMaxLen;      // position of this chunk in the row
  unsigned long long *g = keys_g + row * npow2 + base;
  if (k_first == 2) {
    const auto *s = src + row * src_stride;
    for (int i = threadIdx.x; i < kSortMaxLen; i += kSortThreads) {
      const int64_t pos = base + i;
      unsigned long long k = ~0ull;
      if (pos < cols) k = sort_key<DT>(s[pos], pos, descending);
      keys[i] = k;
    }
  } else {
    for (int i = threadIdx.x; i < kSortMaxLen; i += kSortThreads) keys[i] = g[i];
  }
  __syncthreads();
  for (int64_t k = k_first; k <= k_last; k <<= 1) {
    for (int j = static_cast<int>(k >> 1 < kSortMaxLen ? k >> 1 : kSortMaxLen >> 1); j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < kSortMaxLen / 2; t += kSortThreads) {
        const int lo = ((t & ~(j - 1)) << 1) | (t & (j - 1)), hi = lo | j;
        const bool up = ((base + lo) & k) == 0;
        const unsigned long long a = keys[lo], b = keys[hi];
        if ((a > b) == up) {
          keys[lo] = b;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < kSortMaxLen; i += kSortThreads) g[i] = keys[i];
}

// one compare-exchange step (partners j apart, j >= kSortMaxLen) of stage k on global memory
__global__ void __launch_bounds__(256) sort_global_step_kernel(unsigned long long *__restrict__ keys_g, int npow2, int64_t k, int64_t j) {
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= npow2 / 2) return;
  unsigned long long *g = keys_g + static_cast<int64_t>(blockIdx.y) * npow2;
  const int64_t lo = ((t & ~(j - 1)) << 1) | (t & (j - 1)), hi = lo | j;
  const bool up = (lo & k) == 0;
  const unsigned long long a = g[lo], b = g[hi];
  if ((a > b) == up) {
    g[lo] = b;
    g[hi] = a;
  }
}

template <int DT>
__global__ void __launch_bounds__(256) sort_emit_kernel(const typename SortElem<DT>::type *__restrict__ src, int64_t src_stride,
                                                        const unsigned long long *__restrict__ keys_g, int npow2,
                                                        typename SortElem<DT>::type *__restrict__ dst_value, int64_t val_stride,
                                                        int32_t *__restrict__ dst_index, int64_t idx_stride, int64_t cols) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= cols) return;
  const int64_t row = blockIdx.y;
  const unsigned long long *keys = keys_g + row * npow2;
  const uint32_t idx = static_cast<uint32_t>(keys[i]);
  int64_t at = i;
  if constexpr (kSortFloat<DT>) {
    const int64_t nan = sort_count_nan(keys, cols);          // one load when the row has no NaN
    if (nan) at = sort_place(keys, i, cols, nan);
  }
  if (dst_value) dst_value[row * val_stride + at] = src[row * src_stride + idx];
  if (dst_index) dst_index[row * idx_stride + at] = static_cast<int32_t>(idx);
}

// rows per pass such that the keys fit `budget` bytes of scratch
template <int DT>
int32_t launch_sort_long(const void *src, int64_t ss, void *dv, int64_t vs, int32_t *di, int64_t is, int64_t rows, int64_t cols,
                         int descending, cudaStream_t st) {
  using T = typename SortElem<DT>::type;
  int64_t npow2 = kSortMaxLen;
  while (npow2 < cols) npow2 <<= 1;
  if (npow2 > (int64_t(1) << 30)) return fail(BSIR_ERR_UNSUPPORTED, "sort: rows of %lld elements", (long long)cols);
  const int64_t row_bytes = npow2 * 8;
  const int64_t budget = int64_t(1) << 30;                       // at most 1 GiB of keys at a time
  int64_t rows_per_pass = budget / row_bytes;
  if (rows_per_pass < 1) rows_per_pass = 1;
  if (rows_per_pass > rows) rows_per_pass = rows;
  if (rows_per_pass > 65535) rows_per_pass = 65535;
  char *ws = static_cast<char *>(device_workspace(kScratchCounterBytes + static_cast<size_t>(rows_per_pass * row_bytes), st));
  if (!ws) return BSIR_ERR_WORKSPACE;
  unsigned long long *keys = reinterpret_cast<unsigned long long *>(ws + kScratchCounterBytes);
  // the attribute belongs to the current device's copy of the kernel: set it on every call, not once per process
  cudaFuncSetAttribute(sort_chunks_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSortMaxLen * 8);
  const T *s = static_cast<const T *>(src);
  T *d = static_cast<T *>(dv);
  const int n = static_cast<int>(npow2);
  for (int64_t r0 = 0; r0 < rows; r0 += rows_per_pass) {
    const unsigned nr = static_cast<unsigned>(rows - r0 < rows_per_pass ? rows - r0 : rows_per_pass);
    const dim3 chunks(static_cast<unsigned>(npow2 / kSortMaxLen), nr);
    sort_chunks_kernel<DT><<<chunks, kSortThreads, kSortMaxLen * 8, st>>>(s + r0 * ss, ss, keys, cols, n, descending, 2, kSortMaxLen);
    count_launch();
    for (int64_t k = 2 * kSortMaxLen; k <= npow2; k <<= 1) {
      for (int64_t j = k >> 1; j >= kSortMaxLen; j >>= 1) {
        sort_global_step_kernel<<<dim3(static_cast<unsigned>(ceil_div(npow2 / 2, 256)), nr), 256, 0, st>>>(keys, n, k, j);
        count_launch();
      }
      sort_chunks_kernel<DT><<<chunks, kSortThreads, kSortMaxLen * 8, st>>>(s, ss, keys, cols, n, descending, static_cast<int>(k), static_cast<int>(k));
      count_launch();
    }
    sort_emit_kernel<DT><<<dim3(static_cast<unsigned>(ceil_div(cols, 256)), nr), 256, 0, st>>>(
        s + r0 * ss, ss, keys, n, d ? d + r0 * vs : nullptr, vs, di ? di + r0 * is : nullptr, is, cols);
  }
  return BSIR_OK;
}

template <int DT>
void launch_sort(const void *src, int64_t ss, void *dv, int64_t vs, int32_t *di, int64_t is, int64_t rows, int64_t cols, int descending,
                 cudaStream_t st) {
  using T = typename SortElem<DT>::type;
  int npow2 = 2;
  while (npow2 < cols) npow2 <<= 1;
  const size_t smem = static_cast<size_t>(npow2) * sizeof(unsigned long long);
  if (smem > 48 * 1024)   // per device, so on every such call rather than once per process
    cudaFuncSetAttribute(sort_rows_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSortMaxLen * 8);
  // half a thread per padded element (each step compares pairs), within [32, 512]: short rows do not pay for
  // idle warps at every barrier
  int threads = npow2 / 2 < 32 ? 32 : npow2 / 2 > kSortThreads ? kSortThreads : npow2 / 2;
  sort_rows_kernel<DT><<<static_cast<unsigned>(rows), threads, smem, st>>>(static_cast<const T *>(src), ss, static_cast<T *>(dv), vs, di, is,
                                                                               cols, npow2, descending);
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" int32_t bsir_sort(int32_t dtype, int32_t descending, int64_t rows, int64_t cols, const void *src, int64_t src_row_stride,
                             void *dst_value, int64_t value_row_stride, int32_t *dst_index, int64_t index_row_stride, void *stream) {
  clear_error();
  const bool ok_type = dtype == BSIR_F32 || dtype == BSIR_F16 || dtype == BSIR_BF16 || dtype == BSIR_I8 || dtype == BSIR_I16 || dtype == BSIR_I32;
  if (!ok_type) return fail(BSIR_ERR_DTYPE, "sort: dtype %d (f32, f16, bf16, i8, i16, i32)", dtype);
  if (rows < 0 || cols < 0) return fail(BSIR_ERR_SHAPE, "sort: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (rows == 0 || cols == 0) return BSIR_OK;
  if (!src || (!dst_value && !dst_index)) return fail(BSIR_ERR_NULL, "sort: null pointer");
  if (rows > 0x7fffffffLL) return fail(BSIR_ERR_SHAPE, "sort: %lld rows", (long long)rows);
  if (src_row_stride < cols || (dst_value && value_row_stride < cols) || (dst_index && index_row_stride < cols))
    return fail(BSIR_ERR_STRIDE, "sort: row stride below the row length");
  const int eb = dtype_bytes(dtype);
  if (!aligned_to(src, eb) || !aligned_to(dst_value, eb) || !aligned_to(dst_index, 4)) return fail(BSIR_ERR_ALIGN, "sort: misaligned");
  cudaStream_t st = resolve_stream(stream);
  const int desc = descending != 0;
  if (cols > kSortMaxLen) {   // keys in device scratch, the wide steps of the network on global memory
    int32_t rc;
    switch (dtype) {
      case BSIR_F32: rc = launch_sort_long<BSIR_F32>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
      case BSIR_F16: rc = launch_sort_long<BSIR_F16>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
      case BSIR_BF16: rc = launch_sort_long<BSIR_BF16>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
      case BSIR_I8: rc = launch_sort_long<BSIR_I8>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
      case BSIR_I16: rc = launch_sort_long<BSIR_I16>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
      default: rc = launch_sort_long<BSIR_I32>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
    }
    if (rc != BSIR_OK) return rc;
    count_launch();
    return check_launch("sort");
  }
  switch (dtype) {
    case BSIR_F32: launch_sort<BSIR_F32>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
    case BSIR_F16: launch_sort<BSIR_F16>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
    case BSIR_BF16: launch_sort<BSIR_BF16>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
    case BSIR_I8: launch_sort<BSIR_I8>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
    case BSIR_I16: launch_sort<BSIR_I16>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
    default: launch_sort<BSIR_I32>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); break;
  }
  count_launch();
  return check_launch("sort");
}
