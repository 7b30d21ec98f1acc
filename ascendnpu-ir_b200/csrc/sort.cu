// sort.cu -- hivm.hir.vsort over the last axis: sorted values and the source index of each
// (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:2222-2283).
//
// Order: ascending (or descending) by value; equal values keep their source order (stable), -0 and +0 compare
// equal, NaN sorts after every number when ascending and before every number when descending.  A row becomes
// 64-bit keys  order(value) << 32 | index  (order() maps the element type to unsigned integers that compare
// like the values; descending complements it), so one integer comparison decides value and tie at once and the
// bitonic network -- not stable by itself -- gives a stable result.  A CTA sorts one row in shared memory
// (rows of up to 8192 elements: 64 KB of keys); the values are read back from the source by index, so their
// bits (the sign of a zero, the payload of a NaN) are the source's.
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
    if (f != f) return 0xffffffffu;                 // NaN: after every number
    uint32_t b = __float_as_uint(f);
    if (b == 0x80000000u) b = 0u;                   // -0 ties with +0
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  }
}

template <int DT>
__global__ void __launch_bounds__(kSortThreads) sort_rows_kernel(const typename SortElem<DT>::type *__restrict__ src, int64_t src_stride,
                                                                 typename SortElem<DT>::type *__restrict__ dst_value, int64_t val_stride,
                                                                 int32_t *__restrict__ dst_index, int64_t idx_stride, int64_t cols,
                                                                 int npow2, int descending) {
  extern __shared__ unsigned long long keys[];
  const int64_t row = blockIdx.x;
  const auto *s = src + row * src_stride;
  for (int i = threadIdx.x; i < npow2; i += kSortThreads) {
    unsigned long long k = ~0ull;                   // padding sorts last
    if (i < cols) {
      uint32_t o = sort_order<DT>(s[i]);
      if (descending) o = ~o;
      k = (static_cast<unsigned long long>(o) << 32) | static_cast<uint32_t>(i);
    }
    keys[i] = k;
  }
  __syncthreads();
  for (int k = 2; k <= npow2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < npow2 / 2; t += kSortThreads) {
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
  for (int i = threadIdx.x; i < cols; i += kSortThreads) {
    const uint32_t idx = static_cast<uint32_t>(keys[i]);
    if (dst_value) dst_value[row * val_stride + i] = s[idx];
    if (dst_index) dst_index[row * idx_stride + i] = static_cast<int32_t>(idx);
  }
}

template <int DT>
void launch_sort(const void *src, int64_t ss, void *dv, int64_t vs, int32_t *di, int64_t is, int64_t rows, int64_t cols, int descending,
                 cudaStream_t st) {
  using T = typename SortElem<DT>::type;
  int npow2 = 2;
  while (npow2 < cols) npow2 <<= 1;
  const size_t smem = static_cast<size_t>(npow2) * sizeof(unsigned long long);
  static bool attr_done = false;   // per instantiation
  if (!attr_done) {
    cudaFuncSetAttribute(sort_rows_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSortMaxLen * 8);
    attr_done = true;
  }
  sort_rows_kernel<DT><<<static_cast<unsigned>(rows), kSortThreads, smem, st>>>(static_cast<const T *>(src), ss, static_cast<T *>(dv), vs, di, is,
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
  if (cols > kSortMaxLen) return fail(BSIR_ERR_UNSUPPORTED, "sort: rows of %lld elements (at most %d are sorted in shared memory)", (long long)cols, kSortMaxLen);
  if (rows > 0x7fffffffLL) return fail(BSIR_ERR_SHAPE, "sort: %lld rows", (long long)rows);
  if (src_row_stride < cols || (dst_value && value_row_stride < cols) || (dst_index && index_row_stride < cols))
    return fail(BSIR_ERR_STRIDE, "sort: row stride below the row length");
  const int eb = dtype_bytes(dtype);
  if (!aligned_to(src, eb) || !aligned_to(dst_value, eb) || !aligned_to(dst_index, 4)) return fail(BSIR_ERR_ALIGN, "sort: misaligned");
  cudaStream_t st = resolve_stream(stream);
  const int desc = descending != 0;
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
