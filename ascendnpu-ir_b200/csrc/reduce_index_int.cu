// reduce_index_int.cu -- hfusion.reduce_with_index over integer rows, and its unsigned kinds
// (bishengir/include/bishengir/Dialect/HFusion/IR/HFusionStructuredOps.td:69-137; kinds min / max / minui / maxui,
// HFusionEnums.td:303-311: the *ui kinds compare the same bits as unsigned numbers, the region uses cmpi ugt / ult
// where min / max use sgt / slt, HFusionOps.cpp:1541-1595).  Ties keep the lowest index with tie_break_left, the
// highest otherwise.  The result is decided by (value, index) alone, so threads and warps can be folded in any order:
// one CTA per row, each thread walks its stride of the row, then a shuffle / shared-memory fold.  Integer argmax
// sits beside the hot path (its float form is the configuration's), hence one simple kernel for all widths.
#include <climits>

#include "common.cuh"

namespace bsir {
namespace {

template <class T> struct UnsignedOf;
template <> struct UnsignedOf<int8_t> { using type = uint8_t; };
template <> struct UnsignedOf<int16_t> { using type = uint16_t; };
template <> struct UnsignedOf<int32_t> { using type = uint32_t; };
template <> struct UnsignedOf<int64_t> { using type = uint64_t; };

// a is better than b: strictly better value, or equal value and the index the tie rule prefers
template <class C>
__device__ __forceinline__ bool better(C av, int ai, C bv, int bi, bool is_max, bool left) {
  if (av != bv) return is_max ? av > bv : av < bv;
  return left ? ai < bi : ai > bi;
}

template <class T, bool UNSIGNED>
__global__ void __launch_bounds__(256) rwi_int_kernel(const T *__restrict__ src, int64_t row_stride, int64_t cols, T *__restrict__ dst_val,
                                                      int32_t *__restrict__ dst_idx, int is_max, int left) {
  using C = typename std::conditional<UNSIGNED, typename UnsignedOf<T>::type, T>::type;
  __shared__ C sval[8];
  __shared__ int sidx[8];
  const int64_t row = blockIdx.x;
  const T *x = src + row * row_stride;
  C bv = 0;
  int bi = -1;
  for (int64_t j = threadIdx.x; j < cols; j += 256) {
    const C v = static_cast<C>(x[j]);
    if (bi < 0 || better<C>(v, static_cast<int>(j), bv, bi, is_max, left)) { bv = v; bi = static_cast<int>(j); }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const C ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi >= 0 && (bi < 0 || better<C>(ov, oi, bv, bi, is_max, left))) { bv = ov; bi = oi; }
  }
  if (lane == 0) { sval[warp] = bv; sidx[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sidx[w] >= 0 && (bi < 0 || better<C>(sval[w], sidx[w], bv, bi, is_max, left))) { bv = sval[w]; bi = sidx[w]; }
    // an empty row keeps the identity the reduction starts from and index 0
    if (bi < 0) {
      bi = 0;
      if (UNSIGNED) bv = is_max ? static_cast<C>(0) : static_cast<C>(~static_cast<C>(0));
      else bv = static_cast<C>(is_max ? std::numeric_limits<T>::min() : std::numeric_limits<T>::max());
    }
    dst_val[row] = static_cast<T>(bv);
    dst_idx[row] = bi;
  }
}

template <class T>
void launch(bool uns, const void *src, int64_t rs, int64_t rows, int64_t cols, void *dv, int32_t *di, int is_max, int left, cudaStream_t st) {
  if (uns) rwi_int_kernel<T, true><<<static_cast<unsigned>(rows), 256, 0, st>>>(static_cast<const T *>(src), rs, cols, static_cast<T *>(dv), di, is_max, left);
  else rwi_int_kernel<T, false><<<static_cast<unsigned>(rows), 256, 0, st>>>(static_cast<const T *>(src), rs, cols, static_cast<T *>(dv), di, is_max, left);
}

}  // namespace

int32_t reduce_with_index_int(int32_t kind, int32_t dtype, int32_t tie_break_left, int64_t rows, int64_t cols, const void *src,
                              int64_t src_row_stride, void *dst_value, int32_t *dst_index, cudaStream_t st) {
  const bool uns = kind == BSIR_RWI_MINUI || kind == BSIR_RWI_MAXUI;
  const int is_max = (kind == BSIR_RWI_MAX || kind == BSIR_RWI_MAXUI) ? 1 : 0;
  if (rows < 0 || cols < 0) return fail(BSIR_ERR_SHAPE, "reduce_with_index: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (cols > INT_MAX - 64) return fail(BSIR_ERR_SHAPE, "reduce_with_index: cols exceed the int32 index range");
  if (rows == 0) return BSIR_OK;
  if (!dst_value || !dst_index || (!src && cols > 0)) return fail(BSIR_ERR_NULL, "reduce_with_index: null pointer");
  if (src_row_stride < cols) return fail(BSIR_ERR_STRIDE, "reduce_with_index: row stride < cols");
  const int eb = dtype_bytes(dtype);
  if (!aligned_to(src, eb) || !aligned_to(dst_value, eb) || !aligned_to(dst_index, 4)) return fail(BSIR_ERR_ALIGN, "reduce_with_index: misaligned");
  for (int64_t r0 = 0; r0 < rows; r0 += 0x7fffffffLL) {
    const int64_t nr = rows - r0 < 0x7fffffffLL ? rows - r0 : 0x7fffffffLL;
    const char *s = static_cast<const char *>(src) + r0 * src_row_stride * eb;
    char *dv = static_cast<char *>(dst_value) + r0 * eb;
    switch (dtype) {
      case BSIR_I8: case BSIR_U8: launch<int8_t>(uns || dtype == BSIR_U8, s, src_row_stride, nr, cols, dv, dst_index + r0, is_max, tie_break_left, st); break;
      case BSIR_I16: case BSIR_U16: launch<int16_t>(uns || dtype == BSIR_U16, s, src_row_stride, nr, cols, dv, dst_index + r0, is_max, tie_break_left, st); break;
      case BSIR_I32: case BSIR_U32: launch<int32_t>(uns || dtype == BSIR_U32, s, src_row_stride, nr, cols, dv, dst_index + r0, is_max, tie_break_left, st); break;
      case BSIR_I64: case BSIR_U64: launch<int64_t>(uns || dtype == BSIR_U64, s, src_row_stride, nr, cols, dv, dst_index + r0, is_max, tie_break_left, st); break;
      default: return fail(BSIR_ERR_DTYPE, "reduce_with_index: dtype %d", dtype);
    }
    count_launch();
  }
  return check_launch("reduce_with_index");
}

}  // namespace bsir
