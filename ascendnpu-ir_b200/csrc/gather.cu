// gather.cu -- hivm.hir.vgather (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:1834-1883):
// dst[o][j][k] = src[o][indices[o][j][k]][k] along one axis of contiguous [outer, axis, inner] tensors
// (source, indices and destination have the same rank; the gather axis of the source may have another length,
// test/Dialect/HIVM/hivm-flatten-ops.mlir:1036-1045).  In general a thread per output element: the index and
// destination streams are coalesced, the source reads go where the indices send them; along the last axis, from
// rows of up to 48 KB, the source row is first brought into shared memory.  An index outside the source axis
// leaves its element untouched and raises BSIR_DEVERR_GATHER_INDEX in the device error word.
#include <cstdint>

#include "common.cuh"

namespace bsir {
namespace {

template <typename T, typename I>
__global__ void __launch_bounds__(256) gather_kernel(const T *__restrict__ src, const I *__restrict__ idx, T *__restrict__ dst,
                                                     int64_t total, int64_t src_axis, int64_t dst_axis, int64_t inner, int *err) {
  const int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const int64_t k = inner == 1 ? 0 : e % inner;
  const int64_t o = e / (dst_axis * inner);
  const int64_t i = static_cast<int64_t>(idx[e]);
  if (i < 0 || i >= src_axis) {
    atomicOr(err, BSIR_DEVERR_GATHER_INDEX);
    return;
  }
  dst[e] = src[(o * src_axis + i) * inner + k];
}

// Gather along the last axis (inner = 1) from rows that fit shared memory: a CTA brings its source row in with
// coalesced loads and the indices then send the reads to shared memory instead of to 32-byte sectors of L2, of
// which a 4-byte element uses an eighth.  A long destination row is shared out over several CTAs (each with its own
// copy of the source row).  Four indices are loaded before the first of them is used.
constexpr int kGatherRowBytes = 48 * 1024;

template <typename T, typename I>
__global__ void __launch_bounds__(256) gather_rows_kernel(const T *__restrict__ src, const I *__restrict__ idx, T *__restrict__ dst,
                                                          int64_t src_axis, int64_t dst_axis, int parts, int64_t part_len, int *err) {
  extern __shared__ __align__(16) unsigned char row_raw[];
  T *row = reinterpret_cast<T *>(row_raw);
  const int tid = threadIdx.x;
  const int64_t o = blockIdx.x / parts;
  const int part = static_cast<int>(blockIdx.x % parts);
  const T *src_row = src + o * src_axis;
  const int n = static_cast<int>(src_axis);
  for (int i = tid; i < n; i += 256 * 4) {
    T v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i + u * 256 < n) v[u] = src_row[i + u * 256];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i + u * 256 < n) row[i + u * 256] = v[u];
  }
  __syncthreads();
  const int64_t j0 = part * part_len, j1 = j0 + part_len < dst_axis ? j0 + part_len : dst_axis;
  const I *idx_row = idx + o * dst_axis;
  T *dst_row = dst + o * dst_axis;
  bool bad = false;
  for (int64_t j = j0 + tid; j < j1; j += 256 * 4) {
    int64_t at[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) at[u] = j + u * 256 < j1 ? static_cast<int64_t>(idx_row[j + u * 256]) : 0;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (j + u * 256 < j1) {
        if (at[u] >= 0 && at[u] < src_axis) dst_row[j + u * 256] = row[at[u]];
        else bad = true;
      }
    }
  }
  if (bad) atomicOr(err, BSIR_DEVERR_GATHER_INDEX);
}

template <typename T, typename I>
bool try_gather_rows(const T *s, const I *idx, T *d, int64_t outer, int64_t src_axis, int64_t dst_axis, int64_t inner, int *err, cudaStream_t st) {
  if (inner != 1 || src_axis * static_cast<int64_t>(sizeof(T)) > kGatherRowBytes || dst_axis < 64) return false;
  const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
  int64_t parts = 1;
  if (outer < 2 * sms) {                                       // few rows: cut the destination rows, 1024 elements a part at least
    parts = ceil_div(static_cast<int64_t>(2 * sms), outer);
    const int64_t most = ceil_div(dst_axis, static_cast<int64_t>(1024));
    if (parts > most) parts = most;
  }
  const int64_t part_len = ceil_div(dst_axis, parts);
  parts = ceil_div(dst_axis, part_len);
  if (outer * parts > 0x7fffffffLL) return false;
  gather_rows_kernel<T, I><<<static_cast<unsigned>(outer * parts), 256, static_cast<size_t>(src_axis) * sizeof(T), st>>>(
      s, idx, d, src_axis, dst_axis, static_cast<int>(parts), part_len, err);
  return true;
}

template <typename T>
void launch_gather(int index_dtype, const void *src, const void *idx, void *dst, int64_t total, int64_t src_axis, int64_t dst_axis,
                   int64_t inner, int *err, cudaStream_t st) {
  const unsigned blocks = static_cast<unsigned>(ceil_div(total, 256));
  const T *s = static_cast<const T *>(src);
  T *d = static_cast<T *>(dst);
  const int64_t outer = total / (dst_axis * inner);
  if (index_dtype == BSIR_I16 ? try_gather_rows(s, static_cast<const int16_t *>(idx), d, outer, src_axis, dst_axis, inner, err, st)
      : index_dtype == BSIR_I32 ? try_gather_rows(s, static_cast<const int32_t *>(idx), d, outer, src_axis, dst_axis, inner, err, st)
                                : try_gather_rows(s, static_cast<const int64_t *>(idx), d, outer, src_axis, dst_axis, inner, err, st))
    return;
  if (index_dtype == BSIR_I16) gather_kernel<T, int16_t><<<blocks, 256, 0, st>>>(s, static_cast<const int16_t *>(idx), d, total, src_axis, dst_axis, inner, err);
  else if (index_dtype == BSIR_I32) gather_kernel<T, int32_t><<<blocks, 256, 0, st>>>(s, static_cast<const int32_t *>(idx), d, total, src_axis, dst_axis, inner, err);
  else gather_kernel<T, int64_t><<<blocks, 256, 0, st>>>(s, static_cast<const int64_t *>(idx), d, total, src_axis, dst_axis, inner, err);
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" int32_t bsir_gather(int32_t dtype, int32_t index_dtype, int64_t outer, int64_t src_axis, int64_t dst_axis, int64_t inner,
                               const void *src, const void *indices, void *dst, void *stream) {
  clear_error();
  const int eb = dtype_bytes(dtype);
  if (eb == 0) return fail(BSIR_ERR_DTYPE, "gather: dtype %d", dtype);
  if (index_dtype != BSIR_I16 && index_dtype != BSIR_I32 && index_dtype != BSIR_I64)
    return fail(BSIR_ERR_DTYPE, "gather: index dtype %d (i16, i32, i64)", index_dtype);
  if (outer < 0 || src_axis < 0 || dst_axis < 0 || inner < 0)
    return fail(BSIR_ERR_SHAPE, "gather: [%lld, %lld -> %lld, %lld]", (long long)outer, (long long)src_axis, (long long)dst_axis, (long long)inner);
  const int64_t total = outer * dst_axis * inner;
  if (total == 0) return BSIR_OK;
  if (!src || !indices || !dst) return fail(BSIR_ERR_NULL, "gather: null pointer");
  if (src_axis == 0) return fail(BSIR_ERR_SHAPE, "gather: the source axis is empty");
  if (!aligned_to(src, eb) || !aligned_to(dst, eb) || !aligned_to(indices, dtype_bytes(index_dtype))) return fail(BSIR_ERR_ALIGN, "gather: misaligned");
  if (ceil_div(total, 256) > 0x7fffffffLL) return fail(BSIR_ERR_SHAPE, "gather: %lld elements", (long long)total);
  {   // an element is read where an index sends the read: nothing may have been written there before
    const char *s0 = static_cast<const char *>(src), *s1 = s0 + outer * src_axis * inner * eb;
    const char *d0 = static_cast<const char *>(dst), *d1 = d0 + total * eb;
    if (s0 < d1 && d0 < s1) return fail(BSIR_ERR_UNSUPPORTED, "gather: the destination may not overlap the source");
  }
  int *err = device_error_word();
  if (!err) return fail(BSIR_ERR_WORKSPACE, "gather: no device error word");
  cudaStream_t st = resolve_stream(stream);
  switch (eb) {
    case 1: launch_gather<uint8_t>(index_dtype, src, indices, dst, total, src_axis, dst_axis, inner, err, st); break;
    case 2: launch_gather<uint16_t>(index_dtype, src, indices, dst, total, src_axis, dst_axis, inner, err, st); break;
    case 4: launch_gather<uint32_t>(index_dtype, src, indices, dst, total, src_axis, dst_axis, inner, err, st); break;
    default: launch_gather<uint64_t>(index_dtype, src, indices, dst, total, src_axis, dst_axis, inner, err, st); break;
  }
  count_launch();
  return check_launch("gather");
}
