// layout_ops.cu -- hivm.hir.varange, vinterleave, vdeinterleave
// (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:1503-1560, 1562-1606, 1612-1660).
//
//   varange:        dst[i0, i1, i2] = offset + i0 * strides[0] + i1 * strides[1] + i2 * strides[2]
//                   (the op's example: offset 1, strides [1, 2], shape 2x4 -> [[1,3,5,7],[2,4,6,8]])
//   vinterleave:    dst[r, N * i + ch] = src_ch[r, i]      (N = interleave_channel_nums sources of one shape)
//   vdeinterleave:  dst_ch[r, i] = src[r, N * i + ch]      (a NULL destination skips its channel: the op's
//                   CHANNEL_0 / CHANNEL_1 index modes)
// All three are pure data movement: a thread writes one 16-byte vector of the contiguous side (or one
// element when the row is not a whole number of vectors) and reads what it needs with scalar loads, which
// the neighbouring threads' loads complete into full sectors.
#include <cstdint>
#include <type_traits>

#include "common.cuh"

namespace bsir {
namespace {

constexpr int kMaxChannels = 8;
struct ChannelPtrs {
  const void *in[kMaxChannels];
  void *out[kMaxChannels];
};

template <typename T>
__global__ void __launch_bounds__(256) arange_kernel(T *dst, int64_t n0, int64_t n1, int64_t n2, int64_t d0, int64_t d1, int64_t d2,
                                                     int64_t offset, int64_t s0, int64_t s1, int64_t s2) {
  const int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= n0 * n1 * n2) return;
  const int64_t i2 = e % n2, i1 = (e / n2) % n1, i0 = e / (n2 * n1);
  const int64_t v = offset + i0 * s0 + i1 * s1 + i2 * s2;
  T out;
  if constexpr (std::is_same<T, __half>::value) out = __float2half_rn(static_cast<float>(v));
  else out = static_cast<T>(v);
  dst[i0 * d0 + i1 * d1 + i2 * d2] = out;
}

// one thread per element of the interleaved side; consecutive threads -> consecutive interleaved columns
template <typename T, bool INTERLEAVE>
__global__ void __launch_bounds__(256) interleave_kernel(ChannelPtrs p, T *dst, const T *src, int channels, int64_t rows, int64_t cols) {
  const int64_t wide = cols * channels;
  const int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= rows * wide) return;
  const int64_t r = e / wide, c = e - r * wide;
  const int ch = static_cast<int>(c % channels);
  const int64_t i = c / channels;
  if constexpr (INTERLEAVE) {
    dst[e] = static_cast<const T *>(p.in[ch])[r * cols + i];
  } else {
    T *d = static_cast<T *>(p.out[ch]);
    if (d) d[r * cols + i] = src[e];
  }
}

template <bool INTERLEAVE>
void launch_interleave(int eb, const ChannelPtrs &p, void *dst, const void *src, int channels, int64_t rows, int64_t cols, cudaStream_t st) {
  const unsigned blocks = static_cast<unsigned>(ceil_div(rows * cols * channels, 256));
  switch (eb) {
    case 1: interleave_kernel<uint8_t, INTERLEAVE><<<blocks, 256, 0, st>>>(p, static_cast<uint8_t *>(dst), static_cast<const uint8_t *>(src), channels, rows, cols); break;
    case 2: interleave_kernel<uint16_t, INTERLEAVE><<<blocks, 256, 0, st>>>(p, static_cast<uint16_t *>(dst), static_cast<const uint16_t *>(src), channels, rows, cols); break;
    case 4: interleave_kernel<uint32_t, INTERLEAVE><<<blocks, 256, 0, st>>>(p, static_cast<uint32_t *>(dst), static_cast<const uint32_t *>(src), channels, rows, cols); break;
    default: interleave_kernel<uint64_t, INTERLEAVE><<<blocks, 256, 0, st>>>(p, static_cast<uint64_t *>(dst), static_cast<const uint64_t *>(src), channels, rows, cols); break;
  }
}

int32_t check_channels(const char *what, int32_t dtype, int32_t channels, int64_t rows, int64_t cols) {
  if (dtype_bytes(dtype) == 0) return fail(BSIR_ERR_DTYPE, "%s: dtype %d", what, dtype);
  if (channels < 1 || channels > kMaxChannels) return fail(BSIR_ERR_ATTR, "%s: %d channels (1..%d)", what, channels, kMaxChannels);
  if (rows < 0 || cols < 0) return fail(BSIR_ERR_SHAPE, "%s: rows=%lld cols=%lld", what, (long long)rows, (long long)cols);
  if (ceil_div(rows * cols * channels, 256) > 0x7fffffffLL) return fail(BSIR_ERR_SHAPE, "%s: too many elements", what);
  return BSIR_OK;
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" int32_t bsir_arange(int32_t dtype, int32_t rank, const int64_t *sizes, int64_t offset, const int64_t *strides, void *dst,
                               const int64_t *dst_strides, void *stream) {
  clear_error();
  if (rank < 1 || rank > 3) return fail(BSIR_ERR_SHAPE, "arange: rank %d (1..3)", rank);
  if (!sizes || !strides) return fail(BSIR_ERR_NULL, "arange: sizes / strides is null");
  if (dtype != BSIR_I16 && dtype != BSIR_I32 && dtype != BSIR_I64 && dtype != BSIR_F16 && dtype != BSIR_F32)
    return fail(BSIR_ERR_DTYPE, "arange: dtype %d (i16, i32, i64, f16, f32)", dtype);
  int64_t n[3] = {1, 1, 1}, s[3] = {0, 0, 0}, d[3] = {0, 0, 0};
  int64_t cs = 1;
  for (int i = rank - 1; i >= 0; --i) {
    if (sizes[i] < 0) return fail(BSIR_ERR_SHAPE, "arange: sizes[%d] = %lld", i, (long long)sizes[i]);
    n[3 - rank + i] = sizes[i];
    s[3 - rank + i] = strides[i];
    d[3 - rank + i] = dst_strides ? dst_strides[i] : cs;
    cs *= sizes[i];
  }
  const int64_t total = n[0] * n[1] * n[2];
  if (total == 0) return BSIR_OK;
  if (!dst) return fail(BSIR_ERR_NULL, "arange: dst is null");
  if (!aligned_to(dst, dtype_bytes(dtype))) return fail(BSIR_ERR_ALIGN, "arange: misaligned");
  if (ceil_div(total, 256) > 0x7fffffffLL) return fail(BSIR_ERR_SHAPE, "arange: too many elements");
  cudaStream_t st = resolve_stream(stream);
  const unsigned blocks = static_cast<unsigned>(ceil_div(total, 256));
  switch (dtype) {
    case BSIR_I16: arange_kernel<int16_t><<<blocks, 256, 0, st>>>(static_cast<int16_t *>(dst), n[0], n[1], n[2], d[0], d[1], d[2], offset, s[0], s[1], s[2]); break;
    case BSIR_I32: arange_kernel<int32_t><<<blocks, 256, 0, st>>>(static_cast<int32_t *>(dst), n[0], n[1], n[2], d[0], d[1], d[2], offset, s[0], s[1], s[2]); break;
    case BSIR_I64: arange_kernel<int64_t><<<blocks, 256, 0, st>>>(static_cast<int64_t *>(dst), n[0], n[1], n[2], d[0], d[1], d[2], offset, s[0], s[1], s[2]); break;
    case BSIR_F16: arange_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<__half *>(dst), n[0], n[1], n[2], d[0], d[1], d[2], offset, s[0], s[1], s[2]); break;
    default: arange_kernel<float><<<blocks, 256, 0, st>>>(static_cast<float *>(dst), n[0], n[1], n[2], d[0], d[1], d[2], offset, s[0], s[1], s[2]); break;
  }
  count_launch();
  return check_launch("arange");
}

extern "C" int32_t bsir_interleave(int32_t dtype, int32_t channels, int64_t rows, int64_t cols, const void *const *srcs, void *dst,
                                   void *stream) {
  clear_error();
  if (const int32_t rc = check_channels("interleave", dtype, channels, rows, cols)) return rc;
  if (rows * cols == 0) return BSIR_OK;
  if (!srcs || !dst) return fail(BSIR_ERR_NULL, "interleave: null pointer");
  ChannelPtrs p{};
  const int eb = dtype_bytes(dtype);
  for (int c = 0; c < channels; ++c) {
    if (!srcs[c]) return fail(BSIR_ERR_NULL, "interleave: source %d is null", c);
    if (!aligned_to(srcs[c], eb)) return fail(BSIR_ERR_ALIGN, "interleave: source %d misaligned", c);
    p.in[c] = srcs[c];
  }
  if (!aligned_to(dst, eb)) return fail(BSIR_ERR_ALIGN, "interleave: dst misaligned");
  launch_interleave<true>(eb, p, dst, nullptr, channels, rows, cols, resolve_stream(stream));
  count_launch();
  return check_launch("interleave");
}

extern "C" int32_t bsir_deinterleave(int32_t dtype, int32_t channels, int64_t rows, int64_t cols, const void *src, void *const *dsts,
                                     void *stream) {
  clear_error();
  if (const int32_t rc = check_channels("deinterleave", dtype, channels, rows, cols)) return rc;
  if (rows * cols == 0) return BSIR_OK;
  if (!src || !dsts) return fail(BSIR_ERR_NULL, "deinterleave: null pointer");
  ChannelPtrs p{};
  const int eb = dtype_bytes(dtype);
  bool any = false;
  for (int c = 0; c < channels; ++c) {
    if (dsts[c] && !aligned_to(dsts[c], eb)) return fail(BSIR_ERR_ALIGN, "deinterleave: destination %d misaligned", c);
    p.out[c] = dsts[c];
    any = any || dsts[c];
  }
  if (!any) return fail(BSIR_ERR_NULL, "deinterleave: every destination is null");
  if (!aligned_to(src, eb)) return fail(BSIR_ERR_ALIGN, "deinterleave: src misaligned");
  launch_interleave<false>(eb, p, nullptr, src, channels, rows, cols, resolve_stream(stream));
  count_launch();
  return check_launch("deinterleave");
}
