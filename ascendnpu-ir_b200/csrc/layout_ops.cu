// layout_ops.cu -- hivm.hir.varange, vinterleave, vdeinterleave
// (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:1503-1560, 1562-1606, 1612-1660).
//
//   varange:        dst[i0, i1, i2] = offset + i0 * strides[0] + i1 * strides[1] + i2 * strides[2]
//                   (the op's example: offset 1, strides [1, 2], shape 2x4 -> [[1,3,5,7],[2,4,6,8]])
//   vinterleave:    dst[r, N * i + ch] = src_ch[r, i]      (N = interleave_channel_nums sources of one shape)
//   vdeinterleave:  dst_ch[r, i] = src[r, N * i + ch]      (a NULL destination skips its channel: the op's
//                   CHANNEL_0 / CHANNEL_1 index modes)
// All three are pure data movement.
#include <cstdint>
#include <cstring>
#include <type_traits>

#include "common.cuh"

namespace bsir {
namespace {

constexpr int kMaxChannels = 8;
struct ChannelPtrs {
  const void *in[kMaxChannels];
  void *out[kMaxChannels];
};

// 4-byte elements into rows that start on 16-byte boundaries: a thread writes four consecutive values as one vector
template <typename T>
__global__ void __launch_bounds__(256) arange_vec4_kernel(T *dst, int64_t n0, int64_t n1, int64_t n2, int64_t d0, int64_t d1,
                                                          int64_t offset, int64_t s0, int64_t s1, int64_t s2) {
  static_assert(sizeof(T) == 4, "four elements a 16-byte vector");
  for (int64_t row = blockIdx.y; row < n0 * n1; row += gridDim.y) {
    const int64_t i0 = row / n1, i1 = row - i0 * n1;
    const int64_t v0 = offset + i0 * s0 + i1 * s1;
    T *drow = dst + i0 * d0 + i1 * d1;
    for (int64_t q = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; q * 4 < n2; q += static_cast<int64_t>(gridDim.x) * 256) {
      T out[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) out[e] = static_cast<T>(v0 + (q * 4 + e) * s2);
      uint4 w;
      memcpy(&w, out, 16);
      *reinterpret_cast<uint4 *>(drow + q * 4) = w;
    }
  }
}

// a block row of the grid per (i0, i1), threads along i2: one division a row, none an element
template <typename T>
__global__ void __launch_bounds__(256) arange_kernel(T *dst, int64_t n0, int64_t n1, int64_t n2, int64_t d0, int64_t d1, int64_t d2,
                                                     int64_t offset, int64_t s0, int64_t s1, int64_t s2) {
  for (int64_t row = blockIdx.y; row < n0 * n1; row += gridDim.y) {
    const int64_t i0 = row / n1, i1 = row - i0 * n1;
    const int64_t v0 = offset + i0 * s0 + i1 * s1;
    T *drow = dst + i0 * d0 + i1 * d1;
    for (int64_t c = static_cast<int64_t>(blockIdx.x) * 1024 + threadIdx.x; c < n2; c += static_cast<int64_t>(gridDim.x) * 1024) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t i2 = c + u * 256;
        if (i2 < n2) {
          const int64_t v = v0 + i2 * s2;
          T out;
          if constexpr (std::is_same<T, __half>::value) out = __float2half_rn(static_cast<float>(v));
          else out = static_cast<T>(v);
          drow[i2 * d2] = out;
        }
      }
    }
  }
}

// The operands are contiguous, so interleaving the last axis of [rows, cols] is interleaving the flat arrays:
// dst[N * j + ch] = src_ch[j].  Two channels (the op's default) with 16-byte aligned operands move 16-byte vectors
// -- a thread reads one from each source and writes the two vectors they interleave into, or the other way round;
// everything else takes a thread per j that loops over the channels: no division anywhere, reads coalesced per
// channel, writes contiguous across the warp.
template <typename T>
__global__ void __launch_bounds__(256) interleave2_vec_kernel(const uint4 *__restrict__ a, const uint4 *__restrict__ b, uint4 *__restrict__ dst,
                                                              int64_t nvec) {
  constexpr int V = 16 / sizeof(T);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    const uint4 ra = __ldg(a + v), rb = __ldg(b + v);
    T xa[V], xb[V], o[2 * V];
    memcpy(xa, &ra, 16);
    memcpy(xb, &rb, 16);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      o[2 * k] = xa[k];
      o[2 * k + 1] = xb[k];
    }
    uint4 w[2];
    memcpy(w, o, 32);
    dst[2 * v] = w[0];
    dst[2 * v + 1] = w[1];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) deinterleave2_vec_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ a, uint4 *__restrict__ b,
                                                                int64_t nvec) {
  constexpr int V = 16 / sizeof(T);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    uint4 w[2];
    w[0] = __ldg(src + 2 * v);
    w[1] = __ldg(src + 2 * v + 1);
    T o[2 * V], xa[V], xb[V];
    memcpy(o, w, 32);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      xa[k] = o[2 * k];
      xb[k] = o[2 * k + 1];
    }
    uint4 ra, rb;
    memcpy(&ra, xa, 16);
    memcpy(&rb, xb, 16);
    if (a) a[v] = ra;
    if (b) b[v] = rb;
  }
}

// flat j in [first, n): one thread each, every channel in turn
template <typename T, bool INTERLEAVE>
__global__ void __launch_bounds__(256) interleave_kernel(ChannelPtrs p, T *dst, const T *src, int channels, int64_t first, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t j = first + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride) {
    for (int ch = 0; ch < channels; ++ch) {
      if constexpr (INTERLEAVE) {
        dst[j * channels + ch] = static_cast<const T *>(p.in[ch])[j];
      } else {
        T *d = static_cast<T *>(p.out[ch]);
        if (d) d[j] = src[j * channels + ch];
      }
    }
  }
}

template <typename T, bool INTERLEAVE>
void launch_interleave_typed(const ChannelPtrs &p, void *dst, const void *src, int channels, int64_t n, cudaStream_t st) {
  const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
  const int64_t cap = static_cast<int64_t>(sms) * 16;           // blocks: a grid-stride loop beyond that
  int64_t first = 0;
  if (channels == 2) {
    bool vec = aligned_to(INTERLEAVE ? dst : src, 16);
    for (int c = 0; c < 2; ++c) {
      const void *q = INTERLEAVE ? p.in[c] : p.out[c];
      vec = vec && (q == nullptr || aligned_to(q, 16));
    }
    constexpr int V = 16 / sizeof(T);
    const int64_t nvec = n / V;
    if (vec && nvec > 0) {
      const int64_t want = ceil_div(nvec, static_cast<int64_t>(256));
      const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
      if constexpr (INTERLEAVE)
        interleave2_vec_kernel<T><<<blocks, 256, 0, st>>>(static_cast<const uint4 *>(p.in[0]), static_cast<const uint4 *>(p.in[1]),
                                                          static_cast<uint4 *>(dst), nvec);
      else
        deinterleave2_vec_kernel<T><<<blocks, 256, 0, st>>>(static_cast<const uint4 *>(src), static_cast<uint4 *>(p.out[0]),
                                                            static_cast<uint4 *>(p.out[1]), nvec);
      count_launch();
      first = nvec * V;                                        // the few elements past the last whole vector follow
    }
  }
  if (first < n) {
    const int64_t want = ceil_div(n - first, static_cast<int64_t>(256));
    const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
    interleave_kernel<T, INTERLEAVE><<<blocks, 256, 0, st>>>(p, static_cast<T *>(dst), static_cast<const T *>(src), channels, first, n);
    count_launch();
  }
}

template <bool INTERLEAVE>
void launch_interleave(int eb, const ChannelPtrs &p, void *dst, const void *src, int channels, int64_t rows, int64_t cols, cudaStream_t st) {
  const int64_t n = rows * cols;
  switch (eb) {
    case 1: launch_interleave_typed<uint8_t, INTERLEAVE>(p, dst, src, channels, n, st); break;
    case 2: launch_interleave_typed<uint16_t, INTERLEAVE>(p, dst, src, channels, n, st); break;
    case 4: launch_interleave_typed<uint32_t, INTERLEAVE>(p, dst, src, channels, n, st); break;
    default: launch_interleave_typed<uint64_t, INTERLEAVE>(p, dst, src, channels, n, st); break;
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
  int64_t bx = ceil_div(n[2], static_cast<int64_t>(1024)), by = n[0] * n[1];
  if (bx > 4096) bx = 4096;
  if (by > 65535) by = 65535;                    // the kernel loops over what the grid does not cover
  const dim3 blocks(static_cast<unsigned>(bx), static_cast<unsigned>(by));
  if ((dtype == BSIR_I32 || dtype == BSIR_F32) && d[2] == 1 && n[2] % 4 == 0 && aligned_to(dst, 16) && d[1] % 4 == 0 && d[0] % 4 == 0) {
    int64_t vx = ceil_div(n[2] / 4, static_cast<int64_t>(256));
    if (vx > 4096) vx = 4096;
    const dim3 vblocks(static_cast<unsigned>(vx), static_cast<unsigned>(by));
    if (dtype == BSIR_I32) arange_vec4_kernel<int32_t><<<vblocks, 256, 0, st>>>(static_cast<int32_t *>(dst), n[0], n[1], n[2], d[0], d[1], offset, s[0], s[1], s[2]);
    else arange_vec4_kernel<float><<<vblocks, 256, 0, st>>>(static_cast<float *>(dst), n[0], n[1], n[2], d[0], d[1], offset, s[0], s[1], s[2]);
    count_launch();
    return check_launch("arange");
  }
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
  return check_launch("deinterleave");
}
