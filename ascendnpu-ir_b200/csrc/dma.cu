// dma.cu -- hivm.hir.load with last-dimension padding and hivm.hir.store with an atomic kind
// (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMDMAOps.td:62-215).
//
// load.  dst[..., 0:left] = pad, dst[..., left:left+n] = src[..., 0:n], dst[..., left+n:left+n+right] = pad,
// where n is the source's last extent and pad is the given value (PadValue) or the row's first source
// element (PadFirstElem).  The paddings that are not given are deduced from the destination's last
// extent exactly as the CPU lowering does (bishengir/lib/ExecutionEngine/ConvertHIVMToUpstream.cpp:1140-1166):
// without a right padding everything after the data is padding; with a right padding but no left one
// the left padding takes the difference.  Destination elements beyond left + n + right are not written.
//
// store.  Without an atomic kind a copy (the CPU lowering copies whatever the kind:
// ConvertHIVMToUpstream.cpp:1715).  With add / max / min (the kinds the op allows, HIVMDMAOps.td:176) and the
// bitwise and unsigned kinds of the enum (HIVMAttrs.td:792-803) the destination is combined with the
// source by device-wide atomics, so stores of several streams or GPUs' kernels into one buffer add up.
//
// Row views with unit element stride and 16-byte aligned destination rows move as 16-byte vectors (a padded load
// builds each destination vector from the data, the padding, or both; an adding store of f32 / f16 / bf16 is one
// vector reduction per 16 bytes); everything else takes an element per thread.
#include <cstdint>
#include <cstring>
#include <type_traits>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace bsir {
namespace {

struct DmaShape {
  int64_t d0, d1, n;          // leading extents (collapsed to two) and the source's last extent
  int64_t ss0, ss1, ss2;      // source strides (elements)
  int64_t ds0, ds1, ds2;      // destination strides (elements)
};

// Fills the collapsed rank-3 view; `sizes` are the source's extents.
bool make_shape(int32_t rank, const int64_t *sizes, const int64_t *src_strides, const int64_t *dst_strides,
                int64_t dst_last, DmaShape *s) {
  if (rank < 1 || rank > 3 || !sizes) return false;
  int64_t sz[3] = {1, 1, 1}, ss[3] = {0, 0, 1}, ds[3] = {0, 0, 1};
  int64_t cs = 1, cd = 1;
  for (int i = rank - 1; i >= 0; --i) {
    const int j = 3 - rank + i;
    if (sizes[i] < 0) return false;
    sz[j] = sizes[i];
    ss[j] = src_strides ? src_strides[i] : cs;
    ds[j] = dst_strides ? dst_strides[i] : cd;
    cs *= sizes[i];
    cd *= (i == rank - 1) ? dst_last : sizes[i];
  }
  s->d0 = sz[0]; s->d1 = sz[1]; s->n = sz[2];
  s->ss0 = ss[0]; s->ss1 = ss[1]; s->ss2 = ss[2];
  s->ds0 = ds[0]; s->ds1 = ds[1]; s->ds2 = ds[2];
  return true;
}

template <typename T>
__global__ void __launch_bounds__(256) load_pad_kernel(DmaShape s, const T *__restrict__ src, T *__restrict__ dst,
                                                        int64_t left, int64_t right, int first_elem, T pad) {
  for (int64_t row = blockIdx.y; row < s.d0 * s.d1; row += gridDim.y) {
  const int64_t i0 = row / s.d1, i1 = row % s.d1;
  const T *srow = src + i0 * s.ss0 + i1 * s.ss1;
  T *drow = dst + i0 * s.ds0 + i1 * s.ds1;
  const int64_t width = left + s.n + right;
  const T fill = (first_elem && s.n > 0) ? srow[0] : pad;
  for (int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < width;
       c += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t k = c - left;
    drow[c * s.ds2] = (k >= 0 && k < s.n) ? srow[k * s.ss2] : fill;
  }
  }
}

// ---- atomic combine, one thread per element
__device__ __forceinline__ void atomic_max_f32(float *p, float v) {
  // NaN-propagating maximum by compare-and-swap (atomicMax has no float form)
  unsigned *u = reinterpret_cast<unsigned *>(p);
  unsigned old = *u;
  while (true) {
    const float cur = __uint_as_float(old);
    const float want = maximumf(cur, v);
    if (__float_as_uint(want) == old) return;
    const unsigned seen = atomicCAS(u, old, __float_as_uint(want));
    if (seen == old) return;
    old = seen;
  }
}
__device__ __forceinline__ void atomic_min_f32(float *p, float v) {
  unsigned *u = reinterpret_cast<unsigned *>(p);
  unsigned old = *u;
  while (true) {
    const float cur = __uint_as_float(old);
    const float want = minimumf(cur, v);
    if (__float_as_uint(want) == old) return;
    const unsigned seen = atomicCAS(u, old, __float_as_uint(want));
    if (seen == old) return;
    old = seen;
  }
}

template <typename T, int KIND>
__device__ __forceinline__ void combine(T *p, T v) {
  if constexpr (std::is_same<T, float>::value) {
    if constexpr (KIND == BSIR_ATOMIC_ADD) atomicAdd(p, v);
    else if constexpr (KIND == BSIR_ATOMIC_MAX) atomic_max_f32(p, v);
    else atomic_min_f32(p, v);
  } else if constexpr (std::is_same<T, __half>::value || std::is_same<T, __nv_bfloat16>::value) {
    atomicAdd(p, v);
  } else if constexpr (std::is_same<T, int32_t>::value) {
    if constexpr (KIND == BSIR_ATOMIC_ADD) atomicAdd(p, v);
    else if constexpr (KIND == BSIR_ATOMIC_MAX) atomicMax(p, v);
    else if constexpr (KIND == BSIR_ATOMIC_MIN) atomicMin(p, v);
    else if constexpr (KIND == BSIR_ATOMIC_AND) atomicAnd(p, v);
    else if constexpr (KIND == BSIR_ATOMIC_OR) atomicOr(p, v);
    else if constexpr (KIND == BSIR_ATOMIC_XOR) atomicXor(p, v);
    else if constexpr (KIND == BSIR_ATOMIC_UMAX) atomicMax(reinterpret_cast<unsigned *>(p), static_cast<unsigned>(v));
    else atomicMin(reinterpret_cast<unsigned *>(p), static_cast<unsigned>(v));
  } else {  // 64-bit integers
    using U = unsigned long long;
    using S = long long;
    if constexpr (KIND == BSIR_ATOMIC_ADD) atomicAdd(reinterpret_cast<U *>(p), static_cast<U>(v));
    else if constexpr (KIND == BSIR_ATOMIC_MAX) atomicMax(reinterpret_cast<S *>(p), static_cast<S>(v));
    else if constexpr (KIND == BSIR_ATOMIC_MIN) atomicMin(reinterpret_cast<S *>(p), static_cast<S>(v));
    else if constexpr (KIND == BSIR_ATOMIC_AND) atomicAnd(reinterpret_cast<U *>(p), static_cast<U>(v));
    else if constexpr (KIND == BSIR_ATOMIC_OR) atomicOr(reinterpret_cast<U *>(p), static_cast<U>(v));
    else if constexpr (KIND == BSIR_ATOMIC_XOR) atomicXor(reinterpret_cast<U *>(p), static_cast<U>(v));
    else if constexpr (KIND == BSIR_ATOMIC_UMAX) atomicMax(reinterpret_cast<U *>(p), static_cast<U>(v));
    else atomicMin(reinterpret_cast<U *>(p), static_cast<U>(v));
  }
}

template <typename T, int KIND>
__global__ void __launch_bounds__(256) store_atomic_kernel(DmaShape s, const T *__restrict__ src, T *dst) {
  for (int64_t row = blockIdx.y; row < s.d0 * s.d1; row += gridDim.y) {
  const int64_t i0 = row / s.d1, i1 = row % s.d1;
  const T *srow = src + i0 * s.ss0 + i1 * s.ss1;
  T *drow = dst + i0 * s.ds0 + i1 * s.ds1;
  for (int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < s.n;
       c += static_cast<int64_t>(gridDim.x) * blockDim.x)
    combine<T, KIND>(drow + c * s.ds2, srow[c * s.ss2]);
  }
}

// ---- 16-byte-vector forms.  Both sides are [rows, n] views with unit element stride and one row stride each, the
// destination's rows on 16-byte boundaries.  A thread takes four destination vectors of the flattened
// [rows x vectors per row] space; every source load is issued before the first store.
struct DmaRows {
  int64_t rows, n;            // n: the source's last extent
  int64_t src_rs, dst_rs;     // row strides (elements)
};
bool as_rows(const DmaShape &s, const void *dst, int eb, DmaRows *r) {
  if (s.ss2 != 1 || s.ds2 != 1) return false;
  const bool one = s.d0 == 1 || s.d1 == 1;
  if (!one && (s.ss0 != s.d1 * s.ss1 || s.ds0 != s.d1 * s.ds1)) return false;      // the two leading axes must collapse
  r->rows = s.d0 * s.d1;
  r->n = s.n;
  r->src_rs = s.d1 == 1 ? s.ss0 : s.ss1;
  r->dst_rs = s.d1 == 1 ? s.ds0 : s.ds1;
  if (r->rows == 1) { r->src_rs = 0; r->dst_rs = 0; }
  return aligned_to(dst, 16) && (r->dst_rs * eb) % 16 == 0;
}

constexpr int kDmaThreads = 256;
constexpr int kDmaUnroll = 4;

template <typename T, bool SRC_VEC>
__global__ void __launch_bounds__(kDmaThreads) load_pad_vec_kernel(DmaRows g, const T *__restrict__ src, T *__restrict__ dst, int64_t left,
                                                                    int64_t width, int first_elem, T pad) {
  constexpr int V = 16 / sizeof(T);
  const int64_t vpr = (width + V - 1) / V;          // destination vectors a row; the last may be partial
  const int64_t total = g.rows * vpr;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (kDmaThreads * kDmaUnroll) + threadIdx.x;
  T x[kDmaUnroll][V];
  T fill[kDmaUnroll];
  int64_t row[kDmaUnroll], c0[kDmaUnroll];
#pragma unroll
  for (int u = 0; u < kDmaUnroll; ++u) {
    const int64_t v = base + static_cast<int64_t>(u) * kDmaThreads;
    row[u] = -1;
    if (v < total) {
      row[u] = total <= 0x7fffffff ? static_cast<int64_t>(static_cast<uint32_t>(v) / static_cast<uint32_t>(vpr)) : v / vpr;
      c0[u] = (v - row[u] * vpr) * V;
      const T *srow = src + row[u] * g.src_rs;
      const int64_t k0 = c0[u] - left;              // source column of the vector's first element
      fill[u] = (first_elem && g.n > 0) ? srow[0] : pad;
      if (SRC_VEC && k0 >= 0 && k0 + V <= g.n) {    // inside the data, and the data's vectors line up with the destination's
        const uint4 q = *reinterpret_cast<const uint4 *>(srow + k0);
        memcpy(x[u], &q, 16);
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const int64_t k = k0 + e;
          x[u][e] = (k >= 0 && k < g.n) ? srow[k] : fill[u];
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kDmaUnroll; ++u) {
    if (row[u] < 0) continue;
    T *d = dst + row[u] * g.dst_rs + c0[u];
    if (c0[u] + V <= width) {
      uint4 q;
      memcpy(&q, x[u], 16);
      *reinterpret_cast<uint4 *>(d) = q;
    } else {                                         // the row's last, partial vector: nothing beyond `width` is written
      for (int e = 0; e < V && c0[u] + e < width; ++e) d[e] = x[u][e];
    }
  }
}

// out += x with one reduction of 16 bytes a vector (f32: four adds, f16 / bf16: eight, each rounded as the scalar
// atomic rounds it)
template <typename T>
__device__ __forceinline__ void red_add_vec(T *p, uint4 q) {
  if constexpr (std::is_same<T, float>::value)
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(__uint_as_float(q.x)), "f"(__uint_as_float(q.y)),
                 "f"(__uint_as_float(q.z)), "f"(__uint_as_float(q.w))
                 : "memory");
  else if constexpr (std::is_same<T, __half>::value)
    asm volatile("red.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(q.x), "r"(q.y), "r"(q.z), "r"(q.w) : "memory");
  else
    asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(q.x), "r"(q.y), "r"(q.z), "r"(q.w) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kDmaThreads) store_add_vec_kernel(DmaRows g, const T *__restrict__ src, T *dst) {
  constexpr int V = 16 / sizeof(T);
  const int64_t vpr = g.n / V;
  const int64_t total = g.rows * vpr;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (kDmaThreads * kDmaUnroll) + threadIdx.x;
  uint4 q[kDmaUnroll];
  int64_t off[kDmaUnroll];
#pragma unroll
  for (int u = 0; u < kDmaUnroll; ++u) {
    const int64_t v = base + static_cast<int64_t>(u) * kDmaThreads;
    off[u] = -1;
    if (v < total) {
      const int64_t row = total <= 0x7fffffff ? static_cast<int64_t>(static_cast<uint32_t>(v) / static_cast<uint32_t>(vpr)) : v / vpr;
      const int64_t c = (v - row * vpr) * V;
      off[u] = row * g.dst_rs + c;
      q[u] = *reinterpret_cast<const uint4 *>(src + row * g.src_rs + c);
    }
  }
#pragma unroll
  for (int u = 0; u < kDmaUnroll; ++u)
    if (off[u] >= 0) red_add_vec<T>(dst + off[u], q[u]);
}

dim3 dma_grid(int64_t width, int64_t rows) {
  int64_t bx = ceil_div(width, 256);
  if (bx > 1024) bx = 1024;
  if (bx < 1) bx = 1;
  return dim3(static_cast<unsigned>(bx), static_cast<unsigned>(rows < 65535 ? rows : 65535));   // kernels loop over further rows
}

template <typename T>
int32_t launch_load(const DmaShape &s, const void *src, void *dst, int64_t left, int64_t right, int first_elem,
                    const void *pad_value, cudaStream_t st) {
  T pad{};
  if (pad_value) memcpy(&pad, pad_value, sizeof(T));
  DmaRows g;
  constexpr int V = 16 / sizeof(T);
  const int64_t width = left + s.n + right;
  if (as_rows(s, dst, sizeof(T), &g) && width >= V) {
    const int64_t total = g.rows * ceil_div(width, static_cast<int64_t>(V));
    const int64_t blocks = ceil_div(total, static_cast<int64_t>(kDmaThreads) * kDmaUnroll);
    if (blocks <= 0x7fffffffLL) {
      // the data's 16-byte vectors line up with the destination's when the left padding is whole vectors and the
      // source rows start on 16-byte boundaries
      const bool src_vec = left % V == 0 && aligned_to(src, 16) && (g.src_rs * sizeof(T)) % 16 == 0;
      if (src_vec) load_pad_vec_kernel<T, true><<<static_cast<unsigned>(blocks), kDmaThreads, 0, st>>>(g, static_cast<const T *>(src), static_cast<T *>(dst), left, width, first_elem, pad);
      else load_pad_vec_kernel<T, false><<<static_cast<unsigned>(blocks), kDmaThreads, 0, st>>>(g, static_cast<const T *>(src), static_cast<T *>(dst), left, width, first_elem, pad);
      count_launch();
      return check_launch("load");
    }
  }
  load_pad_kernel<T><<<dma_grid(left + s.n + right, s.d0 * s.d1), 256, 0, st>>>(s, static_cast<const T *>(src), static_cast<T *>(dst), left, right,
                                                                             first_elem, pad);
  count_launch();
  return check_launch("load");
}

template <typename T, int KIND>
int32_t launch_store(const DmaShape &s, const void *src, void *dst, cudaStream_t st) {
  if constexpr (KIND == BSIR_ATOMIC_ADD && (std::is_same<T, float>::value || std::is_same<T, __half>::value || std::is_same<T, __nv_bfloat16>::value)) {
    DmaRows g;
    constexpr int V = 16 / sizeof(T);
    if (as_rows(s, dst, sizeof(T), &g) && s.n % V == 0 && aligned_to(src, 16) && (g.src_rs * sizeof(T)) % 16 == 0) {
      const int64_t blocks = ceil_div(g.rows * (s.n / V), static_cast<int64_t>(kDmaThreads) * kDmaUnroll);
      if (blocks <= 0x7fffffffLL) {
        store_add_vec_kernel<T><<<static_cast<unsigned>(blocks), kDmaThreads, 0, st>>>(g, static_cast<const T *>(src), static_cast<T *>(dst));
        count_launch();
        return check_launch("store");
      }
    }
  }
  store_atomic_kernel<T, KIND><<<dma_grid(s.n, s.d0 * s.d1), 256, 0, st>>>(s, static_cast<const T *>(src), static_cast<T *>(dst));
  count_launch();
  return check_launch("store");
}

template <typename T>
int32_t store_int_kinds(int32_t kind, const DmaShape &s, const void *src, void *dst, cudaStream_t st) {
  switch (kind) {
    case BSIR_ATOMIC_ADD: return launch_store<T, BSIR_ATOMIC_ADD>(s, src, dst, st);
    case BSIR_ATOMIC_MAX: return launch_store<T, BSIR_ATOMIC_MAX>(s, src, dst, st);
    case BSIR_ATOMIC_MIN: return launch_store<T, BSIR_ATOMIC_MIN>(s, src, dst, st);
    case BSIR_ATOMIC_AND: return launch_store<T, BSIR_ATOMIC_AND>(s, src, dst, st);
    case BSIR_ATOMIC_OR: return launch_store<T, BSIR_ATOMIC_OR>(s, src, dst, st);
    case BSIR_ATOMIC_XOR: return launch_store<T, BSIR_ATOMIC_XOR>(s, src, dst, st);
    case BSIR_ATOMIC_UMAX: return launch_store<T, BSIR_ATOMIC_UMAX>(s, src, dst, st);
    case BSIR_ATOMIC_UMIN: return launch_store<T, BSIR_ATOMIC_UMIN>(s, src, dst, st);
    default: return fail(BSIR_ERR_UNSUPPORTED, "store: atomic kind %d", kind);
  }
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" {

int32_t bsir_load(int32_t dtype, int32_t rank, const int64_t *src_sizes, const void *src, const int64_t *src_strides,
                  void *dst, const int64_t *dst_strides, int64_t dst_last, int32_t pad_mode, const void *pad_value,
                  int64_t left_pad, int64_t right_pad, void *stream) {
  clear_error();
  const int eb = dtype_bytes(dtype);
  if (eb == 0) return fail(BSIR_ERR_DTYPE, "load: dtype %d", dtype);
  if (pad_mode < BSIR_PAD_NULL || pad_mode > BSIR_PAD_VALUE) return fail(BSIR_ERR_ATTR, "load: pad_mode %d", pad_mode);
  DmaShape s;
  if (!make_shape(rank, src_sizes, src_strides, dst_strides, dst_last, &s))
    return fail(BSIR_ERR_SHAPE, "load: rank %d (1..3) or negative extent", rank);
  if (pad_mode == BSIR_PAD_NULL) {
    if (dst_last != s.n) return fail(BSIR_ERR_SHAPE, "load: without pad_mode the shapes must match (%lld vs %lld)",
                                     (long long)dst_last, (long long)s.n);
    return bsir_copy(dtype, rank, src_sizes, src, src_strides, dst, dst_strides, stream);
  }
  if (pad_mode == BSIR_PAD_VALUE && !pad_value) return fail(BSIR_ERR_NULL, "load: pad_value is null");
  // paddings that are not given (< 0) take what the destination leaves over
  int64_t left = left_pad, right = right_pad;
  if (right < 0) {
    if (left < 0) left = 0;
    right = dst_last - (s.n + left);
  } else if (left < 0) {
    left = dst_last - (s.n + right);
  }
  if (left < 0 || right < 0 || left + s.n + right > dst_last)
    return fail(BSIR_ERR_SHAPE, "load: paddings %lld + %lld and %lld elements do not fit the destination's %lld",
                (long long)left, (long long)right, (long long)s.n, (long long)dst_last);
  if (s.d0 * s.d1 == 0 || left + s.n + right == 0) return BSIR_OK;
  if (!src || !dst) return fail(BSIR_ERR_NULL, "load: null pointer");
  if (!aligned_to(src, eb) || !aligned_to(dst, eb)) return fail(BSIR_ERR_ALIGN, "load: misaligned");
  cudaStream_t st = resolve_stream(stream);
  const int first = pad_mode == BSIR_PAD_FIRST_ELEM;
  switch (eb) {
    case 1: return launch_load<uint8_t>(s, src, dst, left, right, first, pad_value, st);
    case 2: return launch_load<uint16_t>(s, src, dst, left, right, first, pad_value, st);
    case 4: return launch_load<uint32_t>(s, src, dst, left, right, first, pad_value, st);
    default: return launch_load<uint64_t>(s, src, dst, left, right, first, pad_value, st);
  }
}

int32_t bsir_store(int32_t dtype, int32_t rank, const int64_t *sizes, const void *src, const int64_t *src_strides,
                   void *dst, const int64_t *dst_strides, int32_t atomic_kind, void *stream) {
  if (atomic_kind == BSIR_ATOMIC_NONE) return bsir_copy(dtype, rank, sizes, src, src_strides, dst, dst_strides, stream);
  clear_error();
  const int eb = dtype_bytes(dtype);
  if (eb == 0) return fail(BSIR_ERR_DTYPE, "store: dtype %d", dtype);
  if (atomic_kind == BSIR_ATOMIC_CAS || atomic_kind == BSIR_ATOMIC_XCHG || atomic_kind < 0 || atomic_kind > BSIR_ATOMIC_UMIN)
    return fail(BSIR_ERR_UNSUPPORTED, "store: atomic kind %d is not a combining store", atomic_kind);
  DmaShape s;
  if (!make_shape(rank, sizes, src_strides, dst_strides, sizes ? sizes[rank > 0 ? rank - 1 : 0] : 0, &s))
    return fail(BSIR_ERR_SHAPE, "store: rank %d (1..3) or negative extent", rank);
  if (s.d0 * s.d1 * s.n == 0) return BSIR_OK;
  if (!src || !dst) return fail(BSIR_ERR_NULL, "store: null pointer");
  if (!aligned_to(src, eb) || !aligned_to(dst, eb)) return fail(BSIR_ERR_ALIGN, "store: misaligned");
  cudaStream_t st = resolve_stream(stream);
  switch (dtype) {
    case BSIR_F32:
      if (atomic_kind == BSIR_ATOMIC_ADD) return launch_store<float, BSIR_ATOMIC_ADD>(s, src, dst, st);
      if (atomic_kind == BSIR_ATOMIC_MAX) return launch_store<float, BSIR_ATOMIC_MAX>(s, src, dst, st);
      if (atomic_kind == BSIR_ATOMIC_MIN) return launch_store<float, BSIR_ATOMIC_MIN>(s, src, dst, st);
      break;
    case BSIR_F16:
      if (atomic_kind == BSIR_ATOMIC_ADD) return launch_store<__half, BSIR_ATOMIC_ADD>(s, src, dst, st);
      break;
    case BSIR_BF16:
      if (atomic_kind == BSIR_ATOMIC_ADD) return launch_store<__nv_bfloat16, BSIR_ATOMIC_ADD>(s, src, dst, st);
      break;
    case BSIR_I32:
      return store_int_kinds<int32_t>(atomic_kind, s, src, dst, st);
    case BSIR_U32:
      // unsigned storage: max / min compare unsigned
      return store_int_kinds<int32_t>(atomic_kind == BSIR_ATOMIC_MAX ? BSIR_ATOMIC_UMAX
                                      : atomic_kind == BSIR_ATOMIC_MIN ? BSIR_ATOMIC_UMIN : atomic_kind, s, src, dst, st);
    case BSIR_I64:
      return store_int_kinds<int64_t>(atomic_kind, s, src, dst, st);
    case BSIR_U64:
      return store_int_kinds<int64_t>(atomic_kind == BSIR_ATOMIC_MAX ? BSIR_ATOMIC_UMAX
                                      : atomic_kind == BSIR_ATOMIC_MIN ? BSIR_ATOMIC_UMIN : atomic_kind, s, src, dst, st);
    default:
      break;
  }
  return fail(BSIR_ERR_UNSUPPORTED, "store: no atomic %d for dtype %d (f32: add/max/min; f16, bf16: add; 32/64-bit integers: all)",
              atomic_kind, dtype);
}

}  // extern "C"
