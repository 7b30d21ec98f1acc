// common.cuh -- shared host/device helpers of the sm_100a backend library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <utility>

#include "bsir_b200.h"

struct CUtensorMap_st;   // <cuda.h>: CUtensorMap

namespace bsir {

// ----------------------------------------------------------------------------
// host: errors, streams, device info
// ----------------------------------------------------------------------------
int32_t fail(int32_t status, const char *fmt, ...);  // records the text, returns status
void clear_error();
cudaStream_t resolve_stream(void *stream);           // NULL -> the thread's stream
int32_t check_launch(const char *what);              // cudaGetLastError -> status
void count_launch(int n = 1);

struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int max_smem_optin = 0;
  int cc_major = 0;
};
const DeviceInfo &device_info();  // of the current device (cached per device)

// Library-owned scratch of the current device: grown on demand, zero-filled when
// (re)allocated.  Kernels that use it keep the "counters are zero between calls"
// invariant themselves.  Returns nullptr and records an error on failure.
void *device_workspace(size_t bytes, cudaStream_t stream);
// Device-side error word (one int per device); kernels OR a code into it when a
// bounded wait gives up.
int *device_error_word();
// 2-D tensor map over bytes: `inner` contiguous bytes a row, `outer` rows `pitch` bytes apart, box = box_rows x 128
// bytes, with the 128-byte swizzle unless `swizzle` is false; bytes outside read as zero and are not written.  The
// base must be 16-byte aligned and the pitch a multiple of 16.  False when the driver has no encoder or refuses the
// shape.
bool make_byte_tmap(::CUtensorMap_st *map, const void *ptr, uint64_t inner, uint64_t outer, uint64_t pitch, uint32_t box_rows,
                    bool swizzle = true);
// The first kScratchCounterBytes of any scratch block hold self-resetting counters only (one
// uint32 per row of a launch, at most 65535 rows); everything else starts after them.
constexpr size_t kScratchCounterBytes = 256 * 1024;

// hfusion.reduce_with_index over integer rows / with the unsigned kinds (reduce_index_int.cu)
int32_t reduce_with_index_int(int32_t kind, int32_t dtype, int32_t tie_break_left, int64_t rows, int64_t cols, const void *src,
                              int64_t src_row_stride, void *dst_value, int32_t *dst_index, cudaStream_t st);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// dtype helpers
inline int dtype_bytes(int32_t dt) {
  switch (dt) {
    case BSIR_F32: case BSIR_I32: case BSIR_U32: return 4;
    case BSIR_F16: case BSIR_BF16: case BSIR_I16: case BSIR_U16: return 2;
    case BSIR_I64: case BSIR_U64: return 8;
    case BSIR_I8: case BSIR_U8: case BSIR_BOOL: return 1;
    default: return 0;
  }
}
inline bool dtype_is_float(int32_t dt) { return dt == BSIR_F32 || dt == BSIR_F16 || dt == BSIR_BF16; }
inline bool dtype_is_unsigned(int32_t dt) { return dt >= BSIR_U8 && dt <= BSIR_BOOL; }
inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ----------------------------------------------------------------------------
// programmatic dependent launch
// ----------------------------------------------------------------------------
// A kernel launched with launch_pdl may be scheduled before the kernel ahead of it in the stream has finished, if
// that one called pdl_launch_dependents(); it must call pdl_wait() before its first access to global memory
// (the wait returns when the kernel ahead has completed and its writes are visible).  Kernels ahead that never
// call pdl_launch_dependents() serialise as usual.  BSIR_NO_PDL=1 launches plainly.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
  static const bool off = [] { const char *e = std::getenv("BSIR_NO_PDL"); return e && e[0] == '1'; }();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = off ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// The same with the grid cut into thread-block clusters of `cluster_x` consecutive blocks along x.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, int cluster_x,
                               Args &&...args) {
  static const bool off = [] { const char *e = std::getenv("BSIR_NO_PDL"); return e && e[0] == '1'; }();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(cluster_x);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = off ? 1 : 2;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// ----------------------------------------------------------------------------
// device: element types and conversions
// ----------------------------------------------------------------------------
struct alignas(16) Vec16 {
  uint32_t w[4];
};

// Streaming (read-once) 16-byte global load / store: keep the data out of L1.
__device__ __forceinline__ Vec16 ld_stream(const void *p) {
  Vec16 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(void *p, const Vec16 &v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]),
               "r"(v.w[3])
               : "memory");
}

__device__ __forceinline__ float bf16lo_to_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
// two f32 -> packed bf16x2 (lo = a, hi = b), round to nearest even
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float a, float b) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ float f16lo_to_f32(uint32_t w) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu)));
}
__device__ __forceinline__ float f16hi_to_f32(uint32_t w) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
}

// arith.maximumf / minimumf: NaN-propagating, -0 < +0.
__device__ __forceinline__ float maximumf(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float minimumf(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// Element traits for the float storage types: how many per 16-byte vector and
// how to widen / narrow a packed 32-bit word.
template <int DT> struct FloatTraits;
template <> struct FloatTraits<BSIR_F32> {
  static constexpr int kPerWord = 1;
  __device__ static __forceinline__ void unpack(uint32_t w, float *o) { o[0] = __uint_as_float(w); }
  __device__ static __forceinline__ uint32_t pack(const float *v) { return __float_as_uint(v[0]); }
};
template <> struct FloatTraits<BSIR_BF16> {
  static constexpr int kPerWord = 2;
  __device__ static __forceinline__ void unpack(uint32_t w, float *o) {
    o[0] = bf16lo_to_f32(w);
    o[1] = bf16hi_to_f32(w);
  }
  __device__ static __forceinline__ uint32_t pack(const float *v) { return pack_bf16x2(v[0], v[1]); }
};
template <> struct FloatTraits<BSIR_F16> {
  static constexpr int kPerWord = 2;
  __device__ static __forceinline__ void unpack(uint32_t w, float *o) {
    o[0] = f16lo_to_f32(w);
    o[1] = f16hi_to_f32(w);
  }
  __device__ static __forceinline__ uint32_t pack(const float *v) { return pack_f16x2(v[0], v[1]); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_nan(float v) {  // maximumf across the warp
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = maximumf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_max_num(float v) {  // fmaxf (NaN ignored) across the warp
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace bsir
