// ternary.cu -- hfusion.elemwise_ternary {fma}: out = a * b + c with one rounding
// (bishengir/include/bishengir/Dialect/HFusion/IR/HFusionNamedStructuredOps.yaml:193-272; TernaryFn fma = 1,
// HFusionEnums.td:105-110; the region builds math.fma, bishengir/lib/Dialect/HFusion/IR/HFusionOps.cpp:737-739).
// f32 computes fmaf directly; f16 / bf16 widen to f32, fuse, and round once to the storage type, like every other
// elementwise op here.  (The other ternary function, select, is bsir_select.)  Operands are tensors of rank <= 3 with
// element strides (0 broadcasts a dimension) or scalars; three dense 16-byte aligned tensors stream as 16-byte
// vectors, everything else goes through the indexed kernel.
#include "common.cuh"

namespace bsir {
namespace {

template <int DT> struct TElem { using type = uint16_t; };
template <> struct TElem<BSIR_F32> { using type = float; };

template <int DT>
__device__ __forceinline__ float t_widen(typename TElem<DT>::type v) {
  if constexpr (DT == BSIR_F32) return v;
  else if constexpr (DT == BSIR_F16) return __half2float(__ushort_as_half(v));
  else return __uint_as_float(static_cast<uint32_t>(v) << 16);
}
template <int DT>
__device__ __forceinline__ typename TElem<DT>::type t_narrow(float f) {
  if constexpr (DT == BSIR_F32) return f;
  else if constexpr (DT == BSIR_F16) return __half_as_ushort(__float2half_rn(f));
  else return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

template <int DT>
__global__ void __launch_bounds__(256) fma_vec_kernel(const Vec16 *__restrict__ a, const Vec16 *__restrict__ b, const Vec16 *__restrict__ c,
                                                      Vec16 *__restrict__ out, int64_t nvec) {
  using T = typename TElem<DT>::type;
  constexpr int kPer = 16 / sizeof(T);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const Vec16 va = ld_stream(a + i), vb = ld_stream(b + i), vc = ld_stream(c + i);
    Vec16 vo;
    const T *pa = reinterpret_cast<const T *>(&va), *pb = reinterpret_cast<const T *>(&vb), *pc = reinterpret_cast<const T *>(&vc);
    T *po = reinterpret_cast<T *>(&vo);
#pragma unroll
    for (int e = 0; e < kPer; ++e) po[e] = t_narrow<DT>(fmaf(t_widen<DT>(pa[e]), t_widen<DT>(pb[e]), t_widen<DT>(pc[e])));
    st_stream(out + i, vo);
  }
}

struct TOperand {
  const void *p;       // null: scalar
  int64_t s0, s1, s2;
  uint32_t scalar;
};
template <int DT>
__device__ __forceinline__ float t_fetch(const TOperand &o, int64_t i0, int64_t i1, int64_t i2) {
  using T = typename TElem<DT>::type;
  if (!o.p) {
    if constexpr (DT == BSIR_F32) return __uint_as_float(o.scalar);
    else return t_widen<DT>(static_cast<T>(o.scalar));
  }
  return t_widen<DT>(static_cast<const T *>(o.p)[i0 * o.s0 + i1 * o.s1 + i2 * o.s2]);
}
template <int DT>
__global__ void __launch_bounds__(256) fma_indexed_kernel(TOperand a, TOperand b, TOperand c, void *out, int64_t n0, int64_t n1, int64_t n2,
                                                          int64_t os0, int64_t os1, int64_t os2) {
  using T = typename TElem<DT>::type;
  const int64_t total = n0 * n1 * n2;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t i2 = i % n2, r = i / n2, i1 = r % n1, i0 = r / n1;
    static_cast<T *>(out)[i0 * os0 + i1 * os1 + i2 * os2] =
        t_narrow<DT>(fmaf(t_fetch<DT>(a, i0, i1, i2), t_fetch<DT>(b, i0, i1, i2), t_fetch<DT>(c, i0, i1, i2)));
  }
}

bool dense(const int64_t *st, const int64_t *sizes, int rank) {
  int64_t want = 1;
  for (int i = rank - 1; i >= 0; --i) {
    if (sizes[i] != 1 && st[i] != want) return false;
    want *= sizes[i];
  }
  return true;
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" int32_t bsir_elemwise_ternary(int32_t fn, int32_t dtype, int32_t rank, const int64_t *sizes, const bsir_operand *a,
                                         const bsir_operand *b, const bsir_operand *c, void *out, const int64_t *out_strides,
                                         void *stream) {
  clear_error();
  if (fn != BSIR_TERNARY_FMA) return fail(BSIR_ERR_ATTR, "elemwise_ternary: fn %d (fma = %d; select is bsir_select)", fn, BSIR_TERNARY_FMA);
  if (!dtype_is_float(dtype)) return fail(BSIR_ERR_DTYPE, "elemwise_ternary fma: dtype %d (f32, f16 or bf16)", dtype);
  if (rank < 1 || rank > 3 || !sizes) return fail(BSIR_ERR_SHAPE, "elemwise_ternary: rank %d (1..3)", rank);
  if (!a || !b || !c) return fail(BSIR_ERR_NULL, "elemwise_ternary: null operand");
  int64_t n[3] = {1, 1, 1}, os[3] = {0, 0, 0}, total = 1;
  for (int i = 0; i < rank; ++i) {
    if (sizes[i] < 0) return fail(BSIR_ERR_SHAPE, "elemwise_ternary: negative size");
    n[3 - rank + i] = sizes[i];
    total *= sizes[i];
  }
  if (total == 0) return BSIR_OK;
  if (!out) return fail(BSIR_ERR_NULL, "elemwise_ternary: null output");
  int64_t dense_stride = 1;
  for (int i = rank - 1; i >= 0; --i) { os[3 - rank + i] = out_strides ? out_strides[i] : dense_stride; dense_stride *= sizes[i]; }
  const int eb = dtype_bytes(dtype);
  const bsir_operand *ops[3] = {a, b, c};
  TOperand t[3];
  bool all_dense = !out_strides || dense(out_strides, sizes, rank);
  for (int k = 0; k < 3; ++k) {
    t[k] = TOperand{ops[k]->data, 0, 0, 0, static_cast<uint32_t>(ops[k]->scalar_bits)};
    if (ops[k]->data) {
      if (!aligned_to(ops[k]->data, eb)) return fail(BSIR_ERR_ALIGN, "elemwise_ternary: misaligned operand");
      int64_t st[3] = {0, 0, 0};
      for (int i = 0; i < rank; ++i) st[3 - rank + i] = ops[k]->strides[i];
      t[k].s0 = st[0]; t[k].s1 = st[1]; t[k].s2 = st[2];
      all_dense = all_dense && dense(ops[k]->strides, sizes, rank) && aligned_to(ops[k]->data, 16);
    } else {
      all_dense = false;
    }
  }
  if (!aligned_to(out, eb)) return fail(BSIR_ERR_ALIGN, "elemwise_ternary: misaligned output");
  cudaStream_t st = resolve_stream(stream);
  const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
  const int per = 16 / eb;
  if (all_dense && aligned_to(out, 16) && total % per == 0) {
    const int64_t nvec = total / per;
    const unsigned blocks = static_cast<unsigned>(ceil_div(nvec, 256) < sms * 16 ? ceil_div(nvec, 256) : sms * 16);
    const Vec16 *pa = static_cast<const Vec16 *>(a->data), *pb = static_cast<const Vec16 *>(b->data), *pc = static_cast<const Vec16 *>(c->data);
    if (dtype == BSIR_F32) fma_vec_kernel<BSIR_F32><<<blocks, 256, 0, st>>>(pa, pb, pc, static_cast<Vec16 *>(out), nvec);
    else if (dtype == BSIR_F16) fma_vec_kernel<BSIR_F16><<<blocks, 256, 0, st>>>(pa, pb, pc, static_cast<Vec16 *>(out), nvec);
    else fma_vec_kernel<BSIR_BF16><<<blocks, 256, 0, st>>>(pa, pb, pc, static_cast<Vec16 *>(out), nvec);
  } else {
    const unsigned blocks = static_cast<unsigned>(ceil_div(total, 256) < sms * 16 ? ceil_div(total, 256) : sms * 16);
    if (dtype == BSIR_F32) fma_indexed_kernel<BSIR_F32><<<blocks, 256, 0, st>>>(t[0], t[1], t[2], out, n[0], n[1], n[2], os[0], os[1], os[2]);
    else if (dtype == BSIR_F16) fma_indexed_kernel<BSIR_F16><<<blocks, 256, 0, st>>>(t[0], t[1], t[2], out, n[0], n[1], n[2], os[0], os[1], os[2]);
    else fma_indexed_kernel<BSIR_BF16><<<blocks, 256, 0, st>>>(t[0], t[1], t[2], out, n[0], n[1], n[2], os[0], os[1], os[2]);
  }
  count_launch();
  return check_launch("elemwise_ternary");
}
