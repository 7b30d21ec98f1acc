// ciface.cu -- definitions of the `_mlir_ciface_*` op-library symbols.
//
// Each symbol unpacks MLIR memref descriptors (base = aligned + offset, strides in elements:
// bishengir/lib/Template/include/Utils.h:72-78) and forwards to the typed entry point.  The
// symbol tables live in include/bsir_b200_ciface.h and restate what the reference registers
// (bishengir/lib/Template/lib/Vector/Elementwise/EltWise1D.cpp:1318-1500 and siblings).
// Work is enqueued on the calling thread's stream (bsir_set_stream).
#include "common.cuh"

namespace bsir {
namespace {

template <class M>
inline const void *base_of(const M *m, int dt) {
  return static_cast<const char *>(m->aligned) + m->offset * dtype_bytes(dt);
}
template <class M>
inline void *base_of_mut(M *m, int dt) {
  return static_cast<char *>(m->aligned) + m->offset * dtype_bytes(dt);
}

template <int RANK, class M>
int32_t shapes_match(const char *what, const M *a, const M *b) {
  for (int i = 0; i < RANK; ++i)
    if (a->sizes[i] != b->sizes[i] && a->sizes[i] != 1)
      return fail(BSIR_ERR_SHAPE, "%s: operand size %lld vs result size %lld in dim %d", what, (long long)a->sizes[i],
                  (long long)b->sizes[i], i);
  return BSIR_OK;
}

// Operand from a descriptor; a dimension of size 1 against a larger result broadcasts (stride 0),
// the inline-broadcast form of the HIVM vector ops.
template <int RANK, class M>
bsir_operand operand_of(const M *m, const M *dst, int dt) {
  bsir_operand o{base_of(m, dt), {0, 0, 0}, 0};
  for (int i = 0; i < RANK; ++i) o.strides[i] = (m->sizes[i] == 1 && dst->sizes[i] != 1) ? 0 : m->strides[i];
  return o;
}

template <int RANK, class M>
int32_t vv(const char *what, int fn, int dt, M *a, M *b, M *dst) {
  if (!a || !b || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (int32_t rc = shapes_match<RANK>(what, a, dst)) return rc;
  if (int32_t rc = shapes_match<RANK>(what, b, dst)) return rc;
  bsir_operand oa = operand_of<RANK>(a, dst, dt), ob = operand_of<RANK>(b, dst, dt);
  return bsir_elemwise_binary(fn, dt, RANK, dst->sizes, &oa, &ob, base_of_mut(dst, dt), dst->strides, nullptr);
}
template <int RANK, class M>
int32_t vs(const char *what, int fn, int dt, M *a, uint64_t scalar_bits, M *dst, bool scalar_first) {
  if (!a || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (int32_t rc = shapes_match<RANK>(what, a, dst)) return rc;
  bsir_operand oa = operand_of<RANK>(a, dst, dt), os{nullptr, {0, 0, 0}, scalar_bits};
  return scalar_first
             ? bsir_elemwise_binary(fn, dt, RANK, dst->sizes, &os, &oa, base_of_mut(dst, dt), dst->strides, nullptr)
             : bsir_elemwise_binary(fn, dt, RANK, dst->sizes, &oa, &os, base_of_mut(dst, dt), dst->strides, nullptr);
}
template <int RANK, class M>
int32_t v1(const char *what, int fn, int dt, M *a, M *dst) {
  if (!a || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (int32_t rc = shapes_match<RANK>(what, a, dst)) return rc;
  bsir_operand oa = operand_of<RANK>(a, dst, dt);
  return bsir_elemwise_unary(fn, dt, RANK, dst->sizes, &oa, base_of_mut(dst, dt), dst->strides, nullptr);
}
template <int RANK, class M>
int32_t vcast(const char *what, int sdt, int ddt, M *src, M *dst, uint32_t cast_mode, int overflow) {
  if (!src || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  for (int i = 0; i < RANK; ++i)
    if (src->sizes[i] != dst->sizes[i]) return fail(BSIR_ERR_SHAPE, "%s: size mismatch in dim %d", what, i);
  // CastMode R/A/F/C/Z/O/OVERFLOW carries the same numbering as hfusion.round_mode
  // (bishengir/lib/Template/include/Vector/Cast/CastUtils.h:30-38).
  return bsir_cast(sdt, ddt, static_cast<int32_t>(cast_mode), overflow, RANK, dst->sizes, base_of(src, sdt),
                   src->strides, base_of_mut(dst, ddt), dst->strides, nullptr);
}

template <class T>
inline uint64_t bits_of_scalar(T v) {
  uint64_t b = 0;
  memcpy(&b, &v, sizeof(T));
  return b;
}

int32_t reduce_ar(const char *what, int kind, int dt, bsir_memref_2d *src, bsir_memref_2d *dst) {
  if (!src || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (src->sizes[1] > 1 && src->strides[1] != 1) return fail(BSIR_ERR_STRIDE, "%s: reduced axis must be unit-stride", what);
  if (dst->sizes[0] != src->sizes[0]) return fail(BSIR_ERR_SHAPE, "%s: dst rows", what);
  if (dst->sizes[0] > 1 && dst->strides[0] != 1) return fail(BSIR_ERR_STRIDE, "%s: dst must be dense", what);
  return bsir_reduce_last_axis(kind, dt, src->sizes[0], src->sizes[1], base_of(src, dt),
                               src->sizes[0] > 1 ? src->strides[0] : src->sizes[1], base_of_mut(dst, dt), nullptr);
}
int32_t reduce_r(const char *what, int kind, int dt, bsir_memref_1d *src, bsir_memref_1d *dst) {
  if (!src || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (src->sizes[0] > 1 && src->strides[0] != 1) return fail(BSIR_ERR_STRIDE, "%s: reduced axis must be unit-stride", what);
  return bsir_reduce_last_axis(kind, dt, 1, src->sizes[0], base_of(src, dt), src->sizes[0], base_of_mut(dst, dt), nullptr);
}
int32_t reduce_ra(const char *what, int kind, int dt, bsir_memref_2d *src, bsir_memref_2d *dst) {
  if (!src || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (src->sizes[1] > 1 && src->strides[1] != 1) return fail(BSIR_ERR_STRIDE, "%s: kept axis must be unit-stride", what);
  if (dst->sizes[1] != src->sizes[1]) return fail(BSIR_ERR_SHAPE, "%s: dst cols", what);
  if (dst->sizes[1] > 1 && dst->strides[1] != 1) return fail(BSIR_ERR_STRIDE, "%s: dst must be dense", what);
  return bsir_reduce_first_axis(kind, dt, src->sizes[0], src->sizes[1], base_of(src, dt),
                                src->sizes[0] > 1 ? src->strides[0] : src->sizes[1], base_of_mut(dst, dt), nullptr);
}
int32_t rwi_ar(const char *what, int kind, int left, int dt, bsir_memref_2d *src, bsir_memref_2d *dv, bsir_memref_2d *di,
               bsir_memref_1d *tmp) {
  if (!src || !dv || !di) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (src->sizes[1] > 1 && src->strides[1] != 1) return fail(BSIR_ERR_STRIDE, "%s: reduced axis must be unit-stride", what);
  if ((dv->sizes[0] > 1 && dv->strides[0] != 1) || (di->sizes[0] > 1 && di->strides[0] != 1))
    return fail(BSIR_ERR_STRIDE, "%s: results must be dense", what);
  (void)tmp;  // on-chip temp of the reference; the global scratch here has its own zero-fill contract
  // The device library's NaN rule: the first NaN wins
  // (bishengir/lib/Template/lib/Vector/Reduction/ReduceR_With_Index.cpp:83-125).
  return bsir_reduce_with_index(kind, dt, left, BSIR_RWI_NAN_FIRST, src->sizes[0], src->sizes[1], base_of(src, dt),
                                src->sizes[0] > 1 ? src->strides[0] : src->sizes[1], base_of_mut(dv, dt),
                                static_cast<int32_t *>(base_of_mut(di, BSIR_I32)), nullptr, 0, nullptr);
}
int32_t rwi_r(const char *what, int kind, int left, int dt, bsir_memref_1d *src, bsir_memref_1d *dv, bsir_memref_1d *di) {
  if (!src || !dv || !di) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (src->sizes[0] > 1 && src->strides[0] != 1) return fail(BSIR_ERR_STRIDE, "%s: reduced axis must be unit-stride", what);
  return bsir_reduce_with_index(kind, dt, left, BSIR_RWI_NAN_FIRST, 1, src->sizes[0], base_of(src, dt), src->sizes[0],
                                base_of_mut(dv, dt), static_cast<int32_t *>(base_of_mut(di, BSIR_I32)), nullptr, 0, nullptr);
}

// ---- further HIVM vector ops: descriptors unpacked onto the typed entry points
int32_t cum_ra(const char *what, int kind, int dt, int reverse, bsir_memref_2d *src, bsir_memref_2d *dst) {
  if (!src || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (src->sizes[0] != dst->sizes[0] || src->sizes[1] != dst->sizes[1]) return fail(BSIR_ERR_SHAPE, "%s: shapes differ", what);
  if ((src->sizes[1] > 1 && (src->strides[1] != 1 || dst->strides[1] != 1))) return fail(BSIR_ERR_STRIDE, "%s: last axis must be unit-stride", what);
  return bsir_cumulative(kind, dt, 0, reverse, 1, src->sizes[0], src->sizes[1], base_of(src, dt), src->sizes[0] > 1 ? src->strides[0] : src->sizes[1],
                         base_of_mut(dst, dt), dst->sizes[0] > 1 ? dst->strides[0] : dst->sizes[1], nullptr);
}
int32_t cum_ara(const char *what, int kind, int dt, int reverse, bsir_memref_3d *src, bsir_memref_3d *dst) {
  if (!src || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  for (int i = 0; i < 3; ++i)
    if (src->sizes[i] != dst->sizes[i]) return fail(BSIR_ERR_SHAPE, "%s: shapes differ", what);
  if (src->sizes[2] > 1 && (src->strides[2] != 1 || dst->strides[2] != 1)) return fail(BSIR_ERR_STRIDE, "%s: last axis must be unit-stride", what);
  const int eb = dtype_bytes(dt);
  for (int64_t i = 0; i < src->sizes[0]; ++i) {
    const int32_t rc = bsir_cumulative(kind, dt, 0, reverse, 1, src->sizes[1], src->sizes[2],
                                       static_cast<const char *>(base_of(src, dt)) + i * src->strides[0] * eb,
                                       src->sizes[1] > 1 ? src->strides[1] : src->sizes[2],
                                       static_cast<char *>(base_of_mut(dst, dt)) + i * dst->strides[0] * eb,
                                       dst->sizes[1] > 1 ? dst->strides[1] : dst->sizes[2], nullptr);
    if (rc) return rc;
  }
  return BSIR_OK;
}
int32_t sort_1d(const char *what, int dt, bsir_memref_1d *src, bsir_memref_1d *dst, bsir_memref_1d *index, bool descending) {
  if (!src || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (src->sizes[0] != dst->sizes[0] || (index && index->sizes[0] != src->sizes[0])) return fail(BSIR_ERR_SHAPE, "%s: lengths differ", what);
  if (src->sizes[0] > 1 && (src->strides[0] != 1 || dst->strides[0] != 1 || (index && index->strides[0] != 1)))
    return fail(BSIR_ERR_STRIDE, "%s: unit strides only", what);
  const int64_t n = src->sizes[0];
  return bsir_sort(dt, descending ? 1 : 0, 1, n, base_of(src, dt), n, base_of_mut(dst, dt), n,
                   index ? static_cast<int32_t *>(base_of_mut(index, BSIR_I32)) : nullptr, n, nullptr);
}
template <class M>
bool dense_last(const M *m, int rank) { return m->sizes[rank - 1] <= 1 || m->strides[rank - 1] == 1; }
int32_t interleave_1d(const char *what, int dt, bsir_memref_1d *a, bsir_memref_1d *b, bsir_memref_1d *dst) {
  if (!a || !b || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (a->sizes[0] != b->sizes[0] || dst->sizes[0] != 2 * a->sizes[0]) return fail(BSIR_ERR_SHAPE, "%s: lengths do not compose", what);
  if (!dense_last(a, 1) || !dense_last(b, 1) || !dense_last(dst, 1)) return fail(BSIR_ERR_STRIDE, "%s: unit strides only", what);
  const void *srcs[2] = {base_of(a, dt), base_of(b, dt)};
  return bsir_interleave(dt, 2, 1, a->sizes[0], srcs, base_of_mut(dst, dt), nullptr);
}
// channel `ch` of `channels` (0 = derive the count from the lengths) out of rows x (channels * cols)
int32_t deinterleave_rows(const char *what, int dt, int ch, int channels, int64_t rows, int64_t src_cols, int64_t dst_cols, const void *src, void *dst) {
  if (channels == 0) {
    if (dst_cols <= 0 || src_cols % dst_cols) return fail(BSIR_ERR_SHAPE, "%s: %lld is not a multiple of %lld", what, (long long)src_cols, (long long)dst_cols);
    channels = static_cast<int>(src_cols / dst_cols);
  }
  if (channels < 1 || channels > 8 || src_cols != dst_cols * channels) return fail(BSIR_ERR_SHAPE, "%s: lengths do not compose", what);
  void *dsts[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  dsts[ch] = dst;
  return bsir_deinterleave(dt, channels, rows, dst_cols, src, dsts, nullptr);
}
template <int RANK, class M>
int32_t arange_nd(const char *what, int dt, M *dst, int64_t offset, const int64_t *strides) {
  if (!dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  return bsir_arange(dt, RANK, dst->sizes, offset, strides, base_of_mut(dst, dt), dst->strides, nullptr);
}
// dst = src with its axes permuted: dst axis i is src axis perm[i]
template <int RANK, class M>
int32_t transpose_nd(const char *what, int dt, M *src, M *dst, const int *perm) {
  if (!src || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  int64_t st[3] = {0, 0, 0};
  for (int i = 0; i < RANK; ++i) {
    if (dst->sizes[i] != src->sizes[perm[i]]) return fail(BSIR_ERR_SHAPE, "%s: shapes do not compose", what);
    st[i] = src->strides[perm[i]];
  }
  return bsir_copy(dt, RANK, dst->sizes, base_of(src, dt), st, base_of_mut(dst, dt), dst->strides, nullptr);
}
int32_t gather_1d(const char *what, int dt, bsir_memref_1d *src, bsir_memref_1d *idx, bsir_memref_1d *dst) {
  if (!src || !idx || !dst) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  if (idx->sizes[0] != dst->sizes[0]) return fail(BSIR_ERR_SHAPE, "%s: indices and dst differ in length", what);
  if (!dense_last(src, 1) || !dense_last(idx, 1) || !dense_last(dst, 1)) return fail(BSIR_ERR_STRIDE, "%s: unit strides only", what);
  return bsir_gather(dt, BSIR_I32, 1, src->sizes[0], dst->sizes[0], 1, base_of(src, dt), base_of(idx, BSIR_I32), base_of_mut(dst, dt), nullptr);
}

// hivm.hir.matmul library call: operands in the op's order, bias / descale optional (null = absent)
int32_t matmul_call(const char *what, int in_dt, int out_dt, int bias_dt, int descale_dt, int descale_mode, int ta, int tb,
                    bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_1d *bias, bsir_memref_1d *descale, bsir_memref_2d *C) {
  if (!A || !B || !C || (descale_mode != BSIR_DESCALE_NULL && !descale)) return fail(BSIR_ERR_NULL, "%s: null descriptor", what);
  const int64_t m = ta ? A->sizes[1] : A->sizes[0], k = ta ? A->sizes[0] : A->sizes[1];
  const int64_t n = tb ? B->sizes[0] : B->sizes[1];
  if ((tb ? B->sizes[1] : B->sizes[0]) != k || C->sizes[0] != m || C->sizes[1] != n)
    return fail(BSIR_ERR_SHAPE, "%s: shapes do not compose", what);
  if (bias && bias->sizes[0] != n) return fail(BSIR_ERR_SHAPE, "%s: bias of %lld entries for n = %lld", what, (long long)bias->sizes[0], (long long)n);
  if (descale_mode == BSIR_DESCALE_PER_CHANNEL && descale->sizes[0] != n) return fail(BSIR_ERR_SHAPE, "%s: per-channel descale of %lld entries for n = %lld", what, (long long)descale->sizes[0], (long long)n);
  if (descale_mode == BSIR_DESCALE_PER_TENSOR && descale->sizes[0] != 1) return fail(BSIR_ERR_SHAPE, "%s: per-tensor descale of %lld entries", what, (long long)descale->sizes[0]);
  if ((A->sizes[1] > 1 && A->strides[1] != 1) || (B->sizes[1] > 1 && B->strides[1] != 1) || (n > 1 && C->strides[1] != 1) ||
      (bias && n > 1 && bias->strides[0] != 1) || (descale && descale->sizes[0] > 1 && descale->strides[0] != 1))
    return fail(BSIR_ERR_STRIDE, "%s: innermost dimensions must be unit-stride", what);
  bsir_matmul_desc d{};
  d.in_dtype = in_dt; d.out_dtype = out_dt; d.transpose_a = ta; d.transpose_b = tb;
  d.descale_mode = descale_mode; d.bias_dtype = bias_dt; d.descale_dtype = descale_dt;
  d.m = m; d.n = n; d.k = k; d.batch = 1;
  d.a = base_of(A, in_dt); d.lda = A->strides[0];
  d.b = base_of(B, in_dt); d.ldb = B->strides[0];
  d.bias = bias ? base_of(bias, bias_dt) : nullptr;
  d.descale = descale ? base_of(descale, descale_dt) : nullptr;
  d.out = base_of_mut(C, out_dt); d.ldo = C->strides[0];
  return bsir_matmul(&d, nullptr);
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" {

#define BSIR_DEF_VV(op, fn, rank, tok)                                                                       \
  int32_t _mlir_ciface_##op##_##rank##d_##tok(BSIR_MEMREF_T(rank) * src0, BSIR_MEMREF_T(rank) * src1,        \
                                              BSIR_MEMREF_T(rank) * dst, bsir_memref_1d *) {                 \
    clear_error();                                                                                           \
    return vv<rank>(#op "_" #rank "d_" #tok, fn, BSIR_DT_##tok, src0, src1, dst);                            \
  }
#define BSIR_DEF_VS(op, fn, rank, tok)                                                                       \
  int32_t _mlir_ciface_##op##_vs_##rank##d_##tok(BSIR_MEMREF_T(rank) * src0, BSIR_SCALAR_##tok scalar,       \
                                                 BSIR_MEMREF_T(rank) * dst, bsir_memref_1d *) {              \
    clear_error();                                                                                           \
    return vs<rank>(#op "_vs_" #rank "d_" #tok, fn, BSIR_DT_##tok, src0, bits_of_scalar(scalar), dst, false); \
  }
#define BSIR_DEF_SV(op, fn, rank, tok)                                                                       \
  int32_t _mlir_ciface_##op##_sv_##rank##d_##tok(BSIR_SCALAR_##tok scalar, BSIR_MEMREF_T(rank) * src1,       \
                                                 BSIR_MEMREF_T(rank) * dst, bsir_memref_1d *) {              \
    clear_error();                                                                                           \
    return vs<rank>(#op "_sv_" #rank "d_" #tok, fn, BSIR_DT_##tok, src1, bits_of_scalar(scalar), dst, true);  \
  }
#define BSIR_DEF_V(op, fn, rank, tok)                                                                        \
  int32_t _mlir_ciface_##op##_##rank##d_##tok(BSIR_MEMREF_T(rank) * src0, BSIR_MEMREF_T(rank) * dst,         \
                                              bsir_memref_1d *) {                                            \
    clear_error();                                                                                           \
    return v1<rank>(#op "_" #rank "d_" #tok, fn, BSIR_DT_##tok, src0, dst);                                  \
  }
#define BSIR_DEF_CAST_MODE(s, d, rank)                                                                       \
  int32_t _mlir_ciface_vcast_##s##_to_##d##_##rank##d_with_mode(BSIR_MEMREF_T(rank) * src,                   \
                                                                BSIR_MEMREF_T(rank) * dst, uint32_t cast_mode) { \
    clear_error();                                                                                           \
    return vcast<rank>("vcast_" #s "_to_" #d, BSIR_DT_##s, BSIR_DT_##d, src, dst, cast_mode, BSIR_OVERFLOW_SATURATE); \
  }
#define BSIR_DEF_CAST_OVERFLOW(s, d, rank)                                                                   \
  int32_t _mlir_ciface_vcast_##s##_to_##d##_##rank##d_with_overflow(                                         \
      BSIR_MEMREF_T(rank) * src, BSIR_MEMREF_T(rank) * dst, bsir_memref_1d *, uint32_t cast_mode) {          \
    clear_error();                                                                                           \
    return vcast<rank>("vcast_" #s "_to_" #d, BSIR_DT_##s, BSIR_DT_##d, src, dst, cast_mode, BSIR_OVERFLOW_WRAP); \
  }                                                                                                          \
  int32_t _mlir_ciface_vcast_##s##_to_##d##_##rank##d_with_overflow_no_size_align(                           \
      BSIR_MEMREF_T(rank) * src, BSIR_MEMREF_T(rank) * dst, bsir_memref_1d *, uint32_t cast_mode) {          \
    clear_error();                                                                                           \
    return vcast<rank>("vcast_" #s "_to_" #d, BSIR_DT_##s, BSIR_DT_##d, src, dst, cast_mode, BSIR_OVERFLOW_WRAP); \
  }
#define BSIR_DEF_CAST_TEMP(s, d, rank)                                                                       \
  int32_t _mlir_ciface_vcast_##s##_to_##d##_##rank##d_with_temp(BSIR_MEMREF_T(rank) * src,                   \
                                                                BSIR_MEMREF_T(rank) * dst, bsir_memref_1d *, \
                                                                uint32_t cast_mode) {                        \
    clear_error();                                                                                           \
    return vcast<rank>("vcast_" #s "_to_" #d, BSIR_DT_##s, BSIR_DT_##d, src, dst, cast_mode, BSIR_OVERFLOW_SATURATE); \
  }
/* initvalue is the identity the caller would have filled dst with; dst is write-only here. */
#define BSIR_DEF_REDUCE(name, kind, tok)                                                                     \
  int32_t _mlir_ciface_##name##_ar_##tok(bsir_memref_2d *src0, bsir_memref_2d *dst, bsir_memref_1d *,        \
                                         BSIR_SCALAR_##tok) {                                                \
    clear_error();                                                                                           \
    return reduce_ar(#name "_ar_" #tok, kind, BSIR_DT_##tok, src0, dst);                                     \
  }                                                                                                          \
  int32_t _mlir_ciface_##name##_r_##tok(bsir_memref_1d *src0, bsir_memref_1d *dst, bsir_memref_1d *,         \
                                        BSIR_SCALAR_##tok) {                                                 \
    clear_error();                                                                                           \
    return reduce_r(#name "_r_" #tok, kind, BSIR_DT_##tok, src0, dst);                                       \
  }                                                                                                          \
  int32_t _mlir_ciface_##name##_ra_##tok(bsir_memref_2d *src0, bsir_memref_2d *dst, bsir_memref_1d *,        \
                                         BSIR_SCALAR_##tok) {                                                \
    clear_error();                                                                                           \
    return reduce_ra(#name "_ra_" #tok, kind, BSIR_DT_##tok, src0, dst);                                     \
  }
#define BSIR_DEF_REDUCE_WITH_INDEX(name, kind, left, tok)                                                    \
  int32_t _mlir_ciface_##name##_ar_##tok(bsir_memref_2d *src0, bsir_memref_2d *dst_value,                    \
                                         bsir_memref_2d *dst_index, bsir_memref_1d *tmp_buf,                 \
                                         BSIR_SCALAR_##tok) {                                                \
    clear_error();                                                                                           \
    return rwi_ar(#name "_ar_" #tok, kind, left, BSIR_DT_##tok, src0, dst_value, dst_index, tmp_buf);        \
  }                                                                                                          \
  int32_t _mlir_ciface_##name##_r_##tok(bsir_memref_1d *src0, bsir_memref_1d *dst_value,                     \
                                        bsir_memref_1d *dst_index, bsir_memref_1d *, BSIR_SCALAR_##tok) {    \
    clear_error();                                                                                           \
    return rwi_r(#name "_r_" #tok, kind, left, BSIR_DT_##tok, src0, dst_value, dst_index);                   \
  }

BSIR_FOREACH_ELTWISE_VV(BSIR_DEF_VV, 1)
BSIR_FOREACH_ELTWISE_VV(BSIR_DEF_VV, 2)
BSIR_FOREACH_ELTWISE_VV(BSIR_DEF_VV, 3)
BSIR_FOREACH_ELTWISE_VS(BSIR_DEF_VS, 1)
BSIR_FOREACH_ELTWISE_VS(BSIR_DEF_VS, 2)
BSIR_FOREACH_ELTWISE_VS(BSIR_DEF_VS, 3)
BSIR_FOREACH_ELTWISE_SV(BSIR_DEF_SV, 1)
BSIR_FOREACH_ELTWISE_SV(BSIR_DEF_SV, 2)
BSIR_FOREACH_ELTWISE_SV(BSIR_DEF_SV, 3)
BSIR_FOREACH_ELTWISE_V(BSIR_DEF_V, 1)
BSIR_FOREACH_ELTWISE_V(BSIR_DEF_V, 2)
BSIR_FOREACH_ELTWISE_V(BSIR_DEF_V, 3)
BSIR_FOREACH_CAST_WITH_MODE(BSIR_DEF_CAST_MODE, 1)
BSIR_FOREACH_CAST_WITH_MODE(BSIR_DEF_CAST_MODE, 2)
BSIR_FOREACH_CAST_WITH_OVERFLOW(BSIR_DEF_CAST_OVERFLOW, 1)
BSIR_FOREACH_CAST_WITH_OVERFLOW(BSIR_DEF_CAST_OVERFLOW, 2)
BSIR_FOREACH_CAST_WITH_TEMP(BSIR_DEF_CAST_TEMP, 1)
BSIR_FOREACH_CAST_WITH_TEMP(BSIR_DEF_CAST_TEMP, 2)
BSIR_FOREACH_REDUCE(BSIR_DEF_REDUCE)
BSIR_FOREACH_REDUCE_WITH_INDEX(BSIR_DEF_REDUCE_WITH_INDEX)

#define BSIR_DEF_CUM(tok, op)                                                                                                    \
  int32_t _mlir_ciface_##op##_ra_##tok(bsir_memref_2d *src, bsir_memref_2d *dst) { clear_error(); return cum_ra(#op "_ra", BSIR_KIND_##op, BSIR_DT_##tok, 0, src, dst); } \
  int32_t _mlir_ciface_##op##_ra_reverse_##tok(bsir_memref_2d *src, bsir_memref_2d *dst) { clear_error(); return cum_ra(#op "_ra_reverse", BSIR_KIND_##op, BSIR_DT_##tok, 1, src, dst); } \
  int32_t _mlir_ciface_##op##_ara_##tok(bsir_memref_3d *src, bsir_memref_3d *dst) { clear_error(); return cum_ara(#op "_ara", BSIR_KIND_##op, BSIR_DT_##tok, 0, src, dst); } \
  int32_t _mlir_ciface_##op##_ara_reverse_##tok(bsir_memref_3d *src, bsir_memref_3d *dst) { clear_error(); return cum_ara(#op "_ara_reverse", BSIR_KIND_##op, BSIR_DT_##tok, 1, src, dst); }
#define BSIR_KIND_cumsum 0
#define BSIR_KIND_cumprod 1
BSIR_TYPES_CUM(BSIR_DEF_CUM, cumsum)
BSIR_TYPES_CUM(BSIR_DEF_CUM, cumprod)
#define BSIR_DEF_SORT(tok)                                                                                                       \
  int32_t _mlir_ciface_sort_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *dst, bsir_memref_1d *tmp, bool descending) {            \
    (void)tmp; clear_error(); return sort_1d("sort_1d", BSIR_DT_##tok, src, dst, nullptr, descending);                            \
  }                                                                                                                              \
  int32_t _mlir_ciface_sort_with_index_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *dst, bsir_memref_1d *index, bsir_memref_1d *tmp, bool descending) { \
    (void)tmp; clear_error();                                                                                                    \
    if (!index) return fail(BSIR_ERR_NULL, "sort_with_index_1d: null index descriptor");                                         \
    return sort_1d("sort_with_index_1d", BSIR_DT_##tok, src, dst, index, descending);                                            \
  }
BSIR_TYPES_SORT(BSIR_DEF_SORT)
#define BSIR_DEF_LEAVE(tok, unused)                                                                                              \
  int32_t _mlir_ciface_interleave_1d_##tok(bsir_memref_1d *src0, bsir_memref_1d *src1, bsir_memref_1d *dst, bsir_memref_1d *temp) { \
    (void)temp; clear_error(); return interleave_1d("interleave_1d", BSIR_DT_##tok, src0, src1, dst);                             \
  }                                                                                                                              \
  int32_t _mlir_ciface_deinterleave_channel_0_from_2_channels_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *dst) {               \
    clear_error();                                                                                                               \
    if (!src || !dst || !dense_last(src, 1) || !dense_last(dst, 1)) return fail(BSIR_ERR_STRIDE, "deinterleave: null or strided descriptor"); \
    return deinterleave_rows("deinterleave_channel_0_from_2_channels_1d", BSIR_DT_##tok, 0, 2, 1, src->sizes[0], dst->sizes[0], base_of(src, BSIR_DT_##tok), base_of_mut(dst, BSIR_DT_##tok)); \
  }                                                                                                                              \
  int32_t _mlir_ciface_deinterleave_channel_1_from_2_channels_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *dst) {               \
    clear_error();                                                                                                               \
    if (!src || !dst || !dense_last(src, 1) || !dense_last(dst, 1)) return fail(BSIR_ERR_STRIDE, "deinterleave: null or strided descriptor"); \
    return deinterleave_rows("deinterleave_channel_1_from_2_channels_1d", BSIR_DT_##tok, 1, 2, 1, src->sizes[0], dst->sizes[0], base_of(src, BSIR_DT_##tok), base_of_mut(dst, BSIR_DT_##tok)); \
  }                                                                                                                              \
  int32_t _mlir_ciface_deinterleave_channel_0_from_n_channels_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *dst) {               \
    clear_error();                                                                                                               \
    if (!src || !dst || !dense_last(src, 1) || !dense_last(dst, 1)) return fail(BSIR_ERR_STRIDE, "deinterleave: null or strided descriptor"); \
    return deinterleave_rows("deinterleave_channel_0_from_n_channels_1d", BSIR_DT_##tok, 0, 0, 1, src->sizes[0], dst->sizes[0], base_of(src, BSIR_DT_##tok), base_of_mut(dst, BSIR_DT_##tok)); \
  }                                                                                                                              \
  int32_t _mlir_ciface_deinterleave_channel_0_from_n_channels_2d_##tok(bsir_memref_2d *src, bsir_memref_2d *dst) {               \
    clear_error();                                                                                                               \
    if (!src || !dst || !dense_last(src, 2) || !dense_last(dst, 2) || src->sizes[0] != dst->sizes[0] ||                          \
        (src->sizes[0] > 1 && (src->strides[0] != src->sizes[1] || dst->strides[0] != dst->sizes[1])))                           \
      return fail(BSIR_ERR_STRIDE, "deinterleave_2d: null, mismatched or non-contiguous descriptor");                            \
    return deinterleave_rows("deinterleave_channel_0_from_n_channels_2d", BSIR_DT_##tok, 0, 0, src->sizes[0], src->sizes[1], dst->sizes[1], base_of(src, BSIR_DT_##tok), base_of_mut(dst, BSIR_DT_##tok)); \
  }
BSIR_TYPES_LEAVE(BSIR_DEF_LEAVE, 0)
#define BSIR_DEF_ARANGE(tok)                                                                                                     \
  int32_t _mlir_ciface_arange_1d_##tok(bsir_memref_1d *dst, int64_t offset, int64_t stride) {                                    \
    clear_error(); const int64_t st[1] = {stride}; return arange_nd<1>("arange_1d", BSIR_DT_##tok, dst, offset, st);              \
  }                                                                                                                              \
  int32_t _mlir_ciface_arange_2d_##tok(bsir_memref_2d *dst, int64_t offset, int64_t stride0, int64_t stride1) {                  \
    clear_error(); const int64_t st[2] = {stride0, stride1}; return arange_nd<2>("arange_2d", BSIR_DT_##tok, dst, offset, st);    \
  }                                                                                                                              \
  int32_t _mlir_ciface_arange_3d_##tok(bsir_memref_3d *dst, int64_t offset, int64_t stride0, int64_t stride1, int64_t stride2) { \
    clear_error(); const int64_t st[3] = {stride0, stride1, stride2}; return arange_nd<3>("arange_3d", BSIR_DT_##tok, dst, offset, st); \
  }
BSIR_TYPES_ARANGE(BSIR_DEF_ARANGE)
#define BSIR_DEF_TRANSPOSE(tok)                                                                                                  \
  int32_t _mlir_ciface_transpose_2d_with_last_axis_##tok(bsir_memref_2d *src, bsir_memref_2d *dst) {                             \
    clear_error(); const int perm[2] = {1, 0}; return transpose_nd<2>("transpose_2d_with_last_axis", BSIR_DT_##tok, src, dst, perm); \
  }                                                                                                                              \
  int32_t _mlir_ciface_transpose_3d_with_last_axis_##tok(bsir_memref_3d *src, bsir_memref_3d *dst) {                             \
    clear_error(); const int perm[3] = {2, 1, 0}; return transpose_nd<3>("transpose_3d_with_last_axis", BSIR_DT_##tok, src, dst, perm); \
  }                                                                                                                              \
  int32_t _mlir_ciface_transpose_3d_without_last_axis_##tok(bsir_memref_3d *src, bsir_memref_3d *dst) {                          \
    clear_error(); const int perm[3] = {1, 0, 2}; return transpose_nd<3>("transpose_3d_without_last_axis", BSIR_DT_##tok, src, dst, perm); \
  }
BSIR_TYPES_TRANSPOSE(BSIR_DEF_TRANSPOSE)
#define BSIR_DEF_GATHER(tok)                                                                                                     \
  int32_t _mlir_ciface_gather_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *indices, bsir_memref_1d *dst, bsir_memref_1d *tmp) { \
    (void)tmp; clear_error(); return gather_1d("gather_1d", BSIR_DT_##tok, src, indices, dst);                                    \
  }
BSIR_TYPES_GATHER(BSIR_DEF_GATHER)

#define BSIR_DEF_MM_PLAIN_T(ta, tb, fa, fb, a, c)                                                                   \
  int32_t _mlir_ciface_matmul_Xbias_Xdescale_##ta##_##tb##_TA##a##_TB##a##_TC##c(bsir_memref_2d *A, bsir_memref_2d *B, \
                                                                                 bsir_memref_2d *C) {                \
    clear_error();                                                                                                    \
    return matmul_call("matmul_" #a "_" #c, BSIR_DT_##a, BSIR_DT_##c, BSIR_F32, BSIR_F32, BSIR_DESCALE_NULL, fa, fb, A, B, \
                       nullptr, nullptr, C);                                                                          \
  }
#define BSIR_DEF_MM_PLAIN(a, c) BSIR_MATMUL_TRANSPOSES(BSIR_DEF_MM_PLAIN_T, a, c)
#define BSIR_DEF_MM_BIAS_T(ta, tb, fa, fb, a, c, bt)                                                                  \
  int32_t _mlir_ciface_matmul_bias_TBIAS##bt##_Xdescale_##ta##_##tb##_TA##a##_TB##a##_TC##c(                          \
      bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_1d *bias, bsir_memref_2d *C) {                                \
    clear_error();                                                                                                    \
    if (!bias) return fail(BSIR_ERR_NULL, "matmul with bias: null bias descriptor");                                  \
    return matmul_call("matmul_bias_" #a "_" #c, BSIR_DT_##a, BSIR_DT_##c, BSIR_DT_##bt, BSIR_F32, BSIR_DESCALE_NULL, fa, fb, \
                       A, B, bias, nullptr, C);                                                                       \
  }
#define BSIR_DEF_MM_BIAS(a, c, bt) BSIR_MATMUL_TRANSPOSES(BSIR_DEF_MM_BIAS_T, a, c, bt)
#define BSIR_DEF_MM_DESCALE_T(ta, tb, fa, fb, a, c, dt)                                                               \
  int32_t _mlir_ciface_matmul_Xbias_descalePerChannel_TDESCALE##dt##_##ta##_##tb##_TA##a##_TB##a##_TC##c(             \
      bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_1d *descale, bsir_memref_2d *C) {                             \
    clear_error();                                                                                                    \
    return matmul_call("matmul_descalePerChannel_" #a "_" #c, BSIR_DT_##a, BSIR_DT_##c, BSIR_F32, BSIR_DT_##dt,       \
                       BSIR_DESCALE_PER_CHANNEL, fa, fb, A, B, nullptr, descale, C);                                  \
  }                                                                                                                   \
  int32_t _mlir_ciface_matmul_Xbias_descalePerTensor_TDESCALE##dt##_##ta##_##tb##_TA##a##_TB##a##_TC##c(              \
      bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_1d *descale, bsir_memref_2d *C) {                             \
    clear_error();                                                                                                    \
    return matmul_call("matmul_descalePerTensor_" #a "_" #c, BSIR_DT_##a, BSIR_DT_##c, BSIR_F32, BSIR_DT_##dt,        \
                       BSIR_DESCALE_PER_TENSOR, fa, fb, A, B, nullptr, descale, C);                                   \
  }
#define BSIR_DEF_MM_DESCALE(a, c, dt) BSIR_MATMUL_TRANSPOSES(BSIR_DEF_MM_DESCALE_T, a, c, dt)
#define BSIR_DEF_MM_BOTH_T(ta, tb, fa, fb, a, c, bt, dt)                                                              \
  int32_t _mlir_ciface_matmul_bias_TBIAS##bt##_descalePerChannel_TDESCALE##dt##_##ta##_##tb##_TA##a##_TB##a##_TC##c(  \
      bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_1d *bias, bsir_memref_1d *descale, bsir_memref_2d *C) {       \
    clear_error();                                                                                                    \
    if (!bias) return fail(BSIR_ERR_NULL, "matmul with bias: null bias descriptor");                                  \
    return matmul_call("matmul_bias_descalePerChannel_" #a "_" #c, BSIR_DT_##a, BSIR_DT_##c, BSIR_DT_##bt, BSIR_DT_##dt, \
                       BSIR_DESCALE_PER_CHANNEL, fa, fb, A, B, bias, descale, C);                                     \
  }                                                                                                                   \
  int32_t _mlir_ciface_matmul_bias_TBIAS##bt##_descalePerTensor_TDESCALE##dt##_##ta##_##tb##_TA##a##_TB##a##_TC##c(   \
      bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_1d *bias, bsir_memref_1d *descale, bsir_memref_2d *C) {       \
    clear_error();                                                                                                    \
    if (!bias) return fail(BSIR_ERR_NULL, "matmul with bias: null bias descriptor");                                  \
    return matmul_call("matmul_bias_descalePerTensor_" #a "_" #c, BSIR_DT_##a, BSIR_DT_##c, BSIR_DT_##bt, BSIR_DT_##dt, \
                       BSIR_DESCALE_PER_TENSOR, fa, fb, A, B, bias, descale, C);                                      \
  }
#define BSIR_DEF_MM_BOTH(a, c, bt, dt) BSIR_MATMUL_TRANSPOSES(BSIR_DEF_MM_BOTH_T, a, c, bt, dt)

BSIR_MATMUL_PLAINSETS(BSIR_DEF_MM_PLAIN)
BSIR_MATMUL_BIASSETS(BSIR_DEF_MM_BIAS)
BSIR_MATMUL_DESCALESETS(BSIR_DEF_MM_DESCALE)
BSIR_MATMUL_TYPESETS(BSIR_DEF_MM_BOTH)

}  // extern "C"
