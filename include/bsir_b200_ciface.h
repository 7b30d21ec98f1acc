/*
 * bsir_b200_ciface.h -- the `_mlir_ciface_*` op-library symbols (layer B1).
 *
 * Names follow the reference's builders: `<op>[_vs|_sv]_<rank>d_<dtype>`
 * (concatVectorOpLibraryCallName,
 * bishengir/lib/Dialect/HIVM/IR/LibraryFunctionOpInterface/LibraryFunctionOpInterfaceImpl.cpp:45-53),
 * `vcast_<src>_to_<dst>_<rank>d_{with_mode,with_temp,with_overflow[_no_size_align]}`
 * (same file :194-235) and `reduce_<kind>[_with_index_{left,right}]_{r,ar,ra}_<dtype>`
 * (bishengir/lib/Template/include/Vector/Reduction/ReductionUtils.h:876-1010).
 * The op/dtype tables below restate what the reference registers in
 * bishengir/lib/Template/lib/Vector/Elementwise/EltWise1D.cpp:1318-1500,
 * lib/Vector/Cast/Cast1D.cpp and lib/Vector/Reduction/Reduce{R,AR,RA}*.cpp.
 *
 * Argument order is the reference's.  `tmp_buf`/`tmp` is accepted and ignored
 * (NULL allowed) except by reduce_*_with_index, which uses it as scratch when
 * it is large enough.  half / bfloat16_t scalars travel as their 16 raw bits.
 * This header is included by bsir_b200.h; do not include it on its own.
 */
#ifndef BSIR_B200_CIFACE_H_
#define BSIR_B200_CIFACE_H_
#ifndef __cplusplus
#include <stdbool.h> /* the sort symbols take the reference's `bool descending` */
#endif

/* The reference's library functions return void; these return a bsir_status in the integer return
 * register, which a caller that declared them void simply does not read (the C calling conventions
 * of x86-64 and AArch64 pass no hidden argument for an int32_t result).  Define BSIR_VOID_ABI before
 * including bsir_b200.h to get the reference's exact prototypes -- the declarations MLIR emits for
 * `llvm.emit_c_interface` callees -- and read failures through bsir_last_status() instead. */
#ifdef BSIR_VOID_ABI
#define BSIR_CIFACE_RET void
#else
#define BSIR_CIFACE_RET int32_t
#endif

/* C type of a scalar argument of element type <tok>. */
#define BSIR_SCALAR_float float
#define BSIR_SCALAR_half uint16_t
#define BSIR_SCALAR_bfloat16_t uint16_t
#define BSIR_SCALAR_int8_t int8_t
#define BSIR_SCALAR_int16_t int16_t
#define BSIR_SCALAR_int32_t int32_t
#define BSIR_SCALAR_int64_t int64_t
#define BSIR_SCALAR_uint8_t uint8_t
#define BSIR_SCALAR_uint16_t uint16_t
#define BSIR_SCALAR_uint32_t uint32_t
#define BSIR_SCALAR_uint64_t uint64_t
#define BSIR_SCALAR_bool uint8_t

/* bsir_dtype of element type <tok>. */
#define BSIR_DT_float BSIR_F32
#define BSIR_DT_half BSIR_F16
#define BSIR_DT_bfloat16_t BSIR_BF16
#define BSIR_DT_int8_t BSIR_I8
#define BSIR_DT_int16_t BSIR_I16
#define BSIR_DT_int32_t BSIR_I32
#define BSIR_DT_int64_t BSIR_I64
#define BSIR_DT_uint8_t BSIR_U8
#define BSIR_DT_uint16_t BSIR_U16
#define BSIR_DT_uint32_t BSIR_U32
#define BSIR_DT_uint64_t BSIR_U64
#define BSIR_DT_bool BSIR_BOOL

/* dtype lists: X(op, fn, rank, tok) */
#define BSIR_TYPES_ARITH(X, op, fn, rank) X(op, fn, rank, int16_t) X(op, fn, rank, int32_t) X(op, fn, rank, half) X(op, fn, rank, float)
#define BSIR_TYPES_FLOAT(X, op, fn, rank) X(op, fn, rank, half) X(op, fn, rank, float)
#define BSIR_TYPES_RELU(X, op, fn, rank) X(op, fn, rank, half) X(op, fn, rank, float) X(op, fn, rank, int32_t)
#define BSIR_TYPES_SHIFT(X, op, fn, rank) X(op, fn, rank, int16_t) X(op, fn, rank, int32_t) X(op, fn, rank, uint16_t) X(op, fn, rank, uint32_t)
#define BSIR_TYPES_INTS(X, op, fn, rank)                                                          \
  X(op, fn, rank, bool) X(op, fn, rank, int8_t) X(op, fn, rank, int16_t) X(op, fn, rank, int32_t) \
  X(op, fn, rank, int64_t) X(op, fn, rank, uint8_t) X(op, fn, rank, uint16_t)                     \
  X(op, fn, rank, uint32_t) X(op, fn, rank, uint64_t)
#define BSIR_TYPES_BITS(X, op, fn, rank) \
  BSIR_TYPES_INTS(X, op, fn, rank) X(op, fn, rank, half) X(op, fn, rank, bfloat16_t) X(op, fn, rank, float)

/* vector-vector: (src0, src1, dst, tmp_buf) */
#define BSIR_FOREACH_ELTWISE_VV(X, rank)                   \
  BSIR_TYPES_ARITH(X, vadd, BSIR_BINARY_ADD, rank)         \
  BSIR_TYPES_ARITH(X, vsub, BSIR_BINARY_SUB, rank)         \
  BSIR_TYPES_ARITH(X, vmul, BSIR_BINARY_MUL, rank)         \
  BSIR_TYPES_FLOAT(X, vdiv, BSIR_BINARY_DIV, rank)         \
  BSIR_TYPES_ARITH(X, vmax, BSIR_BINARY_MAX_SIGNED, rank)  \
  BSIR_TYPES_ARITH(X, vmin, BSIR_BINARY_MIN_SIGNED, rank)  \
  BSIR_TYPES_BITS(X, vand, BSIR_BINARY_VAND, rank)         \
  BSIR_TYPES_BITS(X, vor, BSIR_BINARY_VOR, rank)           \
  BSIR_TYPES_INTS(X, vxor, BSIR_BINARY_VXOR, rank)
/* vector-scalar: (src0, scalar, dst, tmp_buf) -> symbol <op>_vs_<rank>d_<tok> */
#define BSIR_FOREACH_ELTWISE_VS(X, rank)                   \
  BSIR_TYPES_ARITH(X, vadds, BSIR_BINARY_ADD, rank)        \
  BSIR_TYPES_ARITH(X, vmuls, BSIR_BINARY_MUL, rank)        \
  BSIR_TYPES_ARITH(X, vmaxs, BSIR_BINARY_MAX_SIGNED, rank) \
  BSIR_TYPES_ARITH(X, vmins, BSIR_BINARY_MIN_SIGNED, rank) \
  BSIR_TYPES_ARITH(X, vsub, BSIR_BINARY_SUB, rank)         \
  BSIR_TYPES_FLOAT(X, vdiv, BSIR_BINARY_DIV, rank)         \
  BSIR_TYPES_SHIFT(X, vshls, BSIR_BINARY_SHLI, rank)       \
  BSIR_TYPES_SHIFT(X, vshrs, BSIR_BINARY_SHRSI, rank)
/* scalar-vector: (scalar, src1, dst, tmp_buf) -> symbol <op>_sv_<rank>d_<tok> */
#define BSIR_FOREACH_ELTWISE_SV(X, rank)           \
  BSIR_TYPES_ARITH(X, vsub, BSIR_BINARY_SUB, rank) \
  BSIR_TYPES_FLOAT(X, vdiv, BSIR_BINARY_DIV, rank)
/* unary: (src0, dst, tmp_buf) */
#define BSIR_FOREACH_ELTWISE_V(X, rank)               \
  BSIR_TYPES_FLOAT(X, vabs, BSIR_UNARY_ABS, rank)     \
  BSIR_TYPES_FLOAT(X, vexp, BSIR_UNARY_EXP, rank)     \
  BSIR_TYPES_FLOAT(X, vln, BSIR_UNARY_LOG, rank)      \
  BSIR_TYPES_FLOAT(X, vsqrt, BSIR_UNARY_SQRT, rank)   \
  BSIR_TYPES_FLOAT(X, vrsqrt, BSIR_UNARY_RSQRT, rank) \
  BSIR_TYPES_FLOAT(X, vrec, BSIR_UNARY_REC, rank)     \
  BSIR_TYPES_RELU(X, vrelu, BSIR_UNARY_RELU, rank)    \
  BSIR_TYPES_BITS(X, vnot, BSIR_UNARY_VNOT, rank)

/* casts with a runtime CastMode: X(src_tok, dst_tok, rank) */
#define BSIR_FOREACH_CAST_WITH_MODE(X, rank)                                                  \
  X(float, float, rank) X(float, half, rank) X(float, bfloat16_t, rank) X(float, int64_t, rank) \
  X(float, int32_t, rank) X(float, int16_t, rank) X(float, int8_t, rank) X(half, float, rank)   \
  X(half, int32_t, rank) X(half, int16_t, rank) X(half, int8_t, rank) X(half, uint8_t, rank)    \
  X(bfloat16_t, float, rank) X(bfloat16_t, int32_t, rank) X(uint8_t, half, rank)                \
  X(int8_t, half, rank) X(int16_t, half, rank) X(int16_t, float, rank) X(int32_t, float, rank)  \
  X(int32_t, int64_t, rank) X(int32_t, int16_t, rank) X(int64_t, int32_t, rank)                 \
  X(int64_t, float, rank)
/* narrowing integer casts that wrap (round_mode = truncwithoverflow) */
#define BSIR_FOREACH_CAST_WITH_OVERFLOW(X, rank) \
  X(int32_t, int8_t, rank) X(int16_t, int8_t, rank) X(int32_t, int16_t, rank) X(int64_t, int32_t, rank)
/* casts from bool / uint8 that take a temp buffer */
#define BSIR_FOREACH_CAST_WITH_TEMP(X, rank)                                                    \
  X(bool, half, rank) X(bool, float, rank) X(bool, bfloat16_t, rank) X(bool, int16_t, rank)     \
  X(bool, int32_t, rank) X(bool, uint16_t, rank) X(bool, uint32_t, rank) X(uint8_t, float, rank) \
  X(uint8_t, bfloat16_t, rank) X(uint8_t, int16_t, rank) X(uint8_t, int32_t, rank)              \
  X(uint8_t, uint16_t, rank) X(uint8_t, uint32_t, rank)

/* reductions: X(name, kind, tok) */
#define BSIR_FOREACH_REDUCE(X)                                                                 \
  X(reduce_sum, BSIR_REDUCE_SUM, int16_t) X(reduce_sum, BSIR_REDUCE_SUM, int32_t)              \
  X(reduce_sum, BSIR_REDUCE_SUM, half) X(reduce_sum, BSIR_REDUCE_SUM, float)                   \
  X(reduce_prod, BSIR_REDUCE_PROD, int16_t) X(reduce_prod, BSIR_REDUCE_PROD, int32_t)          \
  X(reduce_prod, BSIR_REDUCE_PROD, half) X(reduce_prod, BSIR_REDUCE_PROD, float)               \
  X(reduce_max, BSIR_REDUCE_MAX, int16_t) X(reduce_max, BSIR_REDUCE_MAX, int32_t)              \
  X(reduce_max, BSIR_REDUCE_MAX, half) X(reduce_max, BSIR_REDUCE_MAX, float)                   \
  X(reduce_min, BSIR_REDUCE_MIN, int16_t) X(reduce_min, BSIR_REDUCE_MIN, int32_t)              \
  X(reduce_min, BSIR_REDUCE_MIN, half) X(reduce_min, BSIR_REDUCE_MIN, float)                   \
  X(reduce_xori, BSIR_REDUCE_XORI, int8_t) X(reduce_xori, BSIR_REDUCE_XORI, int16_t)           \
  X(reduce_xori, BSIR_REDUCE_XORI, int32_t) X(reduce_xori, BSIR_REDUCE_XORI, int64_t)          \
  X(reduce_ori, BSIR_REDUCE_ORI, int8_t) X(reduce_ori, BSIR_REDUCE_ORI, int16_t)               \
  X(reduce_ori, BSIR_REDUCE_ORI, int32_t) X(reduce_ori, BSIR_REDUCE_ORI, int64_t)              \
  X(reduce_ori, BSIR_REDUCE_ORI, uint8_t) X(reduce_ori, BSIR_REDUCE_ORI, uint16_t)             \
  X(reduce_ori, BSIR_REDUCE_ORI, uint32_t) X(reduce_ori, BSIR_REDUCE_ORI, uint64_t)            \
  X(reduce_andi, BSIR_REDUCE_ANDI, int8_t) X(reduce_andi, BSIR_REDUCE_ANDI, int16_t)           \
  X(reduce_andi, BSIR_REDUCE_ANDI, int32_t) X(reduce_andi, BSIR_REDUCE_ANDI, int64_t)          \
  X(reduce_andi, BSIR_REDUCE_ANDI, uint8_t) X(reduce_andi, BSIR_REDUCE_ANDI, uint16_t)         \
  X(reduce_andi, BSIR_REDUCE_ANDI, uint32_t) X(reduce_andi, BSIR_REDUCE_ANDI, uint64_t)
/* X(name, kind, tie_break_left, tok) */
#define BSIR_FOREACH_REDUCE_WITH_INDEX(X)                                                        \
  X(reduce_max_with_index_left, BSIR_RWI_MAX, 1, half) X(reduce_max_with_index_left, BSIR_RWI_MAX, 1, float)   \
  X(reduce_max_with_index_right, BSIR_RWI_MAX, 0, half) X(reduce_max_with_index_right, BSIR_RWI_MAX, 0, float) \
  X(reduce_min_with_index_left, BSIR_RWI_MIN, 1, half) X(reduce_min_with_index_left, BSIR_RWI_MIN, 1, float)   \
  X(reduce_min_with_index_right, BSIR_RWI_MIN, 0, half) X(reduce_min_with_index_right, BSIR_RWI_MIN, 0, float)

/* ------------------------------ declarations ----------------------------- */
#define BSIR_MEMREF_T(rank) bsir_memref_##rank##d

#define BSIR_DECL_VV(op, fn, rank, tok)                                                   \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##op##_##rank##d_##tok(BSIR_MEMREF_T(rank) *src0,         \
      BSIR_MEMREF_T(rank) *src1, BSIR_MEMREF_T(rank) *dst, bsir_memref_1d *tmp_buf);
#define BSIR_DECL_VS(op, fn, rank, tok)                                                   \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##op##_vs_##rank##d_##tok(BSIR_MEMREF_T(rank) *src0,      \
      BSIR_SCALAR_##tok scalar, BSIR_MEMREF_T(rank) *dst, bsir_memref_1d *tmp_buf);
#define BSIR_DECL_SV(op, fn, rank, tok)                                                   \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##op##_sv_##rank##d_##tok(BSIR_SCALAR_##tok scalar,       \
      BSIR_MEMREF_T(rank) *src1, BSIR_MEMREF_T(rank) *dst, bsir_memref_1d *tmp_buf);
#define BSIR_DECL_V(op, fn, rank, tok)                                                    \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##op##_##rank##d_##tok(BSIR_MEMREF_T(rank) *src0,         \
      BSIR_MEMREF_T(rank) *dst, bsir_memref_1d *tmp_buf);
#define BSIR_DECL_CAST_MODE(s, d, rank)                                                   \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_vcast_##s##_to_##d##_##rank##d_with_mode(                 \
      BSIR_MEMREF_T(rank) *src, BSIR_MEMREF_T(rank) *dst, uint32_t cast_mode);
#define BSIR_DECL_CAST_OVERFLOW(s, d, rank)                                               \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_vcast_##s##_to_##d##_##rank##d_with_overflow(             \
      BSIR_MEMREF_T(rank) *src, BSIR_MEMREF_T(rank) *dst, bsir_memref_1d *tmp,            \
      uint32_t cast_mode);                                                                \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_vcast_##s##_to_##d##_##rank##d_with_overflow_no_size_align( \
      BSIR_MEMREF_T(rank) *src, BSIR_MEMREF_T(rank) *dst, bsir_memref_1d *tmp,            \
      uint32_t cast_mode);
#define BSIR_DECL_CAST_TEMP(s, d, rank)                                                   \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_vcast_##s##_to_##d##_##rank##d_with_temp(                 \
      BSIR_MEMREF_T(rank) *src, BSIR_MEMREF_T(rank) *dst, bsir_memref_1d *temp,           \
      uint32_t cast_mode);
/* (a, r) -> (a, 1): src/dst 2-D; (r) -> (1): 1-D; (r, a) -> (1, a): 2-D */
#define BSIR_DECL_REDUCE(name, kind, tok)                                                 \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##name##_ar_##tok(bsir_memref_2d *src0, bsir_memref_2d *dst, \
      bsir_memref_1d *tmp_buf, BSIR_SCALAR_##tok initvalue);                              \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##name##_r_##tok(bsir_memref_1d *src0, bsir_memref_1d *dst, \
      bsir_memref_1d *tmp_buf, BSIR_SCALAR_##tok initvalue);                              \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##name##_ra_##tok(bsir_memref_2d *src0, bsir_memref_2d *dst, \
      bsir_memref_1d *tmp_buf, BSIR_SCALAR_##tok initvalue);
#define BSIR_DECL_REDUCE_WITH_INDEX(name, kind, left, tok)                                \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##name##_ar_##tok(bsir_memref_2d *src0,                   \
      bsir_memref_2d *dst_value, bsir_memref_2d *dst_index, bsir_memref_1d *tmp_buf,      \
      BSIR_SCALAR_##tok initvalue);                                                       \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##name##_r_##tok(bsir_memref_1d *src0,                    \
      bsir_memref_1d *dst_value, bsir_memref_1d *dst_index, bsir_memref_1d *tmp_buf,      \
      BSIR_SCALAR_##tok initvalue);

BSIR_FOREACH_ELTWISE_VV(BSIR_DECL_VV, 1)
BSIR_FOREACH_ELTWISE_VV(BSIR_DECL_VV, 2)
BSIR_FOREACH_ELTWISE_VV(BSIR_DECL_VV, 3)
BSIR_FOREACH_ELTWISE_VS(BSIR_DECL_VS, 1)
BSIR_FOREACH_ELTWISE_VS(BSIR_DECL_VS, 2)
BSIR_FOREACH_ELTWISE_VS(BSIR_DECL_VS, 3)
BSIR_FOREACH_ELTWISE_SV(BSIR_DECL_SV, 1)
BSIR_FOREACH_ELTWISE_SV(BSIR_DECL_SV, 2)
BSIR_FOREACH_ELTWISE_SV(BSIR_DECL_SV, 3)
BSIR_FOREACH_ELTWISE_V(BSIR_DECL_V, 1)
BSIR_FOREACH_ELTWISE_V(BSIR_DECL_V, 2)
BSIR_FOREACH_ELTWISE_V(BSIR_DECL_V, 3)
BSIR_FOREACH_CAST_WITH_MODE(BSIR_DECL_CAST_MODE, 1)
BSIR_FOREACH_CAST_WITH_MODE(BSIR_DECL_CAST_MODE, 2)
BSIR_FOREACH_CAST_WITH_OVERFLOW(BSIR_DECL_CAST_OVERFLOW, 1)
BSIR_FOREACH_CAST_WITH_OVERFLOW(BSIR_DECL_CAST_OVERFLOW, 2)
BSIR_FOREACH_CAST_WITH_TEMP(BSIR_DECL_CAST_TEMP, 1)
BSIR_FOREACH_CAST_WITH_TEMP(BSIR_DECL_CAST_TEMP, 2)
BSIR_FOREACH_REDUCE(BSIR_DECL_REDUCE)
BSIR_FOREACH_REDUCE_WITH_INDEX(BSIR_DECL_REDUCE_WITH_INDEX)

/* Library symbols of the further HIVM vector ops (declarations in bishengir/lib/Template/include/Vector/:
 * Cumulative/CumsumUtils.h:31-49 and CumprodUtils.h, Sort/SortUtils.h:45-66, Interleave/InterleaveUtils.h:47-58,
 * Deinterleave/DeinterleaveUtils.h:36-45, Arange/ArangeUtils.h:26-49, Transpose/TransposeUtils.h:87-120,
 * Gather/GatherUtils.h:48-54; registered type lists in the matching lib/Template/lib/Vector .cpp files).
 *   cumsum / cumprod _ra_<t>  (src [r, a], dst): running sum / product along the first axis; _ara_ (3-D [a, r, a]):
 *       along the middle axis; _reverse_ from the far end
 *   sort_1d_<t> (src, dst, tmp, descending), sort_with_index_1d_<t> (src, dst, index, tmp, descending)
 *   interleave_1d_<t> (src0, src1, dst, temp); deinterleave_channel_{0,1}_from_2_channels_1d_<t> (src, dst),
 *       deinterleave_channel_0_from_n_channels_{1,2}d_<t> (n = src length / dst length)
 *   arange_{1,2,3}d_<t> (dst, offset, stride...); transpose_2d_with_last_axis_<t> (dst = src^T),
 *       transpose_3d_with_last_axis_<t> ((a, b, c) -> (c, b, a)), transpose_3d_without_last_axis_<t> ((a, b, c) -> (b, a, c))
 *   gather_1d_<t> (src, indices, dst, tmp): dst[i] = src[indices[i]]
 * Scratch arguments (tmp) are accepted and unused. */
#define BSIR_TYPES_CUM(X, ...) X(int16_t, __VA_ARGS__) X(int32_t, __VA_ARGS__) X(half, __VA_ARGS__) X(float, __VA_ARGS__)
#define BSIR_TYPES_SORT(X) X(half) X(float)
#define BSIR_TYPES_LEAVE(X, ...)                                                                     \
  X(half, __VA_ARGS__) X(bfloat16_t, __VA_ARGS__) X(float, __VA_ARGS__) X(int16_t, __VA_ARGS__)     \
  X(int32_t, __VA_ARGS__) X(uint16_t, __VA_ARGS__) X(uint32_t, __VA_ARGS__)
#define BSIR_TYPES_ARANGE(X) X(int16_t) X(int32_t) X(half) X(float) X(int64_t)
#define BSIR_TYPES_TRANSPOSE(X)                                                                      \
  X(uint8_t) X(int8_t) X(uint16_t) X(int16_t) X(half) X(bfloat16_t) X(uint32_t) X(int32_t) X(float)
#define BSIR_TYPES_GATHER(X) X(uint16_t) X(uint32_t) X(int16_t) X(int32_t) X(half) X(float) X(bfloat16_t)

#define BSIR_DECL_CUM(tok, op)                                                                                       \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##op##_ra_##tok(bsir_memref_2d *src, bsir_memref_2d *dst);                   \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##op##_ra_reverse_##tok(bsir_memref_2d *src, bsir_memref_2d *dst);           \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##op##_ara_##tok(bsir_memref_3d *src, bsir_memref_3d *dst);                  \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_##op##_ara_reverse_##tok(bsir_memref_3d *src, bsir_memref_3d *dst);
BSIR_TYPES_CUM(BSIR_DECL_CUM, cumsum)
BSIR_TYPES_CUM(BSIR_DECL_CUM, cumprod)
#define BSIR_DECL_SORT(tok)                                                                                          \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_sort_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *dst, bsir_memref_1d *tmp, bool descending); \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_sort_with_index_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *dst, bsir_memref_1d *index, \
                                                                 bsir_memref_1d *tmp, bool descending);
BSIR_TYPES_SORT(BSIR_DECL_SORT)
#define BSIR_DECL_LEAVE(tok, unused)                                                                                 \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_interleave_1d_##tok(bsir_memref_1d *src0, bsir_memref_1d *src1, bsir_memref_1d *dst, bsir_memref_1d *temp); \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_deinterleave_channel_0_from_2_channels_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *dst); \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_deinterleave_channel_1_from_2_channels_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *dst); \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_deinterleave_channel_0_from_n_channels_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *dst); \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_deinterleave_channel_0_from_n_channels_2d_##tok(bsir_memref_2d *src, bsir_memref_2d *dst);
BSIR_TYPES_LEAVE(BSIR_DECL_LEAVE, 0)
#define BSIR_DECL_ARANGE(tok)                                                                                        \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_arange_1d_##tok(bsir_memref_1d *dst, int64_t offset, int64_t stride);        \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_arange_2d_##tok(bsir_memref_2d *dst, int64_t offset, int64_t stride0, int64_t stride1); \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_arange_3d_##tok(bsir_memref_3d *dst, int64_t offset, int64_t stride0, int64_t stride1, int64_t stride2);
BSIR_TYPES_ARANGE(BSIR_DECL_ARANGE)
#define BSIR_DECL_TRANSPOSE(tok)                                                                                     \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_transpose_2d_with_last_axis_##tok(bsir_memref_2d *src, bsir_memref_2d *dst); \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_transpose_3d_with_last_axis_##tok(bsir_memref_3d *src, bsir_memref_3d *dst); \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_transpose_3d_without_last_axis_##tok(bsir_memref_3d *src, bsir_memref_3d *dst);
BSIR_TYPES_TRANSPOSE(BSIR_DECL_TRANSPOSE)
#define BSIR_DECL_GATHER(tok)                                                                                        \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_gather_1d_##tok(bsir_memref_1d *src, bsir_memref_1d *indices, bsir_memref_1d *dst, bsir_memref_1d *tmp);
BSIR_TYPES_GATHER(BSIR_DECL_GATHER)

/* GEMM library symbols.  Names as the reference's name builder spells them
 * (bishengir/lib/Dialect/HIVM/IR/LibraryFunctionOpInterface/LibraryFunctionOpInterfaceImpl.cpp:470-505,
 * checked by bishengir/test/Conversion/HIVMToStandard/HIVMToStandard/matmul.mlir:13-55):
 *   matmul_{X,}bias[_TBIAS<t>]_{Xdescale | descalePerChannel_TDESCALE<t> | descalePerTensor_TDESCALE<t>}
 *         _{X,}transposeA_{X,}transposeB_TA<t>_TB<t>_TC<t>
 * with the operands in the op's order: A, B, [bias], [descale], C.  The reference's device library registers the
 * eight Xbias_Xdescale variants of half x half -> half and int8 x int8 -> half
 * (bishengir/lib/Template/lib/Cube/GlobalMmad.cpp:176-187); here every bias / descale form exists for those two
 * type sets and for bfloat16_t.  C = descale * (A x B + bias); int8 inputs accumulate in int32 (bias int32_t,
 * descale float or half), 16-bit float inputs in f32 (bias and descale of the operand type or float); the result
 * is rounded to nearest even, half saturating at its range.
 * X(ta, tb): transposeA / transposeB tokens; T(a, c): operand and result element types. */
#define BSIR_MATMUL_TRANSPOSES(X, ...)                                                              \
  X(XtransposeA, XtransposeB, 0, 0, __VA_ARGS__) X(transposeA, XtransposeB, 1, 0, __VA_ARGS__)      \
  X(XtransposeA, transposeB, 0, 1, __VA_ARGS__) X(transposeA, transposeB, 1, 1, __VA_ARGS__)
/* type sets: (TA = TB, TC, bias type) x the descale types offered */
#define BSIR_MATMUL_TYPESETS(X)                                                                     \
  X(half, half, half, half) X(half, half, half, float) X(half, half, float, half) X(half, half, float, float) \
  X(bfloat16_t, bfloat16_t, bfloat16_t, bfloat16_t) X(bfloat16_t, bfloat16_t, bfloat16_t, float)    \
  X(bfloat16_t, bfloat16_t, float, bfloat16_t) X(bfloat16_t, bfloat16_t, float, float)              \
  X(int8_t, half, int32_t, float) X(int8_t, half, int32_t, half)
#define BSIR_MATMUL_PLAINSETS(X) X(half, half) X(bfloat16_t, bfloat16_t) X(int8_t, half)
#define BSIR_MATMUL_BIASSETS(X) X(half, half, half) X(half, half, float) X(bfloat16_t, bfloat16_t, bfloat16_t) X(bfloat16_t, bfloat16_t, float) X(int8_t, half, int32_t)
#define BSIR_MATMUL_DESCALESETS(X) X(half, half, half) X(half, half, float) X(bfloat16_t, bfloat16_t, bfloat16_t) X(bfloat16_t, bfloat16_t, float) X(int8_t, half, float) X(int8_t, half, half)

#define BSIR_DECL_MM_PLAIN_T(ta, tb, fa, fb, a, c)                                                  \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_matmul_Xbias_Xdescale_##ta##_##tb##_TA##a##_TB##a##_TC##c(  \
      bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_2d *C);
#define BSIR_DECL_MM_PLAIN(a, c) BSIR_MATMUL_TRANSPOSES(BSIR_DECL_MM_PLAIN_T, a, c)
#define BSIR_DECL_MM_BIAS_T(ta, tb, fa, fb, a, c, bt)                                               \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_matmul_bias_TBIAS##bt##_Xdescale_##ta##_##tb##_TA##a##_TB##a##_TC##c( \
      bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_1d *bias, bsir_memref_2d *C);
#define BSIR_DECL_MM_BIAS(a, c, bt) BSIR_MATMUL_TRANSPOSES(BSIR_DECL_MM_BIAS_T, a, c, bt)
#define BSIR_DECL_MM_DESCALE_T(ta, tb, fa, fb, a, c, dt)                                            \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_matmul_Xbias_descalePerChannel_TDESCALE##dt##_##ta##_##tb##_TA##a##_TB##a##_TC##c( \
      bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_1d *descale, bsir_memref_2d *C);            \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_matmul_Xbias_descalePerTensor_TDESCALE##dt##_##ta##_##tb##_TA##a##_TB##a##_TC##c( \
      bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_1d *descale, bsir_memref_2d *C);
#define BSIR_DECL_MM_DESCALE(a, c, dt) BSIR_MATMUL_TRANSPOSES(BSIR_DECL_MM_DESCALE_T, a, c, dt)
#define BSIR_DECL_MM_BOTH_T(ta, tb, fa, fb, a, c, bt, dt)                                           \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_matmul_bias_TBIAS##bt##_descalePerChannel_TDESCALE##dt##_##ta##_##tb##_TA##a##_TB##a##_TC##c( \
      bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_1d *bias, bsir_memref_1d *descale, bsir_memref_2d *C); \
  BSIR_API BSIR_CIFACE_RET _mlir_ciface_matmul_bias_TBIAS##bt##_descalePerTensor_TDESCALE##dt##_##ta##_##tb##_TA##a##_TB##a##_TC##c( \
      bsir_memref_2d *A, bsir_memref_2d *B, bsir_memref_1d *bias, bsir_memref_1d *descale, bsir_memref_2d *C);
#define BSIR_DECL_MM_BOTH(a, c, bt, dt) BSIR_MATMUL_TRANSPOSES(BSIR_DECL_MM_BOTH_T, a, c, bt, dt)

BSIR_MATMUL_PLAINSETS(BSIR_DECL_MM_PLAIN)
BSIR_MATMUL_BIASSETS(BSIR_DECL_MM_BIAS)
BSIR_MATMUL_DESCALESETS(BSIR_DECL_MM_DESCALE)
BSIR_MATMUL_TYPESETS(BSIR_DECL_MM_BOTH)

#endif /* BSIR_B200_CIFACE_H_ */
