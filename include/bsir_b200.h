/*
 * bsir_b200.h -- C ABI of the B200 (sm_100a) execution backend for the operator
 * set of BiShengIR's HFusion / HIVM dialects.
 *
 * Three layers, all plain C (pointers + sizes, no C++/torch types):
 *
 *  B1  op-library ABI: the `_mlir_ciface_<op>_<rank>d_<dtype>` symbols that the
 *      reference's HIVMToStandard conversion calls, taking pointers to MLIR
 *      memref descriptors.  Reference declaration macros:
 *      bishengir/lib/Template/include/Vector/VecUtils.h:971-1023 (elementwise),
 *      bishengir/lib/Template/include/Vector/Cast/CastUtils.h:229-301 (vcast),
 *      bishengir/lib/Template/include/Vector/Reduction/ReductionUtils.h:876-1010.
 *      Descriptor: bishengir/lib/Template/include/Utils.h:72-78.
 *      Differences from the reference symbols: (1) the buffers are device (HBM)
 *      pointers, (2) the functions return an int32 status instead of void, and
 *      (3) they enqueue on the stream set with bsir_set_stream() for the
 *      calling thread (default: the legacy default stream), exactly as the
 *      reference enqueues on the ACL stream of its launch.
 *
 *  B2  compiled-kernel ABI: bsir_kernel_register() + bsir_launch(), the
 *      equivalent of `rtFunctionRegister` + `rtKernelLaunch(stub, blockDim,
 *      args, argsSize, smDesc, stream)` used by
 *      bishengir/test/Integration/HIVM/VecAdd/main.cpp:96-113,169-171.
 *      A registered kernel = one op (or fused pattern) + its static shape, the
 *      thing `bishengir-compile` turns an .mlir file into; args are one bare
 *      device pointer per memref argument, inputs first, then outputs.
 *
 *  B3  typed entry points (bsir_<op>): pointers + sizes/strides + attributes,
 *      used by B1/B2 internally and callable directly.
 *
 * Every function is asynchronous with respect to the host (returns after the
 * enqueue), allocates nothing per call, and never aborts: errors come back as
 * a negative bsir_status and bsir_last_error() has the text.
 */
#ifndef BSIR_B200_H_
#define BSIR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSIR_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* status                                                                    */
/* ------------------------------------------------------------------------ */
typedef enum {
  BSIR_OK = 0,
  BSIR_ERR_NULL = -1,        /* a required pointer is null                   */
  BSIR_ERR_SHAPE = -2,       /* negative/mismatched sizes                    */
  BSIR_ERR_STRIDE = -3,      /* layout the kernel cannot address             */
  BSIR_ERR_DTYPE = -4,       /* dtype not legal for this op                  */
  BSIR_ERR_ATTR = -5,        /* illegal attribute / attribute-dtype combo    */
  BSIR_ERR_ALIGN = -6,       /* pointer alignment below the element size     */
  BSIR_ERR_LAUNCH = -7,      /* CUDA reported an error at enqueue            */
  BSIR_ERR_UNKNOWN_KERNEL = -8,
  BSIR_ERR_ARGS = -9,        /* wrong args_size for bsir_launch              */
  BSIR_ERR_WORKSPACE = -10,  /* scratch too small / could not be set up      */
  BSIR_ERR_UNSUPPORTED = -11,
  BSIR_ERR_DEVICE = -12      /* a device-side bounded wait gave up           */
} bsir_status;

BSIR_API const char *bsir_status_string(int32_t status);
/* Text of the last error raised on the calling thread ("" if none). */
BSIR_API const char *bsir_last_error(void);
/* Status of the calling thread's most recent library call (0 = ok): for callers that use the void
 * prototypes of BSIR_VOID_ABI and cannot see the return value. */
BSIR_API int32_t bsir_last_status(void);
BSIR_API const char *bsir_version(void);

/* Stream used by the B1 symbols and by bsir_launch(..., stream == NULL) on the
 * calling thread.  `stream` is a cudaStream_t; NULL = legacy default stream. */
BSIR_API int32_t bsir_set_stream(void *stream);
BSIR_API void *bsir_get_stream(void);

/* ------------------------------------------------------------------------ */
/* element types (names as spelled in library symbols:                      */
/* bishengir/lib/Dialect/HIVM/IR/LibraryFunctionOpInterface/                 */
/* LibraryFunctionOpInterfaceImpl.cpp:45-53)                                 */
/* ------------------------------------------------------------------------ */
typedef enum {
  BSIR_F32 = 0,  /* float       */
  BSIR_F16 = 1,  /* half        */
  BSIR_BF16 = 2, /* bfloat16_t  */
  BSIR_I8 = 3,   /* int8_t      */
  BSIR_I16 = 4,  /* int16_t     */
  BSIR_I32 = 5,  /* int32_t     */
  BSIR_I64 = 6,  /* int64_t     */
  BSIR_U8 = 7,   /* uint8_t     */
  BSIR_U16 = 8,  /* uint16_t    */
  BSIR_U32 = 9,  /* uint32_t    */
  BSIR_U64 = 10, /* uint64_t    */
  BSIR_BOOL = 11 /* bool (i1 stored one per byte) */
} bsir_dtype;

BSIR_API int32_t bsir_dtype_size(int32_t dtype);

/* ------------------------------------------------------------------------ */
/* attributes (integer values as in                                          */
/* bishengir/include/bishengir/Dialect/HFusion/IR/HFusionEnums.td)           */
/* ------------------------------------------------------------------------ */
typedef enum { /* hfusion.round_mode, HFusionEnums.td:122-141 */
  BSIR_ROUND_RINT = 0,
  BSIR_ROUND_ROUND = 1,
  BSIR_ROUND_FLOOR = 2,
  BSIR_ROUND_CEIL = 3,
  BSIR_ROUND_TRUNC = 4,
  BSIR_ROUND_ODD = 5,
  BSIR_ROUND_TRUNCWITHOVERFLOW = 6
} bsir_round_mode;

/* CastMode argument of the vcast library symbols
 * (bishengir/lib/Template/include/Vector/Cast/CastUtils.h:30-38). */
typedef enum {
  BSIR_CASTMODE_R = 0, /* rint  */
  BSIR_CASTMODE_A = 1, /* round */
  BSIR_CASTMODE_F = 2, /* floor */
  BSIR_CASTMODE_C = 3, /* ceil  */
  BSIR_CASTMODE_Z = 4, /* trunc */
  BSIR_CASTMODE_O = 5, /* odd   */
  BSIR_CASTMODE_OVERFLOW = 6
} bsir_cast_mode;

/* How a float->int (or narrowing int) cast treats out-of-range values. */
typedef enum {
  BSIR_OVERFLOW_WRAP = 0,     /* enable_saturate = false: round, then keep the
                                 low bits (two's complement wrap)            */
  BSIR_OVERFLOW_SATURATE = 1, /* enable_saturate = true: clamp to the range of
                                 the destination; NaN -> 0                   */
  /* Device-path rewrites of the reference for f32 -> i8, kept as named
   * variants (never the default):                                          */
  BSIR_OVERFLOW_ASCEND_SATURATE_TRUNC_VIA_F16 = 2, /* Normalize.cpp:3826-3836 */
  BSIR_OVERFLOW_ASCEND_DOUBLE_ROUND_VIA_F16 = 3    /* HIVMDecomposeOp.cpp:101-190 */
} bsir_overflow_mode;

typedef enum { /* hfusion.unary_fn 0..26 (HFusionEnums.td:29-57); 100.. = linalg.unary_fn */
  BSIR_UNARY_RELU = 0, BSIR_UNARY_SQRT = 1, BSIR_UNARY_RSQRT = 2, BSIR_UNARY_REC = 3,
  BSIR_UNARY_VNOT = 4, BSIR_UNARY_TANH = 5, BSIR_UNARY_SIN = 6, BSIR_UNARY_COS = 7,
  BSIR_UNARY_ATAN = 8, BSIR_UNARY_TAN = 9, BSIR_UNARY_ABSI = 10, BSIR_UNARY_ERF = 11,
  BSIR_UNARY_LOG2 = 12, BSIR_UNARY_LOG10 = 13, BSIR_UNARY_LOG1P = 14, BSIR_UNARY_EXP2 = 15,
  BSIR_UNARY_EXPM1 = 16, BSIR_UNARY_ILOGB = 17, BSIR_UNARY_ASIN = 18, BSIR_UNARY_ACOS = 19,
  BSIR_UNARY_ASINH = 20, BSIR_UNARY_ACOSH = 21, BSIR_UNARY_ATANH = 22, BSIR_UNARY_SINH = 23,
  BSIR_UNARY_LGAMMA = 24, BSIR_UNARY_COSH = 25, BSIR_UNARY_NEARBYINT = 26,
  BSIR_UNARY_EXP = 100, BSIR_UNARY_LOG = 101, BSIR_UNARY_ABS = 102, BSIR_UNARY_CEIL = 103,
  BSIR_UNARY_FLOOR = 104, BSIR_UNARY_NEGF = 105, BSIR_UNARY_RECIPROCAL = 106,
  BSIR_UNARY_ROUND = 107, BSIR_UNARY_SQRT_L = 108, BSIR_UNARY_RSQRT_L = 109,
  BSIR_UNARY_SQUARE = 110, BSIR_UNARY_TANH_L = 111, BSIR_UNARY_ERF_L = 112
} bsir_unary_fn;

typedef enum { /* hfusion.binary_fn 0..20 (HFusionEnums.td:62-84); 100.. = linalg.binary_fn */
  BSIR_BINARY_VOR = 0, BSIR_BINARY_VAND = 1, BSIR_BINARY_VXOR = 2, BSIR_BINARY_MINF = 3,
  BSIR_BINARY_MAXF = 4, BSIR_BINARY_POWF = 5, BSIR_BINARY_MOD = 6, BSIR_BINARY_MODUI = 7,
  BSIR_BINARY_SHLI = 8, BSIR_BINARY_SHRSI = 9, BSIR_BINARY_SHRUI = 10, BSIR_BINARY_LDEXP = 11,
  BSIR_BINARY_CEILDIVSI = 12, BSIR_BINARY_CEILDIVUI = 13, BSIR_BINARY_FLOORDIVSI = 14,
  BSIR_BINARY_POWI = 15, BSIR_BINARY_MINNUMF = 16, BSIR_BINARY_MAXNUMF = 17,
  BSIR_BINARY_ATAN2 = 18, BSIR_BINARY_DIVFHP = 19, BSIR_BINARY_COPYSIGN = 20,
  BSIR_BINARY_ADD = 100, BSIR_BINARY_SUB = 101, BSIR_BINARY_MUL = 102, BSIR_BINARY_DIV = 103,
  BSIR_BINARY_DIV_UNSIGNED = 104, BSIR_BINARY_MAX_SIGNED = 105, BSIR_BINARY_MIN_SIGNED = 106,
  BSIR_BINARY_MAX_UNSIGNED = 107, BSIR_BINARY_MIN_UNSIGNED = 108, BSIR_BINARY_POWF_L = 109
} bsir_binary_fn;

typedef enum { /* hfusion.compare_fn */
  BSIR_CMP_VEQ = 0, BSIR_CMP_VNE = 1, BSIR_CMP_VLE = 2, BSIR_CMP_VLT = 3, BSIR_CMP_VGE = 4,
  BSIR_CMP_VGT = 5, BSIR_CMP_VULE = 6, BSIR_CMP_VULT = 7, BSIR_CMP_VUGE = 8, BSIR_CMP_VUGT = 9
} bsir_compare_fn;

typedef enum { /* hivm reduce kinds, HIVMVectorOps.td:1316-1434 */
  BSIR_REDUCE_SUM = 0, BSIR_REDUCE_PROD = 1, BSIR_REDUCE_MAX = 2, BSIR_REDUCE_MIN = 3,
  BSIR_REDUCE_ANY = 4, BSIR_REDUCE_ALL = 5, BSIR_REDUCE_XORI = 6, BSIR_REDUCE_ORI = 7,
  BSIR_REDUCE_ANDI = 8
} bsir_reduce_kind;

typedef enum { /* hfusion.reduce_with_index_kind, HFusionEnums.td:303-311 */
  BSIR_RWI_MIN = 0, BSIR_RWI_MAX = 1, BSIR_RWI_MINUI = 2, BSIR_RWI_MAXUI = 3
} bsir_reduce_with_index_kind;

/* NaN policy of reduce_with_index. */
typedef enum {
  /* What the op's region computes when lowered to loops
   * (HFusionOps.cpp:1506-1523): value = maximumf chain (NaN poisons the value),
   * index moves only on a strict ordered compare, so it stays at the best
   * element seen before the first NaN. */
  BSIR_RWI_NAN_REGION = 0,
  /* Device/Triton rule: the first NaN wins value and index
   * (Normalize.cpp:2688-2777, linalg-to-hfusion.mlir:224-241). */
  BSIR_RWI_NAN_FIRST = 1
} bsir_rwi_nan_mode;

typedef enum { /* #hivm.descale_mode, HIVMAttrs.td:1061-1071 */
  BSIR_DESCALE_NULL = 0, BSIR_DESCALE_PER_CHANNEL = 1, BSIR_DESCALE_PER_TENSOR = 2
} bsir_descale_mode;

/* ------------------------------------------------------------------------ */
/* memref descriptors (MLIR C interface; Template/include/Utils.h:72-78)     */
/* base = aligned + offset (elements); strides in elements                   */
/* ------------------------------------------------------------------------ */
typedef struct { void *allocated; void *aligned; int64_t offset; int64_t sizes[1]; int64_t strides[1]; } bsir_memref_1d;
typedef struct { void *allocated; void *aligned; int64_t offset; int64_t sizes[2]; int64_t strides[2]; } bsir_memref_2d;
typedef struct { void *allocated; void *aligned; int64_t offset; int64_t sizes[3]; int64_t strides[3]; } bsir_memref_3d;

/* ------------------------------------------------------------------------ */
/* B3: typed entry points                                                    */
/* ------------------------------------------------------------------------ */

/* A strided operand of rank <= 3.  stride 0 broadcasts that dimension (the
 * inline `broadcast = [...]` form of HIVM vector ops, HIVMVectorOps.td:55-111).
 * `data` may be NULL for a scalar operand, in which case `scalar_bits` holds
 * the value in the op's element type (low bits). */
typedef struct {
  const void *data;
  int64_t strides[3];
  uint64_t scalar_bits;
} bsir_operand;

/* out = fn(x); elemwise_unary (HFusionNamedStructuredOps.yaml:72-123,
 * bodies HFusionOps.cpp:434-535).  rank in 1..3, sizes[rank..] ignored. */
BSIR_API int32_t bsir_elemwise_unary(int32_t fn, int32_t dtype, int32_t rank, const int64_t *sizes,
                                     const bsir_operand *x, void *out, const int64_t *out_strides,
                                     void *stream);
/* out = fn(a, b); elemwise_binary (yaml:124-190, bodies HFusionOps.cpp:538-639);
 * hivm.hir.vadd/vsub/vmul/vdiv/vmax/vmin/vand/vor/vxor are this with the
 * matching fn (HFusionToHIVM.cpp:327-359). */
BSIR_API int32_t bsir_elemwise_binary(int32_t fn, int32_t dtype, int32_t rank, const int64_t *sizes,
                                      const bsir_operand *a, const bsir_operand *b, void *out,
                                      const int64_t *out_strides, void *stream);
/* out(bool bytes) = a <pred> b; hfusion.compare (HFusionOps.cpp:642-720). */
BSIR_API int32_t bsir_compare(int32_t fn, int32_t dtype, int32_t rank, const int64_t *sizes,
                              const bsir_operand *a, const bsir_operand *b, void *out,
                              const int64_t *out_strides, void *stream);
/* hfusion.elemwise_ternary (yaml:193-272; TernaryFn select = 0, fma = 1, HFusionEnums.td:105-110).  fma is math.fma
 * (HFusionOps.cpp:737-739): out = a * b + c with one rounding, f32 / f16 / bf16; select has its own entry below. */
#define BSIR_TERNARY_SELECT 0
#define BSIR_TERNARY_FMA 1
BSIR_API int32_t bsir_elemwise_ternary(int32_t fn, int32_t dtype, int32_t rank, const int64_t *sizes,
                                       const bsir_operand *a, const bsir_operand *b, const bsir_operand *c,
                                       void *out, const int64_t *out_strides, void *stream);
/* out = cond ? a : b; hfusion.select (HFusionOps.cpp:723-743); cond is bool bytes. */
BSIR_API int32_t bsir_select(int32_t dtype, int32_t rank, const int64_t *sizes,
                             const bsir_operand *cond, const bsir_operand *a, const bsir_operand *b,
                             void *out, const int64_t *out_strides, void *stream);
/* hfusion.cast / hivm.hir.vcast (yaml:373-432, HIVMVectorOps.td:542-635). */
BSIR_API int32_t bsir_cast(int32_t src_dtype, int32_t dst_dtype, int32_t round_mode,
                           int32_t overflow_mode, int32_t rank, const int64_t *sizes,
                           const void *src, const int64_t *src_strides, void *dst,
                           const int64_t *dst_strides, void *stream);
/* hivm.hir.load/store/copy (HIVMDMAOps.td:62-273): identity copy. */
BSIR_API int32_t bsir_copy(int32_t dtype, int32_t rank, const int64_t *sizes, const void *src,
                           const int64_t *src_strides, void *dst, const int64_t *dst_strides,
                           void *stream);

/* hivm.hir.load with last-dimension padding (HIVMDMAOps.td:62-155; PadMode values HIVMAttrs.td:388-401).
 * `src_sizes` are the source's extents (rank 1..3); the destination has the same leading extents and
 * `dst_last` elements in the last one.  dst[..., 0:left] = pad, then the source row, then `right` pads;
 * pad = *pad_value (one element of `dtype`, host memory) or the row's first source element.  A padding
 * given as -1 is deduced from dst_last the way the CPU lowering does (ConvertHIVMToUpstream.cpp:1140-1166);
 * destination elements beyond left + n + right keep their contents.  BSIR_PAD_NULL is a plain copy. */
typedef enum bsir_pad_mode { BSIR_PAD_NULL = 0, BSIR_PAD_FIRST_ELEM = 1, BSIR_PAD_VALUE = 2 } bsir_pad_mode;
BSIR_API int32_t bsir_load(int32_t dtype, int32_t rank, const int64_t *src_sizes, const void *src,
                           const int64_t *src_strides, void *dst, const int64_t *dst_strides,
                           int64_t dst_last, int32_t pad_mode, const void *pad_value, int64_t left_pad,
                           int64_t right_pad, void *stream);
/* hivm.hir.store (HIVMDMAOps.td:157-200; AtomicKind values HIVMAttrs.td:792-803).  BSIR_ATOMIC_NONE copies
 * (as the CPU lowering always does, ConvertHIVMToUpstream.cpp:1715); the other kinds combine the
 * destination with the source through device-wide atomics: f32 add/max/min (max/min propagate NaN),
 * f16/bf16 add, 32- and 64-bit integers every kind but CAS/XCHG; other combinations are refused. */
typedef enum bsir_atomic_kind {
  BSIR_ATOMIC_NONE = 0, BSIR_ATOMIC_ADD = 1, BSIR_ATOMIC_MAX = 2, BSIR_ATOMIC_MIN = 3, BSIR_ATOMIC_AND = 4,
  BSIR_ATOMIC_OR = 5, BSIR_ATOMIC_XOR = 6, BSIR_ATOMIC_CAS = 7, BSIR_ATOMIC_XCHG = 8, BSIR_ATOMIC_UMAX = 9,
  BSIR_ATOMIC_UMIN = 10
} bsir_atomic_kind;
BSIR_API int32_t bsir_store(int32_t dtype, int32_t rank, const int64_t *sizes, const void *src,
                            const int64_t *src_strides, void *dst, const int64_t *dst_strides,
                            int32_t atomic_kind, void *stream);

/* linalg.reduce / hivm.hir.vreduce over the last axis of a [rows, cols] view
 * (Reduction.cpp:101-148).  dst is write-only: dst[r] = reduce(identity, src[r,:]).
 * Float sums accumulate in f32 (f16/bf16 inputs are promoted). */
BSIR_API int32_t bsir_reduce_last_axis(int32_t kind, int32_t dtype, int64_t rows, int64_t cols,
                                       const void *src, int64_t src_row_stride, void *dst,
                                       void *stream);
/* Same over the first axis: dst[c] = reduce(src[:, c]). */
BSIR_API int32_t bsir_reduce_first_axis(int32_t kind, int32_t dtype, int64_t rows, int64_t cols,
                                        const void *src, int64_t src_row_stride, void *dst,
                                        void *stream);

/* Bytes of scratch bsir_reduce_with_index needs for this shape (0 = none). */
BSIR_API int64_t bsir_reduce_with_index_workspace_bytes(int64_t rows, int64_t cols);
/* hfusion.reduce_with_index over the last axis (HFusionStructuredOps.td:69-137,
 * region HFusionOps.cpp:1506-1595).  Ties keep the lowest index when
 * tie_break_left != 0, the highest otherwise.  dst_index is int32.
 * `workspace` may be NULL: the library then uses its own scratch (see "library-owned
 * scratch" below).  A caller-provided workspace must be 16-byte aligned, at least
 * bsir_reduce_with_index_workspace_bytes() long and zero-filled once before its first use;
 * every call leaves it zero-filled again.  One that is too small or misaligned is refused
 * with BSIR_ERR_WORKSPACE (the library never swaps in its own scratch behind the caller's
 * back), and two calls that may overlap on the GPU need a workspace each. */
BSIR_API int32_t bsir_reduce_with_index(int32_t kind, int32_t dtype, int32_t tie_break_left,
                                        int32_t nan_mode, int64_t rows, int64_t cols,
                                        const void *src, int64_t src_row_stride, void *dst_value,
                                        int32_t *dst_index, void *workspace,
                                        int64_t workspace_bytes, void *stream);

/* bsir_reduce_with_index for hosts that cannot let the library allocate: no counterpart in the
 * reference (its device library gets `tmp_buf` from the compiler's memory planner).  The scratch is
 * a fixed 512 KiB array inside the library image, so the call never reaches cudaMalloc or cudaFree.
 * Limits: rows <= 4096 and rows x segments <= 31744 (the 256 x 152064 benchmark shape uses 2560);
 * beyond them the call returns BSIR_ERR_WORKSPACE and enqueues nothing.  The first call on a device
 * looks up the array's device address: make it before any stream capture on that device.  All calls
 * share the array; calls whose kernels can overlap on the GPU race and must be ordered by the caller. */
BSIR_API int32_t bsir_reduce_with_index_static(int32_t kind, int32_t dtype, int32_t tie_break_left,
                                               int32_t nan_mode, int64_t rows, int64_t cols,
                                               const void *src, int64_t src_row_stride, void *dst_value,
                                               int32_t *dst_index, void *stream);

/* Fused LAST_AXIS_PBR pattern RMSNorm
 * (test/bishengir-compile/hfusion/compile-rms-norm-fp16-split-n.mlir:13-71):
 * y = cast_rint(gamma32 * (rstd * x32)), rstd = 1 / sqrt(sum(x32^2) * (1/cols) + eps);
 * rstd_out (same dtype as x, may be NULL) = cast_rint(rstd). */
BSIR_API int32_t bsir_rms_norm(int32_t dtype, int64_t rows, int64_t cols, const void *x,
                               int64_t x_row_stride, const void *gamma, float eps, void *y,
                               int64_t y_row_stride, void *rstd_out, void *stream);
/* A chain of elementwise ops with broadcast operands as ONE kernel: what HFusion's op fusion outlines as a
 * PURE_ELEMWISE / ANY_PB function (FusibleHelper.cpp:52-72).  All arithmetic is f32 with a single
 * rounding at each output (the bf16 policy of LegalizeBF16.cpp:243-275 + SimplifyOps.cpp:105-230).
 * The chain is a tape for an accumulator machine with four temporaries:
 *   LOAD    acc = src                 UNARY   acc = fn(acc)            SAVE  tmp[src] = acc
 *   BINARY  acc = fn(acc, src)        RBINARY acc = fn(src, acc)
 * src is an input operand, a temporary or the immediate.  fn is a bsir_unary_fn / bsir_binary_fn that
 * has an f32 form.  Operands and outputs are f32 / f16 / bf16; an output takes the accumulator
 * (tmp = -1) or a temporary.  At most 8 operands, 24 instructions, 4 outputs.
 *   REDUCE  acc = reduce over the row of acc (fn = BSIR_REDUCE_SUM / PROD / MAX / MIN), broadcast back to the row
 * turns the chain into a LAST_AXIS_PBR function (elementwise + broadcast + last-axis reductions, e.g. a whole
 * RMSNorm, softmax or LayerNorm): the threads of a row keep it in registers across the reductions, so every
 * operand is still read once.  Sums associate as a tree, not left to right.  An output with row_stride = 0 is a
 * [rows] vector and takes a value that is uniform along the row (a reduction result and what is computed from
 * it).  Chains with REDUCE exist only as compiled kernels: 16-byte aligned rows of a multiple of 8 columns, at
 * most 8192 columns per temporary-free bf16 chain (less with f32 operands or temporaries: the row must fit the
 * registers of 1024 threads); otherwise BSIR_ERR_UNSUPPORTED. */
typedef enum bsir_chain_operand_kind {
  BSIR_CHAIN_FULL = 0,        /* [rows, cols], row_stride in elements             */
  BSIR_CHAIN_ROW_VECTOR = 1,  /* [cols], the same for every row (linalg.broadcast dimensions = [0]) */
  BSIR_CHAIN_COL_VECTOR = 2,  /* [rows], one value per row (linalg.broadcast dimensions = [1])      */
  BSIR_CHAIN_SCALAR = 3       /* one element in device memory                     */
} bsir_chain_operand_kind;
typedef enum bsir_chain_op {
  BSIR_CHAIN_LOAD = 0, BSIR_CHAIN_UNARY = 1, BSIR_CHAIN_BINARY = 2, BSIR_CHAIN_RBINARY = 3, BSIR_CHAIN_SAVE = 4,
  BSIR_CHAIN_REDUCE = 5
} bsir_chain_op;
typedef enum bsir_chain_src { BSIR_CHAIN_SRC_OPERAND = 0, BSIR_CHAIN_SRC_TMP = 1, BSIR_CHAIN_SRC_IMM = 2 } bsir_chain_src;
typedef struct bsir_chain_operand { const void *data; int64_t row_stride; int32_t dtype; int32_t kind; } bsir_chain_operand;
typedef struct bsir_chain_instr { int32_t op; int32_t fn; int32_t src_kind; int32_t src; float imm; } bsir_chain_instr;
typedef struct bsir_chain_output { void *data; int64_t row_stride; int32_t dtype; int32_t tmp; } bsir_chain_output;
BSIR_API int32_t bsir_fused_elementwise(int64_t rows, int64_t cols, int32_t n_in, const bsir_chain_operand *ins,
                                        int32_t n_instr, const bsir_chain_instr *tape, int32_t n_out,
                                        const bsir_chain_output *outs, void *stream);
/* How the last bsir_fused_elementwise of this thread ran: 0 nothing was enqueued, 1 the tape interpreter kernel,
 * 2 a kernel compiled for this chain.  By default a chain whose rows are 16-byte aligned multiples of 8 columns
 * is compiled on first use (NVRTC, sm_100a; cached for the life of the process; the first call with a new chain must not sit inside a stream capture) and everything
 * else is interpreted; both give the same bits.  BSIR_CHAIN_JIT=0 always interprets, =1 returns
 * BSIR_ERR_UNSUPPORTED instead of interpreting (no NVRTC in the process, ragged rows). */
BSIR_API int32_t bsir_fused_elementwise_path(void);
/* The CUDA C++ that would be compiled for a chain (data pointers and strides are not read).  flags: bit 0 every
 * tensor is contiguous (flat addressing), bit 1 an output overlaps an operand, bit 2 one block per stretch of a
 * row (the mapping chosen for rows that fill whole blocks) instead of a division per group; for a chain with
 * REDUCE bits 8.. give cols / 8 (the thread geometry depends on the row length; default 512).  Writes at most cap bytes
 * (NUL-terminated) and returns the bytes needed, or a negative bsir_status. */
BSIR_API int64_t bsir_fused_elementwise_source(int32_t n_in, const bsir_chain_operand *ins, int32_t n_instr,
                                               const bsir_chain_instr *tape, int32_t n_out, const bsir_chain_output *outs,
                                               int32_t flags, char *buf, int64_t cap);
/* Compiles that source for sm_100a without touching a device; *cubin_bytes receives the size of the image. */
BSIR_API int32_t bsir_fused_elementwise_compile(int32_t n_in, const bsir_chain_operand *ins, int32_t n_instr,
                                                const bsir_chain_instr *tape, int32_t n_out, const bsir_chain_output *outs,
                                                int32_t flags, int64_t *cubin_bytes);

/* hivm.hir.vcumsum / vcumprod / vcummax / vcummin (HIVMVectorOps.td:1937-2220) over axis 0 or 1 of a [rows, cols]
 * problem: dst[0] = src[0], dst[i] = src[i] (op) dst[i-1] in index order (hivm-lower-to-loops-op.mlir:1558-1599),
 * from the last index backwards with reverse.  f16 / bf16 run in f32 and round once per output; integers wrap
 * in their own width.  propagate_nan (cummax / cummin on floats): NaN poisons what follows (maximumf), else a NaN
 * operand is ignored (maxnumf).  dtype: f32, f16, bf16, i8, i16, i32, i64.  The scan is sequential along its axis
 * (float sums do not associate), so it is fast when the other axis is long. */
typedef enum { BSIR_CUM_SUM = 0, BSIR_CUM_PROD = 1, BSIR_CUM_MAX = 2, BSIR_CUM_MIN = 3 } bsir_cum_kind;
BSIR_API int32_t bsir_cumulative(int32_t kind, int32_t dtype, int32_t axis, int32_t reverse, int32_t propagate_nan,
                                 int64_t rows, int64_t cols, const void *src, int64_t src_row_stride, void *dst,
                                 int64_t dst_row_stride, void *stream);

/* hivm.hir.vgather (HIVMVectorOps.td:1834-1883) on contiguous [outer, axis, inner] tensors:
 * dst[o][j][k] = src[o][indices[o][j][k]][k]; src is [outer, src_axis, inner], indices and dst are
 * [outer, dst_axis, inner].  index_dtype: BSIR_I16 / I32 (the op's types) or I64.  An index outside
 * [0, src_axis) leaves its element untouched and sets BSIR_DEVERR_GATHER_INDEX in the device error word
 * (bsir_device_error).  The destination may not overlap the source (BSIR_ERR_UNSUPPORTED). */
BSIR_API int32_t bsir_gather(int32_t dtype, int32_t index_dtype, int64_t outer, int64_t src_axis, int64_t dst_axis,
                             int64_t inner, const void *src, const void *indices, void *dst, void *stream);

/* hivm.hir.varange (HIVMVectorOps.td:1503-1560): dst[i0, i1, i2] = offset + sum_d i_d * strides[d], converted to
 * dtype (i16, i32, i64, f16, f32); rank 1..3; dst_strides NULL = contiguous. */
BSIR_API int32_t bsir_arange(int32_t dtype, int32_t rank, const int64_t *sizes, int64_t offset, const int64_t *strides,
                             void *dst, const int64_t *dst_strides, void *stream);
/* hivm.hir.vinterleave {interleave_channel_nums = channels} (HIVMVectorOps.td:1562-1606):
 * dst[r, channels * i + ch] = srcs[ch][r, i]; sources contiguous [rows, cols], dst contiguous [rows, channels * cols].
 * hivm.hir.vdeinterleave {channel_num} (1612-1660) is the inverse; a NULL destination skips its channel (the
 * op's CHANNEL_0 / CHANNEL_1 index modes).  At most 8 channels; any element type (moved as bits). */
BSIR_API int32_t bsir_interleave(int32_t dtype, int32_t channels, int64_t rows, int64_t cols, const void *const *srcs,
                                 void *dst, void *stream);
BSIR_API int32_t bsir_deinterleave(int32_t dtype, int32_t channels, int64_t rows, int64_t cols, const void *src,
                                   void *const *dsts, void *stream);

/* hivm.hir.vsort / hfusion.sort {descending, sort_axis = last} (HIVMVectorOps.td:2222-2283): every row sorted by
 * value, with the source index of each sorted element (int32).  The result is the one the reference's lowering
 * produces (n-1 bubble passes of compare-and-swap on `cmpf ugt` / `ult`,
 * bishengir/lib/Dialect/HFusion/Transforms/DecomposeOpInterfaceImpl.cpp:742-838; runner goldens
 * test/Dialect/HFusion/test_sort_2d_asc.mlir:16-19): equal values keep their source order, -0 = +0, and a NaN that
 * starts at position p of its row ends at (p + 1) mod n in either direction, the numbers filling the other places
 * in order.  dst_value or dst_index may be NULL; dst_value may not overlap src (BSIR_ERR_UNSUPPORTED).
 * dtype: f32, f16, bf16, i8, i16, i32.  Rows of up to 4096 elements are sorted in shared memory by one CTA; longer
 * rows (up to 2^30 elements) keep two copies of their 8-byte keys and 1 KB of digit counts per 4096 elements in the
 * library's device scratch (about 16.3 bytes an element, at most 1 GiB at a time: more rows are sorted in turns). */
BSIR_API int32_t bsir_sort(int32_t dtype, int32_t descending, int64_t rows, int64_t cols, const void *src,
                           int64_t src_row_stride, void *dst_value, int64_t value_row_stride, int32_t *dst_index,
                           int64_t index_row_stride, void *stream);

/* Fused softmax over the last axis
 * (test/Dialect/Analysis/VFFusion/MaxParallelKind/softmax_small_shape.mlir:86-117). */
BSIR_API int32_t bsir_softmax(int32_t dtype, int64_t rows, int64_t cols, const void *x,
                              int64_t x_row_stride, void *y, int64_t y_row_stride, void *stream);
/* Per-token dynamic int8 quantisation: scale[r] = max_j |x32[r,j]| / 127,
 * q = hfusion.cast{round_mode, enable_saturate}(x32 / scale[r]) -> i8. */
BSIR_API int32_t bsir_quant_per_token_i8(int32_t dtype, int32_t round_mode, int64_t rows,
                                         int64_t cols, const void *x, int64_t x_row_stride,
                                         int8_t *q, int64_t q_row_stride, float *scale,
                                         void *stream);

/* Bytes of scratch the W8A8 GEMM needs for this problem (0 = none). */
BSIR_API int64_t bsir_matmul_w8a8_workspace_bytes(int64_t m, int64_t n, int64_t k,
                                                  int32_t transpose_b);
/* linalg.matmul i8 x i8 -> i32 (compile-dot-int8-fractal-c.mlir:25) with the
 * composed dequant suffix: out = bf16_rint( f32(acc) * scale_a[m] * scale_b[n] ).
 * a: [m,k] row-major int8 (lda elements per row); b: [k,n] row-major (ldb) or,
 * with transpose_b, [n,k] row-major.  scale_a / scale_b may be NULL (= 1).
 * acc_out (may be NULL): int32 [m,n] row-major accumulators, for parity checks.
 * out (may be NULL when acc_out is given): out_dtype is BSIR_BF16 or BSIR_F16.
 * workspace as for bsir_reduce_with_index (no zero-fill requirement). */
BSIR_API int32_t bsir_matmul_w8a8(int64_t m, int64_t n, int64_t k, const int8_t *a, int64_t lda,
                                  const int8_t *b, int64_t ldb, int32_t transpose_b,
                                  const float *scale_a, const float *scale_b, int32_t out_dtype,
                                  void *out, int64_t ldo, int32_t *acc_out, void *workspace,
                                  int64_t workspace_bytes, void *stream);

/* hivm.hir.matmul, "C = descale * (A * B + bias)" with optional transposed operands
 * (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMMacroOps.td:364-492; descale modes
 * HIVMAttrs.td:1061-1071; the device library's variants
 * bishengir/lib/Template/lib/Cube/GlobalMmad.cpp:176-187 and the names with bias / descale in
 * bishengir/test/Conversion/HIVMToStandard/HIVMToStandard/matmul.mlir:13-55), followed by what the
 * reference inlines into the accumulator's way out (hivm.hir.fixpipe, HIVMDMAOps.td:275-335;
 * InlineFixpipe.cpp:876-884): pre_relu NORMAL_RELU and the pre_quant conversions F322F16, F322BF16 and
 * S322I8.  One description serves linalg.matmul of int8 (int32 accumulation), f16 and bf16 (f32
 * accumulation, Normalize.cpp:8224-8257) and batch_matmul (one launch per batch entry):
 *   acc  = sum_k A[i, k] * B[k, j]                              int32 or f32
 *   v    = f32(acc + bias[j])                                   int32 add for an int8 product
 *   v    = v * scale_a[i]                                       optional, the per-token half of a W8A8 dequant
 *   v    = v * descale[j] (per channel) | descale[0] (per tensor)
 *   v    = maximumf(v, 0)                                       with relu
 *   C    = cast_rint(v): f16 (clamped to its range), bf16, f32, int8 (saturating: S322I8); out_dtype
 *          BSIR_I32 stores acc + bias of an int8 product untouched. */
typedef struct bsir_matmul_desc {
  int32_t in_dtype;      /* BSIR_I8, BSIR_F16 or BSIR_BF16: the type of both A and B                  */
  int32_t out_dtype;     /* BSIR_F16, BSIR_BF16, BSIR_F32, BSIR_I8, and BSIR_I32 for an int8 product   */
  int32_t transpose_a;   /* 0: a is [m, k] rows; 1: a is [k, m] rows                                 */
  int32_t transpose_b;   /* 0: b is [k, n] rows (linalg.matmul); 1: b is [n, k] rows                 */
  int32_t descale_mode;  /* bsir_descale_mode: BSIR_DESCALE_NULL, _PER_CHANNEL or _PER_TENSOR                */
  int32_t relu;          /* 1: maximumf(v, 0) before the final cast                                  */
  int32_t bias_dtype;    /* BSIR_I32 with an int8 product; BSIR_F32, BSIR_F16 or BSIR_BF16 otherwise  */
  int32_t descale_dtype; /* BSIR_F32, BSIR_F16 or BSIR_BF16                                           */
  int64_t m, n, k;
  int64_t batch;         /* >= 1; entry e uses a + e * batch_stride_a and so on (strides in elements) */
  const void *a;
  int64_t lda, batch_stride_a;
  const void *b;
  int64_t ldb, batch_stride_b;
  const void *bias;      /* [n] or NULL                                                              */
  const void *descale;   /* [n] (per channel), [1] (per tensor) or NULL; a device pointer either way */
  const float *scale_a;  /* [m] f32 or NULL                                                          */
  void *out;
  int64_t ldo, batch_stride_out;
  int32_t n_peers;       /* 0: C goes to `out`.  > 0 (at most 8): C goes to every peer_out[i] instead --    */
  void *const *peer_out; /* the same block of each rank's output buffer (N-sharded GEMM, one-sided)        */
} bsir_matmul_desc;
BSIR_API int32_t bsir_matmul(const bsir_matmul_desc *desc, void *stream);

/* W4A16 group-quantised GEMM: out = bf16_rint( a . bf16_rint((q - z) * s) ), f32
 * accumulation.  a: [m,k] bf16 row-major (lda); qweight: int32 [k/8, n], nibble i
 * of word (r, c) (bits 4i..4i+3) is q[8r+i, c]; scales: bf16 [k/group, n];
 * zeros: int32 [k/group, n/8], nibble i of word (g, c) is z[g, 8c+i].
 * Requires k % group == 0, group % 32 == 0, n % 8 == 0. */
BSIR_API int32_t bsir_matmul_w4a16(int64_t m, int64_t n, int64_t k, int64_t group, const void *a,
                                   int64_t lda, const int32_t *qweight, const void *scales,
                                   const int32_t *zeros, void *out, int64_t ldo, void *stream);
/* The same product with the result stored into every peer_out[i] (each rank's copy of the output, already
 * offset to this rank's column block) instead of one `out`: the one-sided form of the N-sharded GEMM. */
BSIR_API int32_t bsir_matmul_w4a16_peers(int64_t m, int64_t n, int64_t k, int64_t group, const void *a,
                                         int64_t lda, const int32_t *qweight, const void *scales,
                                         const int32_t *zeros, int32_t n_peers, void *const *peer_out,
                                         int64_t ldo, void *stream);

/* ------------------------------------------------------------------------ */
/* B2: compiled-kernel ABI                                                   */
/* ------------------------------------------------------------------------ */
typedef enum {
  BSIR_KERNEL_ELEMWISE_BINARY = 0, /* args: a, b, out                          */
  BSIR_KERNEL_ELEMWISE_UNARY = 1,  /* args: x, out                             */
  BSIR_KERNEL_CAST = 2,            /* args: src, dst                           */
  BSIR_KERNEL_RMS_NORM = 3,        /* args: x, gamma, y, rstd (NULL allowed)   */
  BSIR_KERNEL_SOFTMAX = 4,         /* args: x, y                               */
  BSIR_KERNEL_QUANT_PER_TOKEN = 5, /* args: x, q, scale                        */
  BSIR_KERNEL_REDUCE_WITH_INDEX = 6, /* args: src, dst_value, dst_index        */
  BSIR_KERNEL_REDUCE = 7,          /* args: src, dst                           */
  BSIR_KERNEL_MATMUL_W8A8 = 8,     /* args: a, scale_a, b, scale_b, out        */
  BSIR_KERNEL_MATMUL_W4A16 = 9     /* args: a, qweight, scales, zeros, out     */
} bsir_kernel_kind;

/* What `bishengir-compile` would have baked into a kernel object: the op, its
 * attributes and the static shape of the arguments (contiguous row-major). */
typedef struct {
  int32_t kind;      /* bsir_kernel_kind                                        */
  int32_t fn;        /* unary/binary fn, reduce kind or reduce_with_index kind  */
  int32_t dtype;     /* element type of the inputs                              */
  int32_t dst_dtype; /* cast: destination type; matmul: output type             */
  int32_t round_mode;
  int32_t overflow_mode;
  int32_t flags;     /* reduce_with_index: bit0 tie_break_left, bit1 nan_first;
                        matmul_w8a8: bit0 transpose_b                          */
  int32_t rank;
  int64_t sizes[4];  /* elementwise: tensor shape; row ops: rows, cols;
                        matmul: m, n, k, group                                  */
  float eps;         /* rms_norm                                                */
} bsir_kernel_desc;

/* Register (or replace) a kernel under `name`; thread-safe. */
BSIR_API int32_t bsir_kernel_register(const char *name, const bsir_kernel_desc *desc);
BSIR_API int32_t bsir_kernel_unregister(const char *name);
/* Number of pointer arguments the kernel takes, or a negative status. */
BSIR_API int32_t bsir_kernel_num_args(const char *name);
/* rtKernelLaunch analogue: args = array of device pointers, args_size = bytes
 * of that array.  block_dim is a hint (the reference binds its outer tile loop
 * to that many cores) and does not change results.  stream NULL = the stream
 * of bsir_set_stream(). */
BSIR_API int32_t bsir_launch(const char *name, uint32_t block_dim, void **args, size_t args_size,
                             void *stream);

/* ------------------------------------------------------------------------ */
/* device bookkeeping                                                        */
/* ------------------------------------------------------------------------ */
/* Reads and clears the device-side error word of the current device (bits set by kernels: a bounded wait
 * that gave up, BSIR_DEVERR_GATHER_INDEX for a gather index outside its axis); synchronises the device.
 * 0 = clean. */
#define BSIR_DEVERR_GATHER_INDEX 0x100
#define BSIR_DEVERR_PEER_WAIT 0x200
BSIR_API int32_t bsir_device_error(void);
/* Number of kernel launches this library has enqueued in this process. */
BSIR_API int64_t bsir_launch_count(void);
/* Library-owned scratch.  Ops that need global memory beyond their operands (argmax over several
 * CTAs per row, split reductions, rows too long for one CTA, long sorts) and were given no workspace
 * take it from a block the library keeps PER (device, stream): calls on different streams never share
 * counters or partial results; calls on one stream are ordered by the stream.  A stream's block is
 * created, or replaced by a larger one, inside the first call that needs it (cudaMalloc + a clearing
 * memset enqueued on that stream; no host-side wait, and an outgrown block is kept, not freed, because
 * enqueued work may still use it).  That allocation is not allowed during stream capture: a call on
 * a capturing stream that has no block of its own borrows the block handed out last on the device
 * (so "run the ops once, then capture on another stream" works as long as the graph is not replayed
 * while that first stream runs scratch-using ops), and fails with BSIR_ERR_WORKSPACE when there is
 * none large enough -- run the ops once or call bsir_reserve_workspace before capturing.  The per-row
 * counters in a block are reset by the kernels themselves; they stay non-zero only if a kernel died,
 * which also ends the CUDA context.
 *
 * bsir_reserve_workspace: makes the block of `stream` (NULL = the thread's stream) at least `bytes`
 * long and creates the device error word, so that later calls allocate nothing.
 * bsir_release_workspace: waits for the device, then frees every block of the current device. */
BSIR_API int32_t bsir_reserve_workspace(int64_t bytes, void *stream);
BSIR_API int32_t bsir_release_workspace(void);

/* ------------------------------------------------------------------------ */
/* one-sided exchange between the GPUs of a node (N-sharded GEMMs)           */
/* ------------------------------------------------------------------------ */
/* The reference reaches other devices through put / signal wrappers over aclshmem
 * (bishengir/lib/Template/lib/Shmem/Shmem.cpp:27-120); here a GEMM's epilogue stores its block of C into every
 * rank's output buffer (see peer_out in bsir_matmul_desc) and bsir_peer_signal_wait closes the step.
 * bsir_peer_alloc: a buffer of its own allocation with 256 bytes of flags at *flags_offset_out (one uint32 per
 * source rank, zeroed).  bsir_peer_export / _open / _close: CUDA IPC handle (64 bytes) out, mapping of another
 * process's buffer in.  bsir_peer_signal_wait(rank, world, flag_ptrs, epoch, stream): enqueues one small kernel
 * that stores `epoch` into flag[rank] of every peer (release, system scope: everything this stream stored
 * before is visible first) and waits until all of this rank's own flags have reached `epoch`.  The wait gives up
 * after about two seconds with BSIR_DEVERR_PEER_WAIT in the device error word.  flag_ptrs[r] is rank r's flag
 * array as mapped in this process; epochs must grow from call to call.  epoch = 0 takes the step number from a
 * counter in this rank's flag page instead and advances it, which is the form to capture in a CUDA graph (every
 * replay then exchanges a fresh epoch); a buffer is driven either with explicit epochs or with epoch 0 by all
 * ranks, not a mix.  One rank per GPU. */
BSIR_API int32_t bsir_peer_alloc(int64_t payload_bytes, void **ptr_out, int64_t *flags_offset_out);
BSIR_API int32_t bsir_peer_free(void *ptr);
BSIR_API int32_t bsir_peer_export(void *ptr, void *handle64);
BSIR_API int32_t bsir_peer_open(const void *handle64, void **ptr_out);
BSIR_API int32_t bsir_peer_close(void *ptr);
/* Copies the block [rows x row_bytes] at byte_offset (row pitch pitch_bytes, all multiples of 16) of this rank's
 * buffer to the same place in every other rank's buffer: for blocks large enough that the GEMM should write its
 * own copy at full speed (TMA stores) and exchange it in a pass of its own. */
BSIR_API int32_t bsir_peer_push(int32_t rank, int32_t world, void *const *buffer_ptrs, int64_t byte_offset, int64_t rows,
                                int64_t row_bytes, int64_t pitch_bytes, void *stream);
BSIR_API int32_t bsir_peer_signal_wait(int32_t rank, int32_t world, void *const *flag_ptrs, uint32_t epoch, void *stream);

/* ------------------------------------------------------------------------ */
/* B1: op-library symbols                                                    */
/* ------------------------------------------------------------------------ */
/* The full list is generated from the same tables as the definitions; see
 * bsir_b200_ciface.h, included here so that one include declares everything. */
#include "bsir_b200_ciface.h"

#ifdef __cplusplus
}
#endif
#endif /* BSIR_B200_H_ */
