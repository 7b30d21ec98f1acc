// gemm_dense.cu -- dense contractions on the tensor core: hivm.hir.matmul / linalg.matmul of int8 (int32
// accumulation), f16 and bf16 (f32 accumulation) with the accumulator's way out fused in:
//   C = cast_rint( relu( descale * (A * B + bias) * scale_a ) )
// ("C = descale * (A * B + bias)", optional transposed operands:
// bishengir/include/bishengir/Dialect/HIVM/IR/HIVMMacroOps.td:364-492; relu and the F322F16 / F322BF16 / S322I8
// conversions are hivm.hir.fixpipe's pre_relu / pre_quant stages, HIVMDMAOps.td:275-335 and
// bishengir/lib/Dialect/HIVM/Transforms/InlineFixpipe.cpp:876-884; int8 dot:
// bishengir/test/bishengir-compile/hivm/compile-dot-int8-fractal-c.mlir:25; f32 accumulation for 16-bit outputs:
// bishengir/lib/Dialect/HFusion/Transforms/Normalize.cpp:8224-8257; device library variants
// bishengir/lib/Template/lib/Cube/GlobalMmad.cpp:176-187).  The W8A8 GEMM of the hot path is the int8 case with
// a per-row scale_a and a per-channel descale:  out = cast_rint( (sitofp(acc) * scale_a[m]) * scale_b[n] ).
//
// sm_100a design.  A persistent kernel, one CTA per SM, 192 threads in three roles:
//   warp 0     TMA producer: cp.async.bulk.tensor loads of the A tile and the B tile (16 KB + BN x 128 B per
//              128 bytes of K) into a ring of shared-memory stages (128-byte swizzle), completion on mbarriers;
//   warp 1     MMA issuer: one thread issues tcgen05.mma (kind::i8 or kind::f16, M=128, N=BN, 32 bytes of K per
//              instruction) with the accumulator in tensor memory; tcgen05.commit releases stages and
//              publishes tiles;
//   warps 2-5  epilogue: tcgen05.ld the accumulator (each warp its 32 TMEM lanes), bias, scales, relu, final
//              rounding, store (16-bit outputs through shared memory and TMA stores).
// Two accumulator buffers in TMEM (2 x BN columns) let the epilogue of tile i overlap the main loop of tile
// i + 1.  M >= 512 runs on CTA pairs (cta_group::2, 256 x 256 tiles); int8 with at most 24 rows swaps the
// operands (decode kernel).
//
// Either operand comes with K contiguous ("K-major": A as [m, k] rows, B as [n, k] rows = transpose_b) or with
// its other dimension contiguous ("MN-major": A as [k, m] rows = transpose_a, B as [k, n] rows as linalg.matmul
// has it): the shared-memory matrix descriptors and the instruction descriptor's major bits describe the layout,
// so no transpose pass is needed.  Everything about a tile is counted in bytes, which is what makes one kernel
// serve 1-byte and 2-byte operands: a stage holds 128 bytes of K (128 int8 or 64 half values).
//
// Every wait on an mbarrier is bounded: after ~2 s of cycles a waiter sets the device error word and an abort
// flag that all roles poll; the CTA then drains and frees its tensor memory.
//
// Shapes the TMA path cannot address (row pitches that are not multiples of 16 bytes, unaligned bases) run on
// a plain CUDA-core kernel instead.
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "tc_ptx.cuh"

namespace bsir {
namespace {

constexpr int kBM = 128;        // rows of A per tile = TMEM lanes
constexpr int kBK = 128;        // K bytes per stage (one 128-byte swizzle row)
constexpr int kUmmaK = 32;      // K bytes per tcgen05.mma
constexpr int kThreads = 192;

enum : int { KI8 = 0, KBF16 = 1, KF16 = 2 };   // operand kind
template <int KIND> constexpr int kEsize = KIND == KI8 ? 1 : 2;

struct GemmParams {
  int64_t m, n, k;             // k in elements
  const float *scale_a;        // per row, f32, may be null
  const void *descale;         // per channel [n] / per tensor [1], may be null
  const void *bias;            // per channel [n], may be null
  void *out;
  int64_t ldo;
  int32_t descale_dtype, descale_mode, bias_dtype, relu;
  int32_t out_dtype;
  int32_t *acc_out;            // int8 products only: raw accumulators (parity checks)
  int64_t ldacc;
  int *err;
  int m_tiles, n_tiles, k_blocks;
  int tma_out;   // 1: the output tile goes through shared memory and TMA stores (16-bit outputs)
  int n_peers;   // > 0: every store of C goes to each of peer[0 .. n_peers) instead of `out` (one-sided N-sharding)
  void *peer[8];
  // decode kernel, K split over CTAs: one arrival word per tile, two partial-tile slots per CTA, launch tag
  unsigned long long *tile_arrivals;
  int32_t *partials;
  uint32_t launch_tag;
  int dk_levels, dk_len, dk_helpers;   // 0 levels: whole tiles, no scratch
  int dk_vec_out;                      // 1: 16-byte stores of C (n and ldo multiples of 8, 16-byte aligned bases)
  // single-CTA kernel over a batch of products in one launch: the tensor maps are then rank 3 (z = the product) and
  // tile t belongs to product t / (m_tiles * n_tiles); 0 or 1: one product, rank-2 maps
  int batch;
  int64_t out_bs;                      // elements between the outputs of consecutive products
  int split_k;                         // 1: the `batch` "products" are the K parts of one product (rank-2 maps; part z covers
                                       // k blocks [z * k_blocks, (z + 1) * k_blocks) and writes its partial result at z * out_bs)
#ifdef BSIR_DEC_TIMELINE
  unsigned long long *tl;
#endif
};
// Built with -DBSIR_DEC_TIMELINE the decode kernel stamps %globaltimer and clock64() at the points marked TL(i) into
// the buffer whose device address the environment variable BSIR_DEC_TL_PTR holds (32 words of 8 bytes per CTA):
// where a launch's microseconds go (first stage landed, last MMA committed, epilogue done) was read off such stamps.
#ifdef BSIR_DEC_TIMELINE
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define TL(i) do { if (p.tl) { p.tl[blockIdx.x * 32 + (i)] = gtime(); p.tl[blockIdx.x * 32 + 16 + (i)] = clock64(); } } while (0)
#else
#define TL(i) do { } while (0)
#endif
// destination d of the output: the peers' buffers when there are any, else `out`
__device__ __forceinline__ int out_count(const GemmParams &p) { return p.n_peers > 0 ? p.n_peers : 1; }
__device__ __forceinline__ void *out_base(const GemmParams &p, int d) { return p.n_peers > 0 ? p.peer[d] : p.out; }

__device__ __forceinline__ float load_f32_as(const void *p, int32_t dtype, int64_t i) {
  if (dtype == BSIR_F16) return __half2float(__ushort_as_half(static_cast<const unsigned short *>(p)[i]));
  if (dtype == BSIR_BF16) return __uint_as_float(static_cast<uint32_t>(static_cast<const unsigned short *>(p)[i]) << 16);
  return static_cast<const float *>(p)[i];
}

// accumulator word -> f32 value after bias (int8 products add the int32 bias before the conversion)
template <int KIND>
__device__ __forceinline__ float acc_plus_bias(uint32_t acc_bits, uint32_t bias_bits) {
  if constexpr (KIND == KI8) return static_cast<float>(static_cast<int32_t>(acc_bits + bias_bits));
  else return __fadd_rn(__uint_as_float(acc_bits), __uint_as_float(bias_bits));
}
// scales, relu (arith.maximumf(x, 0): NaN stays NaN)
__device__ __forceinline__ float scale_relu(float f, float sa, float sw, int relu) {
  f = __fmul_rn(__fmul_rn(f, sa), sw);
  if (relu) f = maximumf(f, 0.0f);
  return f;
}
__device__ __forceinline__ uint32_t sat_i8_bits(float f) {   // cast{rint, saturate} to int8, NaN -> 0
  int v = __float2int_rn(f);
  v = v < -128 ? -128 : (v > 127 ? 127 : v);
  return static_cast<uint32_t>(v) & 0xffu;
}

template <int KIND>
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == KI8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
template <int KIND>
__device__ __forceinline__ void mma_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == KI8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// instruction descriptor: accumulator format, operand formats, operand majors, N, M
template <int KIND>
__device__ __forceinline__ uint32_t make_idesc(bool a_mn, bool b_mn, int n, int m) {
  uint32_t d;
  if constexpr (KIND == KI8) d = (2u << 4) | (1u << 7) | (1u << 10);          // D = s32, A = B = signed int8
  else if constexpr (KIND == KBF16) d = (1u << 4) | (1u << 7) | (1u << 10);   // D = f32, A = B = bf16
  else d = (1u << 4);                                                         // D = f32, A = B = f16
  return d | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}
// Descriptor of the K step `kk` (32 bytes of K) of an operand tile at `tile`:
//   K-major:  rows of 128 K-bytes, the step is 32 bytes into the row;
//   MN-major: chunks of [kr K-rows x 128 MN-bytes] kr * 128 bytes apart, the step is 32 / esize rows down.
template <int KIND>
__device__ __forceinline__ uint64_t operand_desc(uint32_t tile, int kk, bool mn_major) {
  constexpr int kr = kBK / kEsize<KIND>;           // K rows per stage of an MN-major tile
  constexpr int rows_per_mma = kUmmaK / kEsize<KIND>;
  return mn_major ? make_desc(tile + kk * (rows_per_mma * 128), kr * 128, 1024) : make_desc(tile + kk * kUmmaK, 16, 1024);
}

// ------------------------------------------------------------------ epilogue
// One accumulator tile, seen by one epilogue warp: its 32 TMEM lanes (rows) x BN columns, 32 columns at
// a time.  acc (+ bias) -> f32 -> * scale_a[row] -> * descale[col] -> relu -> output type.  The per-column
// descale and bias of the tile sit in shared memory (sw_s, bias_s); a row's 64 output bytes per chunk of a
// 16-bit output are written to a small shared-memory tile with the 64-byte TMA swizzle (conflict-free) and
// leave through a TMA store, so global memory sees whole sectors and the warp does not wait on the store.
// Without TMA (odd output pitch, 1- and 4-byte outputs) or for the int32 accumulator dump the lanes store
// directly.
constexpr int kEpiStageBytes = 2048;     // 32 rows x 64 bytes, two of them per warp

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y), "r"(src)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, int x, int y, int z, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y), "r"(z), "r"(src)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// zb: the product of a batched launch this tile belongs to (-1: one product, rank-2 output map)
template <int KIND, int BN>
__device__ __forceinline__ void epilogue_tile(const GemmParams &p, const CUtensorMap *tmap_out, uint32_t t_row,
                                              int64_t row, int64_t row_warp0, int64_t n0, int lane, uint8_t *stage_gen,
                                              uint32_t stage_addr, const float *sw_s, const uint32_t *bias_s,
                                              uint32_t &nstores, int zb = -1) {
  const bool row_ok = row < p.m;
  const int64_t out_off = zb > 0 ? static_cast<int64_t>(zb) * p.out_bs : 0;   // in elements of the output
  const float sa = (p.scale_a && row_ok) ? p.scale_a[row] : 1.0f;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 32) {
    uint32_t r[32];
    tmem_ld32(t_row + static_cast<uint32_t>(c0), r);
    tmem_ld_wait();
    const int64_t col0 = n0 + c0;
    if (col0 >= p.n) continue;          // uniform over the warp
    const bool full = col0 + 32 <= p.n;
    if (p.acc_out && row_ok) {
      int32_t *dst = p.acc_out + row * p.ldacc + col0;
      if (full && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<int4 *>(dst + j) = make_int4(static_cast<int>(r[j]), static_cast<int>(r[j + 1]),
                                                         static_cast<int>(r[j + 2]), static_cast<int>(r[j + 3]));
      } else {
        for (int j = 0; j < 32 && col0 + j < p.n; ++j) dst[j] = static_cast<int32_t>(r[j]);
      }
    }
    if (!p.out) continue;
    if (p.out_dtype == BSIR_BF16 || p.out_dtype == BSIR_F16) {
      // straight-line: the output type and relu are decided once per chunk, not per element, so that the 32
      // independent chains can overlap (one warp per scheduler has nothing else to hide latencies with)
      uint32_t packed[16];
      float f[32];
      const float floor_v = p.relu ? 0.0f : __int_as_float(0xff800000);   // maximumf(x, -inf) = x, NaN stays NaN
#pragma unroll
      for (int j4 = 0; j4 < 32; j4 += 4) {
        const float4 sw = *reinterpret_cast<const float4 *>(sw_s + c0 + j4);   // same address in every lane: broadcast
        const uint4 bb = *reinterpret_cast<const uint4 *>(bias_s + c0 + j4);
        f[j4 + 0] = maximumf(__fmul_rn(__fmul_rn(acc_plus_bias<KIND>(r[j4 + 0], bb.x), sa), sw.x), floor_v);
        f[j4 + 1] = maximumf(__fmul_rn(__fmul_rn(acc_plus_bias<KIND>(r[j4 + 1], bb.y), sa), sw.y), floor_v);
        f[j4 + 2] = maximumf(__fmul_rn(__fmul_rn(acc_plus_bias<KIND>(r[j4 + 2], bb.z), sa), sw.z), floor_v);
        f[j4 + 3] = maximumf(__fmul_rn(__fmul_rn(acc_plus_bias<KIND>(r[j4 + 3], bb.w), sa), sw.w), floor_v);
      }
      if (p.out_dtype == BSIR_F16) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          packed[j] = pack_f16x2(fminf(fmaxf(f[2 * j], -65504.0f), 65504.0f), fminf(fmaxf(f[2 * j + 1], -65504.0f), 65504.0f));
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) packed[j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
      }
      if (p.tma_out) {
        const uint32_t b = nstores & 1u;
        // the store that read this buffer two chunks ago must have finished reading it
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        __syncwarp();
        uint8_t *dstrow = stage_gen + b * kEpiStageBytes + lane * 64;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4 *>(dstrow + ((c ^ ((lane >> 1) & 3)) * 16)) =
              make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          if (zb >= 0) tma_store_3d(tmap_out, static_cast<int>(col0), static_cast<int>(row_warp0), zb, stage_addr + b * kEpiStageBytes);
          else tma_store_2d(tmap_out, static_cast<int>(col0), static_cast<int>(row_warp0), stage_addr + b * kEpiStageBytes);
        }
        ++nstores;
      } else if (row_ok) {
        for (int d = 0; d < out_count(p); ++d) {
          uint16_t *dst = static_cast<uint16_t *>(out_base(p, d)) + out_off + row * p.ldo + col0;
          if (full && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              *reinterpret_cast<uint4 *>(dst + 2 * j) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
          } else {
            for (int j = 0; j < 32 && col0 + j < p.n; ++j)
              dst[j] = static_cast<uint16_t>((j & 1) ? (packed[j >> 1] >> 16) : (packed[j >> 1] & 0xffffu));
          }
        }
      }
    } else if (row_ok) {
      // 1-byte (S322I8), 4-byte (f32) and raw int32 outputs: the lanes store directly
      if (p.out_dtype == BSIR_I8) {
        uint32_t packed[8];
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          uint32_t w = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e)
            w |= sat_i8_bits(scale_relu(acc_plus_bias<KIND>(r[j + e], bias_s[c0 + j + e]), sa, sw_s[c0 + j + e], p.relu)) << (8 * e);
          packed[j >> 2] = w;
        }
        for (int d = 0; d < out_count(p); ++d) {
          uint8_t *dst = static_cast<uint8_t *>(out_base(p, d)) + out_off + row * p.ldo + col0;
          if (full && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
            *reinterpret_cast<uint4 *>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            *reinterpret_cast<uint4 *>(dst + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
          } else {
            for (int j = 0; j < 32 && col0 + j < p.n; ++j) dst[j] = static_cast<uint8_t>(packed[j >> 2] >> (8 * (j & 3)));
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (p.out_dtype == BSIR_I32) o[e] = r[j + e] + bias_s[c0 + j + e];
            else o[e] = __float_as_uint(scale_relu(acc_plus_bias<KIND>(r[j + e], bias_s[c0 + j + e]), sa, sw_s[c0 + j + e], p.relu));
          }
          for (int d = 0; d < out_count(p); ++d) {
            uint32_t *dst = static_cast<uint32_t *>(out_base(p, d)) + out_off + row * p.ldo + col0;
            if (full && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
              *reinterpret_cast<uint4 *>(dst + j) = make_uint4(o[0], o[1], o[2], o[3]);
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (col0 + j + e < p.n) dst[j + e] = o[e];
            }
          }
        }
      }
    }
  }
}

// Per-column descale and bias of a tile into this warp's own shared-memory copy (no CTA-wide barrier, so a
// warp that gives up on a bounded wait can never leave the others stuck).
template <int KIND, int BN>
__device__ __forceinline__ void stage_scales(const GemmParams &p, int64_t n0, float *sw_s, uint32_t *bias_s, int lane) {
  const float tensor_scale = (p.descale && p.descale_mode == BSIR_DESCALE_PER_TENSOR) ? load_f32_as(p.descale, p.descale_dtype, 0) : 1.0f;
  for (int i = lane; i < BN; i += 32) {
    const bool in = n0 + i < p.n;
    sw_s[i] = (p.descale && p.descale_mode == BSIR_DESCALE_PER_CHANNEL && in) ? load_f32_as(p.descale, p.descale_dtype, n0 + i) : tensor_scale;
    uint32_t b = 0u;   // int32 0 and +0.0f alike
    if (p.bias && in) {
      if constexpr (KIND == KI8) b = static_cast<const uint32_t *>(p.bias)[n0 + i];
      else b = __float_as_uint(load_f32_as(p.bias, p.bias_dtype, n0 + i));
    }
    bias_s[i] = b;
  }
  __syncwarp();
}

template <int BN>
struct TileCfg {
  static constexpr int kStageA = kBM * kBK;           // 16 KB
  static constexpr int kStageB = BN * kBK;            // BN x 128 B
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);   // + the epilogue's staging
  static constexpr int kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;
  static constexpr int kEpiOff = kStages * kStage + 1024;                      // after the barriers (1 KB reserved)
  static constexpr int kEpiBytes = 4 * 2 * kEpiStageBytes + 2 * (4 * 2 * BN * 4);   // 4 warps x (2 store buffers + descale and bias of two tiles)
  static constexpr int kSmemBytes = kEpiOff + kEpiBytes + 1024 /*alignment slack*/;
};

// ------------------------------------------------------------------ the kernel
template <int KIND, int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads + 32, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_out, GemmParams p) {
  using Cfg = TileCfg<BN>;
  constexpr int kEs = kEsize<KIND>;
  constexpr int kKr = kBK / kEs;                  // K rows (elements) per stage
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // 128-byte swizzle wants 1024-byte aligned tiles
  uint8_t *gen_base = smem_raw + (base - raw);
  const uint32_t bars = base + Cfg::kStages * Cfg::kStage;
  // barrier slots (8 bytes each): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (Cfg::kStages + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * Cfg::kStages + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * Cfg::kStages + 2 + a); };
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen_base + Cfg::kStages * Cfg::kStage + 8 * (2 * Cfg::kStages + 4));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  volatile uint32_t *tiles_started = tmem_slot + 2;     // tiles whose overwriting MMA the first issuer has issued
  // int8 products: two issuing threads (warps 1 and 6), as in the CTA-pair kernel below
  constexpr int kIssuers = KIND == KI8 ? 2 : 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_per = p.m_tiles * p.n_tiles;           // of one product
  const bool batched = p.batch > 1;
  const int total_tiles = tiles_per * (batched ? p.batch : 1);

  pdl_launch_dependents();   // the set-up below overlaps the tail of the kernel ahead (see launch_pdl)
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), kIssuers); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), kIssuers); mbar_init(tempty_bar(a), 4); }
    *abort_flag = 0;
    *tiles_started = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
  pdl_wait();                // no global memory is touched before this
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (coordinates are bytes along the contiguous axis, rows along the other)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int zb = tile / tiles_per, t = tile - zb * tiles_per;
        const int m0 = (t % p.m_tiles) * kBM;
        const int n0 = (t / p.m_tiles) * BN;
        // one product: rank-2 maps; a batch: rank-3 maps, the product is the third coordinate
        auto load = [&](uint32_t dst, const CUtensorMap *map, int x, int y) {
          if (batched && !p.split_k) tma_load_3d(dst, map, x, y, zb, full_bar(stage));
          else tma_load_2d(dst, map, x, y, full_bar(stage));
        };
        const int kb0 = p.split_k ? zb * p.k_blocks : 0;           // K split over CTAs: this part's first k block
        for (int kq = 0; kq < p.k_blocks; ++kq) {
          const int kb = kb0 + kq;
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.err)) { ok = false; break; }
          const uint32_t sa = base + stage * Cfg::kStage;
          const uint32_t sb = sa + Cfg::kStageA;
          mbar_expect_tx(full_bar(stage), Cfg::kStage);
          if constexpr (A_MN) {
            // A is [k, m]: chunks of [kKr k rows x 128 m bytes]
#pragma unroll
            for (int c = 0; c < kBM * kEs / 128; ++c) load(sa + c * (kKr * 128), &tmap_a, m0 * kEs + c * 128, kb * kKr);
          } else {
            load(sa, &tmap_a, kb * kBK, m0);   // [128 m rows x 128 k bytes]
          }
          if constexpr (B_MN) {
            // B is [k, n]: chunks of [kKr k rows x 128 n bytes]
#pragma unroll
            for (int c = 0; c < BN * kEs / 128; ++c) load(sb + c * (kKr * 128), &tmap_b, n0 * kEs + c * 128, kb * kKr);
          } else {
            // B is [n, k]: boxes of [128 n rows x 128 k bytes]
#pragma unroll
            for (int c = 0; c < (BN + 127) / 128; ++c)
              load(sb + c * (128 * kBK), &tmap_b, kb * kBK, n0 + c * 128);
          }
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // loads already issued still write this CTA's shared memory: wait (bounded) for them
        for (int s = 0; s < Cfg::kStages; ++s) {
          for (int i = 0; i < 200000; ++i)
            if (mbar_try_wait(full_bar(s), 0) || mbar_try_wait(full_bar(s), 1)) break;
        }
      }
    }
  } else if (warp == 1 || warp == 6) {
    // ---------------- MMA issuers
    const int issuer = warp == 1 ? 0 : 1;
    if (lane == 0 && issuer < kIssuers) {
      const uint32_t idesc = make_idesc<KIND>(A_MN, B_MN, BN, kBM);
      constexpr int kSteps = kBK / kUmmaK / kIssuers;       // k steps of a block per issuer
      int stage = 0;
      uint32_t phase = 0, tile_seq = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0u, 0u};
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tile_seq) {
        if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * Cfg::kStage;
          const uint32_t sb = sa + Cfg::kStageA;
          if (issuer == 1 && kb == 0) {        // not before the MMA that overwrites the accumulator is on its way
            const long long t0 = clock64();
            while (*tiles_started <= tile_seq) {
              if (*abort_flag || clock64() - t0 > 4000000000LL) {
                *abort_flag = 1;
                if (p.err) atomicOr(p.err, static_cast<int>(kErrGemmWait));
                ok = false;
                break;
              }
            }
            if (!ok) break;
          }
#pragma unroll
          for (int kk = issuer * kSteps; kk < (issuer + 1) * kSteps; ++kk) {
            mma_ss<KIND>(d_tmem, operand_desc<KIND>(sa, kk, A_MN), operand_desc<KIND>(sb, kk, B_MN), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            if (kIssuers > 1 && issuer == 0 && kb == 0 && kk == 0) {
              __threadfence_block();
              *tiles_started = tile_seq + 1u;
            }
          }
          tc_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(tfull_bar(acc));      // accumulator complete
        acc_phase[acc] ^= 1u;
        acc ^= 1;
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5, TMEM lane quadrant = warp % 4
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    uint8_t *stage_gen = gen_base + Cfg::kEpiOff + (warp - 2) * 2 * kEpiStageBytes;
    const uint32_t stage_addr = base + Cfg::kEpiOff + (warp - 2) * 2 * kEpiStageBytes;
    float *sw_all = reinterpret_cast<float *>(gen_base + Cfg::kEpiOff + 4 * 2 * kEpiStageBytes);
    uint32_t *bias_all = reinterpret_cast<uint32_t *>(sw_all + 4 * 2 * BN);
    uint32_t nstores = 0;
    int acc = 0;
    uint32_t acc_phase[2] = {0u, 0u};
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int zb = tile / tiles_per, t = tile - zb * tiles_per;
      const int64_t m0 = static_cast<int64_t>(t % p.m_tiles) * kBM;
      const int64_t n0 = static_cast<int64_t>(t / p.m_tiles) * BN;
      float *sw_s = sw_all + ((warp - 2) * 2 + acc) * BN;
      uint32_t *bias_s = bias_all + ((warp - 2) * 2 + acc) * BN;
      stage_scales<KIND, BN>(p, n0, sw_s, bias_s, lane);         // overlaps the tile's main loop
      if (!mbar_wait(tfull_bar(acc), acc_phase[acc], abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * BN);
      epilogue_tile<KIND, BN>(p, &tmap_out, t_row, m0 + row_in_tile, m0 + quad * 32, n0, lane, stage_gen, stage_addr, sw_s, bias_s, nstores,
                              batched ? zb : -1);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));  // 4 arrivals (one per epilogue warp) free the buffer
      acc_phase[acc] ^= 1u;
      acc ^= 1;
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // shared memory must outlive the stores
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------ decode kernel (few rows of A, int8)
// For m <= 128 the roles of the operands are swapped: out^T[n, m] = W^T[n, k] . a^T[k, m].  The 128
// output columns of a tile are the MMA's M (the TMEM lanes), the rows of `a`, padded to a multiple
// of 16, are its N.  A stage then holds a 16 KB weight tile and only NB x 128 bytes of activations
// instead of a 128-row activation tile that is mostly padding, so the ring is up to 11 stages deep
// and a CTA keeps ~180 KB of weight loads in flight -- this shape is bound by HBM latency x
// bandwidth per SM, not by the tensor core.  Roles and barriers as in the kernel above; the
// epilogue reads the accumulator with lanes = output columns and writes 64-byte runs per row.
// It serves the W8A8 form of the epilogue (f32 per-row and per-channel scales, 16-bit output).
//
// With two thirds of the SMs or fewer holding a tile (N-sharded decode), K is split -- in a way that keeps the
// CTAs that run side by side on the same k blocks of neighbouring tiles, because a weight tile is 128 rows of 128
// bytes and only neighbours in n at the same k make those rows one contiguous stretch of DRAM.  With G CTAs
// and T tiles, G >= T: CTA b < levels * T (levels = G / T) takes k blocks [lvl * len, (lvl + 1) * len) of tile
// b % T, lvl = b / T; the remaining G % T "helper" CTAs share the last range [levels * len, k_blocks), helper h
// taking tiles h, h + helpers, ... one after the other.  len is the smallest block count that leaves a helper no
// more work than anyone else.  Every CTA writes its int32 partial tile to its slot of the scratch block and arrives
// on the tile's word; the CTA that arrives last adds the other parts to its accumulator and runs the epilogue.
// Nobody waits for anybody, int32 addition is exact, so the result has the bits of the unsplit product in every
// schedule.  An arrival word is {launch tag, count}: a count left behind by a launch that failed carries another
// tag and reads as zero; the last arrival writes zero back, so a replayed CUDA graph (same tag) finds it clean.
constexpr int kDecStageW = kBM * kBK;             // weight tile: 128 columns x 128 k
constexpr int kDecMaxStages = 12;
constexpr int kDecSmemBudget = 200 * 1024;

struct DecodeCfg {
  int nb;          // rows of `a` per MMA (multiple of 16, <= 128)
  int stage;       // bytes per stage
  int stages;
  uint32_t smem;   // dynamic shared memory to request
};
inline DecodeCfg decode_cfg(int64_t m) {
  DecodeCfg c;
  c.nb = static_cast<int>((m + 15) / 16 * 16);
  c.stage = kDecStageW + c.nb * kBK;
  c.stages = kDecSmemBudget / c.stage;
  if (c.stages > kDecMaxStages) c.stages = kDecMaxStages;
  c.smem = static_cast<uint32_t>(c.stages * c.stage + 1024 /*barriers*/ + 4096 /*output staging*/ + 1024 /*alignment slack*/);
  return c;
}

__device__ __forceinline__ bool tile_arrive(unsigned long long *word, uint32_t tag, int parts, int *err) {
  unsigned long long old = *reinterpret_cast<volatile unsigned long long *>(word);
  for (int tries = 0; tries < 4096; ++tries) {        // a failed swap means another part arrived: at most parts - 1 of them
    const uint32_t cnt = static_cast<uint32_t>(old >> 32) == tag ? static_cast<uint32_t>(old) : 0u;
    const bool last = static_cast<int>(cnt) + 1 >= parts;
    const unsigned long long next = last ? 0ull : ((static_cast<unsigned long long>(tag) << 32) | (cnt + 1u));
    const unsigned long long prev = atomicCAS(word, old, next);
    if (prev == old) return last;
    old = prev;
  }
  if (err) atomicOr(err, static_cast<int>(kErrGemmWait));
  return false;
}

// Which k blocks of which tiles CTA `b` works on (its s-th segment).  See the plan in the header comment above.
struct DecodeSeg { int tile, kb0, kb1, part; };
__device__ __forceinline__ bool decode_segment(const GemmParams &p, int b, int grid, int s, DecodeSeg &g) {
  if (p.dk_levels == 0) {                                  // whole tiles, round-robin
    g.tile = b + s * grid; g.kb0 = 0; g.kb1 = p.k_blocks; g.part = 0;
    return g.tile < p.n_tiles;
  }
  if (b < p.dk_levels * p.n_tiles) {                       // one k range of one tile
    const int lvl = b / p.n_tiles;
    g.tile = b - lvl * p.n_tiles; g.kb0 = lvl * p.dk_len; g.kb1 = min(p.k_blocks, g.kb0 + p.dk_len); g.part = lvl;
    return s == 0 && g.kb0 < p.k_blocks;
  }
  const int h = b - p.dk_levels * p.n_tiles;               // the last k range of every dk_helpers-th tile
  g.tile = h + s * p.dk_helpers; g.kb0 = p.dk_levels * p.dk_len; g.kb1 = p.k_blocks; g.part = p.dk_levels;
  return g.kb0 < p.k_blocks && g.tile < p.n_tiles;
}

// Four threads issue the MMAs: the thread that issues a tcgen05.mma is held for about 140 cycles by each one
// whatever its shape, so one issuer spent 570 cycles on the four MMAs of a 128-byte k block -- 60 GB/s of weights per
// CTA, which is what bounded this kernel.  Issuer j (warp 1 and the three warps after the epilogue warps) takes the
// j-th 32-byte k step of every block into an accumulator of its own; the epilogue adds the four (int32: exact, so
// the bits do not depend on the order).
constexpr int kDecIssuers = 4;
constexpr int kDecThreads = kThreads + 32 * (kDecIssuers - 1);
// KIND = KI8: the W8A8 form (int32 accumulators, f32 scales).  KIND = KBF16 / KF16: hivm.hir.matmul of few rows with
// f32 accumulators -- each issuer's accumulator is a partial sum over its k steps, the epilogue adds the four in issuer
// order (the same bits on every run) and applies bias, scales and relu as the tile kernels' epilogue does.
template <int KIND, bool W_MN>
__global__ void __launch_bounds__(kDecThreads, 1)
    w8a8_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a, GemmParams p,
                       int nb, int stage_bytes, int nstages) {
  constexpr int kEs = kEsize<KIND>;
  constexpr int kKr = kBK / kEs;                    // K rows of an MN-major weight chunk
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gen_base = smem_raw + (base - raw);
  const uint32_t bars = base + static_cast<uint32_t>(nstages * stage_bytes);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kDecMaxStages + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * kDecMaxStages + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * kDecMaxStages + 2 + a); };
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen_base + nstages * stage_bytes + 8 * (2 * kDecMaxStages + 4));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  volatile int *last_flag = reinterpret_cast<volatile int *>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, grid = gridDim.x;
  // one accumulator per issuer when they fit (4 x 2 x nb columns of tensor memory), else all into one
  const int nacc = nb <= 64 ? kDecIssuers : 1;
  const uint32_t want_cols = static_cast<uint32_t>(2 * nacc * nb);
  const uint32_t tmem_cols = want_cols <= 32 ? 32u : (want_cols <= 64 ? 64u : (want_cols <= 128 ? 128u : (want_cols <= 256 ? 256u : 512u)));
  const float *scale_b = static_cast<const float *>(p.descale);

  // Load number `it` of this CTA uses stage it % nstages.  All segments of a CTA have the same number of k blocks,
  // so load `it` is block it % seg_len of segment it / seg_len.
  DecodeSeg seg0;
  const bool any = decode_segment(p, cta, grid, 0, seg0);
  const int seg_len = any ? seg0.kb1 - seg0.kb0 : 1;
  int nsegs = 0;
  if (any) {
    if (p.dk_levels == 0) nsegs = (p.n_tiles - cta + grid - 1) / grid;
    else if (cta < p.dk_levels * p.n_tiles) nsegs = 1;
    else nsegs = (p.n_tiles - (cta - p.dk_levels * p.n_tiles) + p.dk_helpers - 1) / p.dk_helpers;
  }
  const int total_its = nsegs * seg_len;
  // The producer's cursor: counters that step, no division per load.
  DecodeSeg pseg = seg0;
  int p_seg = 0, p_kb = seg0.kb0, p_stage = 0;
  uint32_t p_round = 0;
  auto issue_next = [&]() {
    const uint32_t sw = base + p_stage * stage_bytes;
    const uint32_t bar = full_bar(p_stage);
    mbar_expect_tx(bar, static_cast<uint32_t>(stage_bytes));
    if constexpr (W_MN) {                                                             // chunks of [kKr k rows x 128 n bytes]
#pragma unroll
      for (int c = 0; c < kBM * kEs / 128; ++c) tma_load_2d(sw + c * (kKr * 128), &tmap_w, pseg.tile * kBM * kEs + c * 128, p_kb * kKr, bar);
    } else {
      tma_load_2d(sw, &tmap_w, p_kb * kBK, pseg.tile * kBM, bar);                     // [128 n rows x 128 k bytes]
    }
    tma_load_2d(sw + kDecStageW, &tmap_a, p_kb * kBK, 0, bar);                       // [nb rows x 128 k bytes]
    if (++p_kb == pseg.kb1) {
      decode_segment(p, cta, grid, ++p_seg, pseg);
      p_kb = pseg.kb0;
    }
    if (++p_stage == nstages) { p_stage = 0; ++p_round; }
  };
  const int preissued = total_its < nstages ? total_its : nstages;
  // Programmatic dependent launch: the next kernel of the stream may be scheduled while this one runs (its
  // blocks take SMs as ours leave them), and this kernel touches global memory only after the one before it
  // has completed -- so launch latency and the barrier / tensor-memory set-up overlap the predecessor's tail.
  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmap_w);
      prefetch_tmap(&tmap_a);
      for (int s = 0; s < nstages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), kDecIssuers); }
      for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), kDecIssuers); mbar_init(tempty_bar(a), 4); }
      *abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    pdl_wait();
    TL(0);
    // The first ring of loads goes out before the CTA meets: a launch this short cannot afford to wait for the
    // tensor-memory allocation first.  One thread issues them in order: the copy engine takes about 200 cycles per
    // 18 KB stage whoever issues it (one load per lane was tried: the ring took as long to go out and its first
    // stage arrived 1.5 us later, the engine having started with another one).
    if (lane == 0)
      for (int it = 0; it < preissued; ++it) issue_next();
    TL(1);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), tmem_cols);
  if (warp != 0) pdl_wait();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer
    if (lane == 0) {
      bool ok = true;
      for (int it = preissued; it < total_its; ++it) {
        if (!mbar_wait(empty_bar(p_stage), (p_round & 1u) ^ 1u, abort_flag, p.err)) { ok = false; break; }
        issue_next();
      }
      if (!ok) {
        for (int s = 0; s < nstages; ++s)
          for (int i = 0; i < 200000; ++i)
            if (mbar_try_wait(full_bar(s), 0) || mbar_try_wait(full_bar(s), 1)) break;
      }
    }
  } else if (warp == 1 || warp >= 6) {
    // ---------------- MMA issuers: warp 1 takes k step 0 of every block, warps 6..8 steps 1..3
    if (lane == 0) {
      const int issuer = warp == 1 ? 0 : warp - 5;
      // D = s32, A (weights) and B (activations) signed int8; A's major per the weight layout; N = nb, M = 128
      const uint32_t idesc = make_idesc<KIND>(W_MN, false, nb, kBM);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0u, 0u};
      bool ok = true;
      DecodeSeg g;
      for (int s = 0; ok && decode_segment(p, cta, grid, s, g); ++s) {
        if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>((acc * nacc + (nacc > 1 ? issuer : 0)) * nb);
        for (int kb = g.kb0; kb < g.kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.err)) { ok = false; break; }
          if (s == 0 && kb == g.kb0 && issuer == 0) TL(2);
          tc_fence_after();
          const uint32_t sw = base + stage * stage_bytes;
          const uint32_t sa = sw + kDecStageW;
          if (nacc > 1) {
            mma_ss<KIND>(d_tmem, operand_desc<KIND>(sw, issuer, W_MN), operand_desc<KIND>(sa, issuer, false), idesc, kb > g.kb0 ? 1u : 0u);
            tc_commit(empty_bar(stage));
          } else if (issuer == 0) {     // one accumulator for all: a single issuer keeps the k steps in order
#pragma unroll
            for (int kk = 0; kk < kBK / kUmmaK; ++kk)
              mma_ss<KIND>(d_tmem, operand_desc<KIND>(sw, kk, W_MN), operand_desc<KIND>(sa, kk, false), idesc, (kb > g.kb0 || kk > 0) ? 1u : 0u);
            tc_commit(empty_bar(stage));
          } else {
            mbar_arrive(empty_bar(stage));
          }
          if (++stage == nstages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (nacc > 1 || issuer == 0) tc_commit(tfull_bar(acc));
        else mbar_arrive(tfull_bar(acc));
        if (issuer == 0) TL(3);
        acc_phase[acc] ^= 1u;
        acc ^= 1;
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5, TMEM lane quadrant = warp % 4; lane = output column
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase[2] = {0u, 0u};
    bool ok = true;
    const size_t slot_words = static_cast<size_t>(nb) * kBM;
    // parts a tile is computed in: the k ranges that are not empty
    int parts = 1;
    if (p.dk_levels > 0) {
      const int lv = (p.k_blocks + p.dk_len - 1) / p.dk_len;
      parts = (lv < p.dk_levels ? lv : p.dk_levels) + (p.dk_levels * p.dk_len < p.k_blocks ? 1 : 0);
    }
    DecodeSeg g;
    for (int s = 0; ok && decode_segment(p, cta, grid, s, g); ++s) {
      const int64_t col = static_cast<int64_t>(g.tile) * kBM + quad * 32 + lane;
      const bool col_ok = col < p.n;
      float sw, bias_col = 0.0f;
      if constexpr (KIND == KI8) {
        sw = (scale_b && col_ok) ? scale_b[col] : 1.0f;
      } else {   // descale of any float type per channel or per tensor, bias per channel
        sw = !p.descale ? 1.0f
             : p.descale_mode == BSIR_DESCALE_PER_TENSOR ? load_f32_as(p.descale, p.descale_dtype, 0)
             : col_ok ? load_f32_as(p.descale, p.descale_dtype, col) : 1.0f;
        bias_col = (p.bias && col_ok) ? load_f32_as(p.bias, p.bias_dtype, col) : 0.0f;
      }
      const float sa_lane = (p.scale_a && lane < p.m) ? p.scale_a[lane] : 1.0f;   // rows 0..31, one per lane
      if (!mbar_wait(tfull_bar(acc), acc_phase[acc], abort_flag, p.err)) { ok = false; break; }
      if (threadIdx.x == 64) TL(4);
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * nacc * nb);
      auto load_sum16 = [&](int c0, uint32_t (&r)[16]) {      // the issuers' accumulators added up, 16 rows of `a`
        tmem_ld16(t_row + static_cast<uint32_t>(c0), r);
        for (int j = 1; j < nacc; ++j) {
          uint32_t q[16];
          tmem_ld16(t_row + static_cast<uint32_t>(j * nb + c0), q);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            if constexpr (KIND == KI8) r[e] += q[e];
            else r[e] = __float_as_uint(__fadd_rn(__uint_as_float(r[e]), __uint_as_float(q[e])));   // issuer order: 0, 1, 2, 3
          }
        }
        tmem_ld_wait();
      };
      bool finish = true;
      int32_t *tile_slots = nullptr;
      if (parts > 1) {
        tile_slots = p.partials + static_cast<size_t>(g.tile) * parts * slot_words;
        int32_t *mine = tile_slots + g.part * slot_words;
        for (int c0 = 0; c0 < nb && c0 < p.m; c0 += 16) {
          uint32_t r[16];
          load_sum16(c0, r);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < p.m) __stcg(mine + static_cast<size_t>(c0 + j) * kBM + quad * 32 + lane, static_cast<int32_t>(r[j]));
        }
        if (threadIdx.x == 64) TL(5);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) TL(6);
        if (warp == 2 && lane == 0) *last_flag = tile_arrive(p.tile_arrivals + g.tile, p.launch_tag, parts, p.err) ? 1 : 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        finish = *last_flag != 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");     // all have read the flag before the next segment's arrival rewrites it
        if (finish) __threadfence();
        if (threadIdx.x == 64) TL(7);
      }
      for (int c0 = 0; c0 < nb && finish; c0 += 16) {
        uint32_t r[16];
        load_sum16(c0, r);
        if (parts > 1 && c0 < p.m) {
          if constexpr (KIND == KI8) {
            for (int q = 0; q < parts; ++q) {
              if (q == g.part) continue;
              const int32_t *theirs = tile_slots + q * slot_words;
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c0 + j < p.m) r[j] += static_cast<uint32_t>(__ldcg(theirs + static_cast<size_t>(c0 + j) * kBM + quad * 32 + lane));
            }
          } else {
            // float parts are added in part order whoever arrived last -- this CTA's own part is read back from its
            // slot like the others -- so the sum is the same from run to run
            // (parts outside, rows inside: sixteen loads in flight a part, not one)
            for (int q = 0; q < parts; ++q) {
              const int32_t *slot = tile_slots + q * slot_words;
              uint32_t v[16];
#pragma unroll
              for (int j = 0; j < 16; ++j)
                v[j] = c0 + j < p.m ? static_cast<uint32_t>(__ldcg(slot + static_cast<size_t>(c0 + j) * kBM + quad * 32 + lane)) : 0u;
#pragma unroll
              for (int j = 0; j < 16; ++j) r[j] = q == 0 ? v[j] : __float_as_uint(__fadd_rn(__uint_as_float(r[j]), __uint_as_float(v[j])));
            }
          }
        }
        // scale and convert; the 16 rows x 32 columns of this warp go through shared memory so that a lane stores
        // 16 bytes of one row (2-byte stores, one per row and lane, cost this epilogue 2.5 us of a 14 us launch)
        uint16_t *stg = reinterpret_cast<uint16_t *>(gen_base + nstages * stage_bytes + 1024) + quad * 512;
        if (threadIdx.x == 64 && c0 == 0) TL(13);
        // straight-line code, no branch per row: one warp per scheduler has only instruction-level parallelism
        // to hide latencies with (a loop with the dtype test and the bounds tests inside ran 220 cycles per row)
        float f[16];
        if (nb <= 32) {
#pragma unroll
          for (int j = 0; j < 16; ++j) f[j] = __shfl_sync(0xffffffffu, sa_lane, (c0 + j) & 31);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) f[j] = (p.scale_a && c0 + j < p.m) ? __ldg(p.scale_a + c0 + j) : 1.0f;
        }
        if constexpr (KIND == KI8) {
#pragma unroll
          for (int j = 0; j < 16; ++j) f[j] = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int32_t>(r[j])), f[j]), sw);
        } else {
          const float floor_v = p.relu ? 0.0f : __int_as_float(0xff800000);   // maximumf(x, -inf) = x, NaN stays NaN
#pragma unroll
          for (int j = 0; j < 16; ++j) f[j] = maximumf(__fmul_rn(__fmul_rn(__fadd_rn(__uint_as_float(r[j]), bias_col), f[j]), sw), floor_v);
        }
        if (p.acc_out && col_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < p.m) p.acc_out[static_cast<int64_t>(c0 + j) * p.ldacc + col] = static_cast<int32_t>(r[j]);
        }
        uint32_t pk[8];
        if (p.out_dtype == BSIR_F16) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            pk[j] = pack_f16x2(fminf(fmaxf(f[2 * j], -65504.0f), 65504.0f), fminf(fmaxf(f[2 * j + 1], -65504.0f), 65504.0f));
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) pk[j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
        }
        if (p.dk_vec_out) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            stg[(2 * j) * 32 + lane] = static_cast<uint16_t>(pk[j] & 0xffffu);
            stg[(2 * j + 1) * 32 + lane] = static_cast<uint16_t>(pk[j] >> 16);
          }
        } else if (p.out && col_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const uint16_t bits = static_cast<uint16_t>((j & 1) ? (pk[j >> 1] >> 16) : (pk[j >> 1] & 0xffffu));
            if (c0 + j < p.m)
              for (int d = 0; d < out_count(p); ++d) static_cast<uint16_t *>(out_base(p, d))[static_cast<int64_t>(c0 + j) * p.ldo + col] = bits;
          }
        }
        if (threadIdx.x == 64 && c0 == 0) TL(14);
        if (p.dk_vec_out) {
          __syncwarp();
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const int id = lane + 32 * t, rr = id >> 2, part = id & 3;
            const int64_t row = c0 + rr, col0 = static_cast<int64_t>(g.tile) * kBM + quad * 32 + part * 8;
            if (row < p.m && col0 < p.n) {
              const uint4 v = *reinterpret_cast<const uint4 *>(stg + rr * 32 + part * 8);
              for (int d = 0; d < out_count(p); ++d)
                *reinterpret_cast<uint4 *>(static_cast<uint16_t *>(out_base(p, d)) + row * p.ldo + col0) = v;
            }
          }
          __syncwarp();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (threadIdx.x == 64) TL(8 + (s < 4 ? s : 4));
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      acc_phase[acc] ^= 1u;
      acc ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ------------------------------------------------------------------ CTA-pair kernel (cta_group::2)
// Two CTAs of a cluster share one 256 x 256 tile: CTA r owns rows [128 r, 128 r + 128) of A and the
// accumulator rows that go with them, and loads only columns [128 r, 128 r + 128) of the B tile; the
// tensor cores of both SMs read both halves of B.  Per SM that is 32 KB of shared-memory fill per
// 128 bytes of K instead of 48 KB, and half as many MMA instructions per flop for the issuing
// thread -- the two things that bound the single-CTA kernel.  Only the leader (cluster rank 0)
// issues MMAs; both CTAs' TMA loads complete on the leader's barrier; tcgen05.commit multicasts the
// "stage free" and "accumulator ready" arrivals to both CTAs (no TMA load is multicast).
constexpr int kPairStages = 6;
constexpr int kPairStageA = kBM * kBK;          // 16 KB: this CTA's 128 rows of A
constexpr int kPairStageB = 128 * kBK;          // 16 KB: this CTA's 128 columns of B
constexpr int kPairStage = kPairStageA + kPairStageB;
constexpr int kPairEpiOff = kPairStages * kPairStage + 1024;   // barriers get 1 KB
constexpr int kPairSmem = kPairEpiOff + 4 * 2 * kEpiStageBytes + 2 * (4 * 2 * 256 * 4) + 1024;
constexpr int kPairBN = 256;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {   // arrives on `bar` in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(static_cast<uint16_t>(3))
               : "memory");
}

// Int8 products have two issuing threads in the leader CTA (warps 1 and 6): the thread that issues a tcgen05.mma is
// held about 140 cycles by each, four per k block are 560 cycles, and the arithmetic of the block is 512.  Thread 0
// takes k steps 0 and 1 of every block, thread 1 steps 2 and 3, into the same accumulator: int32 sums do not depend
// on the order.  The second thread's first MMA of a tile waits until the first thread has issued the one that
// overwrites the accumulator.  Float products keep one issuer: their sums would depend on the order of arrival.
constexpr int kPairThreads = kThreads + 32;
template <int KIND, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_out, GemmParams p) {
  constexpr int kEs = kEsize<KIND>;
  constexpr int kKr = kBK / kEs;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gen_base = smem_raw + (base - raw);
  const uint32_t bars = base + kPairStages * kPairStage;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kPairStages + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * kPairStages + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * kPairStages + 2 + a); };
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen_base + kPairStages * kPairStage + 8 * (2 * kPairStages + 4));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  volatile uint32_t *tiles_started = tmem_slot + 2;     // tiles whose overwriting MMA the first issuer has issued
  constexpr int kIssuers = KIND == KI8 ? 2 : 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int m_tiles2 = (p.m_tiles + 1) / 2;            // tiles of 256 rows
  const int total_tiles = m_tiles2 * p.n_tiles;         // p.n_tiles counts 256-wide tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), kIssuers); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), kIssuers); mbar_init(tempty_bar(a), 8); }
    *abort_flag = 0;
    *tiles_started = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // both CTAs' barriers are initialised before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs): own half of the operands, completion on the leader's barrier
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += npairs) {
        const int m0 = (tile % m_tiles2) * 256 + static_cast<int>(rank) * 128;
        const int n0 = (tile / m_tiles2) * kPairBN + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.err)) { ok = false; break; }
          const uint32_t sa = base + stage * kPairStage;
          const uint32_t sb = sa + kPairStageA;
          const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * kPairStage);   // both CTAs' bytes
          if constexpr (A_MN) {
#pragma unroll
            for (int c = 0; c < kEs; ++c) tma_load_2d_pair(sa + c * (kKr * 128), &tmap_a, m0 * kEs + c * 128, kb * kKr, leader_full);
          } else {
            tma_load_2d_pair(sa, &tmap_a, kb * kBK, m0, leader_full);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int c = 0; c < kEs; ++c) tma_load_2d_pair(sb + c * (kKr * 128), &tmap_b, n0 * kEs + c * 128, kb * kKr, leader_full);
          } else {
            tma_load_2d_pair(sb, &tmap_b, kb * kBK, n0, leader_full);
          }
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1 || warp == 6) {
    // ---------------- MMA issuers: leader CTA only
    const int issuer = warp == 1 ? 0 : 1;
    if (lane == 0 && rank == 0 && issuer < kIssuers) {
      const uint32_t idesc = make_idesc<KIND>(A_MN, B_MN, kPairBN, 256);
      constexpr int kSteps = kBK / kUmmaK / kIssuers;       // k steps of a block per issuer
      int stage = 0;
      uint32_t phase = 0, tile_seq = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0u, 0u};
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += npairs, ++tile_seq) {
        if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kPairBN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * kPairStage;
          const uint32_t sb = sa + kPairStageA;
          if (issuer == 1 && kb == 0) {        // not before the MMA that overwrites the accumulator is on its way
            const long long t0 = clock64();
            while (*tiles_started <= tile_seq) {
              if (*abort_flag || clock64() - t0 > 4000000000LL) {
                *abort_flag = 1;
                if (p.err) atomicOr(p.err, static_cast<int>(kErrGemmWait));
                ok = false;
                break;
              }
            }
            if (!ok) break;
          }
#pragma unroll
          for (int kk = issuer * kSteps; kk < (issuer + 1) * kSteps; ++kk) {
            mma_ss_pair<KIND>(d_tmem, operand_desc<KIND>(sa, kk, A_MN), operand_desc<KIND>(sb, kk, B_MN), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            if (kIssuers > 1 && issuer == 0 && kb == 0 && kk == 0) {
              __threadfence_block();
              *tiles_started = tile_seq + 1u;
            }
          }
          tc_commit_pair(empty_bar(stage));
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit_pair(tfull_bar(acc));
        acc_phase[acc] ^= 1u;
        acc ^= 1;
      }
    }
  } else {
    // ---------------- epilogue (both CTAs): own 128 accumulator rows x 256 columns
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    uint8_t *stage_gen = gen_base + kPairEpiOff + (warp - 2) * 2 * kEpiStageBytes;
    const uint32_t stage_addr = base + kPairEpiOff + (warp - 2) * 2 * kEpiStageBytes;
    float *sw_all = reinterpret_cast<float *>(gen_base + kPairEpiOff + 4 * 2 * kEpiStageBytes);
    uint32_t *bias_all = reinterpret_cast<uint32_t *>(sw_all + 4 * 2 * kPairBN);
    uint32_t nstores = 0;
    int acc = 0;
    uint32_t acc_phase[2] = {0u, 0u};
    bool ok = true;
    for (int tile = pair; tile < total_tiles && ok; tile += npairs) {
      const int64_t m0 = static_cast<int64_t>(tile % m_tiles2) * 256 + static_cast<int64_t>(rank) * 128;
      const int64_t n0 = static_cast<int64_t>(tile / m_tiles2) * kPairBN;
      float *sw_s = sw_all + ((warp - 2) * 2 + acc) * kPairBN;
      uint32_t *bias_s = bias_all + ((warp - 2) * 2 + acc) * kPairBN;
      stage_scales<KIND, kPairBN>(p, n0, sw_s, bias_s, lane);
      if (!mbar_wait(tfull_bar(acc), acc_phase[acc], abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * kPairBN);
      epilogue_tile<KIND, kPairBN>(p, &tmap_out, t_row, m0 + row_in_tile, m0 + quad * 32, n0, lane, stage_gen, stage_addr, sw_s, bias_s, nstores);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));   // 8 arrivals (4 warps x 2 CTAs) at the leader
      acc_phase[acc] ^= 1u;
      acc ^= 1;
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // the peer may still be signalling into this CTA / reading its shared memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ------------------------------------------------------------------ plain fallback (any layout, any alignment)
template <int KIND>
__global__ void __launch_bounds__(256) gemm_simple_kernel(GemmParams p, const void *__restrict__ a, int64_t lda, int transpose_a,
                                                          const void *__restrict__ b, int64_t ldb, int transpose_b) {
  const int64_t col = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t row = blockIdx.y;
  if (col >= p.n || row >= p.m) return;
  const int64_t a0 = transpose_a ? row : row * lda, as = transpose_a ? lda : 1;
  const int64_t b0 = transpose_b ? col * ldb : col, bs = transpose_b ? 1 : ldb;
  uint32_t acc_bits;
  if constexpr (KIND == KI8) {
    const int8_t *ap = static_cast<const int8_t *>(a), *bp = static_cast<const int8_t *>(b);
    int32_t acc = 0;
    for (int64_t kk = 0; kk < p.k; ++kk) acc += static_cast<int32_t>(ap[a0 + kk * as]) * static_cast<int32_t>(bp[b0 + kk * bs]);
    acc_bits = static_cast<uint32_t>(acc);
    if (p.acc_out) p.acc_out[row * p.ldacc + col] = acc;
  } else {
    const uint16_t *ap = static_cast<const uint16_t *>(a), *bp = static_cast<const uint16_t *>(b);
    float acc = 0.0f;
    for (int64_t kk = 0; kk < p.k; ++kk) {
      float x, y;
      if constexpr (KIND == KBF16) {
        x = __uint_as_float(static_cast<uint32_t>(ap[a0 + kk * as]) << 16);
        y = __uint_as_float(static_cast<uint32_t>(bp[b0 + kk * bs]) << 16);
      } else {
        x = __half2float(__ushort_as_half(ap[a0 + kk * as]));
        y = __half2float(__ushort_as_half(bp[b0 + kk * bs]));
      }
      acc = __fadd_rn(acc, __fmul_rn(x, y));
    }
    acc_bits = __float_as_uint(acc);
  }
  if (!p.out) return;
  uint32_t bias_bits = 0u;
  if (p.bias) {
    if constexpr (KIND == KI8) bias_bits = static_cast<const uint32_t *>(p.bias)[col];
    else bias_bits = __float_as_uint(load_f32_as(p.bias, p.bias_dtype, col));
  }
  if (p.out_dtype == BSIR_I32) {
    for (int d = 0; d < out_count(p); ++d) static_cast<uint32_t *>(out_base(p, d))[row * p.ldo + col] = acc_bits + bias_bits;
    return;
  }
  const float sa = p.scale_a ? p.scale_a[row] : 1.0f;
  float sw = 1.0f;
  if (p.descale && p.descale_mode == BSIR_DESCALE_PER_CHANNEL) sw = load_f32_as(p.descale, p.descale_dtype, col);
  else if (p.descale && p.descale_mode == BSIR_DESCALE_PER_TENSOR) sw = load_f32_as(p.descale, p.descale_dtype, 0);
  const float f = scale_relu(acc_plus_bias<KIND>(acc_bits, bias_bits), sa, sw, p.relu);
  for (int d = 0; d < out_count(p); ++d) {
    void *ob = out_base(p, d);
    if (p.out_dtype == BSIR_F16) static_cast<uint16_t *>(ob)[row * p.ldo + col] = __half_as_ushort(__float2half_rn(fminf(fmaxf(f, -65504.0f), 65504.0f)));
    else if (p.out_dtype == BSIR_BF16) static_cast<uint16_t *>(ob)[row * p.ldo + col] = __bfloat16_as_ushort(__float2bfloat16_rn(f));
    else if (p.out_dtype == BSIR_I8) static_cast<uint8_t *>(ob)[row * p.ldo + col] = static_cast<uint8_t>(sat_i8_bits(f));
    else static_cast<float *>(ob)[row * p.ldo + col] = f;
  }
}

// ------------------------------------------------------------------ host side
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
    else
      cudaGetLastError();
  });
  return fn;
}

// Output [m, n] of 2-byte elements: box = [32 rows x 32 columns (64 bytes)], 64-byte swizzle.
bool make_out_tmap(CUtensorMap *map, void *ptr, uint64_t n, uint64_t m, uint64_t ldo) {
  EncodeFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {n, m};
  cuuint64_t strides[1] = {ldo * 2u};
  cuuint32_t box[2] = {32u, 32u};
  cuuint32_t estr[2] = {1u, 1u};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 2-D byte tensor map (operands of either width are addressed in bytes): `inner` contiguous bytes per row,
// `outer` rows of pitch `pitch` bytes, box = [box_rows x 128 bytes], 128-byte swizzle, out-of-range bytes read
// as zero.
bool make_tmap(CUtensorMap *map, const void *ptr, uint64_t inner, uint64_t outer, uint64_t pitch, uint32_t box_rows) {
  EncodeFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch};
  cuuint32_t box[2] = {128u, box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same maps over a batch of matrices `bstride` bytes apart (rank 3, one matrix a box).
bool make_tmap3(CUtensorMap *map, const void *ptr, uint64_t inner, uint64_t outer, uint64_t batch, uint64_t pitch, uint64_t bstride,
                uint32_t box_rows) {
  EncodeFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[3] = {inner, outer, batch};
  cuuint64_t strides[2] = {pitch, bstride};
  cuuint32_t box[3] = {128u, box_rows, 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool make_out_tmap3(CUtensorMap *map, void *ptr, uint64_t n, uint64_t m, uint64_t batch, uint64_t ldo, uint64_t out_bs) {
  EncodeFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[3] = {n, m, batch};
  cuuint64_t strides[2] = {ldo * 2u, out_bs * 2u};
  cuuint32_t box[3] = {32u, 32u, 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int KIND, int BN, bool A_MN, bool B_MN>
int32_t launch_tc(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tout, GemmParams p, cudaStream_t st) {
  using Cfg = TileCfg<BN>;
  // the attribute is per device and cheap to set
  cudaFuncSetAttribute(gemm_tc_kernel<KIND, BN, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  p.n_tiles = static_cast<int>(ceil_div(p.n, BN));
  const int64_t total = static_cast<int64_t>(p.m_tiles) * p.n_tiles * (p.batch > 1 ? p.batch : 1);
  int grid = device_info().sm_count > 0 ? device_info().sm_count : 148;
  if (grid > total) grid = static_cast<int>(total);
  launch_pdl(gemm_tc_kernel<KIND, BN, A_MN, B_MN>, dim3(grid), dim3(kThreads + 32), Cfg::kSmemBytes, st, ta, tb, tout, p);
  count_launch();
  return check_launch("matmul");
}
template <int KIND, bool A_MN, bool B_MN>
int32_t launch_tc_bn(int bn, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tout, const GemmParams &p, cudaStream_t st) {
  if (bn == 256) return launch_tc<KIND, 256, A_MN, B_MN>(ta, tb, tout, p, st);
  if constexpr (!B_MN) {
    if (bn == 64) return launch_tc<KIND, 64, A_MN, B_MN>(ta, tb, tout, p, st);
  }
  return launch_tc<KIND, 128, A_MN, B_MN>(ta, tb, tout, p, st);
}
template <int KIND, bool A_MN, bool B_MN>
int32_t launch_pair(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tout, GemmParams p, cudaStream_t st) {
  p.n_tiles = static_cast<int>(ceil_div(p.n, kPairBN));
  int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
  int grid = sms & ~1;
  const int total = static_cast<int>(ceil_div(p.m, 256)) * p.n_tiles;
  if (grid > 2 * total) grid = 2 * total;
  cudaFuncSetAttribute(gemm_pair_kernel<KIND, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
  gemm_pair_kernel<KIND, A_MN, B_MN><<<grid, kPairThreads, kPairSmem, st>>>(ta, tb, tout, p);
  count_launch();
  return check_launch("matmul (CTA pairs)");
}

// Tile width: the widest N tile whose tile count still covers the SMs reasonably.
int pick_bn(int64_t m, int64_t n, int sm_count, bool b_mn, int64_t batch = 1) {
  const int64_t m_tiles = ceil_div(m, kBM) * batch;
  const int min_bn = b_mn ? 128 : 64;
  int best = 256;
  double best_eff = -1.0;
  for (int bn = 256; bn >= min_bn; bn >>= 1) {
    const int64_t tiles = m_tiles * ceil_div(n, bn);
    const int64_t rounds = ceil_div(tiles, sm_count);
    double eff = static_cast<double>(tiles) / static_cast<double>(rounds * sm_count);
    if (bn == 256) eff *= 1.0; else if (bn == 128) eff *= 0.93; else eff *= 0.85;  // narrower tiles re-read A more
    if (eff > best_eff + 1e-9) { best_eff = eff; best = bn; }
  }
  return best;
}

struct Operands {
  const void *a;
  int64_t lda;
  int transpose_a;
  const void *b;
  int64_t ldb;
  int transpose_b;
};

// Second step of a float product whose K was split over CTAs: the `parts` f32 partial products of every element are
// added in part order (so the result is the same from run to run) and go through the epilogue's arithmetic --
// bias, per-row scale, descale, relu, conversion -- exactly as epilogue_tile applies it to an accumulator.
__global__ void __launch_bounds__(256) splitk_finish_kernel(GemmParams p, const float *__restrict__ partials, int parts, int64_t part_stride,
                                                            int64_t ldp) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = p.m * p.n;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t row = i / p.n, col = i - row * p.n;
    float acc = partials[row * ldp + col];
    for (int e = 1; e < parts; ++e) acc = __fadd_rn(acc, partials[e * part_stride + row * ldp + col]);
    const float sa = p.scale_a ? p.scale_a[row] : 1.0f;
    const float sw = !p.descale ? 1.0f
                     : p.descale_mode == BSIR_DESCALE_PER_CHANNEL ? load_f32_as(p.descale, p.descale_dtype, col)
                                                                  : load_f32_as(p.descale, p.descale_dtype, 0);
    const float bias = p.bias ? load_f32_as(p.bias, p.bias_dtype, col) : 0.0f;
    const float f = scale_relu(__fadd_rn(acc, bias), sa, sw, p.relu);
    const int64_t o = row * p.ldo + col;
    if (p.out_dtype == BSIR_BF16) static_cast<__nv_bfloat16 *>(p.out)[o] = __float2bfloat16_rn(f);
    else if (p.out_dtype == BSIR_F16) static_cast<__half *>(p.out)[o] = __float2half_rn(fminf(fmaxf(f, -65504.0f), 65504.0f));
    else if (p.out_dtype == BSIR_I8) static_cast<uint8_t *>(p.out)[o] = static_cast<uint8_t>(sat_i8_bits(f));
    else static_cast<float *>(p.out)[o] = f;
  }
}

// `batch` products of one shape, `bsa` / `bsb` / `p.out_bs` elements apart, in one launch of the single-CTA kernel over
// rank-3 tensor maps.  false: not possible here (alignment, no encoder, tiles too many for int) -- the caller then
// launches product by product.
template <int KIND>
bool run_gemm_batched(GemmParams p, const Operands &o, int64_t batch, int64_t bsa, int64_t bsb, cudaStream_t st, int32_t *rc) {
  constexpr int es = kEsize<KIND>;
  const int64_t m = p.m, n = p.n, k = p.k;
  p.m_tiles = static_cast<int>(ceil_div(m, kBM));
  p.k_blocks = static_cast<int>(ceil_div(k * es, kBK));
  const bool a_mn = o.transpose_a != 0, b_mn = o.transpose_b == 0;
  if (!(k > 0 && device_info().cc_major >= 10 && aligned_to(o.a, 16) && aligned_to(o.b, 16) && (o.lda * es) % 16 == 0 &&
        (o.ldb * es) % 16 == 0 && (bsa * es) % 16 == 0 && (bsb * es) % 16 == 0 && encode_fn() != nullptr && batch <= 65535))
    return false;
  const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
  const int bn = pick_bn(m, n, sms, b_mn, batch);
  if (static_cast<int64_t>(p.m_tiles) * ceil_div(n, bn) * batch > 0x3fffffffLL) return false;
  CUtensorMap ta, tb, tout;
  memset(&tout, 0, sizeof(tout));
  const bool out16 = p.out_dtype == BSIR_BF16 || p.out_dtype == BSIR_F16;
  p.tma_out = (p.out && out16 && aligned_to(p.out, 16) && p.ldo % 8 == 0 && p.out_bs % 8 == 0 &&
               make_out_tmap3(&tout, p.out, static_cast<uint64_t>(n), static_cast<uint64_t>(m), static_cast<uint64_t>(batch),
                              static_cast<uint64_t>(p.ldo), static_cast<uint64_t>(p.out_bs))) ? 1 : 0;
  const uint32_t kr = static_cast<uint32_t>(kBK / es);
  const uint64_t ub = static_cast<uint64_t>(batch);
  bool ok = a_mn ? make_tmap3(&ta, o.a, static_cast<uint64_t>(m) * es, static_cast<uint64_t>(k), ub, static_cast<uint64_t>(o.lda) * es, static_cast<uint64_t>(bsa) * es, kr)
                 : make_tmap3(&ta, o.a, static_cast<uint64_t>(k) * es, static_cast<uint64_t>(m), ub, static_cast<uint64_t>(o.lda) * es, static_cast<uint64_t>(bsa) * es, kBM);
  if (b_mn) ok = ok && make_tmap3(&tb, o.b, static_cast<uint64_t>(n) * es, static_cast<uint64_t>(k), ub, static_cast<uint64_t>(o.ldb) * es, static_cast<uint64_t>(bsb) * es, kr);
  else ok = ok && make_tmap3(&tb, o.b, static_cast<uint64_t>(k) * es, static_cast<uint64_t>(n), ub, static_cast<uint64_t>(o.ldb) * es, static_cast<uint64_t>(bsb) * es, bn < 128 ? bn : 128);
  if (!ok) return false;
  p.batch = static_cast<int>(batch);
  if (a_mn) *rc = b_mn ? launch_tc_bn<KIND, true, true>(bn, ta, tb, tout, p, st) : launch_tc_bn<KIND, true, false>(bn, ta, tb, tout, p, st);
  else *rc = b_mn ? launch_tc_bn<KIND, false, true>(bn, ta, tb, tout, p, st) : launch_tc_bn<KIND, false, false>(bn, ta, tb, tout, p, st);
  return true;
}

// One [m, k] x [k, n] product.  p holds the epilogue; sizes are validated by the callers.
template <int KIND>
int32_t run_gemm(GemmParams p, const Operands &o, bool classic_w8a8, cudaStream_t st) {
  constexpr int es = kEsize<KIND>;
  const int64_t m = p.m, n = p.n, k = p.k;
  p.m_tiles = static_cast<int>(ceil_div(m, kBM));
  p.k_blocks = static_cast<int>(ceil_div(k * es, kBK));
  const bool a_mn = o.transpose_a != 0, b_mn = o.transpose_b == 0;
  const bool tma_ok = k > 0 && device_info().cc_major >= 10 && aligned_to(o.a, 16) && aligned_to(o.b, 16) && (o.lda * es) % 16 == 0 &&
                      (o.ldb * es) % 16 == 0 && encode_fn() != nullptr;
  if (tma_ok) {
    CUtensorMap ta, tb, tout;
    memset(&tout, 0, sizeof(tout));
    const bool out16 = p.out_dtype == BSIR_BF16 || p.out_dtype == BSIR_F16;
    p.tma_out = (p.out && p.n_peers == 0 && out16 && aligned_to(p.out, 16) && p.ldo % 8 == 0 &&
                 make_out_tmap(&tout, p.out, static_cast<uint64_t>(n), static_cast<uint64_t>(m), static_cast<uint64_t>(p.ldo))) ? 1 : 0;
    int bn = pick_bn(m, n, device_info().sm_count > 0 ? device_info().sm_count : 148, b_mn);
    const char *force = std::getenv("BSIR_W8A8_PATH");
    // BSIR_W8A8_PATH=1 / 2 forces the single-CTA / CTA-pair kernel (tests use it on small shapes)
    const bool want_pair = (force && force[0] == '2') ||
                           (!(force && force[0] == '1') && m >= 192 && ceil_div(m, 256) * ceil_div(n, 256) >= 56);   // measured, k 4096, n 14336: m = 128 19.2 / 14.8 us (pair / single CTA), 192 19.3 / 19.8, 384 27.9 / 31.1, 511 28.3 / 31.4
    // Float products with too few tiles for the SMs: K is split into `parts` (4 or 8 whole shares of k blocks), every
    // part a "product" of a batched launch that writes its f32 partial result into scratch, and a second launch adds
    // the parts in order and applies the epilogue.  A tile of K = 4096 is 64 k blocks of four MMAs from one issuing
    // thread -- 19 us of MMA issue alone, whatever the tile's width; so the widest tile that leaves the most parts wins.
    int parts = 1;
    if constexpr (KIND != KI8) {
      const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
      // (measured, bf16, K = N = 4096, device time: m = 1 24.3 -> 20.6 us, 16 24.4 -> 21.2, 128 24.6 -> 24.5, 512 26.8 -> 37.7 --
      // the partial results of many rows cost more than the split saves, so it is for few rows only; up to 128 rows when K is
      // very long: n = 4096, k = 14336, m = 128 72.9 -> 41.2 us)
      if ((m <= 64 || (m <= 128 && p.k_blocks >= 128)) && !want_pair && p.n_peers == 0 && p.out && !p.acc_out && !force && (k * es) % kBK == 0 && std::getenv("BSIR_GEMM_NO_SPLITK") == nullptr) {
        for (int cand = 256; cand >= (b_mn ? 128 : 64); cand >>= 1) {
          const int64_t tiles = static_cast<int64_t>(p.m_tiles) * ceil_div(n, static_cast<int64_t>(cand));
          for (int c = 8; c > parts && c >= 4; c >>= 1)          // (two parts do not pay for the second launch: n = 14336, m = 64 27 -> 39 us)
            if (p.k_blocks % c == 0 && p.k_blocks / c >= 4 && tiles * c <= sms) { parts = c; bn = cand; break; }
        }
      }
    }
    const uint32_t kr = static_cast<uint32_t>(kBK / es);
    // A: [m rows x k bytes] boxes of 128 rows, or (transposed) [k rows x m bytes] boxes of kr rows
    bool ok = a_mn ? make_tmap(&ta, o.a, static_cast<uint64_t>(m) * es, static_cast<uint64_t>(k), static_cast<uint64_t>(o.lda) * es, kr)
                   : make_tmap(&ta, o.a, static_cast<uint64_t>(k) * es, static_cast<uint64_t>(m), static_cast<uint64_t>(o.lda) * es, kBM);
    if (b_mn) ok = ok && make_tmap(&tb, o.b, static_cast<uint64_t>(n) * es, static_cast<uint64_t>(k), static_cast<uint64_t>(o.ldb) * es, kr);
    else ok = ok && make_tmap(&tb, o.b, static_cast<uint64_t>(k) * es, static_cast<uint64_t>(n), static_cast<uint64_t>(o.ldb) * es, bn < 128 ? bn : 128);
    if (ok && want_pair) {
      // CTA pairs: A as before; B boxes of 128 columns (MN-major: kr rows of 128 bytes) / 128 rows (K-major)
      CUtensorMap tb2;
      const bool ok2 = b_mn ? make_tmap(&tb2, o.b, static_cast<uint64_t>(n) * es, static_cast<uint64_t>(k), static_cast<uint64_t>(o.ldb) * es, kr)
                            : make_tmap(&tb2, o.b, static_cast<uint64_t>(k) * es, static_cast<uint64_t>(n), static_cast<uint64_t>(o.ldb) * es, 128);
      if (ok2) {
        if (a_mn) return b_mn ? launch_pair<KIND, true, true>(ta, tb2, tout, p, st) : launch_pair<KIND, true, false>(ta, tb2, tout, p, st);
        return b_mn ? launch_pair<KIND, false, true>(ta, tb2, tout, p, st) : launch_pair<KIND, false, false>(ta, tb2, tout, p, st);
      }
    }
    if constexpr (KIND != KI8) {
      const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
      if (!ok) parts = 1;
      // up to 48 rows with a 16-bit result take the decode form below, which shares a tile's k blocks out itself
      if (parts > 1 && !a_mn && m <= 48 && out16 && std::getenv("BSIR_GEMM_NO_FLOAT_DECODE") == nullptr) parts = 1;
      if (parts > 1) {
        const int64_t ldp = (n + 3) / 4 * 4;                       // f32 rows on 16-byte boundaries
        const int64_t part_elems = m * ldp;
        char *ws = static_cast<char *>(device_workspace(kScratchCounterBytes + static_cast<size_t>(parts) * part_elems * 4, st));
        if (ws) {
          float *partials = reinterpret_cast<float *>(ws + kScratchCounterBytes);
          GemmParams q{};
          q.m = m; q.n = n; q.k = k / parts;
          q.m_tiles = p.m_tiles; q.k_blocks = p.k_blocks / parts;
          q.out = partials; q.ldo = ldp; q.out_dtype = BSIR_F32; q.out_bs = part_elems;
          q.err = p.err;
          q.batch = parts; q.split_k = 1;
          int32_t rc;
          if (a_mn) rc = b_mn ? launch_tc_bn<KIND, true, true>(bn, ta, tb, tout, q, st) : launch_tc_bn<KIND, true, false>(bn, ta, tb, tout, q, st);
          else rc = b_mn ? launch_tc_bn<KIND, false, true>(bn, ta, tb, tout, q, st) : launch_tc_bn<KIND, false, false>(bn, ta, tb, tout, q, st);
          if (rc != BSIR_OK) return rc;
          int64_t blocks = ceil_div(m * n, static_cast<int64_t>(256));
          if (blocks > sms * 8) blocks = sms * 8;
          launch_pdl(splitk_finish_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, st, p, static_cast<const float *>(partials), parts,
                     part_elems, ldp);
          count_launch();
          return check_launch("matmul (K split)");
        }
      }
    }
    {
      // few rows: operands swapped, deep ring of weight tiles (BSIR_W8A8_PATH=3 forces it for m <= 128, =1 avoids it)
      // measured on B200 (k 4096, n 14336), this kernel against the 128-row-tile one: m = 16 12.5 / 19.8 us, 32 13.0 / 14.5,
      // 48 13.9 / 14.6, 64 14.7 / 14.6, 96 18.0 / 14.8.  Float products take it with 16-bit outputs (its store path).
      const bool decode_form = KIND == KI8 ? classic_w8a8 : (out16 && !p.acc_out && std::getenv("BSIR_GEMM_NO_FLOAT_DECODE") == nullptr);
      const bool want_decode = decode_form && !a_mn && ((force && force[0] == '3') ? m <= 128 : (!force && m <= 48));
      if (ok && want_decode) {
        const DecodeCfg dc = decode_cfg(m);
        CUtensorMap tw, tact;
        // weights [k, n] (MN-major): chunks of kr k rows x 128 n bytes; [n, k]: boxes of 128 n rows x 128 k bytes
        bool ok3 = b_mn ? make_tmap(&tw, o.b, static_cast<uint64_t>(n) * es, static_cast<uint64_t>(k), static_cast<uint64_t>(o.ldb) * es, kr)
                        : make_tmap(&tw, o.b, static_cast<uint64_t>(k) * es, static_cast<uint64_t>(n), static_cast<uint64_t>(o.ldb) * es, kBM);
        ok3 = ok3 && make_tmap(&tact, o.a, static_cast<uint64_t>(k) * es, static_cast<uint64_t>(m), static_cast<uint64_t>(o.lda) * es, static_cast<uint32_t>(dc.nb));
        if (ok3) {
          p.n_tiles = static_cast<int>(ceil_div(n, kBM));
          const int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
          const int64_t items = static_cast<int64_t>(p.n_tiles) * p.k_blocks;
          int grid = p.n_tiles < sms ? p.n_tiles : sms;
          // K is split over CTAs when whole tiles would leave SMs idle (BSIR_W8A8_SPLITK=0: never)
          const char *split_env = std::getenv("BSIR_W8A8_SPLITK");
          p.partials = nullptr;
          p.tile_arrivals = nullptr;
          p.dk_levels = p.dk_len = p.dk_helpers = 0;
          p.launch_tag = 0;
#ifdef BSIR_DEC_TIMELINE
          { const char *e = std::getenv("BSIR_DEC_TL_PTR"); p.tl = e ? reinterpret_cast<unsigned long long *>(std::strtoull(e, nullptr, 0)) : nullptr; }
#endif
          p.dk_vec_out = (p.out || p.n_peers > 0) && n % 8 == 0 && p.ldo % 8 == 0 && (p.n_peers > 0 || aligned_to(p.out, 16));
          for (int d = 0; d < p.n_peers; ++d) p.dk_vec_out = p.dk_vec_out && aligned_to(p.peer[d], 16);
          // 112 CTAs already stream n = 14336 at the HBM rate, so K is split only when a third of the SMs or more would idle
          if (!(split_env && split_env[0] == '0') && p.n_tiles * 3 <= sms * 2 && p.k_blocks > 1 && static_cast<size_t>(p.n_tiles) * 8 <= kScratchCounterBytes) {
            // at most six parts per tile: the CTA that arrives last reads the others' partial tiles one after the other
            int64_t g2 = items < sms ? items : sms;
            if (g2 > static_cast<int64_t>(p.n_tiles) * 6) g2 = static_cast<int64_t>(p.n_tiles) * 6;
            const int levels = static_cast<int>(g2 / p.n_tiles), helpers = static_cast<int>(g2 % p.n_tiles);
            int len;
            if (helpers == 0) {
              len = static_cast<int>(ceil_div(p.k_blocks, levels));
            } else {
              const int64_t q = ceil_div(p.n_tiles, helpers);              // tiles per helper
              len = static_cast<int>(ceil_div(static_cast<int64_t>(p.k_blocks) * q, 1 + levels * q));
            }
            if (len < 1) len = 1;
            if (len * 10 <= p.k_blocks * 9) {                                // worth it: the longest share shrinks by a tenth or more
              const int lv = static_cast<int>(ceil_div(p.k_blocks, len));
              const int parts = (lv < levels ? lv : levels) + (levels * len < p.k_blocks ? 1 : 0);
              const size_t need = kScratchCounterBytes + static_cast<size_t>(p.n_tiles) * parts * dc.nb * kBM * sizeof(int32_t);
              char *ws = static_cast<char *>(device_workspace(need, st));
              if (!ws) return BSIR_ERR_WORKSPACE;
              static std::atomic<uint32_t> tag{0};
              uint32_t t = ++tag;
              if (t == 0) t = ++tag;
              p.tile_arrivals = reinterpret_cast<unsigned long long *>(ws);
              p.partials = reinterpret_cast<int32_t *>(ws + kScratchCounterBytes);
              p.launch_tag = t;
              p.dk_levels = levels; p.dk_len = len; p.dk_helpers = helpers;
              grid = static_cast<int>(g2);
            }
          }
          if (b_mn) {
            cudaFuncSetAttribute(w8a8_decode_kernel<KIND, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dc.smem));
            launch_pdl(w8a8_decode_kernel<KIND, true>, dim3(grid), dim3(kDecThreads), dc.smem, st, tw, tact, p, dc.nb, dc.stage, dc.stages);
          } else {
            cudaFuncSetAttribute(w8a8_decode_kernel<KIND, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dc.smem));
            launch_pdl(w8a8_decode_kernel<KIND, false>, dim3(grid), dim3(kDecThreads), dc.smem, st, tw, tact, p, dc.nb, dc.stage, dc.stages);
          }
          count_launch();
          return check_launch("matmul (decode)");
        }
      }
    }
    if (ok) {
      if (a_mn) return b_mn ? launch_tc_bn<KIND, true, true>(bn, ta, tb, tout, p, st) : launch_tc_bn<KIND, true, false>(bn, ta, tb, tout, p, st);
      return b_mn ? launch_tc_bn<KIND, false, true>(bn, ta, tb, tout, p, st) : launch_tc_bn<KIND, false, false>(bn, ta, tb, tout, p, st);
    }
  }
  if (k == 0 && p.acc_out) cudaMemsetAsync(p.acc_out, 0, static_cast<size_t>(m) * n * 4, st);   // empty contraction
  const dim3 grid(static_cast<unsigned>(ceil_div(n, 256)), static_cast<unsigned>(m));
  if (m > 65535) return fail(BSIR_ERR_UNSUPPORTED, "matmul: unaligned operands with m > 65535");
  gemm_simple_kernel<KIND><<<grid, 256, 0, st>>>(p, o.a, o.lda, o.transpose_a, o.b, o.ldb, o.transpose_b);
  count_launch();
  return check_launch("matmul (plain path)");
}

bool is_float_param(int32_t dt) { return dt == BSIR_F32 || dt == BSIR_F16 || dt == BSIR_BF16; }

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" int64_t bsir_matmul_w8a8_workspace_bytes(int64_t, int64_t, int64_t, int32_t) { return 0; }

extern "C" int32_t bsir_matmul_w8a8(int64_t m, int64_t n, int64_t k, const int8_t *a, int64_t lda, const int8_t *b,
                                    int64_t ldb, int32_t transpose_b, const float *scale_a, const float *scale_b,
                                    int32_t out_dtype, void *out, int64_t ldo, int32_t *acc_out, void *workspace,
                                    int64_t workspace_bytes, void *stream) {
  (void)workspace;
  (void)workspace_bytes;
  clear_error();
  if (m < 0 || n < 0 || k < 0) return fail(BSIR_ERR_SHAPE, "matmul_w8a8: m=%lld n=%lld k=%lld", (long long)m, (long long)n, (long long)k);
  if (m == 0 || n == 0) return BSIR_OK;
  if (!out && !acc_out) return fail(BSIR_ERR_NULL, "matmul_w8a8: neither out nor acc_out given");
  if (k > 0 && (!a || !b)) return fail(BSIR_ERR_NULL, "matmul_w8a8: null operand");
  if (out && out_dtype != BSIR_BF16 && out_dtype != BSIR_F16) return fail(BSIR_ERR_DTYPE, "matmul_w8a8: out dtype %d (bf16 or f16)", out_dtype);
  if (lda < k || ldb < (transpose_b ? k : n) || (out && ldo < n)) return fail(BSIR_ERR_STRIDE, "matmul_w8a8: leading dimension too small");
  if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL) return fail(BSIR_ERR_SHAPE, "matmul_w8a8: dimension exceeds int32");
  if ((out && !aligned_to(out, 2)) || !aligned_to(acc_out, 4) || !aligned_to(scale_a, 4) || !aligned_to(scale_b, 4))
    return fail(BSIR_ERR_ALIGN, "matmul_w8a8: misaligned");
  GemmParams p{};
  p.m = m; p.n = n; p.k = k;
  p.scale_a = scale_a;
  p.descale = scale_b; p.descale_dtype = BSIR_F32; p.descale_mode = scale_b ? BSIR_DESCALE_PER_CHANNEL : BSIR_DESCALE_NULL;
  p.out = out; p.ldo = ldo; p.out_dtype = out_dtype;
  p.acc_out = acc_out; p.ldacc = n;
  p.err = device_error_word();
  const Operands o{a, lda, 0, b, ldb, transpose_b};
  return run_gemm<KI8>(p, o, true, resolve_stream(stream));
}

extern "C" int32_t bsir_matmul(const bsir_matmul_desc *d, void *stream) {
  clear_error();
  if (!d) return fail(BSIR_ERR_NULL, "matmul: null descriptor");
  const int32_t in = d->in_dtype;
  if (in != BSIR_I8 && in != BSIR_F16 && in != BSIR_BF16) return fail(BSIR_ERR_DTYPE, "matmul: operand dtype %d (i8, f16 or bf16)", in);
  const bool int_in = in == BSIR_I8;
  const int32_t od = d->out_dtype;
  if (!(od == BSIR_F16 || od == BSIR_BF16 || od == BSIR_F32 || od == BSIR_I8 || (od == BSIR_I32 && int_in)))
    return fail(BSIR_ERR_DTYPE, "matmul: out dtype %d (f16, bf16, f32, i8; i32 for an int8 product)", od);
  if (d->m < 0 || d->n < 0 || d->k < 0 || d->batch < 0) return fail(BSIR_ERR_SHAPE, "matmul: m=%lld n=%lld k=%lld batch=%lld", (long long)d->m, (long long)d->n, (long long)d->k, (long long)d->batch);
  if (d->m == 0 || d->n == 0 || d->batch == 0) return BSIR_OK;
  if (d->n_peers < 0 || d->n_peers > 8 || (d->n_peers > 0 && !d->peer_out)) return fail(BSIR_ERR_ARGS, "matmul: n_peers %d (0..8)", d->n_peers);
  if ((d->n_peers == 0 && !d->out) || (d->k > 0 && (!d->a || !d->b))) return fail(BSIR_ERR_NULL, "matmul: null operand");
  for (int i = 0; i < d->n_peers; ++i)
    if (!d->peer_out[i] || !aligned_to(d->peer_out[i], dtype_bytes(d->out_dtype))) return fail(BSIR_ERR_NULL, "matmul: peer_out[%d]", i);
  if (d->m > 0x7fffffffLL || d->n > 0x7fffffffLL || d->k > 0x7fffffffLL) return fail(BSIR_ERR_SHAPE, "matmul: dimension exceeds int32");
  if (d->lda < (d->transpose_a ? d->m : d->k) || d->ldb < (d->transpose_b ? d->k : d->n) || d->ldo < d->n)
    return fail(BSIR_ERR_STRIDE, "matmul: leading dimension too small");
  if (d->descale_mode < BSIR_DESCALE_NULL || d->descale_mode > BSIR_DESCALE_PER_TENSOR) return fail(BSIR_ERR_ATTR, "matmul: descale_mode %d", d->descale_mode);
  if (d->descale_mode != BSIR_DESCALE_NULL && !d->descale) return fail(BSIR_ERR_NULL, "matmul: descale_mode %d without a descale operand", d->descale_mode);
  if (d->descale_mode != BSIR_DESCALE_NULL && !is_float_param(d->descale_dtype)) return fail(BSIR_ERR_DTYPE, "matmul: descale dtype %d (f32, f16 or bf16)", d->descale_dtype);
  if (d->bias && (int_in ? d->bias_dtype != BSIR_I32 : !is_float_param(d->bias_dtype)))
    return fail(BSIR_ERR_DTYPE, "matmul: bias dtype %d (i32 with int8 operands, f32 / f16 / bf16 otherwise)", d->bias_dtype);
  const int es = int_in ? 1 : 2;
  const int os = dtype_bytes(od);
  if (!aligned_to(d->a, es) || !aligned_to(d->b, es) || (d->out && !aligned_to(d->out, os)) || !aligned_to(d->scale_a, 4) ||
      (d->bias && !aligned_to(d->bias, dtype_bytes(d->bias_dtype))) ||
      (d->descale && d->descale_mode != BSIR_DESCALE_NULL && !aligned_to(d->descale, dtype_bytes(d->descale_dtype))))
    return fail(BSIR_ERR_ALIGN, "matmul: misaligned");
  cudaStream_t st = resolve_stream(stream);
  GemmParams p{};
  p.m = d->m; p.n = d->n; p.k = d->k;
  p.scale_a = d->scale_a;
  p.descale = d->descale_mode != BSIR_DESCALE_NULL ? d->descale : nullptr;
  p.descale_dtype = d->descale_dtype; p.descale_mode = d->descale_mode;
  p.bias = d->bias; p.bias_dtype = d->bias_dtype;
  p.relu = d->relu ? 1 : 0;
  p.ldo = d->ldo; p.out_dtype = od;
  p.err = device_error_word();
  p.n_peers = d->n_peers;
  // the W8A8 form of the epilogue (what the decode kernel serves): f32 scales, no bias, no relu, 16-bit output
  const bool classic = int_in && !d->bias && !d->relu && (od == BSIR_BF16 || od == BSIR_F16) && !d->transpose_a &&
                       (d->descale_mode == BSIR_DESCALE_NULL || (d->descale_mode == BSIR_DESCALE_PER_CHANNEL && d->descale_dtype == BSIR_F32));
  // a batch of small products: one launch over rank-3 tensor maps (a launch a product leaves the GPU to one product's
  // few tiles at a time: 8 x [512,1024] x [1024,512] bf16 took 72 us on the device, product after product).  Products
  // large enough for the CTA-pair kernel, or int8 products of the decode shape, keep their kernels, one launch each.
  if (d->batch > 1 && d->n_peers == 0 && d->out && std::getenv("BSIR_GEMM_NO_BATCH_LAUNCH") == nullptr) {
    const bool pair_sized = d->m >= 192 && ceil_div(d->m, static_cast<int64_t>(256)) * ceil_div(d->n, static_cast<int64_t>(256)) >= 56;
    const bool decode_sized = classic && d->m <= 48;
    if (!pair_sized && !decode_sized) {
      p.out = d->out;
      p.out_bs = d->batch_stride_out;
      const Operands o{d->a, d->lda, d->transpose_a ? 1 : 0, d->b, d->ldb, d->transpose_b ? 1 : 0};
      int32_t rc = BSIR_OK;
      const bool done = in == BSIR_I8 ? run_gemm_batched<KI8>(p, o, d->batch, d->batch_stride_a, d->batch_stride_b, st, &rc)
                        : in == BSIR_BF16 ? run_gemm_batched<KBF16>(p, o, d->batch, d->batch_stride_a, d->batch_stride_b, st, &rc)
                                          : run_gemm_batched<KF16>(p, o, d->batch, d->batch_stride_a, d->batch_stride_b, st, &rc);
      if (done) return rc;
      p.out_bs = 0;
    }
  }
  for (int64_t e = 0; e < d->batch; ++e) {
    p.out = d->n_peers > 0 ? d->peer_out[0] : static_cast<char *>(d->out) + e * d->batch_stride_out * os;
    for (int i = 0; i < d->n_peers; ++i) p.peer[i] = static_cast<char *>(d->peer_out[i]) + e * d->batch_stride_out * os;
    if (d->n_peers > 0) p.out = p.peer[0];
    const Operands o{static_cast<const char *>(d->a) + e * d->batch_stride_a * es, d->lda, d->transpose_a ? 1 : 0,
                     static_cast<const char *>(d->b) + e * d->batch_stride_b * es, d->ldb, d->transpose_b ? 1 : 0};
    int32_t rc;
    if (in == BSIR_I8) rc = run_gemm<KI8>(p, o, classic, st);
    else if (in == BSIR_BF16) rc = run_gemm<KBF16>(p, o, false, st);
    else rc = run_gemm<KF16>(p, o, false, st);
    if (rc != BSIR_OK) return rc;
  }
  return BSIR_OK;
}
