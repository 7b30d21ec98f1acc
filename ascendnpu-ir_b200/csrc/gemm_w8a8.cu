// gemm_w8a8.cu -- linalg.matmul i8 x i8 -> i32 with the fused dequant suffix
//   out[m, n] = cast_rint( (sitofp(acc[m, n]) * scale_a[m]) * scale_b[n] )
// (int8 dot: bishengir/test/bishengir-compile/hivm/compile-dot-int8-fractal-c.mlir:25; the global
// GEMM with a descale epilogue is hivm.hir.matmul, bishengir/include/bishengir/Dialect/HIVM/IR/HIVMMacroOps.td:364-492;
// device library variants bishengir/lib/Template/lib/Cube/GlobalMmad.cpp:176-187).
//
// sm_100a design.  A persistent kernel, one CTA per SM, 192 threads in three roles:
//   warp 0     TMA producer: cp.async.bulk.tensor loads of the A tile [128 x 128 B] and the B tile
//              into a ring of shared-memory stages (128-byte swizzle), completion on mbarriers;
//   warp 1     MMA issuer: one thread issues tcgen05.mma.kind::i8 (M=128, N=BN, K=32) with the int32
//              accumulator in tensor memory; tcgen05.commit releases stages and publishes tiles;
//   warps 2-5  epilogue: tcgen05.ld the accumulator (each warp its 32 TMEM lanes), convert to f32,
//              apply both scales, round to bf16/f16, store.
// Two accumulator buffers in TMEM (2 x BN columns) let the epilogue of tile i overlap the main
// loop of tile i + 1.
//
// B comes either as [n, k] rows (transpose_b, "K-major" for the tensor core) or, as linalg.matmul has
// it, as [k, n] rows ("MN-major"): the shared-memory matrix descriptor and the instruction
// descriptor's b_major bit describe the layout, so no transpose pass is needed.
//
// Every wait on an mbarrier is bounded: after ~2 s of cycles a waiter sets the device error word
// and an abort flag that all roles poll; the CTA then drains and frees its tensor memory.
//
// Shapes the TMA path cannot address (row pitches that are not multiples of 16 bytes, unaligned
// bases) run on a plain CUDA-core kernel instead.
#include <cstdlib>
#include <mutex>

#include "tc_ptx.cuh"

namespace bsir {
namespace {

constexpr int kBM = 128;        // rows of A per tile = TMEM lanes
constexpr int kBK = 128;        // K bytes per stage (one 128-byte swizzle row)
constexpr int kUmmaK = 32;      // K per tcgen05.mma for 8-bit operands
constexpr int kThreads = 192;

struct GemmParams {
  int64_t m, n, k;
  const float *scale_a;
  const float *scale_b;
  void *out;
  int64_t ldo;
  int32_t out_dtype;
  int32_t *acc_out;
  int64_t ldacc;
  int *err;
  int m_tiles, n_tiles, k_blocks;
  int tma_out;   // 1: the output tile goes through shared memory and TMA stores
};

// ------------------------------------------------------------------ epilogue
// One accumulator tile, seen by one epilogue warp: its 32 TMEM lanes (rows) x BN columns, 32 columns at
// a time.  acc -> f32 -> * scale_a[row] -> * scale_b[col] -> bf16/f16.  The per-column scales of the
// tile sit in shared memory (sw_s); a row's 64 output bytes per chunk are written to a small
// shared-memory tile with the 64-byte TMA swizzle (conflict-free) and leave through a TMA store, so
// global memory sees whole sectors and the warp does not wait on the store.  Without TMA (odd output
// pitch) or for the int32 accumulator dump the lanes store directly.
constexpr int kEpiStageBytes = 2048;     // 32 rows x 64 bytes, two of them per warp

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y), "r"(src)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int BN>
__device__ __forceinline__ void epilogue_tile(const GemmParams &p, const CUtensorMap *tmap_out, uint32_t t_row,
                                              int64_t row, int64_t row_warp0, int64_t n0, int lane, uint8_t *stage_gen,
                                              uint32_t stage_addr, const float *sw_s, uint32_t &nstores) {
  const bool row_ok = row < p.m;
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
    uint32_t packed[16];
#pragma unroll
    for (int j4 = 0; j4 < 32; j4 += 4) {
      const float4 sw = *reinterpret_cast<const float4 *>(sw_s + c0 + j4);   // same address in every lane: broadcast
      const float swv[4] = {sw.x, sw.y, sw.z, sw.w};
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        float f0 = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int32_t>(r[j4 + j])), sa), swv[j]);
        float f1 = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int32_t>(r[j4 + j + 1])), sa), swv[j + 1]);
        if (p.out_dtype == BSIR_F16) {
          f0 = fminf(fmaxf(f0, -65504.0f), 65504.0f);
          f1 = fminf(fmaxf(f1, -65504.0f), 65504.0f);
          packed[(j4 + j) >> 1] = pack_f16x2(f0, f1);
        } else {
          packed[(j4 + j) >> 1] = pack_bf16x2(f0, f1);
        }
      }
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
      if (lane == 0) tma_store_2d(tmap_out, static_cast<int>(col0), static_cast<int>(row_warp0), stage_addr + b * kEpiStageBytes);
      ++nstores;
    } else if (row_ok) {
      uint16_t *dst = static_cast<uint16_t *>(p.out) + row * p.ldo + col0;
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
}

// Per-column scales of a tile into this warp's own shared-memory copy (no CTA-wide barrier, so a warp
// that gives up on a bounded wait can never leave the others stuck).
template <int BN>
__device__ __forceinline__ void stage_scales(const GemmParams &p, int64_t n0, float *sw_s, int lane) {
  for (int i = lane; i < BN; i += 32) sw_s[i] = (p.scale_b && n0 + i < p.n) ? p.scale_b[n0 + i] : 1.0f;
  __syncwarp();
}

template <int BN>
struct TileCfg {
  static constexpr int kStageA = kBM * kBK;           // 16 KB
  static constexpr int kStageB = BN * kBK;            // BN x 128 B
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);   // + 16.5-18 KB of epilogue staging
  static constexpr int kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;
  static constexpr int kEpiOff = kStages * kStage + 1024;                      // after the barriers (1 KB reserved)
  static constexpr int kEpiBytes = 4 * 2 * kEpiStageBytes + 4 * 2 * BN * 4;     // 4 warps x (2 store buffers + scales of two tiles)
  static constexpr int kSmemBytes = kEpiOff + kEpiBytes + 1024 /*alignment slack*/;
};

// ------------------------------------------------------------------ the kernel
template <int BN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
    w8a8_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_out, GemmParams p) {
  using Cfg = TileCfg<BN>;
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = p.m_tiles * p.n_tiles;

  pdl_launch_dependents();   // the set-up below overlaps the tail of the kernel ahead (see launch_pdl)
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
    *abort_flag = 0;
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
    // ---------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.m_tiles) * kBM;
        const int n0 = (tile / p.m_tiles) * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.err)) { ok = false; break; }
          const uint32_t sa = base + stage * Cfg::kStage;
          const uint32_t sb = sa + Cfg::kStageA;
          mbar_expect_tx(full_bar(stage), Cfg::kStage);
          tma_load_2d(sa, &tmap_a, kb * kBK, m0, full_bar(stage));
          if constexpr (B_MN) {
            // B is [k, n]: one box of [128 k rows x 128 n bytes] per 128-wide column chunk
#pragma unroll
            for (int c = 0; c < BN / 128; ++c) tma_load_2d(sb + c * (kBK * 128), &tmap_b, n0 + c * 128, kb * kBK, full_bar(stage));
          } else {
            // B is [n, k]: boxes of [128 n rows x 128 k bytes]
#pragma unroll
            for (int c = 0; c < (BN + 127) / 128; ++c)
              tma_load_2d(sb + c * (128 * kBK), &tmap_b, kb * kBK, n0 + c * 128, full_bar(stage));
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
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0) {
      // instruction descriptor: D = s32, A = B = signed int8, A K-major, B per layout, N, M
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((B_MN ? 1u : 0u) << 16) |
                             (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0u, 0u};
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * Cfg::kStage;
          const uint32_t sb = sa + Cfg::kStageA;
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            const uint64_t adesc = make_desc(sa + kk * kUmmaK, 16, 1024);
            const uint64_t bdesc = B_MN ? make_desc(sb + kk * (kUmmaK * 128), kBK * 128, 1024)
                                        : make_desc(sb + kk * kUmmaK, 16, 1024);
            mma_i8(d_tmem, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
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
    uint32_t nstores = 0;
    int acc = 0;
    uint32_t acc_phase[2] = {0u, 0u};
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int64_t m0 = static_cast<int64_t>(tile % p.m_tiles) * kBM;
      const int64_t n0 = static_cast<int64_t>(tile / p.m_tiles) * BN;
      float *sw_s = sw_all + ((warp - 2) * 2 + acc) * BN;
      stage_scales<BN>(p, n0, sw_s, lane);         // overlaps the tile's main loop
      if (!mbar_wait(tfull_bar(acc), acc_phase[acc], abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * BN);
      epilogue_tile<BN>(p, &tmap_out, t_row, m0 + row_in_tile, m0 + quad * 32, n0, lane, stage_gen, stage_addr, sw_s, nstores);
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

// ------------------------------------------------------------------ decode kernel (few rows of A)
// For m <= 128 the roles of the operands are swapped: out^T[n, m] = W^T[n, k] . a^T[k, m].  The 128
// output columns of a tile are the MMA's M (the TMEM lanes), the rows of `a`, padded to a multiple
// of 16, are its N.  A stage then holds a 16 KB weight tile and only NB x 128 bytes of activations
// instead of a 128-row activation tile that is mostly padding, so the ring is up to 11 stages deep
// and a CTA keeps ~180 KB of weight loads in flight -- this shape is bound by HBM latency x
// bandwidth per SM, not by the tensor core.  Roles and barriers as in the kernel above; the
// epilogue reads the accumulator with lanes = output columns and writes 64-byte runs per row.
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
  c.smem = static_cast<uint32_t>(c.stages * c.stage + 1024 /*barriers*/ + 1024 /*alignment slack*/);
  return c;
}

template <bool W_MN>
__global__ void __launch_bounds__(kThreads, 1)
    w8a8_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a, GemmParams p,
                       int nb, int stage_bytes, int nstages) {
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = p.n_tiles;
  const uint32_t tmem_cols = 2 * nb < 32 ? 32u : (2 * nb <= 64 ? 64u : (2 * nb <= 128 ? 128u : 256u));

  // (tile, k block) pairs of this CTA in issue order; pair `it` uses stage it % nstages
  const int my_tiles = (total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int total_its = my_tiles * p.k_blocks;
  auto issue = [&](int it) {
    const int tile = static_cast<int>(blockIdx.x) + (it / p.k_blocks) * static_cast<int>(gridDim.x);
    const int kb = it % p.k_blocks, stage = it % nstages;
    const int n0 = tile * kBM;
    const uint32_t sw = base + stage * stage_bytes;
    mbar_expect_tx(full_bar(stage), static_cast<uint32_t>(stage_bytes));
    if constexpr (W_MN) tma_load_2d(sw, &tmap_w, n0, kb * kBK, full_bar(stage));   // [128 k rows x 128 n bytes]
    else tma_load_2d(sw, &tmap_w, kb * kBK, n0, full_bar(stage));                 // [128 n rows x 128 k bytes]
    tma_load_2d(sw + kDecStageW, &tmap_a, kb * kBK, 0, full_bar(stage));          // [nb rows x 128 k bytes]
  };
  const int preissued = total_its < nstages ? total_its : nstages;
  // Programmatic dependent launch: the next kernel of the stream may be scheduled while this one runs (its
  // blocks take SMs as ours leave them), and this kernel touches global memory only after the one before it
  // has completed -- so launch latency and the barrier / tensor-memory set-up overlap the predecessor's tail.
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < nstages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    pdl_wait();
    // the first ring of loads goes out before the CTA meets: a launch this short (about 9 us of
    // transfer) cannot afford to wait for the tensor-memory allocation first
    for (int it = 0; it < preissued; ++it) issue(it);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), tmem_cols);
  if (threadIdx.x != 0) pdl_wait();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer
    if (lane == 0) {
      bool ok = true;
      for (int it = preissued; it < total_its; ++it) {
        const int stage = it % nstages;
        const uint32_t phase = static_cast<uint32_t>(it / nstages) & 1u;
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.err)) { ok = false; break; }
        issue(it);
      }
      if (!ok) {
        for (int s = 0; s < nstages; ++s)
          for (int i = 0; i < 200000; ++i)
            if (mbar_try_wait(full_bar(s), 0) || mbar_try_wait(full_bar(s), 1)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0) {
      // D = s32, A (weights) and B (activations) signed int8; A's major per the weight layout; N = nb, M = 128
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((W_MN ? 1u : 0u) << 15) |
                             (static_cast<uint32_t>(nb >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0u, 0u};
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * nb);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = base + stage * stage_bytes;
          const uint32_t sa = sw + kDecStageW;
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            const uint64_t wdesc = W_MN ? make_desc(sw + kk * (kUmmaK * 128), kBK * 128, 1024) : make_desc(sw + kk * kUmmaK, 16, 1024);
            const uint64_t adesc = make_desc(sa + kk * kUmmaK, 16, 1024);
            mma_i8(d_tmem, wdesc, adesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));
          if (++stage == nstages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(tfull_bar(acc));
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
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int64_t col = static_cast<int64_t>(tile) * kBM + quad * 32 + lane;
      const bool col_ok = col < p.n;
      const float sw = (p.scale_b && col_ok) ? p.scale_b[col] : 1.0f;
      const float sa_lane = (p.scale_a && lane < p.m) ? p.scale_a[lane] : 1.0f;   // rows 0..31, one per lane
      if (!mbar_wait(tfull_bar(acc), acc_phase[acc], abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * nb);
      for (int c0 = 0; c0 < nb; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(t_row + static_cast<uint32_t>(c0), r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int64_t row = c0 + j;
          if (row >= p.m) break;               // uniform over the warp
          const int32_t v = static_cast<int32_t>(r[j]);
          // all lanes take part in the shuffle (row is uniform over the warp)
          const float sa = row < 32 ? __shfl_sync(0xffffffffu, sa_lane, static_cast<int>(row)) : (p.scale_a ? __ldg(p.scale_a + row) : 1.0f);
          if (p.acc_out && col_ok) p.acc_out[row * p.ldacc + col] = v;
          if (p.out && col_ok) {
            float f = __fmul_rn(__fmul_rn(static_cast<float>(v), sa), sw);
            uint16_t bits;
            if (p.out_dtype == BSIR_F16) {
              f = fminf(fmaxf(f, -65504.0f), 65504.0f);
              bits = static_cast<uint16_t>(pack_f16x2(f, 0.0f) & 0xffffu);
            } else {
              bits = static_cast<uint16_t>(pack_bf16x2(f, 0.0f) & 0xffffu);
            }
            static_cast<uint16_t *>(p.out)[row * p.ldo + col] = bits;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
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
// 128-deep K block instead of 48 KB, and half as many MMA instructions per flop for the issuing
// thread -- the two things that bound the single-CTA kernel.  Only the leader (cluster rank 0)
// issues MMAs; both CTAs' TMA loads complete on the leader's barrier; tcgen05.commit multicasts the
// "stage free" and "accumulator ready" arrivals to both CTAs (no TMA load is multicast).
constexpr int kPairStages = 6;
constexpr int kPairStageA = kBM * kBK;          // 16 KB: this CTA's 128 rows of A
constexpr int kPairStageB = 128 * kBK;          // 16 KB: this CTA's 128 columns of B
constexpr int kPairStage = kPairStageA + kPairStageB;
constexpr int kPairEpiOff = kPairStages * kPairStage + 1024;   // barriers get 1 KB
constexpr int kPairSmem = kPairEpiOff + 4 * 2 * kEpiStageBytes + 4 * 2 * 256 * 4 + 1024;
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
__device__ __forceinline__ void mma_i8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    w8a8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_out, GemmParams p) {
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int m_tiles2 = (p.m_tiles + 1) / 2;            // tiles of 256 rows
  const int total_tiles = m_tiles2 * p.n_tiles;         // p.n_tiles counts 256-wide tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }
    *abort_flag = 0;
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
          tma_load_2d_pair(sa, &tmap_a, kb * kBK, m0, leader_full);
          if constexpr (B_MN) tma_load_2d_pair(sb, &tmap_b, n0, kb * kBK, leader_full);
          else tma_load_2d_pair(sb, &tmap_b, kb * kBK, n0, leader_full);
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: leader CTA only
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((B_MN ? 1u : 0u) << 16) |
                             (static_cast<uint32_t>(kPairBN >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0u, 0u};
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += npairs) {
        if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kPairBN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * kPairStage;
          const uint32_t sb = sa + kPairStageA;
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            const uint64_t adesc = make_desc(sa + kk * kUmmaK, 16, 1024);
            const uint64_t bdesc = B_MN ? make_desc(sb + kk * (kUmmaK * 128), kBK * 128, 1024)
                                        : make_desc(sb + kk * kUmmaK, 16, 1024);
            mma_i8_pair(d_tmem, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
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
    uint32_t nstores = 0;
    int acc = 0;
    uint32_t acc_phase[2] = {0u, 0u};
    bool ok = true;
    for (int tile = pair; tile < total_tiles && ok; tile += npairs) {
      const int64_t m0 = static_cast<int64_t>(tile % m_tiles2) * 256 + static_cast<int64_t>(rank) * 128;
      const int64_t n0 = static_cast<int64_t>(tile / m_tiles2) * kPairBN;
      float *sw_s = sw_all + ((warp - 2) * 2 + acc) * kPairBN;
      stage_scales<kPairBN>(p, n0, sw_s, lane);
      if (!mbar_wait(tfull_bar(acc), acc_phase[acc], abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * kPairBN);
      epilogue_tile<kPairBN>(p, &tmap_out, t_row, m0 + row_in_tile, m0 + quad * 32, n0, lane, stage_gen, stage_addr, sw_s, nstores);
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

// ------------------------------------------------------------------ plain fallback (any layout)
__global__ void __launch_bounds__(256) w8a8_simple_kernel(GemmParams p, const int8_t *__restrict__ a, int64_t lda,
                                                          const int8_t *__restrict__ b, int64_t ldb, int transpose_b) {
  const int64_t col = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t row = blockIdx.y;
  if (col >= p.n || row >= p.m) return;
  int32_t acc = 0;
  const int8_t *ar = a + row * lda;
  if (transpose_b) {
    const int8_t *br = b + col * ldb;
    for (int64_t kk = 0; kk < p.k; ++kk) acc += static_cast<int32_t>(ar[kk]) * static_cast<int32_t>(br[kk]);
  } else {
    for (int64_t kk = 0; kk < p.k; ++kk) acc += static_cast<int32_t>(ar[kk]) * static_cast<int32_t>(b[kk * ldb + col]);
  }
  if (p.acc_out) p.acc_out[row * p.ldacc + col] = acc;
  if (p.out) {
    float f = static_cast<float>(acc);
    if (p.scale_a) f = __fmul_rn(f, p.scale_a[row]);
    if (p.scale_b) f = __fmul_rn(f, p.scale_b[col]);
    uint16_t *dst = static_cast<uint16_t *>(p.out) + row * p.ldo + col;
    if (p.out_dtype == BSIR_F16) *dst = __half_as_ushort(__float2half_rn(fminf(fmaxf(f, -65504.0f), 65504.0f)));
    else *dst = __bfloat16_as_ushort(__float2bfloat16_rn(f));
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

// 2-D uint8 tensor map: `inner` contiguous bytes per row, `outer` rows of pitch `pitch` bytes,
// box = [box_rows x 128 bytes], 128-byte swizzle, out-of-range bytes read as zero.
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

template <int BN, bool B_MN>
int32_t launch_tc(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tout, GemmParams p, cudaStream_t st) {
  using Cfg = TileCfg<BN>;
  // the attribute is per device and cheap to set
  cudaFuncSetAttribute(w8a8_tc_kernel<BN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  p.n_tiles = static_cast<int>(ceil_div(p.n, BN));
  const int total = p.m_tiles * p.n_tiles;
  int grid = device_info().sm_count > 0 ? device_info().sm_count : 148;
  if (grid > total) grid = total;
  launch_pdl(w8a8_tc_kernel<BN, B_MN>, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, st, ta, tb, tout, p);
  count_launch();
  return check_launch("matmul_w8a8");
}

// Tile width: the widest N tile whose tile count still covers the SMs reasonably.
int pick_bn(int64_t m, int64_t n, int sm_count, bool b_mn) {
  const int64_t m_tiles = ceil_div(m, kBM);
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
  cudaStream_t st = resolve_stream(stream);
  GemmParams p{};
  p.m = m; p.n = n; p.k = k;
  p.scale_a = scale_a; p.scale_b = scale_b;
  p.out = out; p.ldo = ldo; p.out_dtype = out_dtype;
  p.acc_out = acc_out; p.ldacc = n;
  p.err = device_error_word();
  p.m_tiles = static_cast<int>(ceil_div(m, kBM));
  p.k_blocks = static_cast<int>(ceil_div(k, kBK));

  const bool tma_ok = k > 0 && device_info().cc_major >= 10 && aligned_to(a, 16) && aligned_to(b, 16) && lda % 16 == 0 &&
                      ldb % 16 == 0 && encode_fn() != nullptr;
  if (tma_ok) {
    CUtensorMap ta, tb, tout;
    memset(&tout, 0, sizeof(tout));
    p.tma_out = (out && aligned_to(out, 16) && ldo % 8 == 0 && make_out_tmap(&tout, out, static_cast<uint64_t>(n), static_cast<uint64_t>(m), static_cast<uint64_t>(ldo))) ? 1 : 0;
    const bool b_mn = !transpose_b;
    const int bn = pick_bn(m, n, device_info().sm_count > 0 ? device_info().sm_count : 148, b_mn);
    bool ok = make_tmap(&ta, a, static_cast<uint64_t>(k), static_cast<uint64_t>(m), static_cast<uint64_t>(lda), kBM);
    if (b_mn) ok = ok && make_tmap(&tb, b, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(ldb), kBK);
    else ok = ok && make_tmap(&tb, b, static_cast<uint64_t>(k), static_cast<uint64_t>(n), static_cast<uint64_t>(ldb), bn < 128 ? bn : 128);
    const char *force = std::getenv("BSIR_W8A8_PATH");
    // BSIR_W8A8_PATH=1 / 2 forces the single-CTA / CTA-pair kernel (tests use it on small shapes)
    const bool want_pair = (force && force[0] == '2') ||
                           (!(force && force[0] == '1') && m >= 512 && ceil_div(m, 256) * ceil_div(n, 256) >= 74);
    if (ok && want_pair) {
      // CTA pairs: A boxes of 128 rows as before; B boxes of 128 columns (MN-major) / 128 rows (K-major)
      CUtensorMap tb2;
      bool ok2 = b_mn ? make_tmap(&tb2, b, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(ldb), kBK)
                      : make_tmap(&tb2, b, static_cast<uint64_t>(k), static_cast<uint64_t>(n), static_cast<uint64_t>(ldb), 128);
      if (ok2) {
        p.n_tiles = static_cast<int>(ceil_div(n, kPairBN));
        int sms = device_info().sm_count > 0 ? device_info().sm_count : 148;
        int grid = sms & ~1;
        const int total = static_cast<int>(ceil_div(m, 256)) * p.n_tiles;
        if (grid > 2 * total) grid = 2 * total;
        if (b_mn) {
          cudaFuncSetAttribute(w8a8_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
          w8a8_pair_kernel<true><<<grid, kThreads, kPairSmem, st>>>(ta, tb2, tout, p);
        } else {
          cudaFuncSetAttribute(w8a8_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
          w8a8_pair_kernel<false><<<grid, kThreads, kPairSmem, st>>>(ta, tb2, tout, p);
        }
        count_launch();
        return check_launch("matmul_w8a8 (CTA pairs)");
      }
    }
    // few rows: operands swapped, deep ring of weight tiles (BSIR_W8A8_PATH=3 forces it for m <= 128, =1 avoids it)
    // measured on B200 (k 4096, n 14336): 13.5-16 us against 19-20 us for m <= 24, slower from m = 32 on
    const bool want_decode = (force && force[0] == '3') ? m <= 128 : (!force && m <= 24);
    if (ok && want_decode) {
      const DecodeCfg dc = decode_cfg(m);
      CUtensorMap tw, tact;
      bool ok3 = b_mn ? make_tmap(&tw, b, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(ldb), kBK)
                      : make_tmap(&tw, b, static_cast<uint64_t>(k), static_cast<uint64_t>(n), static_cast<uint64_t>(ldb), kBM);
      ok3 = ok3 && make_tmap(&tact, a, static_cast<uint64_t>(k), static_cast<uint64_t>(m), static_cast<uint64_t>(lda), static_cast<uint32_t>(dc.nb));
      if (ok3) {
        p.n_tiles = static_cast<int>(ceil_div(n, kBM));
        int grid = device_info().sm_count > 0 ? device_info().sm_count : 148;
        if (grid > p.n_tiles) grid = p.n_tiles;
        if (b_mn) {
          cudaFuncSetAttribute(w8a8_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dc.smem));
          launch_pdl(w8a8_decode_kernel<true>, dim3(grid), dim3(kThreads), dc.smem, st, tw, tact, p, dc.nb, dc.stage, dc.stages);
        } else {
          cudaFuncSetAttribute(w8a8_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dc.smem));
          launch_pdl(w8a8_decode_kernel<false>, dim3(grid), dim3(kThreads), dc.smem, st, tw, tact, p, dc.nb, dc.stage, dc.stages);
        }
        count_launch();
        return check_launch("matmul_w8a8 (decode)");
      }
    }
    if (ok) {
      if (b_mn) return bn == 256 ? launch_tc<256, true>(ta, tb, tout, p, st) : launch_tc<128, true>(ta, tb, tout, p, st);
      return bn == 256 ? launch_tc<256, false>(ta, tb, tout, p, st)
                       : bn == 128 ? launch_tc<128, false>(ta, tb, tout, p, st) : launch_tc<64, false>(ta, tb, tout, p, st);
    }
  }
  if (k == 0) {
    // empty contraction: accumulators are zero
    if (acc_out) cudaMemsetAsync(acc_out, 0, static_cast<size_t>(m) * n * 4, st);
  }
  const dim3 grid(static_cast<unsigned>(ceil_div(n, 256)), static_cast<unsigned>(m));
  if (m > 65535) return fail(BSIR_ERR_UNSUPPORTED, "matmul_w8a8: unaligned operands with m > 65535");
  w8a8_simple_kernel<<<grid, 256, 0, st>>>(p, a, lda, b, ldb, transpose_b);
  count_launch();
  return check_launch("matmul_w8a8 (plain path)");
}
