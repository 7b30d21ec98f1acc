// gemm_w4a16.cu -- W4A16 group-quantised GEMM for decode-sized M (memory-bound on the weights):
//   w[k, n]  = cast_rint_bf16( (q[k, n] - z[k / group, n]) * s[k / group, n] )
//   out[m,n] = cast_rint_bf16( sum_k a[m, k] * w[k, n] ),  f32 accumulation.
// The reference has no group-dequant primitive; this is the composed prefix (i4 -> f32, subtract,
// multiply by the broadcast scale, cast) in front of linalg.matmul (int4 support in the reference:
// vcast i4 <-> f16, bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:574; the `enable_i4`
// mmad mark, bishengir/lib/Conversion/HFusionToHIVM/Matmul.cpp:199-206).  The packing is this
// project's: qweight int32 [k/8, n], nibble t of word (r, c) = q[8r + t, c]; scales bf16 [k/group, n];
// zeros int32 [k/group, n/8], nibble t of word (g, c) = z[g, 8c + t].
//
// Streaming kernel (w4a16_mma_kernel).  One CTA owns 64 output columns and all of K; its 8 warps take
// contiguous K slices and meet in shared memory at the end.  A thread streams 16-byte pieces of
// qweight (4 columns x 8 k values), dequantises in registers with packed bf16 arithmetic and feeds
// mma.sync.m16n8k16 with the weights as the A operand (see the kernel's comment):
//   (word >> 4i) & 0x000F000F | 0x43004300 is the bf16 pair (128 + q[k_i], 128 + q[k_i+4]);
//   subtracting (128 + z) is exact and the product with s rounds once, exactly like the f32
//   computation it restates ((q - z) * s needs 13 bits).
// The k order inside an MMA is free as long as both operands use the same one, so the nibble pairs
// (i, i + 4) are taken as they come and the activations' 8-element pieces are permuted to match with
// two byte permutes.  Row blocks of 9..16 rows run the tensor-memory kernel further down; larger M
// runs once per 16 rows (decode path; large M belongs on a dense GEMM).
#include <cstdlib>
#include <mutex>

#include "tc_ptx.cuh"

namespace bsir {
namespace {

constexpr int kWarps = 8;
constexpr int kPrefetch = 4;  // k32 steps of weights in flight per warp

struct W4Params {
  int64_t m, n, k, group;
  const uint16_t *a;
  int64_t lda;
  const uint32_t *qw;
  const uint16_t *scales;
  const uint32_t *zeros;
  uint16_t *out;
  int64_t ldo;
  int n_peers;          // > 0: every store of the result goes to each of peer[0 .. n_peers) instead of `out`
  uint16_t *peer[8];
};
__device__ __forceinline__ void store_out(const W4Params &p, int64_t index, uint16_t bits) {
  if (p.n_peers == 0) { p.out[index] = bits; return; }
  for (int d = 0; d < p.n_peers; ++d) p.peer[d][index] = bits;
}

__device__ __forceinline__ void mma_bf16_16816(float *c, const uint32_t *a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// (w >> shift) & 0x000f000f | 0x43004300 as one lop3: written as separate and / or the assembler
// keeps two instructions (measured: one more instruction per nibble pair).
__device__ __forceinline__ uint32_t nibble_pair_bf16(uint32_t w, int shift) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w >> shift), "r"(0x000f000fu), "r"(0x43004300u));
  return r;
}
__device__ __forceinline__ uint4 ldg_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// out^T = W^T . a^T on mma.sync.m16n8k16: the dequantised weights are the MMA's A operand (16 output
// columns x 16 k), the activations its B operand (16 k x 8 rows of `a`).  A lane holds weight words of
// four adjacent columns (one 16-byte piece = 4 columns x 8 k); columns (c0, c1) and (c2, c3) are the
// tile rows (g, g + 8) of two MMA tiles, and the two nibble-pair halves of a word are two k blocks.
// Lane (g, t) supplies k = 8 t + {0,4,1,5} (first MMA) and 8 t + {2,6,3,7} (second) of the 32-k step,
// and reads the activation row g at exactly those k (one 16-byte load, two byte permutes per MMA).
// MT = number of 8-row blocks of `a` (1 for m <= 8: the decode case needs half the MMAs and accumulators).
template <int NP, int MT>
__global__ void __launch_bounds__(kWarps * 32, NP == 1 ? 3 : 2) w4a16_mma_kernel(W4Params p, int64_t m0) {
  constexpr int kCols = 32 * NP;   // output columns per CTA
  __shared__ float red[kWarps][8 * MT][kCols + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t col_base = static_cast<int64_t>(blockIdx.x) * kCols;
  const int steps = static_cast<int>(p.k / 32);
  const int per_warp = (steps + kWarps - 1) / kWarps;
  const int s_begin = min(steps, warp * per_warp);
  const int s_end = min(steps, s_begin + per_warp);
  const int64_t rows_left = p.m - m0;
  pdl_launch_dependents();   // the next launch may be scheduled while this one runs (launch_pdl) ...
  pdl_wait();                // ... and this one reads global memory only after the kernel ahead has completed

  // this thread's columns: piece j covers col_base + 32 j + 4 g + {0..3}; n is a multiple of 8, so a
  // piece is all in or all out.  Everything is addressed through pointers that advance by a fixed
  // stride (weights: one step = 4 word rows; scales / zeros: one group), counters are 32-bit.
  bool col_ok[NP];
  const uint32_t *wp[NP];       // weights of the step kPrefetch ahead
  const uint16_t *sp[NP];       // scales of the next group
  const uint32_t *zp[NP];       // zero words of the next group
  int zshift[NP];
  const int64_t wstride = 4 * p.n;
  const int steps_per_group = static_cast<int>(p.group / 32);
  const int first_group = s_begin / steps_per_group;
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    const int64_t c = col_base + 32 * j + 4 * g;
    col_ok[j] = c < p.n;
    const int64_t cc = col_ok[j] ? c : 0;
    wp[j] = p.qw + (static_cast<int64_t>(s_begin) * 4 + t) * p.n + cc;
    sp[j] = p.scales + static_cast<int64_t>(first_group) * p.n + cc;
    zp[j] = p.zeros + static_cast<int64_t>(first_group) * (p.n / 8) + cc / 8;
    zshift[j] = 4 * static_cast<int>(cc % 8);
  }
  bool row_ok[MT];
  const uint16_t *ap[MT];
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    row_ok[r] = g + 8 * r < rows_left;
    ap[r] = p.a + (m0 + (row_ok[r] ? g + 8 * r : 0)) * p.lda + static_cast<int64_t>(s_begin) * 32 + 8 * t;
  }

  float acc[NP][2][MT][4];   // [piece][column pair][row block][d0..d3]
#pragma unroll
  for (int j = 0; j < NP; ++j)
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2)
#pragma unroll
      for (int r = 0; r < MT; ++r)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][c2][r][e] = 0.0f;

  // Everything a step needs is requested ahead of its use: weights kPrefetch steps ahead, the
  // activations one step ahead, the scales and zero points one group ahead.  A warp runs only
  // k / (32 * kWarps) steps, so a single exposed round trip per step or per group would dominate.
  int loads_left = s_end - s_begin;     // weight steps not yet requested
  auto load_pieces = [&](uint4 (&dst)[NP]) {
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      dst[j] = make_uint4(0u, 0u, 0u, 0u);
      if (loads_left > 0 && col_ok[j]) dst[j] = ldg_stream16(wp[j]);
      wp[j] += wstride;
    }
    --loads_left;
  };
  uint4 pre[kPrefetch][NP];
#pragma unroll
  for (int d = 0; d < kPrefetch; ++d) load_pieces(pre[d]);

  int groups_left = s_begin < s_end ? (s_end - 1) / steps_per_group - first_group + 1 : 0;
  uint2 next_sc[NP];
  uint32_t next_zw[NP];
  auto load_group = [&]() {
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      next_sc[j] = make_uint2(0u, 0u);
      next_zw[j] = 0u;
      if (groups_left > 0 && col_ok[j]) {
        next_sc[j] = __ldg(reinterpret_cast<const uint2 *>(sp[j]));
        next_zw[j] = __ldg(zp[j]) >> zshift[j];
      }
      sp[j] += p.n;
      zp[j] += p.n / 8;
    }
    --groups_left;
  };
  int a_left = s_end - s_begin;
  uint4 next_a[MT];
  auto load_a = [&]() {
#pragma unroll
    for (int r = 0; r < MT; ++r) {
      next_a[r] = make_uint4(0u, 0u, 0u, 0u);
      if (a_left > 0 && row_ok[r]) next_a[r] = __ldg(reinterpret_cast<const uint4 *>(ap[r]));
      ap[r] += 32;
    }
    --a_left;
  };
  // The activation and scale loads further down are only one step / one group ahead of their use,
  // far less than an L2 round trip: ask for all of this warp's lines now, so that they hit in L1.
  for (int sidx = 1; sidx < s_end - s_begin; ++sidx) {
#pragma unroll
    for (int r = 0; r < MT; ++r)
      if (row_ok[r]) asm volatile("prefetch.global.L1 [%0];" ::"l"(ap[r] + 32 * sidx));
  }
  for (int gi = 1; gi < groups_left; ++gi) {
#pragma unroll
    for (int j = 0; j < NP; ++j)
      if (col_ok[j]) {
        asm volatile("prefetch.global.L1 [%0];" ::"l"(sp[j] + gi * p.n));
        asm volatile("prefetch.global.L1 [%0];" ::"l"(zp[j] + gi * (p.n / 8)));
      }
  }
  load_group();
  load_a();

  uint32_t zz[NP][4], ss[NP][4];  // per column: bf16x2 (128 + z, 128 + z) and (s, s)
  int to_group_end = 0;           // steps left in the current group

  for (int base = s_begin; base < s_end; base += kPrefetch) {
#pragma unroll
    for (int d = 0; d < kPrefetch; ++d) {
      const int step = base + d;
      if (step >= s_end) break;
      // weights of this step; refill the slot with the step kPrefetch ahead
      uint4 w[NP];
#pragma unroll
      for (int j = 0; j < NP; ++j) w[j] = pre[d][j];
      load_pieces(pre[d]);
      if (to_group_end == 0) {
        to_group_end = steps_per_group - step % steps_per_group;
#pragma unroll
        for (int j = 0; j < NP; ++j) {
          const uint32_t s01[4] = {next_sc[j].x & 0xffffu, next_sc[j].x >> 16, next_sc[j].y & 0xffffu, next_sc[j].y >> 16};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            ss[j][i] = s01[i] | (s01[i] << 16);
            const uint32_t z = (next_zw[j] >> (4 * i)) & 0xfu;
            zz[j][i] = (0x4300u | z) * 0x00010001u;
          }
        }
        load_group();
      }
      --to_group_end;
      // activations of row g (+8): 8 consecutive k as the pairs (e0,e4) (e1,e5) | (e2,e6) (e3,e7)
      uint32_t fb[MT][2][2];   // [row block][k block][b0, b1]
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        const uint4 ra = next_a[r];
        fb[r][0][0] = __byte_perm(ra.x, ra.z, 0x5410);
        fb[r][0][1] = __byte_perm(ra.x, ra.z, 0x7632);
        fb[r][1][0] = __byte_perm(ra.y, ra.w, 0x5410);
        fb[r][1][1] = __byte_perm(ra.y, ra.w, 0x7632);
      }
      load_a();
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        const uint32_t words[4] = {w[j].x, w[j].y, w[j].z, w[j].w};
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t dq[2][4];   // [column of the pair][nibble pair q]: (k_q, k_{q+4})
#pragma unroll
          for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint32_t v = nibble_pair_bf16(words[2 * c2 + i], 4 * q);  // (128 + q_k, 128 + q_{k+4})
              dq[i][q] = bf16x2_mul(bf16x2_sub(v, zz[j][2 * c2 + i]), ss[j][2 * c2 + i]);
            }
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
            // A fragment: a0 (row g, k 2t..) a1 (row g+8, k 2t..) a2 (row g, k 2t+8..) a3 (row g+8, k 2t+8..)
            const uint32_t fa[4] = {dq[0][2 * kb], dq[1][2 * kb], dq[0][2 * kb + 1], dq[1][2 * kb + 1]};
#pragma unroll
            for (int r = 0; r < MT; ++r) mma_bf16_16816(acc[j][c2][r], fa, fb[r][kb][0], fb[r][kb][1]);
          }
        }
      }
    }
  }

  // D fragment: d0,d1 -> tile row g (column word 2 c2), rows 2t, 2t+1 of `a`; d2,d3 -> tile row g+8
  // (column word 2 c2 + 1).  CTA column of (piece j, word i) = 32 j + 4 g + i.
#pragma unroll
  for (int j = 0; j < NP; ++j)
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2)
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        const int c0 = 32 * j + 4 * g + 2 * c2, mr = 8 * r + 2 * t;
        red[warp][mr][c0] = acc[j][c2][r][0];
        red[warp][mr + 1][c0] = acc[j][c2][r][1];
        red[warp][mr][c0 + 1] = acc[j][c2][r][2];
        red[warp][mr + 1][c0 + 1] = acc[j][c2][r][3];
      }
  __syncthreads();
  for (int o = threadIdx.x; o < 8 * MT * kCols; o += kWarps * 32) {
    const int r = o / kCols, c = o % kCols;
    if (r >= rows_left || col_base + c >= p.n) continue;
    float s = 0.0f;
#pragma unroll
    for (int wq = 0; wq < kWarps; ++wq) s += red[wq][r][c];
    store_out(p, (m0 + r) * p.ldo + col_base + c, __bfloat16_as_ushort(__float2bfloat16_rn(s)));
  }
}

// ------------------------------------------------------------------ tensor-memory path (tcgen05)
// out^T[n, m] = W^T[n, k] . a^T[k, m]: the 128 output columns of a CTA are the 128 lanes of tensor
// memory, the (at most 16) rows of `a` are the MMA's N.  Roles in a CTA of 672 threads:
//   warp 16     TMA producer.  A stage of the ring holds 256 k: one box of packed weights
//               [32 word rows x 128 columns] (16 KB) and four boxes of activations [16 rows x 64 k]
//               (2 KB each, 128-byte swizzle: the tensor core's K-major layout as TMA writes it);
//   warps 0-15  dequantisers: thread = one output column.  Each reads its column's words from the
//               stage, turns every word into four bf16 pairs (k_i, k_i+4) and stores them into its own
//               TMEM lane (tcgen05.st); warp w owns lane quadrant w % 4 and chunk w / 4 of every stage;
//   warps 17-20 first put every 16-byte piece of the stage's activations into the pair order the nibble
//               trick produces (k 0,4,1,5,2,6,3,7; in place, the swizzle only moves whole pieces), then
//               one thread per warp issues tcgen05.mma.kind::f16 for its chunk: A operand from tensor
//               memory, B = the activations in the stage, f32 accumulator in tensor memory.
// Nothing is staged up front except the scales and zero points, so the ring is as deep as shared
// memory allows (8 stages = 128 KB of weight loads in flight per SM): the shape is bound by HBM
// latency x bandwidth per SM.  All waits are bounded.
constexpr int kTcCols = 128;            // output columns per CTA
constexpr int kTcStageRows = 32;        // word rows per weight stage (= 256 k)
constexpr int kTcWeightBytes = kTcStageRows * kTcCols * 4;   // 16 KB
constexpr int kTcActBytes = 4 * 2048;                        // four chunks of 16 rows x 128 B
constexpr int kTcStageBytes = kTcWeightBytes + kTcActBytes;  // 24 KB
constexpr int kTcMaxStages = 8;
constexpr int kTcABufs = 8;             // 64-k chunks of dequantised weights in TMEM (8 x 32 columns)
constexpr int kTcDqWarps = 16;          // dequantising warps: 4 lane quadrants x 4 chunks of a stage
constexpr int kTcMmaWarps = 4;          // fix-up + MMA-issuing warps; chunk c belongs to issuer c % 4
constexpr int kTcFixWarps = 4;          // warps that put the activations into the nibble-pair order
constexpr int kTcThreads = (kTcDqWarps + 1 + kTcMmaWarps + kTcFixWarps) * 32;
constexpr int kTcSmemBudget = 222 * 1024;

struct TcLayout {
  int stages;
  uint32_t sc_off, zp_off, bar_off, bytes;
};
__host__ __device__ inline TcLayout tc_layout(int64_t k, int64_t group) {
  TcLayout L;
  const uint32_t ngroups = static_cast<uint32_t>(k / group);
  const uint32_t tail = ngroups * kTcCols * 2u + ngroups * 64u + 512u;   // scales, zero words, barriers
  int st = static_cast<int>((kTcSmemBudget - 1024 - static_cast<int>(tail)) / kTcStageBytes);
  L.stages = st > kTcMaxStages ? kTcMaxStages : st;
  L.sc_off = static_cast<uint32_t>(L.stages > 0 ? L.stages : 0) * kTcStageBytes;
  L.zp_off = L.sc_off + ngroups * kTcCols * 2u;
  L.bar_off = (L.zp_off + ngroups * 64u + 15u) & ~15u;
  L.bytes = L.bar_off + 512u + 1024u;
  return L;
}

__global__ void __launch_bounds__(kTcThreads, 1)
    w4a16_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a, W4Params p,
                    int64_t m0, int *err) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gen = smem_raw + (base - raw);
  const TcLayout L = tc_layout(p.k, p.group);
  const int nstages = L.stages;
  const int nchunks = static_cast<int>(p.k / 64);
  const int ngroups = static_cast<int>(p.k / p.group);
  const uint32_t bars = base + L.bar_off;
  auto wfull = [&](int s) { return bars + 8u * s; };
  auto wempty = [&](int s) { return bars + 8u * (kTcMaxStages + s); };
  auto aready = [&](int s) { return bars + 8u * (2 * kTcMaxStages + s); };
  auto afull = [&](int b) { return bars + 8u * (3 * kTcMaxStages + b); };
  auto aempty = [&](int b) { return bars + 8u * (3 * kTcMaxStages + kTcABufs + b); };
  const uint32_t dfull = bars + 8u * (3 * kTcMaxStages + 2 * kTcABufs);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(gen + L.bar_off + 8 * (3 * kTcMaxStages + 2 * kTcABufs + 1));
  uint16_t *sm_scales = reinterpret_cast<uint16_t *>(gen + L.sc_off);
  uint32_t *sm_zeros = reinterpret_cast<uint32_t *>(gen + L.zp_off);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kTcCols;
  const int nstages_total = (nchunks + 3) / 4;   // stages of 4 chunks

  auto issue_stage = [&](int s) {
    const int slot = s % nstages;
    const uint32_t dst = base + slot * kTcStageBytes;
    mbar_expect_tx(wfull(slot), kTcStageBytes);
    tma_load_2d(dst, &tmap_w, static_cast<int>(n0), s * kTcStageRows, wfull(slot));
#pragma unroll
    for (int c = 0; c < 4; ++c)
      tma_load_2d(dst + kTcWeightBytes + c * 2048, &tmap_a, (s * 4 + c) * 64, static_cast<int>(m0), wfull(slot));
  };
  const int preissued = nstages_total < nstages ? nstages_total : nstages;
  pdl_launch_dependents();   // barrier set-up and the tensor-memory allocation overlap the kernel ahead (launch_pdl)
  if (warp == kTcDqWarps && lane == 0) {
    for (int s = 0; s < nstages; ++s) {
      mbar_init(wfull(s), 1);
      mbar_init(wempty(s), kTcDqWarps + kTcMmaWarps);
      mbar_init(aready(s), kTcFixWarps * 32);
    }
    for (int b = 0; b < kTcABufs; ++b) { mbar_init(afull(b), 4); mbar_init(aempty(b), 1); }
    mbar_init(dfull, kTcMmaWarps);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    pdl_wait();
    // the first ring of loads goes out before the CTA meets
    for (int s = 0; s < preissued; ++s) issue_stage(s);
  } else {
    if (warp == kTcDqWarps + 1) tmem_alloc(smem_u32(tmem_slot), 512);
    pdl_wait();              // global memory is read from here on
  }
  // scales and zero points of all groups of this CTA's columns, every load issued before the first store
  {
    const int nvec = ngroups * (kTcCols / 8);                 // 8 bf16 per vector
    for (int i0 = threadIdx.x; i0 < nvec; i0 += 2 * kTcThreads) {
      uint4 sv[2];
      uint32_t zv[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = i0 + u * kTcThreads;
        const int gi = i / (kTcCols / 8), c8 = i % (kTcCols / 8);
        sv[u] = make_uint4(0u, 0u, 0u, 0u);
        zv[u] = 0u;
        if (i < nvec && n0 + 8 * c8 < p.n) {
          sv[u] = *reinterpret_cast<const uint4 *>(p.scales + static_cast<int64_t>(gi) * p.n + n0 + 8 * c8);
          zv[u] = p.zeros[static_cast<int64_t>(gi) * (p.n / 8) + n0 / 8 + c8];
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = i0 + u * kTcThreads;
        if (i < nvec) {
          reinterpret_cast<uint4 *>(sm_scales)[i] = sv[u];
          sm_zeros[i] = zv[u];
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // One f32 accumulator (16 columns) per issuing warp; the epilogue adds them.  A tcgen05.mma costs its
  // issuing thread ~70 cycles and a commit ~130 whatever the MMA's size, and these MMAs are tiny
  // (128 x 16 x 16), so a single issuer would be the bottleneck: four warps issue side by side.
  const uint32_t tmem_d = tmem_base;            // columns 0..63
  const uint32_t tmem_a0 = tmem_base + 64;      // kTcABufs x 32 columns of packed bf16 pairs

  if (warp == kTcDqWarps) {
    if (lane == 0) {
      bool ok = true;
      int slot = preissued % nstages;
      uint32_t phase = static_cast<uint32_t>(preissued / nstages) & 1u;
      for (int s = preissued; s < nstages_total; ++s) {
        if (!mbar_wait_relaxed(wempty(slot), phase ^ 1u, abort_flag, err)) { ok = false; break; }
        issue_stage(s);
        if (++slot == nstages) { slot = 0; phase ^= 1u; }
      }
      if (!ok)
        for (int s = 0; s < nstages; ++s)
          for (int i = 0; i < 200000; ++i)
            if (mbar_try_wait(wfull(s), 0) || mbar_try_wait(wfull(s), 1)) break;
    }
  } else if (warp > kTcDqWarps + kTcMmaWarps) {
    // ---------------- activation fix-up: every 16-byte piece of the stage into the nibble-pair k order
    const int tix = (warp - kTcDqWarps - kTcMmaWarps - 1) * 32 + lane;
    int slot = 0;
    uint32_t phase = 0u;
    for (int s = 0; s < nstages_total; ++s) {
      if (!mbar_wait_relaxed(wfull(slot), phase, abort_flag, err)) break;
      uint8_t *act = gen + slot * kTcStageBytes + kTcWeightBytes;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 *piece = reinterpret_cast<uint4 *>(act) + tix + u * 128;
        const uint4 v = *piece;
        uint4 o;
        o.x = __byte_perm(v.x, v.z, 0x5410);  // (e0, e4)
        o.y = __byte_perm(v.x, v.z, 0x7632);  // (e1, e5)
        o.z = __byte_perm(v.y, v.w, 0x5410);  // (e2, e6)
        o.w = __byte_perm(v.y, v.w, 0x7632);  // (e3, e7)
        *piece = o;
      }
      fence_proxy_async();
      mbar_arrive(aready(slot));
      if (++slot == nstages) { slot = 0; phase ^= 1u; }
    }
  } else if (warp > kTcDqWarps) {
    // ---------------- MMA issue: one thread per warp, chunk c of a stage belongs to issuer c
    // D = f32, A = B = bf16, both K-major, N = 16, M = 128
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(16 >> 3) << 17) |
                             (static_cast<uint32_t>(128 >> 4) << 24);
      const int issuer = warp - kTcDqWarps - 1;
      uint32_t aphase = 0u;   // one parity bit per TMEM buffer
      int slot = 0;
      uint32_t phase = 0u;
      for (int s = 0; s < nstages_total; ++s) {
        const int c = s * 4 + issuer;
        if (c < nchunks) {
          const int b = c % kTcABufs;
          if (!mbar_wait(aready(slot), phase, abort_flag, err) || !mbar_wait(afull(b), (aphase >> b) & 1u, abort_flag, err)) break;
          aphase ^= 1u << b;
          tc_fence_after();
          const uint32_t act_addr = base + slot * kTcStageBytes + kTcWeightBytes + static_cast<uint32_t>(issuer) * 2048u;
#pragma unroll
          for (int j = 0; j < 4; ++j)   // 4 x K=16 per 64-k chunk; 8 TMEM columns and 32 bytes of smem each
            mma_f16_ts(tmem_d + static_cast<uint32_t>(issuer * 16), tmem_a0 + static_cast<uint32_t>(b * 32 + j * 8),
                       make_desc(act_addr + j * 32, 16, 1024), idesc, (c >= kTcMmaWarps || j > 0) ? 1u : 0u);
          // one commit per chunk: when the stage's four commits and its sixteen reader arrivals are in, the
          // stage can be refilled, and the unpackers know the tensor-memory buffers of that stage are drained
          tc_commit(wempty(slot));
        } else {
          mbar_arrive(wempty(slot));
        }
        if (++slot == nstages) { slot = 0; phase ^= 1u; }
      }
      tc_commit(dfull);   // arrives once this issuer's MMAs are done (immediately if it had none)
    }
  } else {
    // ---------------- dequantisers
    const int quad = warp & 3, sub = warp >> 2;       // sub: which chunk of every stage this warp owns
    const int tid_n = quad * 32 + lane;                 // TMEM lane = column within the tile
    const int64_t n = n0 + tid_n;
    const bool n_ok = n < p.n;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int chunks_per_group = static_cast<int>(p.group / 64);
    bool ok = true;
    int cur_group = -1;
    uint32_t zz = 0x43004300u, ss = 0u;
    // The tensor-memory store of a chunk completes while the next chunk is read and dequantised: the
    // wait for it, and the arrival that hands the chunk to the MMA issuers, come just before the
    // next store.  The stage's weights are released as soon as its words are in registers.
    int pending_buf = -1;
    auto hand_over = [&]() {
      if (pending_buf < 0) return;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(afull(pending_buf));
      pending_buf = -1;
    };
    int slot = 0;
    uint32_t phase = 0u;
    int slot2 = 0;            // slot and phase of the stage two before this one: its MMAs read the
    uint32_t phase2 = 0u;     // tensor-memory buffer this stage's chunk is about to overwrite
    for (int s = 0; s < nstages_total && ok; ++s) {
      if (!mbar_wait_relaxed(wfull(slot), phase, abort_flag, err)) { ok = false; break; }
      const uint32_t *st = reinterpret_cast<const uint32_t *>(gen + slot * kTcStageBytes);
      const int cs = sub;                             // chunk of the stage this warp owns
      const int c = s * 4 + cs;                       // global chunk
      uint32_t words[8];
      if (c < nchunks) {
#pragma unroll
        for (int r = 0; r < 8; ++r) words[r] = st[(cs * 8 + r) * kTcCols + tid_n];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(wempty(slot));
      if (c < nchunks) {
        const int b = c % kTcABufs;
        const int grp = c / chunks_per_group;
        if (grp != cur_group) {
          cur_group = grp;
          const uint32_t sv = sm_scales[grp * kTcCols + tid_n];
          const uint32_t z = (sm_zeros[grp * 16 + (tid_n >> 3)] >> (4 * (tid_n & 7))) & 0xfu;
          ss = sv | (sv << 16);
          zz = (0x4300u | z) * 0x00010001u;
        }
        uint32_t qv[32];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t v = nibble_pair_bf16(words[r], 4 * q);
            qv[r * 4 + q] = bf16x2_mul(bf16x2_sub(v, zz), ss);
          }
        }
        hand_over();   // the previous chunk's store
        // the buffer must have been drained by the MMAs that read it kTcABufs chunks (two stages) ago:
        // the "stage empty" barrier of that stage completes only after its four MMA commits
        if (s >= 2) {
          if (!mbar_wait_relaxed(wempty(slot2), phase2, abort_flag, err)) { ok = false; }
          tc_fence_after();
        }
        tmem_st32(tmem_a0 + lane_addr + static_cast<uint32_t>(b * 32), qv);
        pending_buf = b;
      }
      if (s >= 2 && ++slot2 == nstages) { slot2 = 0; phase2 ^= 1u; }
      if (++slot == nstages) { slot = 0; phase ^= 1u; }
    }
    hand_over();
    // ---------------- epilogue: the four warps of half 0 read the accumulator
    if (sub == 0 && ok) {
      if (mbar_wait(dfull, 0, abort_flag, err)) {
        tc_fence_after();
        float accs[16];
#pragma unroll
        for (int mm = 0; mm < 16; ++mm) accs[mm] = 0.0f;
        const int nacc = nchunks < kTcMmaWarps ? nchunks : kTcMmaWarps;   // issuers that had a chunk
        for (int a8 = 0; a8 < nacc; ++a8) {
          uint32_t t16[16];
          tmem_ld16(tmem_d + lane_addr + static_cast<uint32_t>(a8 * 16), t16);
          tmem_ld_wait();
#pragma unroll
          for (int mm = 0; mm < 16; ++mm) accs[mm] += __uint_as_float(t16[mm]);
        }
        uint32_t r[16];
#pragma unroll
        for (int mm = 0; mm < 16; ++mm) r[mm] = __float_as_uint(accs[mm]);
        const int64_t rows_left = p.m - m0;
        if (n_ok) {
#pragma unroll
          for (int mm = 0; mm < 16; ++mm)
            if (mm < rows_left) store_out(p, (m0 + mm) * p.ldo + n, __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[mm]))));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kTcDqWarps + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------ folded-scale kernel (tcgen05, bf16 operands from shared memory)
// out[m, n] = sum over groups g of  s[g, n] * ( sum_{k in g} a[m, k] * (q[k, n] - 8)  -  (z[g, n] - 8) * A[g, m] ),
// A[g, m] = sum_{k in g} a[m, k].  The inner sum is a bf16 x bf16 product on the tensor core; a packed word turns
// into its eight operand values q - 8 with twelve instructions (four shifts, four lop3, four exact sub.bf16x2) and
// no per-weight multiplication or rounding -- the zero point and the scale act once per group and column, on the
// group's accumulator, in the epilogue.  The exact-rounding kernels above spend fifteen instructions per word.  Against the oracle (every dequantised weight
// rounded to bf16 first) the result differs by those roundings: a relative RMS of about 1e-3, inside the 2e-2 bar.
//
// One CTA per 128 output columns, all of K.  Roles: warp 0 issues TMA loads (a stage = 64 k: 4 KB of packed weights
// + the 16 x 64 activations), warps 6-21 turn a packed stage into the tensor core's K-major bf16 tile (128 rows =
// output columns x 128 bytes, 128-byte swizzle) in a ring of operand slots and put the activations into the same
// nibble-pair k order, warps 1-4 issue the MMAs (stage s is issued by warp 1 + s % 4: four MMAs M = 128, N = 16,
// K = 16 into one of that issuer's two accumulators), warps 5-8 add the accumulators of a finished group's stages
// and fold them into f32 partial sums held in registers.  Stage s always uses operand slot s % 4, packed slot s % 24,
// dequantising team s % 4 and issuer s % 4: every barrier has the same waiters in every phase (a waiter that sits
// out a phase cannot tell the phase it wants from the one two before it).
constexpr int kFoldCols = 128;
constexpr int kFoldPStage = 8 * kFoldCols * 4 + 2048;        // packed weights + activations: 6 KB
constexpr int kFoldPStages = 24;     // 144 KB of packed stages in flight: a CTA streams what it keeps in flight per memory latency
constexpr int kFoldOStage = kFoldCols * 128 + 2048;          // bf16 weight tile + permuted activations: 18 KB
constexpr int kFoldOStages = 4;
constexpr int kFoldDqWarps = 16;
constexpr int kFoldIssuers = 4;          // the thread that issues a tcgen05.mma is held about 140 cycles by each: stage s is issuer s % 4's
constexpr int kFoldThreads = (1 + kFoldIssuers + 4 + kFoldDqWarps) * 32;
constexpr int kFoldMaxGroups = 512;

// Nibbles t and t + 4 of a packed word as the bf16 pair (q_t - 8, q_{t+4} - 8): 16 + q is the bf16 with bit pattern
// 0x4180 | q << 3 (one shift, one lop3), and subtracting 24 is exact.  The operand is centred because the tensor
// core adds the products of one instruction with about 13 bits below the largest addend: with 128 + q as the operand
// (no subtraction) the group sums came back with a relative error of 2^-11.6, which the zero-point term magnified.
__device__ __forceinline__ uint32_t centred_pair_bf16(uint32_t w, int t) {
  uint32_t r;
  const uint32_t sh = t == 0 ? (w << 3) : (w >> (4 * t - 3));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(sh), "r"(0x00780078u), "r"(0x41804180u));
  return bf16x2_sub(r, 0x41C041C0u);        // 24.0 in both halves
}

__device__ __forceinline__ void mma_bf16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

inline size_t fold_smem_bytes(int64_t groups) {
  return 1024 /*alignment*/ + static_cast<size_t>(kFoldOStages) * kFoldOStage + static_cast<size_t>(kFoldPStages) * kFoldPStage +
         static_cast<size_t>(groups) * 16 * 4 /*activation sums*/ + 4096 /*output staging*/ + 1024 /*barriers*/;
}

__global__ void __launch_bounds__(kFoldThreads, 1)
    w4a16_fold_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a, W4Params p, int64_t m0, int *err) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;                    // operand slots first: 1024-byte aligned swizzle atoms
  uint8_t *gen = smem_raw + (base - raw);
  const uint32_t o_base = base, p_base = base + kFoldOStages * kFoldOStage;
  const int groups = static_cast<int>(p.k / p.group), spg = static_cast<int>(p.group / 64), nstages = static_cast<int>(p.k / 64);
  float *asum = reinterpret_cast<float *>(gen + kFoldOStages * kFoldOStage + kFoldPStages * kFoldPStage);   // [groups][16]
  uint16_t *stg = reinterpret_cast<uint16_t *>(reinterpret_cast<uint8_t *>(asum) + static_cast<size_t>(groups) * 64);
  const uint32_t bars = smem_u32(stg) + 4096;
  auto full_p = [&](int s) { return bars + 8u * s; };
  auto empty_p = [&](int s) { return bars + 8u * (kFoldPStages + s); };
  auto full_o = [&](int s) { return bars + 8u * (2 * kFoldPStages + s); };
  auto empty_o = [&](int s) { return bars + 8u * (2 * kFoldPStages + kFoldOStages + s); };
  auto tfull = [&](int a) { return bars + 8u * (2 * kFoldPStages + 2 * kFoldOStages + a); };                        // a = issuer * 2 + buffer
  auto tempty = [&](int a) { return bars + 8u * (2 * kFoldPStages + 2 * kFoldOStages + 2 * kFoldIssuers + a); };
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(reinterpret_cast<uint8_t *>(stg) + 4096 + 8 * (2 * kFoldPStages + 2 * kFoldOStages + 4 * kFoldIssuers));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kFoldCols;
  const int rows = static_cast<int>(p.m - m0 < 16 ? p.m - m0 : 16);

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_w);
    prefetch_tmap(&tmap_a);
    for (int s = 0; s < kFoldPStages; ++s) { mbar_init(full_p(s), 1); mbar_init(empty_p(s), 4); }
    for (int s = 0; s < kFoldOStages; ++s) { mbar_init(full_o(s), 4); mbar_init(empty_o(s), 1); }
    for (int a = 0; a < 2 * kFoldIssuers; ++a) { mbar_init(tfull(a), 1); mbar_init(tempty(a), 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 128);
  pdl_wait();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer
    if (lane == 0) {
      int slot = 0;
      uint32_t round = 0;
      bool ok = true;
      for (int s = 0; s < nstages; ++s) {
        if (!mbar_wait(empty_p(slot), (round & 1u) ^ 1u, abort_flag, err)) { ok = false; break; }
        const uint32_t dst = p_base + slot * kFoldPStage;
        mbar_expect_tx(full_p(slot), kFoldPStage);
        tma_load_2d(dst, &tmap_w, n0, s * 8, full_p(slot));                               // [8 word rows x 128 columns]
        tma_load_2d(dst + 8 * kFoldCols * 4, &tmap_a, s * 64, static_cast<int>(m0), full_p(slot));   // [16 rows x 64 k]
        if (++slot == kFoldPStages) { slot = 0; ++round; }
      }
      if (!ok) {
        for (int q = 0; q < kFoldPStages; ++q)
          for (int i = 0; i < 200000; ++i)
            if (mbar_try_wait(full_p(q), 0) || mbar_try_wait(full_p(q), 1)) break;
      }
    }
  } else if (warp <= kFoldIssuers + 4) {
    // sums of the activations per (group, row), by the issuing and the folding warps together (they have nothing
    // else to do yet): every load of a pair is issued before the first is used
    {
      const int t12 = (warp - 1) * 32 + lane;
      for (int pr = t12; pr < groups * 16; pr += (kFoldIssuers + 4) * 32) {
        const int g = pr >> 4, r = pr & 15;
        float sum = 0.0f;
        if (r < rows) {
          const uint4 *src = reinterpret_cast<const uint4 *>(p.a + (m0 + r) * p.lda + static_cast<int64_t>(g) * p.group);
          for (int i0 = 0; i0 < static_cast<int>(p.group / 8); i0 += 16) {
            uint4 v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = (i0 + i < static_cast<int>(p.group / 8)) ? __ldg(src + i0 + i) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
              for (int j = 0; j < 4; ++j) sum += __uint_as_float(w[j] << 16) + __uint_as_float(w[j] & 0xffff0000u);
            }
          }
        }
        asum[pr] = sum;
      }
      asm volatile("bar.sync 1, %0;" ::"n"((kFoldIssuers + 4) * 32) : "memory");
    }
    if (warp <= kFoldIssuers) {
    // ---------------- MMA issuers
    if (lane == 0) {
      const int issuer = warp - 1;
      // D = f32, A = B = bf16, both K-major, N = 16, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(16 >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
      bool ok = true;
      static_assert(kFoldIssuers == kFoldOStages, "an issuer per operand slot");
      // spg is 1, 2 or 4: every stage of this issuer belongs to another group, its c-th stage (c = s / 4) goes to its
      // accumulator c % 2, whose (c / 2)-th use this is
      for (int s = issuer; s < nstages && ok; s += kFoldIssuers) {
        const int c = s / kFoldIssuers, buf = c & 1;
        const uint32_t use = static_cast<uint32_t>(c >> 1);
        if (!mbar_wait(tempty(issuer * 2 + buf), (use & 1u) ^ 1u, abort_flag, err)) { ok = false; break; }
        if (!mbar_wait(full_o(issuer), static_cast<uint32_t>(c) & 1u, abort_flag, err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>((issuer * 2 + buf) * 16);
        const uint32_t wt = o_base + issuer * kFoldOStage, at = wt + kFoldCols * 128;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_bf16_ss(d_tmem, make_desc(wt + kk * 32, 16, 1024), make_desc(at + kk * 32, 16, 1024), idesc, kk > 0 ? 1u : 0u);
        tc_commit(empty_o(issuer));
        tc_commit(tfull(issuer * 2 + buf));
      }
    }
    } else {
    // ---------------- group fold + output: warps 2..5, TMEM lane quadrant = warp % 4; lane = output column
    const int quad = warp & 3;
    const int64_t col = static_cast<int64_t>(n0) + quad * 32 + lane;
    const bool col_ok = col < p.n;
    const int64_t cc = col_ok ? col : 0;
    float part[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) part[j] = 0.0f;
    bool ok = true;
    float s_next = __uint_as_float(static_cast<uint32_t>(p.scales[cc]) << 16);
    uint32_t z_next = (p.zeros[cc >> 3] >> (4 * (cc & 7))) & 0xfu;
    for (int g = 0; g < groups && ok; ++g) {
      const float sc = s_next, zc = static_cast<float>(static_cast<int>(z_next) - 8);
      if (g + 1 < groups) {
        s_next = __uint_as_float(static_cast<uint32_t>(p.scales[static_cast<int64_t>(g + 1) * p.n + cc]) << 16);
        z_next = (p.zeros[static_cast<int64_t>(g + 1) * (p.n >> 3) + (cc >> 3)] >> (4 * (cc & 7))) & 0xfu;
      }
      // the accumulators of this group's stages (stage s: issuer s % 4, its accumulator (s / 4) % 2), added in stage order
      uint32_t r[16];
      for (int i = 0; i < spg && ok; ++i) {
        const int st = g * spg + i, issuer = st & (kFoldIssuers - 1), c = st / kFoldIssuers, a2 = issuer * 2 + (c & 1);
        if (!mbar_wait(tfull(a2), static_cast<uint32_t>(c >> 1) & 1u, abort_flag, err)) { ok = false; break; }
        tc_fence_after();
        uint32_t q[16];
        tmem_ld16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(a2 * 16), q);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty(a2));
#pragma unroll
        for (int e = 0; e < 16; ++e) r[e] = i == 0 ? q[e] : __float_as_uint(__uint_as_float(r[e]) + __uint_as_float(q[e]));
      }
      if (!ok) break;
      const float4 *as4 = reinterpret_cast<const float4 *>(asum + g * 16);
#pragma unroll
      for (int j4 = 0; j4 < 4; ++j4) {
        const float4 av = as4[j4];          // same address in every lane: broadcast
        part[4 * j4 + 0] = fmaf(sc, fmaf(-zc, av.x, __uint_as_float(r[4 * j4 + 0])), part[4 * j4 + 0]);
        part[4 * j4 + 1] = fmaf(sc, fmaf(-zc, av.y, __uint_as_float(r[4 * j4 + 1])), part[4 * j4 + 1]);
        part[4 * j4 + 2] = fmaf(sc, fmaf(-zc, av.z, __uint_as_float(r[4 * j4 + 2])), part[4 * j4 + 2]);
        part[4 * j4 + 3] = fmaf(sc, fmaf(-zc, av.w, __uint_as_float(r[4 * j4 + 3])), part[4 * j4 + 3]);
      }
    }
    if (ok) {
      uint32_t pk[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) pk[j] = pack_bf16x2(part[2 * j], part[2 * j + 1]);
      const bool vec = p.n % 8 == 0 && p.ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(p.n_peers ? p.peer[0] : p.out) & 15u) == 0 && p.n_peers <= 1;
      uint16_t *wst = stg + quad * 512;                     // this warp's 16 rows x 32 columns
      if (vec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          wst[(2 * j) * 32 + lane] = static_cast<uint16_t>(pk[j] & 0xffffu);
          wst[(2 * j + 1) * 32 + lane] = static_cast<uint16_t>(pk[j] >> 16);
        }
        __syncwarp();
        uint16_t *dst = p.n_peers ? p.peer[0] : p.out;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          const int id = lane + 32 * t, rr = id >> 2, part4 = id & 3;
          const int64_t c0 = static_cast<int64_t>(n0) + quad * 32 + part4 * 8;
          if (rr < rows && c0 < p.n)
            *reinterpret_cast<uint4 *>(dst + (m0 + rr) * p.ldo + c0) = *reinterpret_cast<const uint4 *>(wst + rr * 32 + part4 * 8);
        }
      } else if (col_ok) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (j < rows) store_out(p, (m0 + j) * p.ldo + col, static_cast<uint16_t>((j & 1) ? (pk[j >> 1] >> 16) : (pk[j >> 1] & 0xffffu)));
      }
    }
    }
  } else {
    // ---------------- packed words -> bf16 operand tile; activations into the nibble-pair k order
    // Four teams of four warps; team t owns operand slot t and takes stages t, t + 4, ...: the teams work on four
    // different stages at once, so the latency of a stage's hand-over (barrier round trips, the proxy fence) is hidden
    // by the other three.  A thread converts the eight words of one column and one 16-byte piece of activations.
    const int dw = warp - (1 + kFoldIssuers + 4), team = dw >> 2, tw = dw & 3;
    static_assert(kFoldOStages == 4 && kFoldDqWarps == 16 && kFoldPStages % 4 == 0, "one operand slot per team");
    uint8_t *ost = gen + team * kFoldOStage;
    const int c = tw * 32 + lane;                                  // column = row of the operand tile
    int pslot = team;
    uint32_t pround = 0, oround = 0;
    bool ok = true;
    for (int s = team; s < nstages && ok; s += 4, ++oround) {
      if (!mbar_wait(full_p(pslot), pround & 1u, abort_flag, err)) { ok = false; break; }
      const uint8_t *pst = gen + kFoldOStages * kFoldOStage + pslot * kFoldPStage;
      uint32_t w[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) w[r] = reinterpret_cast<const uint32_t *>(pst)[r * kFoldCols + c];
      const uint4 av = *reinterpret_cast<const uint4 *>(pst + 8 * kFoldCols * 4 + c * 16);
      if (!mbar_wait(empty_o(team), (oround & 1u) ^ 1u, abort_flag, err)) { ok = false; break; }
#pragma unroll
      for (int r = 0; r < 8; ++r)
        *reinterpret_cast<uint4 *>(ost + c * 128 + ((r ^ (c & 7)) << 4)) =
            make_uint4(centred_pair_bf16(w[r], 0), centred_pair_bf16(w[r], 1), centred_pair_bf16(w[r], 2), centred_pair_bf16(w[r], 3));
      // (a0 .. a7) -> (a0, a4, a1, a5, a2, a6, a3, a7), piece by piece in the swizzled tile
      *reinterpret_cast<uint4 *>(ost + kFoldCols * 128 + c * 16) =
          make_uint4(__byte_perm(av.x, av.z, 0x5410), __byte_perm(av.x, av.z, 0x7632), __byte_perm(av.y, av.w, 0x5410), __byte_perm(av.y, av.w, 0x7632));
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) { mbar_arrive(full_o(team)); mbar_arrive(empty_p(pslot)); }
      pslot += 4;
      if (pslot >= kFoldPStages) { pslot -= kFoldPStages; ++pround; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
}

// Plain path: any alignment; one thread per output column, one row block of up to 4 rows.
__global__ void __launch_bounds__(128) w4a16_plain_kernel(W4Params p, int64_t m0) {
  const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= p.n) return;
  const int64_t row = m0 + blockIdx.y;
  if (row >= p.m) return;
  float acc = 0.0f;
  for (int64_t kk = 0; kk < p.k; ++kk) {
    const int64_t grp = kk / p.group;
    const uint32_t q = (p.qw[(kk / 8) * p.n + c] >> (4 * (kk % 8))) & 0xfu;
    const uint32_t z = (p.zeros[grp * (p.n / 8) + c / 8] >> (4 * (c % 8))) & 0xfu;
    const float s = __uint_as_float(static_cast<uint32_t>(p.scales[grp * p.n + c]) << 16);
    const float wv = __bfloat162float(__float2bfloat16_rn(__fmul_rn(static_cast<float>(q) - static_cast<float>(z), s)));
    const float av = __uint_as_float(static_cast<uint32_t>(p.a[row * p.lda + kk]) << 16);
    acc = __fmaf_rn(av, wv, acc);
  }
  store_out(p, row * p.ldo + c, __bfloat16_as_ushort(__float2bfloat16_rn(acc)));
}

// ------------------------------------------------------------------ host helpers for the tcgen05 path
using EncodeFnW4 = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFnW4 encode_fn_w4() {
  static EncodeFnW4 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFnW4>(sym);
    else
      cudaGetLastError();
  });
  return fn;
}

// qweight as a 2-D int32 tensor [k/8 rows, n columns]; box = [32 rows x 128 columns], no swizzle.
bool make_weight_tmap(CUtensorMap *map, const uint32_t *qw, int64_t n, int64_t k, int box_rows = kTcStageRows) {
  EncodeFnW4 enc = encode_fn_w4();
  if (!enc) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(k / 8)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(n) * 4u};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kTcCols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1u, 1u};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<uint32_t *>(qw), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// activations as a 2-D bf16 tensor [m rows, k]; box = [16 rows x 64 k] (128 bytes per row), 128-byte
// swizzle: a box lands in the tensor core's K-major layout; rows beyond m read as zeros
bool make_act_tmap(CUtensorMap *map, const uint16_t *a, int64_t m, int64_t k, int64_t lda) {
  EncodeFnW4 enc = encode_fn_w4();
  if (!enc) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(m)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(lda) * 2u};
  cuuint32_t box[2] = {64u, 16u};
  cuuint32_t estr[2] = {1u, 1u};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(a), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace
}  // namespace bsir

using namespace bsir;

static int32_t matmul_w4a16_impl(int64_t m, int64_t n, int64_t k, int64_t group, const void *a, int64_t lda,
                                 const int32_t *qweight, const void *scales, const int32_t *zeros, void *out,
                                 int64_t ldo, int32_t n_peers, void *const *peer_out, void *stream) {
  clear_error();
  if (n_peers < 0 || n_peers > 8 || (n_peers > 0 && !peer_out)) return fail(BSIR_ERR_ARGS, "matmul_w4a16: n_peers %d (0..8)", n_peers);
  for (int i = 0; i < n_peers; ++i)
    if (!peer_out[i] || !aligned_to(peer_out[i], 2)) return fail(BSIR_ERR_NULL, "matmul_w4a16: peer_out[%d]", i);
  if (n_peers > 0) out = peer_out[0];
  if (m < 0 || n < 0 || k < 0) return fail(BSIR_ERR_SHAPE, "matmul_w4a16: m=%lld n=%lld k=%lld", (long long)m, (long long)n, (long long)k);
  if (group <= 0 || group % 32 || k % group || n % 8)
    return fail(BSIR_ERR_SHAPE, "matmul_w4a16: need group %% 32 == 0, k %% group == 0, n %% 8 == 0 (group=%lld k=%lld n=%lld)",
                (long long)group, (long long)k, (long long)n);
  if (m == 0 || n == 0) return BSIR_OK;
  if (!out || (k > 0 && (!a || !qweight || !scales || !zeros))) return fail(BSIR_ERR_NULL, "matmul_w4a16: null pointer");
  if (lda < k || ldo < n) return fail(BSIR_ERR_STRIDE, "matmul_w4a16: leading dimension too small");
  if (!aligned_to(a, 2) || !aligned_to(out, 2) || !aligned_to(qweight, 4) || !aligned_to(scales, 2) || !aligned_to(zeros, 4))
    return fail(BSIR_ERR_ALIGN, "matmul_w4a16: misaligned");
  cudaStream_t st = resolve_stream(stream);
  W4Params p{m, n, k, group, static_cast<const uint16_t *>(a), lda, reinterpret_cast<const uint32_t *>(qweight),
             static_cast<const uint16_t *>(scales), reinterpret_cast<const uint32_t *>(zeros),
             static_cast<uint16_t *>(out), ldo, n_peers, {}};
  for (int i = 0; i < n_peers; ++i) p.peer[i] = static_cast<uint16_t *>(peer_out[i]);
  const bool fast = k > 0 && aligned_to(a, 16) && lda % 8 == 0 && aligned_to(qweight, 16) && aligned_to(scales, 16);
  // tensor-memory path: needs sm_100, k <= 4096 (activations resident in shared memory), groups that are
  // whole 64-k chunks and a weight pitch TMA can address
  // Two kernels stream the packed weights.  Blocks of up to 8 rows (decode) run the register
  // dequantisation + mma.sync kernel, whose MMA count halves for 8 rows; taller blocks run the
  // tensor-memory kernel (tcgen05), where the MMA cost does not depend on the rows: legacy mma.sync
  // tiles cost about 32 cycles per SM sub-core on this GPU.  BSIR_W4A16_PATH=m / t forces one of them.
  const char *force = std::getenv("BSIR_W4A16_PATH");
  const bool tc_ok = fast && device_info().cc_major >= 10 && group % 64 == 0 && k % 64 == 0 && tc_layout(k, group).stages >= 2;
  if (!fast) {
    for (int64_t m0 = 0; m0 < m; m0 += 65535) {
      const int64_t mr = m - m0 < 65535 ? m - m0 : 65535;
      const dim3 grid(static_cast<unsigned>(ceil_div(n, 128)), static_cast<unsigned>(mr));
      w4a16_plain_kernel<<<grid, 128, 0, st>>>(p, m0);
      count_launch();
    }
    return check_launch("matmul_w4a16");
  }
  // The folded-scale kernel (scale and zero point applied per group in the epilogue) runs on request only
  // (BSIR_W4A16_PATH=f): it is correct and halves the dequantisation work, but with the weights as the MMA's A
  // operand a 128-column tile needs K / 16 MMAs, and an SM accepts one tcgen05.mma per 115-140 cycles whatever its
  // shape -- 15-17 us for K = 4096 before anything else (measured 36-41 us with one, four and eight issuing
  // threads).  The form that would pay has the weights as the B operand (N = 256 per MMA) and K split over all SMs.
  const bool fold_ok = fast && device_info().cc_major >= 10 && (group == 64 || group == 128 || group == 256) && k % 64 == 0 && k / group <= kFoldMaxGroups &&
                       fold_smem_bytes(k / group) <= 226 * 1024 && n_peers <= 1;
  if (fold_ok && force && force[0] == 'f') {
    CUtensorMap fw, fa;
    if (make_weight_tmap(&fw, p.qw, n, k, 8) && make_act_tmap(&fa, p.a, m, k, lda)) {
      const size_t smem = fold_smem_bytes(k / group);
      cudaFuncSetAttribute(w4a16_fold_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      for (int64_t m0 = 0; m0 < m; m0 += 16) {
        launch_pdl(w4a16_fold_kernel, dim3(static_cast<unsigned>(ceil_div(n, kFoldCols))), dim3(kFoldThreads), smem, st, fw, fa, p, m0,
                   device_error_word());
        count_launch();
      }
      return check_launch("matmul_w4a16 (folded scales)");
    }
  }
  CUtensorMap tw, ta;
  bool have_map = false;
  for (int64_t m0 = 0; m0 < m; m0 += 16) {
    const bool one_block = m - m0 <= 8;
    bool use_tc = tc_ok && !one_block;
    if (force && force[0] == 'm') use_tc = false;
    if (force && force[0] == 't') use_tc = tc_ok;
    if (use_tc && !have_map) {
      have_map = make_weight_tmap(&tw, p.qw, n, k) && make_act_tmap(&ta, p.a, m, k, lda);
      if (!have_map) use_tc = false;
    }
    if (use_tc) {
      const size_t smem = tc_layout(k, group).bytes;
      cudaFuncSetAttribute(w4a16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      launch_pdl(w4a16_tc_kernel, dim3(static_cast<unsigned>(ceil_div(n, kTcCols))), dim3(kTcThreads), smem, st, tw, ta, p, m0,
                 device_error_word());
    } else {
      const unsigned blocks = static_cast<unsigned>(ceil_div(n, 64));
      if (one_block) launch_pdl(w4a16_mma_kernel<2, 1>, dim3(blocks), dim3(kWarps * 32), 0, st, p, m0);
      else launch_pdl(w4a16_mma_kernel<2, 2>, dim3(blocks), dim3(kWarps * 32), 0, st, p, m0);
    }
    count_launch();
  }
  return check_launch("matmul_w4a16");
}

extern "C" int32_t bsir_matmul_w4a16(int64_t m, int64_t n, int64_t k, int64_t group, const void *a, int64_t lda,
                                     const int32_t *qweight, const void *scales, const int32_t *zeros, void *out,
                                     int64_t ldo, void *stream) {
  return matmul_w4a16_impl(m, n, k, group, a, lda, qweight, scales, zeros, out, ldo, 0, nullptr, stream);
}

extern "C" int32_t bsir_matmul_w4a16_peers(int64_t m, int64_t n, int64_t k, int64_t group, const void *a, int64_t lda,
                                           const int32_t *qweight, const void *scales, const int32_t *zeros, int32_t n_peers,
                                           void *const *peer_out, int64_t ldo, void *stream) {
  if (n_peers <= 0) return fail(BSIR_ERR_ARGS, "matmul_w4a16_peers: n_peers %d", n_peers);
  return matmul_w4a16_impl(m, n, k, group, a, lda, qweight, scales, zeros, nullptr, ldo, n_peers, peer_out, stream);
}
