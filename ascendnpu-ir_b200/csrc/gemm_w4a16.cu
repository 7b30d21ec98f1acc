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
// Kernel.  One CTA owns 64 output columns and all of K; its 8 warps take contiguous K slices and
// meet in shared memory at the end.  A thread streams 16-byte pieces of qweight (4 columns x 8 k
// values), dequantises in registers with packed bf16 arithmetic and feeds mma.sync.m16n8k16:
//   (word >> 4i) & 0x000F000F | 0x43004300 is the bf16 pair (128 + q[k_i], 128 + q[k_i+4]);
//   subtracting (128 + z) is exact and the product with s rounds once, exactly like the f32
//   computation it restates ((q - z) * s needs 13 bits).
// The k order inside an MMA is free as long as A uses the same one, so the nibble pairs (i, i + 4)
// are taken as they come and A's 8-element pieces are permuted to match with two byte permutes.
// M up to 16 is one MMA row block; larger M runs the kernel once per 16 rows (decode path; large M
// belongs on a dense GEMM).
#include "common.cuh"

namespace bsir {
namespace {

constexpr int kColsPerCta = 64;
constexpr int kWarps = 8;
constexpr int kPrefetch = 3;  // k32 steps of weights in flight per warp

struct W4Params {
  int64_t m, n, k, group;
  const uint16_t *a;
  int64_t lda;
  const uint32_t *qw;
  const uint16_t *scales;
  const uint32_t *zeros;
  uint16_t *out;
  int64_t ldo;
};

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
__device__ __forceinline__ uint4 ldg_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// One k32 step of one 32-column piece: 4 weight words (columns 4g..4g+3, 8 k values each).
struct Piece {
  uint4 w;
};

__global__ void __launch_bounds__(kWarps * 32, 2) w4a16_mma_kernel(W4Params p, int64_t m0) {
  __shared__ float red[kWarps][16][kColsPerCta + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t col_base = static_cast<int64_t>(blockIdx.x) * kColsPerCta;
  const int64_t steps = p.k / 32;
  const int64_t per_warp = (steps + kWarps - 1) / kWarps;
  const int64_t s_begin = warp * per_warp;
  const int64_t s_end = s_begin + per_warp < steps ? s_begin + per_warp : steps;
  const int64_t rows_left = p.m - m0;
  const bool row_lo_ok = g < rows_left, row_hi_ok = g + 8 < rows_left;
  const uint16_t *a_lo = p.a + (m0 + g) * p.lda;
  const uint16_t *a_hi = p.a + (m0 + g + 8) * p.lda;

  // this thread's columns: piece j (0, 1) covers col_base + 32 j + 4 g + {0..3}
  int64_t col[2];
  bool col_ok[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    col[j] = col_base + 32 * j + 4 * g;
    col_ok[j] = col[j] < p.n;  // n is a multiple of 8, so a piece is all in or all out
  }

  float acc[2][4][4];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[j][i][e] = 0.0f;

  auto load_piece = [&](int64_t step, int j) -> uint4 {
    if (step < s_end && col_ok[j]) return ldg_stream16(p.qw + (step * 4 + t) * p.n + col[j]);
    return make_uint4(0u, 0u, 0u, 0u);
  };

  uint4 pre[kPrefetch][2];
#pragma unroll
  for (int d = 0; d < kPrefetch; ++d)
#pragma unroll
    for (int j = 0; j < 2; ++j) pre[d][j] = load_piece(s_begin + d, j);

  uint32_t zz[2][4], ss[2][4];  // per column: bf16x2 (128 + z, 128 + z) and (s, s)
  int64_t cur_group = -1;

  for (int64_t step = s_begin; step < s_end; ++step) {
    // weights of this step; refill the slot with the step kPrefetch ahead
    uint4 w[2];
    {
      const int slot = static_cast<int>((step - s_begin) % kPrefetch);
#pragma unroll
      for (int d = 0; d < kPrefetch; ++d)
        if (d == slot) {
#pragma unroll
          for (int j = 0; j < 2; ++j) { w[j] = pre[d][j]; pre[d][j] = load_piece(step + kPrefetch, j); }
        }
    }
    // this thread's k values of the step: 32 step + 8 t + {0..7}
    const int64_t k0 = step * 32 + 8 * t;
    const int64_t grp = k0 / p.group;
    if (grp != cur_group) {
      cur_group = grp;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint2 sc = make_uint2(0u, 0u);
        uint32_t zw = 0u;
        if (col_ok[j]) {
          sc = *reinterpret_cast<const uint2 *>(p.scales + grp * p.n + col[j]);
          zw = p.zeros[grp * (p.n / 8) + col[j] / 8] >> (4 * (col[j] % 8));
        }
        const uint32_t s01[4] = {sc.x & 0xffffu, sc.x >> 16, sc.y & 0xffffu, sc.y >> 16};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ss[j][i] = s01[i] | (s01[i] << 16);
          const uint32_t z = (zw >> (4 * i)) & 0xfu;
          zz[j][i] = (0x4300u | z) * 0x00010001u;
        }
      }
    }
    // A pieces (8 consecutive k) permuted to the pair order (e0,e4) (e1,e5) (e2,e6) (e3,e7)
    uint4 ra = make_uint4(0u, 0u, 0u, 0u), rb = make_uint4(0u, 0u, 0u, 0u);
    if (row_lo_ok) ra = *reinterpret_cast<const uint4 *>(a_lo + k0);
    if (row_hi_ok) rb = *reinterpret_cast<const uint4 *>(a_hi + k0);
    uint32_t fa[2][4];  // [mma][a0..a3]
    fa[0][0] = __byte_perm(ra.x, ra.z, 0x5410);  // row g   : (e0, e4)
    fa[0][2] = __byte_perm(ra.x, ra.z, 0x7632);  // row g   : (e1, e5)
    fa[1][0] = __byte_perm(ra.y, ra.w, 0x5410);  //           (e2, e6)
    fa[1][2] = __byte_perm(ra.y, ra.w, 0x7632);  //           (e3, e7)
    fa[0][1] = __byte_perm(rb.x, rb.z, 0x5410);  // row g+8
    fa[0][3] = __byte_perm(rb.x, rb.z, 0x7632);
    fa[1][1] = __byte_perm(rb.y, rb.w, 0x5410);
    fa[1][3] = __byte_perm(rb.y, rb.w, 0x7632);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t words[4] = {w[j].x, w[j].y, w[j].z, w[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t wd = words[i];
        uint32_t b[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t v = ((wd >> (4 * q)) & 0x000f000fu) | 0x43004300u;  // (128 + q_k, 128 + q_{k+4})
          b[q] = bf16x2_mul(bf16x2_sub(v, zz[j][i]), ss[j][i]);
        }
        mma_bf16_16816(acc[j][i], fa[0], b[0], b[1]);  // k pairs (0,4) and (1,5)
        mma_bf16_16816(acc[j][i], fa[1], b[2], b[3]);  // k pairs (2,6) and (3,7)
      }
    }
  }

  // C fragment: c0,c1 -> row g, tile columns 2t, 2t+1; c2,c3 -> row g+8.  Tile column nn of piece j,
  // word i is CTA column 32 j + 4 nn + i.
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c0 = 32 * j + 4 * (2 * t) + i, c1 = 32 * j + 4 * (2 * t + 1) + i;
      red[warp][g][c0] = acc[j][i][0];
      red[warp][g][c1] = acc[j][i][1];
      red[warp][g + 8][c0] = acc[j][i][2];
      red[warp][g + 8][c1] = acc[j][i][3];
    }
  __syncthreads();
  for (int o = threadIdx.x; o < 16 * kColsPerCta; o += kWarps * 32) {
    const int r = o / kColsPerCta, c = o % kColsPerCta;
    if (r >= rows_left || col_base + c >= p.n) continue;
    float s = 0.0f;
#pragma unroll
    for (int wq = 0; wq < kWarps; ++wq) s += red[wq][r][c];
    p.out[(m0 + r) * p.ldo + col_base + c] = __bfloat16_as_ushort(__float2bfloat16_rn(s));
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
  p.out[row * p.ldo + c] = __bfloat16_as_ushort(__float2bfloat16_rn(acc));
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" int32_t bsir_matmul_w4a16(int64_t m, int64_t n, int64_t k, int64_t group, const void *a, int64_t lda,
                                     const int32_t *qweight, const void *scales, const int32_t *zeros, void *out,
                                     int64_t ldo, void *stream) {
  clear_error();
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
             static_cast<uint16_t *>(out), ldo};
  const bool fast = k > 0 && aligned_to(a, 16) && lda % 8 == 0 && aligned_to(qweight, 16) && aligned_to(scales, 8);
  if (fast) {
    const unsigned blocks = static_cast<unsigned>(ceil_div(n, kColsPerCta));
    for (int64_t m0 = 0; m0 < m; m0 += 16) {
      w4a16_mma_kernel<<<blocks, kWarps * 32, 0, st>>>(p, m0);
      count_launch();
    }
  } else {
    for (int64_t m0 = 0; m0 < m; m0 += 65535) {
      const int64_t mr = m - m0 < 65535 ? m - m0 : 65535;
      const dim3 grid(static_cast<unsigned>(ceil_div(n, 128)), static_cast<unsigned>(mr));
      w4a16_plain_kernel<<<grid, 128, 0, st>>>(p, m0);
      count_launch();
    }
  }
  return check_launch("matmul_w4a16");
}
