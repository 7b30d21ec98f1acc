// transpose.cu -- tiled 2-D (optionally batched) transposition for copies whose source is a transposed view.
//
// hivm.hir.vtranspose (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:1439-1501) and
// linalg.transpose with a permutation that swaps the last two axes reach the library as a copy with a
// permuted source.  An element-wise strided copy reads 2..8 bytes per 32-byte sector; here a CTA moves a
// tile of 64 source rows x 128 bytes through shared memory so that both the global loads and the global
// stores are 16-byte accesses of full 128-byte lines.
//
// Shared-memory layout: the tile is 64 rows of 32 words; word w of row r sits at column w ^ f(r), with f a
// multiple of 4 that changes every 16 / ES rows (ES = element size).  Writing a row segment as one 16-byte
// store and reading a column of words for one 16-byte output vector are then both free of bank conflicts.
#include <cstdint>

#include "common.cuh"

namespace bsir {
namespace {

constexpr int kTileRows = 64;       // source rows per tile (= columns of a destination tile)
constexpr int kTileWords = 32;      // 128 bytes of source columns per tile
constexpr int kTrThreads = 256;

struct TrParams {
  const char *src;
  char *dst;
  int64_t rows, cols;               // of the source matrix [rows][cols]; the destination is [cols][rows]
  int64_t src_row, dst_row;         // row strides in elements
  int64_t src_batch, dst_batch;     // batch strides in elements
  int aligned;                      // 16-byte accesses are legal for full tiles
};

template <int ES>
__device__ __forceinline__ int swz(int r) {
  constexpr int RPV = 16 / ES;                      // source rows that make one 16-byte destination vector
  constexpr int VL = ES == 1 ? 4 : 8, WL = 32 / VL;
  return ((r / RPV) % VL) * WL;
}

template <int ES>
__global__ void __launch_bounds__(kTrThreads) transpose_kernel(const TrParams p) {
  __shared__ uint32_t tile[kTileRows][kTileWords];
  constexpr int TC = kTileWords * 4 / ES;           // source columns per tile
  constexpr int RPV = 16 / ES;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * kTileRows, c0 = static_cast<int64_t>(blockIdx.x) * TC;
  const char *src = p.src + static_cast<int64_t>(blockIdx.z) * p.src_batch * ES;
  char *dst = p.dst + static_cast<int64_t>(blockIdx.z) * p.dst_batch * ES;
  const bool full = p.aligned && r0 + kTileRows <= p.rows && c0 + TC <= p.cols;

  if (!full) {
    // edge tile (or an unaligned problem): element copies, destination-major so that the stores coalesce
    for (int i = threadIdx.x; i < kTileRows * TC; i += kTrThreads) {
      const int r = i % kTileRows, c = i / kTileRows;
      if (r0 + r < p.rows && c0 + c < p.cols) {
        const char *s = src + ((r0 + r) * p.src_row + c0 + c) * ES;
        char *d = dst + ((c0 + c) * p.dst_row + r0 + r) * ES;
        if (ES == 1) *d = *s;
        else if (ES == 2) *reinterpret_cast<uint16_t *>(d) = *reinterpret_cast<const uint16_t *>(s);
        else if (ES == 4) *reinterpret_cast<uint32_t *>(d) = *reinterpret_cast<const uint32_t *>(s);
        else *reinterpret_cast<uint64_t *>(d) = *reinterpret_cast<const uint64_t *>(s);
      }
    }
    return;
  }

  // ---- load: 64 rows x 8 vectors of 16 bytes, two per thread
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int r = threadIdx.x / 8 + 32 * j, v = threadIdx.x % 8;
    const Vec16 d = ld_stream(src + ((r0 + r) * p.src_row + c0) * ES + v * 16);
    *reinterpret_cast<uint4 *>(&tile[r][(4 * v) ^ swz<ES>(r)]) = make_uint4(d.w[0], d.w[1], d.w[2], d.w[3]);
  }
  __syncthreads();

  // ---- store: a task = one unit of source columns (a word; an element for 8-byte types) x one group of RPV rows
  constexpr int VL = ES == 1 ? 4 : 8, WL = 32 / VL;
  constexpr int UW = ES == 8 ? 2 : 1;               // words per unit
  constexpr int NU = kTileWords / UW;               // units per tile row
  constexpr int UL = WL / UW;                       // unit lanes per warp step
  constexpr int NV = kTileRows / RPV;               // row groups per tile
  constexpr int kTasks = NU * NV;
  for (int q = threadIdx.x; q < kTasks; q += kTrThreads) {
    const int ul = q % UL, vl = (q / UL) % VL, rest = q / (UL * VL);
    const int unit = (rest % (NU / UL)) * UL + ul, vg = (rest / (NU / UL)) * VL + vl;
    const int rr = vg * RPV;                        // first source row of the group
    const int f = swz<ES>(rr);                      // the same for all rows of the group
    if constexpr (ES == 4) {
      Vec16 o;
#pragma unroll
      for (int i = 0; i < 4; ++i) o.w[i] = tile[rr + i][unit ^ f];
      st_stream(dst + ((c0 + unit) * p.dst_row + r0 + rr) * 4, o);
    } else if constexpr (ES == 8) {
      Vec16 o;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint2 e = *reinterpret_cast<const uint2 *>(&tile[rr + i][(2 * unit) ^ f]);
        o.w[2 * i] = e.x;
        o.w[2 * i + 1] = e.y;
      }
      st_stream(dst + ((c0 + unit) * p.dst_row + r0 + rr) * 8, o);
    } else if constexpr (ES == 2) {
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = tile[rr + i][unit ^ f];
      Vec16 lo, hi;                                 // destination rows 2 unit and 2 unit + 1
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        lo.w[i] = __byte_perm(w[2 * i], w[2 * i + 1], 0x5410);
        hi.w[i] = __byte_perm(w[2 * i], w[2 * i + 1], 0x7632);
      }
      st_stream(dst + ((c0 + 2 * unit) * p.dst_row + r0 + rr) * 2, lo);
      st_stream(dst + ((c0 + 2 * unit + 1) * p.dst_row + r0 + rr) * 2, hi);
    } else {
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) w[i] = tile[rr + i][unit ^ f];
#pragma unroll
      for (int b = 0; b < 4; ++b) {                 // destination row 4 unit + b takes byte b of every word
        Vec16 o;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t x = __byte_perm(w[4 * i], w[4 * i + 1], 0x0040 + 0x11 * b);      // bytes b of words 0, 1
          const uint32_t y = __byte_perm(w[4 * i + 2], w[4 * i + 3], 0x0040 + 0x11 * b);  // bytes b of words 2, 3
          o.w[i] = __byte_perm(x, y, 0x5410);
        }
        st_stream(dst + ((c0 + 4 * unit + b) * p.dst_row + r0 + rr), o);
      }
    }
  }
}

}  // namespace

// dst[b][i][j] = src[b][j][i]: the source matrix is [rows][cols] (row stride src_row), the destination
// [cols][rows] (row stride dst_row); strides in elements.  false: the geometry is outside the grid limits.
bool launch_transpose(int elem_bytes, const void *src, void *dst, int64_t batch, int64_t rows, int64_t cols, int64_t src_row,
                      int64_t dst_row, int64_t src_batch, int64_t dst_batch, cudaStream_t st) {
  const int64_t tc = kTileWords * 4 / elem_bytes;
  const int64_t gx = ceil_div(cols, tc), gy = ceil_div(rows, kTileRows);
  if (gx > 0x7fffffffLL || gy > 65535 || batch > 65535 || batch < 1) return false;
  TrParams p{static_cast<const char *>(src), static_cast<char *>(dst), rows, cols, src_row, dst_row, src_batch, dst_batch, 0};
  auto mult16 = [&](int64_t elems) { return (elems * elem_bytes) % 16 == 0; };
  p.aligned = aligned_to(src, 16) && aligned_to(dst, 16) && mult16(src_row) && mult16(dst_row) && (batch == 1 || (mult16(src_batch) && mult16(dst_batch)));
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(batch));
  switch (elem_bytes) {
    case 1: transpose_kernel<1><<<grid, kTrThreads, 0, st>>>(p); break;
    case 2: transpose_kernel<2><<<grid, kTrThreads, 0, st>>>(p); break;
    case 4: transpose_kernel<4><<<grid, kTrThreads, 0, st>>>(p); break;
    case 8: transpose_kernel<8><<<grid, kTrThreads, 0, st>>>(p); break;
    default: return false;
  }
  return true;
}

}  // namespace bsir
