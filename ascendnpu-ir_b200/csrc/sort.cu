// sort.cu -- hivm.hir.vsort over the last axis: sorted values and the source index of each
// (bishengir/include/bishengir/Dialect/HIVM/IR/HIVMVectorOps.td:2222-2283).
//
// The result is the one the reference's lowering of hfusion.sort produces: n-1 bubble passes of n-1 adjacent
// compare-and-swaps on `cmpf ugt` (ascending) / `cmpf ult` (descending), `cmpi sgt` / `slt` for integers
// (bishengir/lib/Dialect/HFusion/Transforms/DecomposeOpInterfaceImpl.cpp:742-838).  In closed form: equal values
// keep their source order (stable; -0 and +0 are equal); a pair holding a NaN always swaps, which moves every NaN
// one place to the left per pass and carries the one at the front to the end, so a NaN that starts at position p
// ends at (p + 1) mod n whatever the direction; the numbers fill the other places in order.
//
// A row becomes 64-bit keys  order(value) << 32 | index  (order() maps the element type to unsigned integers
// that compare like the values; descending complements it; NaN is the largest key in both directions), so one
// integer comparison decides value and tie at once and the bitonic network -- not stable by itself -- gives a
// stable result with the NaNs at the end in source order; the write-out then moves them to their places.  Short
// rows (a few hundred elements) are sorted this way by one CTA in shared memory; longer ones by stable radix
// passes on the same keys (below): in one CTA's shared memory up to 4096 elements, over device scratch beyond.
// The values' bits are the source's -- the sign of a zero, the payload of a NaN: the network's write-out reads
// them back by index; the radix paths rebuild them from the key and read back only zeros and NaNs.
#include <cstdint>
#include <cstdlib>

#include "common.cuh"

namespace bsir {
namespace {

constexpr int kSortThreads = 512;
constexpr int kSortMaxLen = 8192;

template <int DT> struct SortElem;
template <> struct SortElem<BSIR_F32> { using type = float; };
template <> struct SortElem<BSIR_F16> { using type = uint16_t; };
template <> struct SortElem<BSIR_BF16> { using type = uint16_t; };
template <> struct SortElem<BSIR_I8> { using type = int8_t; };
template <> struct SortElem<BSIR_I16> { using type = int16_t; };
template <> struct SortElem<BSIR_I32> { using type = int32_t; };

// unsigned integers that compare like the values
template <int DT>
__device__ __forceinline__ uint32_t sort_order(typename SortElem<DT>::type v) {
  if constexpr (DT == BSIR_I8 || DT == BSIR_I16 || DT == BSIR_I32) {
    return static_cast<uint32_t>(static_cast<int32_t>(v)) ^ 0x80000000u;
  } else {
    float f;
    if constexpr (DT == BSIR_F32) f = v;
    else if constexpr (DT == BSIR_F16) f = __half2float(__ushort_as_half(v));
    else f = __uint_as_float(static_cast<uint32_t>(v) << 16);
    if (f != f) return 0xffffffffu;                 // NaN: no number maps here (+inf is 0xff800000)
    uint32_t b = __float_as_uint(f);
    if (b == 0x80000000u) b = 0u;                   // -0 ties with +0
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  }
}

template <int DT> constexpr bool kSortFloat = DT == BSIR_F32 || DT == BSIR_F16 || DT == BSIR_BF16;

template <int DT>
__device__ __forceinline__ unsigned long long sort_key(typename SortElem<DT>::type v, int64_t pos, int descending) {
  uint32_t o = sort_order<DT>(v);
  if (descending && !(kSortFloat<DT> && o == 0xffffffffu)) o = ~o;      // a NaN key stays the largest
  return (static_cast<unsigned long long>(o) << 32) | static_cast<uint32_t>(pos);
}

__device__ __forceinline__ bool sort_key_is_nan(unsigned long long k) { return (k >> 32) == 0xffffffffull && k != ~0ull; }

// Where element i of the sorted keys (numbers first, then the row's `nan` NaNs in source order) goes in a row of
// `cols`.  The NaN from source position p goes to (p + 1) mod cols; number r takes the r-th place no NaN took:
// with the NaN places T[0] < T[1] < ... ascending, that is r + #{j : T[j] - j <= r}.
__device__ __forceinline__ int64_t sort_place(const unsigned long long *keys, int64_t i, int64_t cols, int64_t nan) {
  const int64_t numbers = cols - nan;
  if (i >= numbers) {
    const int64_t p = static_cast<uint32_t>(keys[i]);
    return p + 1 == cols ? 0 : p + 1;
  }
  const bool wrap = static_cast<uint32_t>(keys[cols - 1]) == cols - 1;   // the last NaN sits at the row's end
  int64_t lo = 0, hi = nan;                                             // first j with T[j] - j > i
  while (lo < hi) {
    const int64_t j = (lo + hi) >> 1;
    const int64_t t = wrap ? (j == 0 ? 0 : static_cast<int64_t>(static_cast<uint32_t>(keys[numbers + j - 1])) + 1)
                           : static_cast<int64_t>(static_cast<uint32_t>(keys[numbers + j])) + 1;
    if (t - j <= i) lo = j + 1; else hi = j;
  }
  return i + lo;
}

// number of NaN keys at the end of a sorted row (keys[0 .. cols))
__device__ __forceinline__ int64_t sort_count_nan(const unsigned long long *keys, int64_t cols) {
  if (!sort_key_is_nan(keys[cols - 1])) return 0;
  int64_t lo = 0, hi = cols - 1;                                        // first NaN key
  while (lo < hi) {
    const int64_t m = (lo + hi) >> 1;
    if (sort_key_is_nan(keys[m])) hi = m; else lo = m + 1;
  }
  return cols - lo;
}

template <int DT>
__global__ void __launch_bounds__(kSortThreads) sort_rows_kernel(const typename SortElem<DT>::type *__restrict__ src, int64_t src_stride,
                                                                 typename SortElem<DT>::type *__restrict__ dst_value, int64_t val_stride,
                                                                 int32_t *__restrict__ dst_index, int64_t idx_stride, int64_t cols,
                                                                 int npow2, int descending) {
  extern __shared__ unsigned long long keys[];
  const int64_t row = blockIdx.x;
  const auto *s = src + row * src_stride;
  for (int i = threadIdx.x; i < npow2; i += blockDim.x) {
    unsigned long long k = ~0ull;                   // padding sorts last
    if (i < cols) k = sort_key<DT>(s[i], i, descending);
    keys[i] = k;
  }
  __syncthreads();
  for (int k = 2; k <= npow2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < npow2 / 2; t += blockDim.x) {
        const int lo = ((t & ~(j - 1)) << 1) | (t & (j - 1)), hi = lo | j;   // the pair this step compares
        const bool up = (lo & k) == 0;
        const unsigned long long a = keys[lo], b = keys[hi];
        if ((a > b) == up) {
          keys[lo] = b;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  int64_t nan = 0;
  if constexpr (kSortFloat<DT>) nan = sort_count_nan(keys, cols);
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    const uint32_t idx = static_cast<uint32_t>(keys[i]);
    const int64_t at = nan ? sort_place(keys, i, cols, nan) : i;
    if (dst_value) dst_value[row * val_stride + at] = s[idx];
    if (dst_index) dst_index[row * idx_stride + at] = static_cast<int32_t>(idx);
  }
}

// ------------------------------------------------------------------ rows longer than one CTA's shared memory
// A least-significant-digit radix sort, eight bits a pass, over keys kept in device scratch ([rows][cols] 64-bit
// words, two copies).  Every pass is stable, so equal values stay in source order without the index taking part;
// only the bits that can differ are visited (four passes for 32-bit elements, two for 16-bit ones, one for int8).
// A pass is three launches over tiles of 4096 keys: count the digits of each tile; turn the counts of a row, in
// (digit, tile) order, into the place where each tile's run of each digit starts; move the keys.  Nothing is
// counted with atomics on global memory and no tile waits for another, so the result does not depend on timing.
constexpr int kRadixTile = 4096;
constexpr int kRadixThreads = 256;
constexpr int kRadixWarps = kRadixThreads / 32;
constexpr int kRadixIters = kRadixTile / kRadixThreads;       // keys per thread

// The bits the passes sort on, in the upper half of the key.  32-bit elements use all 32 bits of their order; narrower
// ones put their 16 (8) ordered bits at the top, so the digits below hold nothing that could differ between two
// elements whose upper digits agree.  A NaN is 0xffffffff in both directions and no number maps there.
template <int DT>
__device__ __forceinline__ uint32_t radix_order(typename SortElem<DT>::type v, int descending) {
  // selects, no branches: the loads of a thread's keys must not wait for one another behind a jump
  uint32_t o;
  bool nan = false;
  if constexpr (DT == BSIR_I8) {
    o = (static_cast<uint32_t>(static_cast<uint8_t>(v)) ^ 0x80u) << 24;
  } else if constexpr (DT == BSIR_I16) {
    o = (static_cast<uint32_t>(static_cast<uint16_t>(v)) ^ 0x8000u) << 16;
  } else if constexpr (DT == BSIR_I32) {
    o = static_cast<uint32_t>(v) ^ 0x80000000u;
  } else if constexpr (DT == BSIR_F16) {
    uint32_t h = v;
    nan = (h & 0x7fffu) > 0x7c00u;
    h = h == 0x8000u ? 0u : h;                                // -0 ties with +0
    o = ((h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u)) << 16;
  } else {
    uint32_t b;
    if constexpr (DT == BSIR_F32) b = __float_as_uint(v);
    else b = static_cast<uint32_t>(v) << 16;                  // bf16: the lower half follows from the sign bit
    nan = (b & 0x7fffffffu) > 0x7f800000u;
    b = b == 0x80000000u ? 0u : b;
    o = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  }
  o = descending ? ~o : o;
  return nan ? 0xffffffffu : o;
}
template <int DT> constexpr int kRadixFirstShift = (DT == BSIR_F32 || DT == BSIR_I32) ? 0 : DT == BSIR_I8 ? 24 : 16;

// digit counts of one tile -> hist[row][digit][tile]
template <int DT, bool FIRST>
__global__ void __launch_bounds__(kRadixThreads) radix_count_kernel(const typename SortElem<DT>::type *__restrict__ src, int64_t src_stride,
                                                                    const unsigned long long *__restrict__ keys_in, int64_t cols, int descending,
                                                                    int shift, uint32_t *__restrict__ hist, int64_t ntiles) {
  __shared__ uint32_t count[4][256];                          // four copies: fewer adds meet on one word when the digits are few
  const int tid = threadIdx.x, warp = tid >> 5;
  const int64_t row = blockIdx.y, tile = blockIdx.x, base = tile * kRadixTile;
#pragma unroll
  for (int c = 0; c < 4; ++c) count[c][tid] = 0;
  __syncthreads();
  const auto *src_row = src + row * src_stride;
  const unsigned long long *keys_row = keys_in + row * cols;
  uint32_t order[kRadixIters];
  if constexpr (FIRST) {
    typename SortElem<DT>::type raw[kRadixIters];
#pragma unroll
    for (int i = 0; i < kRadixIters; ++i) {
      const int64_t pos = base + i * kRadixThreads + tid;
      raw[i] = pos < cols ? src_row[pos] : typename SortElem<DT>::type(0);
    }
#pragma unroll
    for (int i = 0; i < kRadixIters; ++i) order[i] = radix_order<DT>(raw[i], descending);
  } else {
#pragma unroll
    for (int i = 0; i < kRadixIters; ++i) {
      const int64_t pos = base + i * kRadixThreads + tid;
      order[i] = pos < cols ? static_cast<uint32_t>(keys_row[pos] >> 32) : 0u;
    }
  }
#pragma unroll
  for (int i = 0; i < kRadixIters; ++i)
    if (base + i * kRadixThreads + tid < cols) atomicAdd(&count[warp & 3][(order[i] >> shift) & 255u], 1u);
  __syncthreads();
  hist[(row * 256 + tid) * ntiles + tile] = count[0][tid] + count[1][tid] + count[2][tid] + count[3][tid];
}

// hist[row] holds 256 x ntiles counts; in (digit, tile) order each becomes the sum of the ones before it
constexpr int kRadixOffsetsTiles = 44;                         // rows of up to this many tiles take the counts into shared memory
__global__ void __launch_bounds__(kRadixThreads) radix_offsets_kernel(uint32_t *__restrict__ hist, int64_t ntiles) {
  __shared__ uint32_t total[256];
  __shared__ uint32_t warp_sum[kRadixWarps];
  __shared__ uint32_t staged[256 * kRadixOffsetsTiles];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t *h = hist + static_cast<int64_t>(blockIdx.x) * 256 * ntiles;
  if (ntiles <= kRadixOffsetsTiles) {
    // one coalesced read, thread d walks digit d's tiles in shared memory, one coalesced write
    const int nt = static_cast<int>(ntiles), entries = 256 * nt;
    for (int e = tid; e < entries; e += kRadixThreads) staged[e] = h[e];
    __syncthreads();
    uint32_t mine = 0;
    for (int t = 0; t < nt; ++t) mine += staged[tid * nt + t];
    uint32_t incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    uint32_t running = incl - mine;
    for (int w = 0; w < warp; ++w) running += warp_sum[w];
    for (int t = 0; t < nt; ++t) {
      const uint32_t c = staged[tid * nt + t];
      staged[tid * nt + t] = running;
      running += c;
    }
    __syncthreads();
    for (int e = tid; e < entries; e += kRadixThreads) h[e] = staged[e];
    return;
  }
  for (int d = warp; d < 256; d += kRadixWarps) {
    uint32_t sum = 0;
    for (int64_t t = lane; t < ntiles; t += 32) sum += h[d * ntiles + t];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) total[d] = sum;
  }
  __syncthreads();
  {   // exclusive scan of the 256 digit totals
    const uint32_t mine = total[tid];
    uint32_t incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    uint32_t before = 0;
    for (int w = 0; w < warp; ++w) before += warp_sum[w];
    total[tid] = before + incl - mine;
  }
  __syncthreads();
  for (int d = warp; d < 256; d += kRadixWarps) {
    uint32_t running = total[d];
    for (int64_t t0 = 0; t0 < ntiles; t0 += 32) {
      const int64_t t = t0 + lane;
      const uint32_t mine = t < ntiles ? h[d * ntiles + t] : 0u;
      uint32_t incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (t < ntiles) h[d * ntiles + t] = running + incl - mine;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
}

// One pass over one tile of 256 * ITERS keys (in registers; a warp owns 32 * ITERS consecutive keys and takes them
// 32 at a time in order): the tile's keys end up in shared memory in the order of the digit at `shift`, source order
// kept within a digit.  Within a group of 32 a key's rank among the keys of its digit is the number of lower lanes
// with that digit (the lanes of a digit meet in a word of shared memory, each setting its bit), and the warp's running count of the digit carries the rank from group to group; the warps'
// counts are then chained behind one another, digit by digit.  Returns, for digit threadIdx.x, where its keys start
// in the tile.  `warp_valid` is how many of the warp's keys exist (the row may end inside the tile).
template <int ITERS>
struct RadixShared {
  unsigned long long sorted[kRadixThreads * ITERS];
  uint32_t lanes[kRadixWarps][256];                            // per warp and digit: the lanes holding it in the current group
  uint16_t count[kRadixWarps][256];                            // at most 4096 keys a tile
  uint32_t warp_sum[kRadixWarps];
};

template <int ITERS>
__device__ __forceinline__ uint32_t radix_tile_pass(RadixShared<ITERS> &sm, const unsigned long long (&key)[ITERS], int warp_valid, int shift) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int w = 0; w < kRadixWarps; ++w) {
    sm.count[w][tid] = 0;
    sm.lanes[w][tid] = 0;
  }
  __syncthreads();                                            // also: every reader of sm.sorted from the pass before is done
  uint32_t rank2[(ITERS + 1) / 2];                            // two 16-bit ranks a word
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    // The lanes with this key's digit, found by each lane setting its bit in the digit's word: one shared-memory
    // operation a key where eight ballots would take some forty instructions a group.
    const bool valid = i * 32 + lane < warp_valid;
    const uint32_t digit = static_cast<uint32_t>(key[i] >> (32 + shift)) & 255u;
    if (valid) atomicOr(&sm.lanes[warp][digit], 1u << lane);
    __syncwarp();
    uint32_t peers = 0, before = 0;
    if (valid) {
      peers = sm.lanes[warp][digit];
      before = sm.count[warp][digit];
    }
    __syncwarp();
    const uint32_t below = __popc(peers & ((1u << lane) - 1));
    if (valid && below == 0) {
      sm.count[warp][digit] = static_cast<uint16_t>(before + __popc(peers));
      sm.lanes[warp][digit] = 0;
    }
    __syncwarp();
    if (i & 1) rank2[i >> 1] |= (before + below) << 16;
    else rank2[i >> 1] = before + below;
  }
  __syncthreads();
  uint32_t start;
  {
    uint32_t mine = 0;
#pragma unroll
    for (int w = 0; w < kRadixWarps; ++w) mine += sm.count[w][tid];
    uint32_t incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) sm.warp_sum[warp] = incl;
    __syncthreads();
    start = incl - mine;
    for (int w = 0; w < warp; ++w) start += sm.warp_sum[w];
    uint32_t running = start;
#pragma unroll
    for (int w = 0; w < kRadixWarps; ++w) {
      const uint32_t c = sm.count[w][tid];
      sm.count[w][tid] = static_cast<uint16_t>(running);
      running += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    if (i * 32 + lane < warp_valid) {
      const uint32_t digit = static_cast<uint32_t>(key[i] >> (32 + shift)) & 255u;
      sm.sorted[sm.count[warp][digit] + ((rank2[i >> 1] >> (16 * (i & 1))) & 0xffffu)] = key[i];
    }
  }
  __syncthreads();
  return start;
}

__device__ __forceinline__ int radix_warp_valid(int64_t cols, int64_t warp_base, int per_warp) {
  const int64_t left = cols - warp_base;
  return left <= 0 ? 0 : left < per_warp ? static_cast<int>(left) : per_warp;
}

// Moves the keys of one tile to their places of this pass: the tile, in digit order in shared memory, goes out in
// runs, so that the stores of a warp fall into a few stretches of the row instead of 32 places.
template <int DT, bool FIRST>
__global__ void __launch_bounds__(kRadixThreads, 3) radix_move_kernel(const typename SortElem<DT>::type *__restrict__ src, int64_t src_stride,
                                                                      const unsigned long long *__restrict__ keys_in,
                                                                      unsigned long long *__restrict__ keys_out, int64_t cols, int descending,
                                                                      int shift, const uint32_t *__restrict__ hist, int64_t ntiles) {
  __shared__ RadixShared<kRadixIters> sm;
  __shared__ uint32_t to_row[256];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row = blockIdx.y, tile = blockIdx.x;
  const int64_t base = tile * kRadixTile + warp * (kRadixTile / kRadixWarps);
  const auto *src_row = src + row * src_stride;
  const unsigned long long *keys_row = keys_in + row * cols;
  unsigned long long key[kRadixIters];
  if constexpr (FIRST) {   // every load first, the keys from them afterwards
    typename SortElem<DT>::type raw[kRadixIters];
#pragma unroll
    for (int i = 0; i < kRadixIters; ++i) {
      const int64_t pos = base + i * 32 + lane;
      raw[i] = pos < cols ? src_row[pos] : typename SortElem<DT>::type(0);
    }
#pragma unroll
    for (int i = 0; i < kRadixIters; ++i)
      key[i] = (static_cast<unsigned long long>(radix_order<DT>(raw[i], descending)) << 32) | static_cast<uint32_t>(base + i * 32 + lane);
  } else {
#pragma unroll
    for (int i = 0; i < kRadixIters; ++i) {
      const int64_t pos = base + i * 32 + lane;
      key[i] = pos < cols ? keys_row[pos] : 0ull;
    }
  }
  const uint32_t start = radix_tile_pass<kRadixIters>(sm, key, radix_warp_valid(cols, base, kRadixTile / kRadixWarps), shift);
  to_row[tid] = hist[(row * 256 + tid) * ntiles + tile] - start;   // turns a place in the tile into the place in the row
  __syncthreads();
  const int64_t left = cols - tile * kRadixTile;
  const int in_tile = left < kRadixTile ? static_cast<int>(left) : kRadixTile;
  unsigned long long *out_row = keys_out + row * cols;
#pragma unroll 4
  for (int j = tid; j < in_tile; j += kRadixThreads) {
    const unsigned long long k = sm.sorted[j];
    const uint32_t digit = static_cast<uint32_t>(k >> (32 + shift)) & 255u;
    out_row[to_row[digit] + static_cast<uint32_t>(j)] = k;
  }
}

// The element a key stands for, from the key alone; false for a zero (either sign maps to the same key) or a NaN,
// whose bits are the source's.
template <int DT>
__device__ __forceinline__ bool radix_value(uint32_t o, int descending, typename SortElem<DT>::type &v) {
  if (kSortFloat<DT> && o == 0xffffffffu) return false;
  if (descending) o = ~o;
  if constexpr (DT == BSIR_I32) { v = static_cast<int32_t>(o ^ 0x80000000u); return true; }
  else if constexpr (DT == BSIR_I16) { v = static_cast<int16_t>((o >> 16) ^ 0x8000u); return true; }
  else if constexpr (DT == BSIR_I8) { v = static_cast<int8_t>((o >> 24) ^ 0x80u); return true; }
  else if constexpr (DT == BSIR_F16) {
    const uint32_t h = (o & 0x80000000u) ? (o >> 16) & 0x7fffu : (~o >> 16) & 0xffffu;
    v = static_cast<uint16_t>(h);
    return h != 0;
  } else {
    const uint32_t b = (o & 0x80000000u) ? o & 0x7fffffffu : ~o;
    if constexpr (DT == BSIR_F32) v = __uint_as_float(b);
    else v = static_cast<uint16_t>(b >> 16);
    return b != 0;
  }
}

template <int DT>
__global__ void __launch_bounds__(256) sort_emit_kernel(const typename SortElem<DT>::type *__restrict__ src, int64_t src_stride,
                                                        const unsigned long long *__restrict__ keys_g, int64_t keys_stride,
                                                        typename SortElem<DT>::type *__restrict__ dst_value, int64_t val_stride,
                                                        int32_t *__restrict__ dst_index, int64_t idx_stride, int64_t cols, int descending) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= cols) return;
  const int64_t row = blockIdx.y;
  const unsigned long long *keys = keys_g + row * keys_stride;
  const unsigned long long key = keys[i];
  const uint32_t idx = static_cast<uint32_t>(key);
  int64_t at = i;
  if constexpr (kSortFloat<DT>) {
    const int64_t nan = sort_count_nan(keys, cols);          // one load when the row has no NaN
    if (nan) at = sort_place(keys, i, cols, nan);
  }
  if (dst_value) {
    typename SortElem<DT>::type v;
    if (!radix_value<DT>(static_cast<uint32_t>(key >> 32), descending, v)) v = src[row * src_stride + idx];
    dst_value[row * val_stride + at] = v;
  }
  if (dst_index) dst_index[row * idx_stride + at] = static_cast<int32_t>(idx);
}

// Rows of up to 256 * ITERS elements: one CTA sorts a row with every pass in shared memory and writes values and
// indices itself.
template <int DT, int ITERS>
__global__ void __launch_bounds__(kRadixThreads, ITERS > 8 ? 3 : 4) radix_rows_kernel(const typename SortElem<DT>::type *__restrict__ src,
                                                                                        int64_t src_stride,
                                                                                        typename SortElem<DT>::type *__restrict__ dst_value,
                                                                                        int64_t val_stride, int32_t *__restrict__ dst_index,
                                                                                        int64_t idx_stride, int cols, int descending) {
  __shared__ RadixShared<ITERS> sm;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row = blockIdx.x;
  const auto *s = src + row * src_stride;
  const int base = warp * 32 * ITERS;
  const int warp_valid = radix_warp_valid(cols, base, 32 * ITERS);
  unsigned long long key[ITERS];
  {   // every load first, the keys from them afterwards
    typename SortElem<DT>::type raw[ITERS];
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int pos = base + i * 32 + lane;
      raw[i] = pos < cols ? s[pos] : typename SortElem<DT>::type(0);
    }
#pragma unroll
    for (int i = 0; i < ITERS; ++i)
      key[i] = (static_cast<unsigned long long>(radix_order<DT>(raw[i], descending)) << 32) | static_cast<uint32_t>(base + i * 32 + lane);
  }
  for (int shift = kRadixFirstShift<DT>; shift < 32; shift += 8) {
    radix_tile_pass<ITERS>(sm, key, warp_valid, shift);
    if (shift < 24) {
#pragma unroll
      for (int i = 0; i < ITERS; ++i) {
        const int pos = base + i * 32 + lane;
        if (pos < cols) key[i] = sm.sorted[pos];
      }
    }
  }
  int64_t nan = 0;
  if constexpr (kSortFloat<DT>) nan = sort_count_nan(sm.sorted, cols);
  for (int i = tid; i < cols; i += kRadixThreads) {
    const unsigned long long k = sm.sorted[i];
    const uint32_t idx = static_cast<uint32_t>(k);
    const int64_t at = nan ? sort_place(sm.sorted, i, cols, nan) : i;
    if (dst_value) {
      typename SortElem<DT>::type v;
      if (!radix_value<DT>(static_cast<uint32_t>(k >> 32), descending, v)) v = s[idx];
      dst_value[row * val_stride + at] = v;
    }
    if (dst_index) dst_index[row * idx_stride + at] = static_cast<int32_t>(idx);
  }
}

template <int DT>
void launch_radix_rows(const void *src, int64_t ss, void *dv, int64_t vs, int32_t *di, int64_t is, int64_t rows, int64_t cols, int descending,
                       cudaStream_t st) {
  using T = typename SortElem<DT>::type;
  const T *s = static_cast<const T *>(src);
  T *d = static_cast<T *>(dv);
  const unsigned g = static_cast<unsigned>(rows);
  const int n = static_cast<int>(cols);
  if (cols <= kRadixThreads * 2) radix_rows_kernel<DT, 2><<<g, kRadixThreads, 0, st>>>(s, ss, d, vs, di, is, n, descending);
  else if (cols <= kRadixThreads * 4) radix_rows_kernel<DT, 4><<<g, kRadixThreads, 0, st>>>(s, ss, d, vs, di, is, n, descending);
  else if (cols <= kRadixThreads * 8) radix_rows_kernel<DT, 8><<<g, kRadixThreads, 0, st>>>(s, ss, d, vs, di, is, n, descending);
  else radix_rows_kernel<DT, 16><<<g, kRadixThreads, 0, st>>>(s, ss, d, vs, di, is, n, descending);
}

// as many rows at a time as fit `budget` bytes of scratch (two copies of the keys and the digit counts)
template <int DT>
int32_t launch_sort_long(const void *src, int64_t ss, void *dv, int64_t vs, int32_t *di, int64_t is, int64_t rows, int64_t cols,
                         int descending, cudaStream_t st) {
  using T = typename SortElem<DT>::type;
  if (cols > (int64_t(1) << 30)) return fail(BSIR_ERR_UNSUPPORTED, "sort: rows of %lld elements", (long long)cols);
  const int64_t ntiles = ceil_div(cols, static_cast<int64_t>(kRadixTile));
  const int64_t keys_bytes = (cols * 8 + 255) / 256 * 256, hist_bytes = ntiles * 256 * 4;
  const int64_t row_bytes = 2 * keys_bytes + hist_bytes;
  const int64_t budget = int64_t(1) << 30;
  int64_t rows_per_pass = budget / row_bytes;
  if (rows_per_pass < 1) rows_per_pass = 1;
  if (rows_per_pass > rows) rows_per_pass = rows;
  if (rows_per_pass > 65535) rows_per_pass = 65535;
  char *ws = static_cast<char *>(device_workspace(kScratchCounterBytes + static_cast<size_t>(rows_per_pass * row_bytes), st));
  if (!ws) return BSIR_ERR_WORKSPACE;
  // each row's keys start where the row index times cols puts them; the two copies and the counts follow one another
  unsigned long long *keys_a = reinterpret_cast<unsigned long long *>(ws + kScratchCounterBytes);
  unsigned long long *keys_b = reinterpret_cast<unsigned long long *>(ws + kScratchCounterBytes + rows_per_pass * keys_bytes);
  uint32_t *hist = reinterpret_cast<uint32_t *>(ws + kScratchCounterBytes + 2 * rows_per_pass * keys_bytes);
  const T *s = static_cast<const T *>(src);
  T *d = static_cast<T *>(dv);
  for (int64_t r0 = 0; r0 < rows; r0 += rows_per_pass) {
    const unsigned nr = static_cast<unsigned>(rows - r0 < rows_per_pass ? rows - r0 : rows_per_pass);
    const dim3 tiles(static_cast<unsigned>(ntiles), nr);
    const unsigned long long *in = nullptr;
    unsigned long long *out = keys_a;
    for (int shift = kRadixFirstShift<DT>; shift < 32; shift += 8) {
      if (!in) radix_count_kernel<DT, true><<<tiles, kRadixThreads, 0, st>>>(s + r0 * ss, ss, nullptr, cols, descending, shift, hist, ntiles);
      else radix_count_kernel<DT, false><<<tiles, kRadixThreads, 0, st>>>(s, ss, in, cols, descending, shift, hist, ntiles);
      radix_offsets_kernel<<<nr, kRadixThreads, 0, st>>>(hist, ntiles);
      if (!in) radix_move_kernel<DT, true><<<tiles, kRadixThreads, 0, st>>>(s + r0 * ss, ss, nullptr, out, cols, descending, shift, hist, ntiles);
      else radix_move_kernel<DT, false><<<tiles, kRadixThreads, 0, st>>>(s, ss, in, out, cols, descending, shift, hist, ntiles);
      count_launch();
      count_launch();
      count_launch();
      in = out;
      out = out == keys_a ? keys_b : keys_a;
    }
    sort_emit_kernel<DT><<<dim3(static_cast<unsigned>(ceil_div(cols, 256)), nr), 256, 0, st>>>(
        s + r0 * ss, ss, in, cols, d ? d + r0 * vs : nullptr, vs, di ? di + r0 * is : nullptr, is, cols, descending);
  }
  return BSIR_OK;
}

template <int DT>
void launch_sort(const void *src, int64_t ss, void *dv, int64_t vs, int32_t *di, int64_t is, int64_t rows, int64_t cols, int descending,
                 cudaStream_t st) {
  using T = typename SortElem<DT>::type;
  int npow2 = 2;
  while (npow2 < cols) npow2 <<= 1;
  const size_t smem = static_cast<size_t>(npow2) * sizeof(unsigned long long);
  if (smem > 48 * 1024)   // per device, so on every such call rather than once per process
    cudaFuncSetAttribute(sort_rows_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSortMaxLen * 8);
  // half a thread per padded element (each step compares pairs), within [32, 512]: short rows do not pay for
  // idle warps at every barrier
  int threads = npow2 / 2 < 32 ? 32 : npow2 / 2 > kSortThreads ? kSortThreads : npow2 / 2;
  sort_rows_kernel<DT><<<static_cast<unsigned>(rows), threads, smem, st>>>(static_cast<const T *>(src), ss, static_cast<T *>(dv), vs, di, is,
                                                                               cols, npow2, descending);
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" int32_t bsir_sort(int32_t dtype, int32_t descending, int64_t rows, int64_t cols, const void *src, int64_t src_row_stride,
                             void *dst_value, int64_t value_row_stride, int32_t *dst_index, int64_t index_row_stride, void *stream) {
  clear_error();
  const bool ok_type = dtype == BSIR_F32 || dtype == BSIR_F16 || dtype == BSIR_BF16 || dtype == BSIR_I8 || dtype == BSIR_I16 || dtype == BSIR_I32;
  if (!ok_type) return fail(BSIR_ERR_DTYPE, "sort: dtype %d (f32, f16, bf16, i8, i16, i32)", dtype);
  if (rows < 0 || cols < 0) return fail(BSIR_ERR_SHAPE, "sort: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (rows == 0 || cols == 0) return BSIR_OK;
  if (!src || (!dst_value && !dst_index)) return fail(BSIR_ERR_NULL, "sort: null pointer");
  if (rows > 0x7fffffffLL) return fail(BSIR_ERR_SHAPE, "sort: %lld rows", (long long)rows);
  if (src_row_stride < cols || (dst_value && value_row_stride < cols) || (dst_index && index_row_stride < cols))
    return fail(BSIR_ERR_STRIDE, "sort: row stride below the row length");
  const int eb = dtype_bytes(dtype);
  if (!aligned_to(src, eb) || !aligned_to(dst_value, eb) || !aligned_to(dst_index, 4)) return fail(BSIR_ERR_ALIGN, "sort: misaligned");
  if (dst_value) {   // zeros and NaNs are read back from the source after other values have been written
    const char *s0 = static_cast<const char *>(src), *s1 = s0 + ((rows - 1) * src_row_stride + cols) * eb;
    const char *d0 = static_cast<const char *>(dst_value), *d1 = d0 + ((rows - 1) * value_row_stride + cols) * eb;
    if (s0 < d1 && d0 < s1) return fail(BSIR_ERR_UNSUPPORTED, "sort: the sorted values may not overlap the source");
  }
  cudaStream_t st = resolve_stream(stream);
  const int desc = descending != 0;
  // Which of the three ways: rows above one tile of the radix sort (4096) keep their keys in device scratch and
  // take the radix passes; rows of `radix_from` elements or more that fit a tile are radix-sorted by one CTA in
  // shared memory; shorter rows by the bitonic network.
  // (measured on [rows, cols] with rows * cols = 8M: the network wins up to 256 columns of 32-bit elements, 128 of 16-bit ones)
  int64_t radix_from = eb == 4 ? 385 : eb == 2 ? 225 : 129;
  if (const char *e = std::getenv("BSIR_SORT_RADIX_FROM")) { const long c = std::atol(e); if (c >= 2 && c <= kSortMaxLen) radix_from = c; }
  const int way = cols > kSortMaxLen || (cols >= radix_from && cols > kRadixTile) ? 2 : cols >= radix_from ? 1 : 0;
  int32_t rc = BSIR_OK;
#define BSIR_SORT_CASE(DT)                                                                                                      \
  case DT:                                                                                                                      \
    if (way == 2) rc = launch_sort_long<DT>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); \
    else if (way == 1) launch_radix_rows<DT>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st); \
    else launch_sort<DT>(src, src_row_stride, dst_value, value_row_stride, dst_index, index_row_stride, rows, cols, desc, st);  \
    break;
  switch (dtype) {
    BSIR_SORT_CASE(BSIR_F32)
    BSIR_SORT_CASE(BSIR_F16)
    BSIR_SORT_CASE(BSIR_BF16)
    BSIR_SORT_CASE(BSIR_I8)
    BSIR_SORT_CASE(BSIR_I16)
    default:
    BSIR_SORT_CASE(BSIR_I32)
  }
#undef BSIR_SORT_CASE
  if (rc != BSIR_OK) return rc;
  count_launch();
  return check_launch("sort");
}
