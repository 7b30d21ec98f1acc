// peer.cu -- one-sided exchange between the GPUs of a node: buffers every rank can store into, and the flag
// step that closes an exchange.
//
// The N-sharded GEMMs write their block of C straight into every rank's copy of the output (ordinary global
// stores through the peer mapping, issued by the GEMM's epilogue) instead of handing a local block to an
// all-gather.  What remains of the collective is a barrier: "every rank's stores into my buffer have landed".
// This is the role the reference gives its aclshmem wrappers -- put the data, then signal
// (bishengir/lib/Template/lib/Shmem/Shmem.cpp:27-120; comm_params on hivm.hir.mix_matmul,
// bishengir/include/bishengir/Dialect/HIVM/IR/HIVMMacroOps.td:494-520).
//
//   bsir_peer_alloc / bsir_peer_free        a device buffer of its own cudaMalloc (an IPC handle names a whole
//                                           allocation) with a flag page behind the payload
//   bsir_peer_export / open / close         CUDA IPC handle out, peer mapping in
//   bsir_peer_signal_wait                   one small kernel: a system-scope release store of `epoch` into
//                                           flag[my rank] of every peer, then a bounded acquire wait until all
//                                           of this rank's flags have reached `epoch`
// Stream order puts the signal behind the GEMM whose stores it announces.  Nothing here is a TMA or multicast
// access to another GPU's memory, and every wait gives up after about two seconds, records
// BSIR_DEVERR_PEER_WAIT in the device error word and returns, so a rank that never arrives costs the others an
// error status, not a hang.  One rank per GPU: the waiting kernels of different ranks must be able to run at
// the same time.
#include "common.cuh"

namespace bsir {
namespace {

constexpr int kMaxPeers = 16;
struct PeerFlags {
  uint32_t *flags[kMaxPeers];   // flags[r]: rank r's flag array (uint32 per source rank), as mapped in this process
};

// epoch == 0: the step number lives in this rank's flag page (word kEpochWord) and advances by one per launch, so
// a launch captured in a CUDA graph exchanges a fresh epoch at every replay.  All ranks must then use this form
// for every exchange on the buffer, so that their counters stay in step.
constexpr int kEpochWord = 32;

__global__ void peer_signal_wait_kernel(PeerFlags pf, int rank, int world, uint32_t epoch, int *err) {
  __shared__ uint32_t e_sh;
  if (threadIdx.x == 0) e_sh = epoch != 0u ? epoch : pf.flags[rank][kEpochWord] + 1u;
  __syncthreads();
  const uint32_t e = e_sh;
  const int r = threadIdx.x;
  if (r < world && r != rank) {
    __threadfence_system();   // the stores of the kernels ahead in this stream are ordered before the flag
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pf.flags[r] + rank), "r"(e) : "memory");
    const uint32_t *mine = pf.flags[rank] + r;
    const long long t0 = clock64();
    for (uint32_t spin = 0;; ++spin) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (static_cast<int32_t>(v - e) >= 0) break;                 // flags only grow; wrap-around safe
      if ((spin & 63u) == 63u && clock64() - t0 > 4000000000LL) {    // about two seconds
        if (err) atomicOr(err, BSIR_DEVERR_PEER_WAIT);
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && epoch == 0u) pf.flags[rank][kEpochWord] = e;
}

// Copies a [rows x row_bytes] block (row pitch `pitch` bytes, the same in every buffer) from this rank's buffer to
// the same place in each peer's: 16-byte loads of local memory, 16-byte stores through the peer mappings, a warp on
// 512 contiguous bytes.  Used for large blocks, where a GEMM writes its own copy through TMA at full speed and the
// exchange is worth a pass of its own; small blocks are stored by the GEMM's epilogue directly.
struct PushDst {
  char *dst[kMaxPeers];
};
__global__ void __launch_bounds__(256) peer_push_kernel(const char *__restrict__ src, PushDst pd, int n_dst, int64_t rows,
                                                        int64_t vec_per_row, int64_t pitch) {
  const int64_t total = rows * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row, c = i - r * vec_per_row;
    const int64_t off = r * pitch + c * 16;
    const uint4 v = *reinterpret_cast<const uint4 *>(src + off);
    for (int d = 0; d < n_dst; ++d) *reinterpret_cast<uint4 *>(pd.dst[d] + off) = v;
  }
}

}  // namespace
}  // namespace bsir

using namespace bsir;

extern "C" {

int32_t bsir_peer_alloc(int64_t payload_bytes, void **ptr_out, int64_t *flags_offset_out) {
  clear_error();
  if (payload_bytes < 0 || !ptr_out || !flags_offset_out) return fail(BSIR_ERR_NULL, "peer_alloc: bad arguments");
  const size_t payload = (static_cast<size_t>(payload_bytes) + 255u) & ~static_cast<size_t>(255u);
  void *p = nullptr;
  if (cudaMalloc(&p, payload + 256) != cudaSuccess) {
    cudaGetLastError();
    return fail(BSIR_ERR_WORKSPACE, "peer_alloc: cannot allocate %zu bytes", payload + 256);
  }
  cudaMemset(p, 0, payload + 256);
  *ptr_out = p;
  *flags_offset_out = static_cast<int64_t>(payload);
  return BSIR_OK;
}
int32_t bsir_peer_free(void *ptr) {
  if (ptr && cudaFree(ptr) != cudaSuccess) { cudaGetLastError(); return fail(BSIR_ERR_WORKSPACE, "peer_free: cudaFree failed"); }
  return BSIR_OK;
}
int32_t bsir_peer_export(void *ptr, void *handle64) {
  clear_error();
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!ptr || !handle64) return fail(BSIR_ERR_NULL, "peer_export: null argument");
  const cudaError_t e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t *>(handle64), ptr);
  if (e != cudaSuccess) { cudaGetLastError(); return fail(BSIR_ERR_UNSUPPORTED, "peer_export: %s", cudaGetErrorString(e)); }
  return BSIR_OK;
}
int32_t bsir_peer_open(const void *handle64, void **ptr_out) {
  clear_error();
  if (!handle64 || !ptr_out) return fail(BSIR_ERR_NULL, "peer_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  const cudaError_t e = cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { cudaGetLastError(); return fail(BSIR_ERR_UNSUPPORTED, "peer_open: %s", cudaGetErrorString(e)); }
  return BSIR_OK;
}
int32_t bsir_peer_close(void *ptr) {
  if (ptr && cudaIpcCloseMemHandle(ptr) != cudaSuccess) { cudaGetLastError(); return fail(BSIR_ERR_UNSUPPORTED, "peer_close failed"); }
  return BSIR_OK;
}

int32_t bsir_peer_push(int32_t rank, int32_t world, void *const *buffer_ptrs, int64_t byte_offset, int64_t rows, int64_t row_bytes,
                       int64_t pitch_bytes, void *stream) {
  clear_error();
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || !buffer_ptrs) return fail(BSIR_ERR_ARGS, "peer_push: rank %d of %d", rank, world);
  if (rows < 0 || row_bytes < 0 || pitch_bytes < row_bytes) return fail(BSIR_ERR_SHAPE, "peer_push: rows=%lld row_bytes=%lld pitch=%lld", (long long)rows, (long long)row_bytes, (long long)pitch_bytes);
  if (rows == 0 || row_bytes == 0 || world == 1) return BSIR_OK;
  if (row_bytes % 16 || pitch_bytes % 16 || byte_offset % 16) return fail(BSIR_ERR_ALIGN, "peer_push: offsets and sizes must be multiples of 16 bytes");
  PushDst pd{};
  int n = 0;
  for (int r = 0; r < world; ++r) {
    if (!buffer_ptrs[r] || !aligned_to(buffer_ptrs[r], 16)) return fail(BSIR_ERR_NULL, "peer_push: buffer pointer %d", r);
    if (r != rank) pd.dst[n++] = static_cast<char *>(buffer_ptrs[r]) + byte_offset;
  }
  const int64_t total = rows * (row_bytes / 16);
  int64_t blocks = ceil_div(total, 256 * 4);
  const int64_t cap = static_cast<int64_t>(device_info().sm_count > 0 ? device_info().sm_count : 148) * 8;
  if (blocks > cap) blocks = cap;
  peer_push_kernel<<<static_cast<unsigned>(blocks), 256, 0, resolve_stream(stream)>>>(static_cast<const char *>(buffer_ptrs[rank]) + byte_offset, pd, n, rows,
                                                                                      row_bytes / 16, pitch_bytes);
  count_launch();
  return check_launch("peer_push");
}

int32_t bsir_peer_signal_wait(int32_t rank, int32_t world, void *const *flag_ptrs, uint32_t epoch, void *stream) {
  clear_error();
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return fail(BSIR_ERR_ARGS, "peer_signal_wait: rank %d of %d (at most %d)", rank, world, kMaxPeers);
  if (!flag_ptrs) return fail(BSIR_ERR_NULL, "peer_signal_wait: null flag pointers");
  PeerFlags pf{};
  for (int r = 0; r < world; ++r) {
    if (!flag_ptrs[r] || !aligned_to(flag_ptrs[r], 4)) return fail(BSIR_ERR_NULL, "peer_signal_wait: flag pointer %d", r);
    pf.flags[r] = static_cast<uint32_t *>(flag_ptrs[r]);
  }
  peer_signal_wait_kernel<<<1, 32, 0, resolve_stream(stream)>>>(pf, rank, world, epoch, device_error_word());
  count_launch();
  return check_launch("peer_signal_wait");
}

}  // extern "C"
