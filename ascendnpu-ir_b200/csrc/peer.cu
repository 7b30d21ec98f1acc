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

__global__ void peer_signal_wait_kernel(PeerFlags pf, int rank, int world, uint32_t epoch, int *err) {
  const int r = threadIdx.x;
  if (r >= world) return;
  if (r != rank) {
    __threadfence_system();   // the stores of the kernels ahead in this stream are ordered before the flag
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pf.flags[r] + rank), "r"(epoch) : "memory");
  }
  const uint32_t *mine = pf.flags[rank] + r;
  if (r == rank) return;
  const long long t0 = clock64();
  for (uint32_t spin = 0;; ++spin) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (static_cast<int32_t>(v - epoch) >= 0) return;          // flags only grow; wrap-around safe
    if ((spin & 63u) == 63u && clock64() - t0 > 4000000000LL) {   // about two seconds
      if (err) atomicOr(err, BSIR_DEVERR_PEER_WAIT);
      return;
    }
    __nanosleep(200);
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
