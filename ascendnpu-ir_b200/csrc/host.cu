// host.cu -- host layer of the library: status/error text, per-thread stream,
// per-device info and scratch, and the compiled-kernel registry behind
// bsir_kernel_register() / bsir_launch().
//
// bsir_launch() is the counterpart of the reference's host-side launch
//   void *args[] = {in0, in1, out};
//   rtKernelLaunch(stub, blockDim, args, sizeof(args), nullptr, stream);
// (bishengir/test/Integration/HIVM/VecAdd/main.cpp:169-171): a kernel is looked
// up by name and receives one bare device pointer per memref argument, inputs
// first, outputs last, exactly like a kernel compiled with static shapes
// (enable-static-bare-ptr, bishengir/include/bishengir/Tools/bishengir-compile/Options.td:149-156).
#include <cuda.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace bsir {

static thread_local char tl_error[512] = {0};
static thread_local int32_t tl_status = 0;
static thread_local cudaStream_t tl_stream = nullptr;
static std::atomic<long long> g_launches{0};

int32_t fail(int32_t status, const char *fmt, ...) {
  tl_status = status;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
  return status;
}
void clear_error() { tl_error[0] = 0; tl_status = 0; }
cudaStream_t resolve_stream(void *stream) { return stream ? static_cast<cudaStream_t>(stream) : tl_stream; }
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int32_t check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(BSIR_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return BSIR_OK;
}

static constexpr int kMaxDevices = 64;
struct ScratchBlock {
  void *ptr = nullptr;
  size_t bytes = 0;
};
struct PerDevice {
  std::once_flag once;
  DeviceInfo info;
  std::mutex mu;
  // Library-owned scratch: one block per stream that ever asked for one, so that calls on different streams never
  // share counters or partial results.  A block that became too small is replaced and kept in `retired` until
  // bsir_release_workspace(): a launch already enqueued may still be using it, and nothing here waits for the GPU.
  std::map<cudaStream_t, ScratchBlock> scratch;
  std::vector<void *> retired;
  ScratchBlock last;   // the block handed out most recently (what a capturing stream borrows)
  int *error_word = nullptr;
};
static PerDevice g_dev[kMaxDevices];

static PerDevice *current() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return nullptr;
  PerDevice *p = &g_dev[d];
  std::call_once(p->once, [p, d] {
    p->info.device = d;
    cudaDeviceGetAttribute(&p->info.sm_count, cudaDevAttrMultiProcessorCount, d);
    cudaDeviceGetAttribute(&p->info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, d);
    cudaDeviceGetAttribute(&p->info.cc_major, cudaDevAttrComputeCapabilityMajor, d);
  });
  return p;
}

const DeviceInfo &device_info() {
  static DeviceInfo none;
  PerDevice *p = current();
  return p ? p->info : none;
}

// Scratch of at least `bytes` for work enqueued on `stream`.  Steady state: a map lookup, no CUDA call.  When the
// stream has no block yet, or one too small, a new one is allocated and cleared on `stream`, which orders the
// clearing before the caller's kernels without the host waiting.  A capturing stream cannot allocate: it borrows the
// block handed out last on this device if that one is large enough (the usual recipe -- warm up on one stream,
// capture on another -- then just works; the graph must not be replayed while other work uses that stream's
// scratch), and fails with a message otherwise.
void *device_workspace(size_t bytes, cudaStream_t stream) {
  PerDevice *p = current();
  if (!p) { fail(BSIR_ERR_WORKSPACE, "no current CUDA device"); return nullptr; }
  std::lock_guard<std::mutex> lock(p->mu);
  auto it = p->scratch.find(stream);
  if (it != p->scratch.end() && it->second.ptr && it->second.bytes >= bytes) {
    p->last = it->second;
    return it->second.ptr;
  }
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) cudaGetLastError();
  if (cap != cudaStreamCaptureStatusNone) {
    if (p->last.ptr && p->last.bytes >= bytes) return p->last.ptr;
    fail(BSIR_ERR_WORKSPACE, "%zu bytes of scratch are needed but the stream is being captured: run the op once, or call "
         "bsir_reserve_workspace, before the capture begins", bytes);
    return nullptr;
  }
  size_t want = size_t(1) << 20;
  while (want < bytes) want <<= 1;
  void *q = nullptr;
  if (cudaMalloc(&q, want) != cudaSuccess) {
    cudaGetLastError();
    fail(BSIR_ERR_WORKSPACE, "cannot allocate %zu bytes of device scratch", want);
    return nullptr;
  }
  if (cudaMemsetAsync(q, 0, want, stream) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(q);
    fail(BSIR_ERR_WORKSPACE, "cannot clear %zu bytes of device scratch", want);
    return nullptr;
  }
  ScratchBlock &b = p->scratch[stream];
  if (b.ptr) p->retired.push_back(b.ptr);
  b.ptr = q;
  b.bytes = want;
  p->last = b;
  return q;
}

bool make_byte_tmap(CUtensorMap *map, const void *ptr, uint64_t inner, uint64_t outer, uint64_t pitch, uint32_t box_rows, bool swizzle) {
  using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn enc = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      enc = reinterpret_cast<EncodeFn>(sym);
    else
      cudaGetLastError();
  });
  if (!enc) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch};
  cuuint32_t box[2] = {128u, box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int *device_error_word() {
  PerDevice *p = current();
  if (!p) return nullptr;
  std::lock_guard<std::mutex> lock(p->mu);
  if (!p->error_word) {
    if (cudaMalloc(reinterpret_cast<void **>(&p->error_word), sizeof(int)) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    cudaMemset(p->error_word, 0, sizeof(int));
  }
  return p->error_word;
}

// ----------------------------------------------------------------------------
// compiled-kernel registry
// ----------------------------------------------------------------------------
static std::mutex g_reg_mu;
static std::map<std::string, bsir_kernel_desc> &registry() {
  static std::map<std::string, bsir_kernel_desc> r;
  return r;
}

static int num_args_of(const bsir_kernel_desc &d) {
  switch (d.kind) {
    case BSIR_KERNEL_ELEMWISE_BINARY: return 3;
    case BSIR_KERNEL_ELEMWISE_UNARY: return 2;
    case BSIR_KERNEL_CAST: return 2;
    case BSIR_KERNEL_RMS_NORM: return 4;
    case BSIR_KERNEL_SOFTMAX: return 2;
    case BSIR_KERNEL_QUANT_PER_TOKEN: return 3;
    case BSIR_KERNEL_REDUCE_WITH_INDEX: return 3;
    case BSIR_KERNEL_REDUCE: return 2;
    case BSIR_KERNEL_MATMUL_W8A8: return 5;
    case BSIR_KERNEL_MATMUL_W4A16: return 5;
    default: return -1;
  }
}

static void contiguous_strides(int rank, const int64_t *sizes, int64_t *strides) {
  int64_t s = 1;
  for (int i = rank - 1; i >= 0; --i) { strides[i] = s; s *= sizes[i]; }
  for (int i = rank; i < 3; ++i) strides[i] = 0;
}

}  // namespace bsir

using namespace bsir;

extern "C" {

const char *bsir_status_string(int32_t s) {
  switch (s) {
    case BSIR_OK: return "ok";
    case BSIR_ERR_NULL: return "null pointer";
    case BSIR_ERR_SHAPE: return "bad shape";
    case BSIR_ERR_STRIDE: return "unsupported stride";
    case BSIR_ERR_DTYPE: return "unsupported dtype";
    case BSIR_ERR_ATTR: return "bad attribute";
    case BSIR_ERR_ALIGN: return "misaligned pointer";
    case BSIR_ERR_LAUNCH: return "CUDA launch error";
    case BSIR_ERR_UNKNOWN_KERNEL: return "unknown kernel";
    case BSIR_ERR_ARGS: return "bad kernel arguments";
    case BSIR_ERR_WORKSPACE: return "workspace error";
    case BSIR_ERR_UNSUPPORTED: return "unsupported";
    case BSIR_ERR_DEVICE: return "device-side wait gave up";
    default: return "unknown status";
  }
}
const char *bsir_last_error(void) { return tl_error; }
int32_t bsir_last_status(void) { return tl_status; }
const char *bsir_version(void) { return "bsir_b200 0.1 (sm_100a)"; }

int32_t bsir_set_stream(void *stream) {
  tl_stream = static_cast<cudaStream_t>(stream);
  return BSIR_OK;
}
void *bsir_get_stream(void) { return tl_stream; }
int32_t bsir_dtype_size(int32_t dtype) { return dtype_bytes(dtype); }
int64_t bsir_launch_count(void) { return g_launches.load(); }

int32_t bsir_device_error(void) {
  int *w = device_error_word();
  if (!w) return fail(BSIR_ERR_WORKSPACE, "no device error word");
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return check_launch("bsir_device_error");
  cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(w, 0, sizeof(int));
  return v;
}

int32_t bsir_release_workspace(void) {
  PerDevice *p = current();
  if (!p) return fail(BSIR_ERR_WORKSPACE, "no current CUDA device");
  std::lock_guard<std::mutex> lock(p->mu);
  if (!p->scratch.empty() || !p->retired.empty()) cudaDeviceSynchronize();   // nothing enqueued may still use a block
  for (auto &kv : p->scratch)
    if (kv.second.ptr) cudaFree(kv.second.ptr);
  for (void *q : p->retired) cudaFree(q);
  p->scratch.clear();
  p->retired.clear();
  p->last = ScratchBlock{};
  return BSIR_OK;
}

int32_t bsir_reserve_workspace(int64_t bytes, void *stream) {
  clear_error();
  if (bytes < 0) return fail(BSIR_ERR_SHAPE, "bsir_reserve_workspace: %lld bytes", (long long)bytes);
  if (!device_workspace(static_cast<size_t>(bytes), resolve_stream(stream))) return BSIR_ERR_WORKSPACE;
  if (!device_error_word()) return fail(BSIR_ERR_WORKSPACE, "bsir_reserve_workspace: no device error word");
  return BSIR_OK;
}

int32_t bsir_kernel_register(const char *name, const bsir_kernel_desc *desc) {
  clear_error();
  if (!name || !desc) return fail(BSIR_ERR_NULL, "bsir_kernel_register: null argument");
  if (num_args_of(*desc) < 0) return fail(BSIR_ERR_ATTR, "bsir_kernel_register: unknown kind %d", desc->kind);
  if (desc->rank < 0 || desc->rank > 4) return fail(BSIR_ERR_SHAPE, "bsir_kernel_register: rank %d", desc->rank);
  std::lock_guard<std::mutex> lock(g_reg_mu);
  registry()[name] = *desc;
  return BSIR_OK;
}
int32_t bsir_kernel_unregister(const char *name) {
  if (!name) return fail(BSIR_ERR_NULL, "bsir_kernel_unregister: null name");
  std::lock_guard<std::mutex> lock(g_reg_mu);
  return registry().erase(name) ? BSIR_OK : fail(BSIR_ERR_UNKNOWN_KERNEL, "kernel '%s' is not registered", name);
}
int32_t bsir_kernel_num_args(const char *name) {
  if (!name) return fail(BSIR_ERR_NULL, "bsir_kernel_num_args: null name");
  std::lock_guard<std::mutex> lock(g_reg_mu);
  auto it = registry().find(name);
  if (it == registry().end()) return fail(BSIR_ERR_UNKNOWN_KERNEL, "kernel '%s' is not registered", name);
  return num_args_of(it->second);
}

int32_t bsir_launch(const char *name, uint32_t block_dim, void **args, size_t args_size, void *stream) {
  (void)block_dim;  // tiling is chosen per shape by each op; the hint does not change results
  clear_error();
  if (!name || !args) return fail(BSIR_ERR_NULL, "bsir_launch: null argument");
  bsir_kernel_desc d;
  {
    std::lock_guard<std::mutex> lock(g_reg_mu);
    auto it = registry().find(name);
    if (it == registry().end()) return fail(BSIR_ERR_UNKNOWN_KERNEL, "kernel '%s' is not registered", name);
    d = it->second;
  }
  const int na = num_args_of(d);
  if (args_size != sizeof(void *) * static_cast<size_t>(na))
    return fail(BSIR_ERR_ARGS, "kernel '%s' takes %d pointers (%zu bytes), got %zu bytes", name, na,
                sizeof(void *) * static_cast<size_t>(na), args_size);
  void *st = stream ? stream : static_cast<void *>(tl_stream);
  int64_t strides[3];
  const int rank3 = d.rank > 3 ? 3 : d.rank;
  switch (d.kind) {
    case BSIR_KERNEL_ELEMWISE_BINARY: {
      contiguous_strides(rank3, d.sizes, strides);
      bsir_operand a{args[0], {strides[0], strides[1], strides[2]}, 0};
      bsir_operand b{args[1], {strides[0], strides[1], strides[2]}, 0};
      return bsir_elemwise_binary(d.fn, d.dtype, rank3, d.sizes, &a, &b, args[2], strides, st);
    }
    case BSIR_KERNEL_ELEMWISE_UNARY: {
      contiguous_strides(rank3, d.sizes, strides);
      bsir_operand x{args[0], {strides[0], strides[1], strides[2]}, 0};
      return bsir_elemwise_unary(d.fn, d.dtype, rank3, d.sizes, &x, args[1], strides, st);
    }
    case BSIR_KERNEL_CAST:
      contiguous_strides(rank3, d.sizes, strides);
      return bsir_cast(d.dtype, d.dst_dtype, d.round_mode, d.overflow_mode, rank3, d.sizes, args[0], strides,
                       args[1], strides, st);
    case BSIR_KERNEL_RMS_NORM:
      return bsir_rms_norm(d.dtype, d.sizes[0], d.sizes[1], args[0], d.sizes[1], args[1], d.eps, args[2],
                           d.sizes[1], args[3], st);
    case BSIR_KERNEL_SOFTMAX:
      return bsir_softmax(d.dtype, d.sizes[0], d.sizes[1], args[0], d.sizes[1], args[1], d.sizes[1], st);
    case BSIR_KERNEL_QUANT_PER_TOKEN:
      return bsir_quant_per_token_i8(d.dtype, d.round_mode, d.sizes[0], d.sizes[1], args[0], d.sizes[1],
                                     static_cast<int8_t *>(args[1]), d.sizes[1], static_cast<float *>(args[2]), st);
    case BSIR_KERNEL_REDUCE_WITH_INDEX:
      return bsir_reduce_with_index(d.fn, d.dtype, d.flags & 1, (d.flags >> 1) & 1, d.sizes[0], d.sizes[1], args[0],
                                    d.sizes[1], args[1], static_cast<int32_t *>(args[2]), nullptr, 0, st);
    case BSIR_KERNEL_REDUCE:
      return bsir_reduce_last_axis(d.fn, d.dtype, d.sizes[0], d.sizes[1], args[0], d.sizes[1], args[1], st);
    case BSIR_KERNEL_MATMUL_W8A8: {
      const int64_t m = d.sizes[0], n = d.sizes[1], k = d.sizes[2];
      const int tb = d.flags & 1;
      return bsir_matmul_w8a8(m, n, k, static_cast<const int8_t *>(args[0]), k, static_cast<const int8_t *>(args[2]),
                              tb ? k : n, tb, static_cast<const float *>(args[1]),
                              static_cast<const float *>(args[3]), d.dst_dtype, args[4], n, nullptr, nullptr, 0, st);
    }
    case BSIR_KERNEL_MATMUL_W4A16: {
      const int64_t m = d.sizes[0], n = d.sizes[1], k = d.sizes[2], g = d.sizes[3];
      return bsir_matmul_w4a16(m, n, k, g, args[0], k, static_cast<const int32_t *>(args[1]), args[2],
                               static_cast<const int32_t *>(args[3]), args[4], n, st);
    }
    default:
      return fail(BSIR_ERR_ATTR, "kernel '%s': unknown kind %d", name, d.kind);
  }
}

}  // extern "C"
