// Runtime plumbing of the C ABI: allocation, copies, the ambient stream,
// streams / events / graphs and the API counters.  Same symbols and return
// conventions as the reference's kernels-cuda/runtime.cu, so that
// crates/kernels (memory.rs:469-496, graph.rs:268-290, backend.rs:1724-1770)
// links against this library unchanged.
#include "common.cuh"

#include <atomic>
#include <dlfcn.h>
#include <string.h>

namespace {

std::atomic<cudaStream_t> g_active{nullptr};     // legacy default stream until set
std::atomic<cudaStream_t> g_prefetch{nullptr};

struct Counters {
  std::atomic<uint64_t> v[15];
};
Counters g_counters{};
enum {
  C_MALLOC, C_FREE, C_H2D, C_H2D_B, C_D2H, C_D2H_B, C_D2D, C_D2D_B, C_D2DA, C_D2DA_B,
  C_MEMSET, C_MEMSET_B, C_SYNC, C_SSYNC, C_GRAPH
};
inline void bump(int idx, uint64_t by = 1) { g_counters.v[idx].fetch_add(by, std::memory_order_relaxed); }

void *raw(qwen36_device_ptr_t p) { return reinterpret_cast<void *>(static_cast<uintptr_t>(p.ptr)); }
cudaStream_t cs(qwen36_cuda_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

void set_str(char *dst, size_t cap, const char *src) {
  if (cap == 0) return;
  dst[0] = '\0';
  if (src != nullptr) {
    strncpy(dst, src, cap - 1);
    dst[cap - 1] = '\0';
  }
}

// Path of the shared object that provides `symbol`, if `soname` can be opened.
void library_path(const char *soname, const char *symbol, char *dst, size_t cap) {
  set_str(dst, cap, nullptr);
  void *h = dlopen(soname, RTLD_LAZY | RTLD_NOLOAD);
  if (h == nullptr) h = dlopen(soname, RTLD_LAZY);
  if (h == nullptr) return;
  Dl_info info{};
  void *sym = dlsym(h, symbol);
  if (sym != nullptr && dladdr(sym, &info) != 0) set_str(dst, cap, info.dli_fname);
}

__global__ void increment_i32_kernel(int32_t *target) { atomicAdd(target, 1); }

__global__ void advance_positions_kernel(int32_t *positions, size_t count, int32_t delta) {
  const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i < count) positions[i] += delta;
}

// Read-only walk that pulls a range into L2 (one 16-byte load per thread per
// step, result folded into a value that is never stored unless it is a
// sentinel no data produces).
__global__ void l2_warm_kernel(const uint4 *base, size_t n16, unsigned *sink) {
  unsigned acc = 0;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n16;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint4 v = __ldg(base + i);
    acc ^= v.x ^ v.y ^ v.z ^ v.w;
  }
  if (acc == 0xdeadbeefu && sink != nullptr) *sink = acc;
}

}  // namespace

using q36::cuda_status;

extern "C" {

qwen36_cuda_stream_t qwen36_internal_active_stream(void) {
  return reinterpret_cast<qwen36_cuda_stream_t>(g_active.load(std::memory_order_acquire));
}
qwen36_cuda_stream_t qwen36_internal_prefetch_stream(void) {
  return reinterpret_cast<qwen36_cuda_stream_t>(g_prefetch.load(std::memory_order_acquire));
}
qwen36_cuda_stream_t qwen36_get_active_stream(void) { return qwen36_internal_active_stream(); }
void qwen36_set_active_stream(qwen36_cuda_stream_t s) { g_active.store(cs(s), std::memory_order_release); }
qwen36_cuda_stream_t qwen36_get_prefetch_stream(void) { return qwen36_internal_prefetch_stream(); }
void qwen36_set_prefetch_stream(qwen36_cuda_stream_t s) { g_prefetch.store(cs(s), std::memory_order_release); }

int qwen36_cuda_malloc(qwen36_device_allocation_t *out, size_t bytes) {
  if (out == nullptr) return QWEN36_STATUS_NULL_POINTER;
  out->ptr.ptr = 0;                       // a failed call leaves an empty allocation behind, as in the reference
  out->bytes = 0;
  if (bytes == 0) return QWEN36_STATUS_INVALID_ARGUMENT;
  void *p = nullptr;
  bump(C_MALLOC);
  const cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return QWEN36_STATUS_CUDA_ERROR;
  out->ptr.ptr = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(p));
  out->bytes = bytes;
  return QWEN36_STATUS_SUCCESS;
}

int qwen36_cuda_free(qwen36_device_ptr_t p) {
  if (p.ptr == 0) return QWEN36_STATUS_SUCCESS;
  bump(C_FREE);
  return cuda_status(cudaFree(raw(p)));
}

int qwen36_cuda_memcpy_h2d(qwen36_device_ptr_t dst, const void *src, size_t bytes) {
  if (dst.ptr == 0 || src == nullptr) return QWEN36_STATUS_NULL_POINTER;
  bump(C_H2D); bump(C_H2D_B, bytes);
  return cuda_status(cudaMemcpy(raw(dst), src, bytes, cudaMemcpyHostToDevice));
}

int qwen36_cuda_memcpy_d2h(void *dst, qwen36_device_ptr_t src, size_t bytes) {
  if (dst == nullptr || src.ptr == 0) return QWEN36_STATUS_NULL_POINTER;
  bump(C_D2H); bump(C_D2H_B, bytes);
  return cuda_status(cudaMemcpy(dst, raw(src), bytes, cudaMemcpyDeviceToHost));
}

int qwen36_cuda_memcpy_d2d(qwen36_device_ptr_t dst, qwen36_device_ptr_t src, size_t bytes) {
  if (dst.ptr == 0 || src.ptr == 0) return QWEN36_STATUS_NULL_POINTER;
  bump(C_D2D); bump(C_D2D_B, bytes);
  return cuda_status(cudaMemcpy(raw(dst), raw(src), bytes, cudaMemcpyDeviceToDevice));
}

int qwen36_cuda_memcpy_d2d_async(qwen36_device_ptr_t dst, qwen36_device_ptr_t src, size_t bytes) {
  if (dst.ptr == 0 || src.ptr == 0) return QWEN36_STATUS_NULL_POINTER;
  bump(C_D2DA); bump(C_D2DA_B, bytes);
  return cuda_status(cudaMemcpyAsync(raw(dst), raw(src), bytes, cudaMemcpyDeviceToDevice, q36::stream()));
}

int qwen36_cuda_memset(qwen36_device_ptr_t dst, int value, size_t bytes) {
  if (dst.ptr == 0) return QWEN36_STATUS_NULL_POINTER;
  bump(C_MEMSET); bump(C_MEMSET_B, bytes);
  return cuda_status(cudaMemset(raw(dst), value, bytes));
}

int qwen36_cuda_memset_async(qwen36_device_ptr_t dst, int value, size_t bytes) {
  if (dst.ptr == 0) return QWEN36_STATUS_NULL_POINTER;
  bump(C_MEMSET); bump(C_MEMSET_B, bytes);
  return cuda_status(cudaMemsetAsync(raw(dst), value, bytes, q36::stream()));
}

int qwen36_cuda_synchronize(void) {
  bump(C_SYNC);
  return cuda_status(cudaDeviceSynchronize());
}

int qwen36_cuda_get_diagnostics(qwen36_cuda_diagnostics_t *out) {
  if (out == nullptr) return QWEN36_STATUS_NULL_POINTER;
  memset(out, 0, sizeof(*out));
  out->active_device = -1;
  library_path("libcuda.so.1", "cuInit", out->libcuda_path, sizeof(out->libcuda_path));
  library_path("libcudart.so", "cudaGetDeviceCount", out->cudart_path, sizeof(out->cudart_path));
  cudaError_t first = cudaSuccess;
  auto note = [&](cudaError_t e) { if (first == cudaSuccess && e != cudaSuccess) first = e; };
  note(cudaDriverGetVersion(&out->driver_version));
  note(cudaRuntimeGetVersion(&out->runtime_version));
  note(cudaGetDeviceCount(&out->device_count));
  if (first == cudaSuccess && out->device_count > 0) {
    note(cudaGetDevice(&out->active_device));
    cudaDeviceProp prop{};
    if (first == cudaSuccess && cudaGetDeviceProperties(&prop, out->active_device) == cudaSuccess) {
      out->sm_major = prop.major;
      out->sm_minor = prop.minor;
      out->multiprocessor_count = prop.multiProcessorCount;
      out->total_global_mem = prop.totalGlobalMem;
      set_str(out->device_name, sizeof(out->device_name), prop.name);
    }
  }
  out->last_cuda_error = static_cast<int>(first);
  set_str(out->last_cuda_error_name, sizeof(out->last_cuda_error_name), cudaGetErrorName(first));
  set_str(out->last_cuda_error_string, sizeof(out->last_cuda_error_string), cudaGetErrorString(first));
  return first == cudaSuccess ? QWEN36_STATUS_SUCCESS : QWEN36_STATUS_CUDA_ERROR;
}

int qwen36_cuda_counters_reset(void) {
  for (auto &c : g_counters.v) c.store(0, std::memory_order_relaxed);
  return QWEN36_STATUS_SUCCESS;
}

int qwen36_cuda_counters_read(qwen36_cuda_counters_t *out) {
  if (out == nullptr) return QWEN36_STATUS_NULL_POINTER;
  uint64_t *dst = reinterpret_cast<uint64_t *>(out);   // 15 consecutive uint64_t fields
  for (int i = 0; i < 15; ++i) dst[i] = g_counters.v[i].load(std::memory_order_relaxed);
  return QWEN36_STATUS_SUCCESS;
}

int qwen36_cuda_set_l2_access_window(qwen36_device_ptr_t base, size_t bytes, float hit_ratio) {
  if (base.ptr == 0 || bytes == 0) return QWEN36_STATUS_INVALID_ARGUMENT;
  cudaStreamAttrValue attr{};
  attr.accessPolicyWindow.base_ptr = raw(base);
  attr.accessPolicyWindow.num_bytes = bytes;
  attr.accessPolicyWindow.hitRatio = hit_ratio;
  attr.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
  attr.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
  return cuda_status(cudaStreamSetAttribute(q36::stream(), cudaStreamAttributeAccessPolicyWindow, &attr));
}

int qwen36_cuda_clear_l2_access_window(void) {
  cudaStreamAttrValue attr{};
  attr.accessPolicyWindow.num_bytes = 0;
  const cudaError_t e = cudaStreamSetAttribute(q36::stream(), cudaStreamAttributeAccessPolicyWindow, &attr);
  if (e != cudaSuccess) return QWEN36_STATUS_CUDA_ERROR;
  return cuda_status(cudaCtxResetPersistingL2Cache());
}

int qwen36_l2_prefetch(qwen36_device_ptr_t base, size_t bytes, int target_cta_count) {
  cudaStream_t s = g_prefetch.load(std::memory_order_acquire);
  if (s == nullptr || base.ptr == 0 || bytes == 0 || (base.ptr & 15u) != 0) return QWEN36_STATUS_INVALID_ARGUMENT;
  if (bytes < 16) return QWEN36_STATUS_SUCCESS;      // fewer bytes than one 16-byte read: nothing to warm
  const int ctas = target_cta_count > 0 ? target_cta_count : 128;
  l2_warm_kernel<<<ctas, 256, 0, s>>>(static_cast<const uint4 *>(raw(base)), bytes / 16, nullptr);
  return q36::launch_status();
}

int qwen36_cuda_stream_create(qwen36_cuda_stream_t *out) {
  if (out == nullptr) return QWEN36_STATUS_NULL_POINTER;
  cudaStream_t s = nullptr;
  const cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  if (e != cudaSuccess) return QWEN36_STATUS_CUDA_ERROR;
  *out = reinterpret_cast<qwen36_cuda_stream_t>(s);
  return QWEN36_STATUS_SUCCESS;
}

int qwen36_cuda_stream_destroy(qwen36_cuda_stream_t s) {
  return s == nullptr ? QWEN36_STATUS_SUCCESS : cuda_status(cudaStreamDestroy(cs(s)));
}

int qwen36_cuda_stream_synchronize(qwen36_cuda_stream_t s) {
  bump(C_SSYNC);
  return cuda_status(cudaStreamSynchronize(cs(s)));
}

int qwen36_cuda_event_create(qwen36_cuda_event_t *out) {
  if (out == nullptr) return QWEN36_STATUS_NULL_POINTER;
  cudaEvent_t ev = nullptr;
  const cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
  if (e != cudaSuccess) return QWEN36_STATUS_CUDA_ERROR;
  *out = reinterpret_cast<qwen36_cuda_event_t>(ev);
  return QWEN36_STATUS_SUCCESS;
}

int qwen36_cuda_event_destroy(qwen36_cuda_event_t ev) {
  return ev == nullptr ? QWEN36_STATUS_SUCCESS : cuda_status(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(ev)));
}

int qwen36_cuda_event_record(qwen36_cuda_event_t ev, qwen36_cuda_stream_t s) {
  if (ev == nullptr) return QWEN36_STATUS_NULL_POINTER;
  return cuda_status(cudaEventRecord(reinterpret_cast<cudaEvent_t>(ev), cs(s)));
}

int qwen36_cuda_stream_wait_event(qwen36_cuda_stream_t s, qwen36_cuda_event_t ev) {
  if (ev == nullptr) return QWEN36_STATUS_NULL_POINTER;
  return cuda_status(cudaStreamWaitEvent(cs(s), reinterpret_cast<cudaEvent_t>(ev), 0));
}

int qwen36_cuda_stream_begin_capture(qwen36_cuda_stream_t s) {
  return cuda_status(cudaStreamBeginCapture(cs(s), cudaStreamCaptureModeThreadLocal));
}

int qwen36_cuda_stream_end_capture(qwen36_cuda_stream_t s, qwen36_cuda_graph_t *out) {
  if (out == nullptr) return QWEN36_STATUS_NULL_POINTER;
  cudaGraph_t g = nullptr;
  const cudaError_t e = cudaStreamEndCapture(cs(s), &g);
  if (e != cudaSuccess) return QWEN36_STATUS_CUDA_ERROR;
  *out = reinterpret_cast<qwen36_cuda_graph_t>(g);
  return QWEN36_STATUS_SUCCESS;
}

int qwen36_cuda_graph_instantiate(qwen36_cuda_graph_t g, qwen36_cuda_graph_exec_t *out) {
  if (g == nullptr || out == nullptr) return QWEN36_STATUS_NULL_POINTER;
  cudaGraphExec_t x = nullptr;
  const cudaError_t e = cudaGraphInstantiate(&x, reinterpret_cast<cudaGraph_t>(g), 0);
  if (e != cudaSuccess) return QWEN36_STATUS_CUDA_ERROR;
  *out = reinterpret_cast<qwen36_cuda_graph_exec_t>(x);
  return QWEN36_STATUS_SUCCESS;
}

int qwen36_cuda_graph_destroy(qwen36_cuda_graph_t g) {
  return g == nullptr ? QWEN36_STATUS_SUCCESS : cuda_status(cudaGraphDestroy(reinterpret_cast<cudaGraph_t>(g)));
}

int qwen36_cuda_graph_exec_destroy(qwen36_cuda_graph_exec_t x) {
  return x == nullptr ? QWEN36_STATUS_SUCCESS
                      : cuda_status(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(x)));
}

int qwen36_cuda_graph_launch(qwen36_cuda_graph_exec_t x, qwen36_cuda_stream_t s) {
  if (x == nullptr) return QWEN36_STATUS_NULL_POINTER;
  bump(C_GRAPH);
  return cuda_status(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(x), cs(s)));
}

int qwen36_increment_i32(qwen36_device_ptr_t target) {
  if (target.ptr == 0) return QWEN36_STATUS_INVALID_ARGUMENT;     // the reference's code for a null target
  increment_i32_kernel<<<1, 1, 0, q36::stream()>>>(static_cast<int32_t *>(raw(target)));
  return q36::launch_status();
}

int qwen36_mtp_assume_accept_chain_advance(qwen36_device_ptr_t position_i32, size_t draft_count,
                                           size_t position_count, int32_t position_delta) {
  // argument checks and codes of kernels-cuda/runtime.cu:257-266
  if (position_i32.ptr == 0) return QWEN36_STATUS_INVALID_ARGUMENT;
  if (draft_count == 0 || draft_count > 4 || position_count == 0 || position_delta <= 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const unsigned blocks = static_cast<unsigned>((position_count + 127) / 128);
  advance_positions_kernel<<<blocks, 128, 0, q36::stream()>>>(static_cast<int32_t *>(raw(position_i32)),
                                                              position_count, position_delta);
  return q36::launch_status();
}

}  // extern "C"
