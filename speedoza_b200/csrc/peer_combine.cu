// Multi-GPU combine steps over NVLink peer memory (no counterpart in the single-GPU reference).
//
// The sharded lm_head and the sharded int8 KV attention end in a tiny exchange: every rank has one
// (value, index) pair per token, or one (m, l, o) partial per q head, and every rank needs the
// combination of all of them.  Through a collective library that costs 20-30 us of latency for a
// few KB.  Here every rank owns an inbox that the other ranks of the node have mapped (CUDA IPC).
// One kernel per rank PUSHES its piece into every peer's inbox with plain peer stores, raises a
// flag there, waits on its own (local) flags and combines the pieces out of its own memory: one
// NVLink crossing, no round trip, a few microseconds.
//
//   * plain st over NVLink only: no multicast objects, no TMA, no remote polling;
//   * every wait is bounded (a few seconds at most), after which the kernel poisons its output (NaN
//     rows, token 0xFFFFFFFF), writes the number of the failed call into state[2] and sets a sticky
//     process-wide error word, so the failure shows in the data a caller reads anyway;
//   * the call number lives in device memory and is advanced by the kernel itself, so a CUDA graph
//     that holds the launch can be replayed;
//   * two inbox slots alternate by call number: a rank can be at most one call ahead of a peer (it
//     needs that peer's flag of the current call to finish), so the slot it overwrites there was
//     consumed one call earlier.
#include "common.cuh"

#include <math.h>

#include "lse_merge.cuh"
#include "peer_combine.cuh"

namespace {

using q36::as_ptr;

constexpr uint32_t kMaxWorld = 16;
constexpr uint32_t kSpinLimit = 1u << 21;          // x (200 ns back-off + one local load): 1-2 s
constexpr uint32_t kEagerPolls = 1024;             // polls without back-off: the common case ends here

__device__ unsigned int g_peer_error = 0;

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_u32(uint32_t *p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_peer_v4(float *p, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ uint32_t ld_inbox_u32(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// state[0] = number of completed calls, state[1] = CTAs of the running call that are done,
// state[2] = number of the first call whose wait ran out (0 = none), state[3] unused.
__device__ __forceinline__ uint32_t begin_call(const uint32_t *state) {
  return *reinterpret_cast<const volatile uint32_t *>(state) + 1u;
}
__device__ __forceinline__ void end_call(uint32_t *state, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(&state[1], 1u) == gridDim.x - 1) {   // every CTA has read state[0] by now
    state[1] = 0;
    *reinterpret_cast<volatile uint32_t *>(state) = epoch;
  }
}

// After this CTA's pushes: thread p raises flag `slot_of_cta` of this rank in peer p's flag array,
// then waits for peer p's flag in the local array.  flags layout: [world][flags_per_rank].
__device__ bool signal_and_wait(uint32_t *const *peer_flags, uint32_t *state, uint32_t world, uint32_t rank,
                                uint32_t epoch, uint32_t flags_per_rank, uint32_t flag) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();                                             // all pushes of the CTA are issued
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(peer_flags[threadIdx.x] + static_cast<size_t>(rank) * flags_per_rank + flag, epoch);
    const uint32_t *mine = peer_flags[rank] + static_cast<size_t>(threadIdx.x) * flags_per_rank + flag;
    uint32_t spin = 0;
    // call numbers only grow; a peer that is already one call ahead has also finished this one
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (++spin > kSpinLimit) {
        ok = 0;
        atomicExch(&g_peer_error, 1u);
        atomicCAS(&state[2], 0u, epoch);
        break;
      }
      if (spin > kEagerPolls) __nanosleep(200);
    }
  }
  __syncthreads();
  return ok != 0;
}

// One CTA of 256 threads per q head.  Inbox: [2 slots][world][q_heads][row] floats, a row =
// o[head_dim], m, l, padded to a multiple of four floats so that rows start on 16-byte boundaries
// and go out as 16-byte peer stores.  The local input is n_parts split partials per head ([heads, n_parts(, head_dim)],
// n_parts = 1: one finished partial per head); they are merged first, with the arithmetic of the
// single-GPU merge kernel, and the result goes straight into the peers' inboxes.
__global__ void __launch_bounds__(q36::kMergeThreads)
attention_peer_merge_kernel(const float *__restrict__ part_o, const float *__restrict__ part_m,
                            const float *__restrict__ part_l, uint32_t n_parts, float *const *peer_inbox,
                            uint32_t *const *peer_flags, uint32_t *state, __nv_bfloat16 *__restrict__ out,
                            uint32_t world, uint32_t rank, uint32_t heads, uint32_t head_dim) {
  asm volatile("griddepcontrol.wait;" ::: "memory");          // the partials come from the kernel before
  __shared__ float s_parts[q36::kMergeThreads];
  __shared__ float s_red[q36::kMergeThreads / 32];
  const uint32_t h = blockIdx.x;
  const uint32_t epoch = begin_call(state);
  const uint32_t row = (head_dim + 2u + 3u) & ~3u;
  const size_t slot = static_cast<size_t>(epoch & 1u) * world * heads * row;
  float local_m, local_l;
  q36::lse_weights(part_m + static_cast<size_t>(h) * n_parts, part_l + static_cast<size_t>(h) * n_parts, n_parts,
                   s_parts, s_red, local_m, local_l);
  const float *my_o = part_o + static_cast<size_t>(h) * n_parts * head_dim;
  auto value_at = [&](uint32_t d) {
    return d < head_dim ? q36::lse_accumulate(my_o, s_parts, n_parts, head_dim, d)
                        : (d == head_dim ? local_m : (d == head_dim + 1u ? local_l : 0.f));
  };
  for (uint32_t d = threadIdx.x * 4u; d < row; d += blockDim.x * 4u) {
    const float4 v = make_float4(value_at(d), value_at(d + 1u), value_at(d + 2u), value_at(d + 3u));
    const size_t at = slot + (static_cast<size_t>(rank) * heads + h) * row + d;
    for (uint32_t p = 0; p < world; ++p) st_peer_v4(peer_inbox[p] + at, v);
  }
  if (signal_and_wait(peer_flags, state, world, rank, epoch, heads, h)) {
    const uint32_t *inbox = reinterpret_cast<const uint32_t *>(peer_inbox[rank] + slot);
    __shared__ float s_w[kMaxWorld];
    __shared__ float s_den;
    if (threadIdx.x < 32) {
      // the arithmetic of the single-GPU merge (kv_merge_kernel: one part per lane, butterfly
      // reductions), so that both routes give the same bits
      const uint32_t p = threadIdx.x;
      const size_t at = (static_cast<size_t>(p) * heads + h) * row + head_dim;
      const float my_m = p < world ? __uint_as_float(ld_inbox_u32(inbox + at)) : -INFINITY;
      const float my_l = p < world ? __uint_as_float(ld_inbox_u32(inbox + at + 1)) : 0.f;
      float M = my_m;
      for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
      const float w = my_m == -INFINITY ? 0.f : __expf(my_m - M);
      if (p < kMaxWorld) s_w[p] = w;
      float den = w * my_l;
      for (int off = 16; off > 0; off >>= 1) den += __shfl_xor_sync(0xffffffffu, den, off);
      if (p == 0) s_den = den;
    }
    __syncthreads();
    for (uint32_t d = threadIdx.x; d < head_dim; d += blockDim.x) {
      float v[kMaxWorld], acc = 0.f;
#pragma unroll
      for (uint32_t p = 0; p < kMaxWorld; ++p)                  // all loads first, then the sum in rank order
        v[p] = p < world ? __uint_as_float(ld_inbox_u32(inbox + (static_cast<size_t>(p) * heads + h) * row + d)) : 0.f;
#pragma unroll
      for (uint32_t p = 0; p < kMaxWorld; ++p)
        if (p < world) acc = fmaf(s_w[p], v[p], acc);
      out[static_cast<size_t>(h) * head_dim + d] = __float2bfloat16(s_den > 0.f ? __fdiv_rn(acc, s_den) : 0.f);
    }
  } else {
    for (uint32_t d = threadIdx.x; d < head_dim; d += blockDim.x)   // a peer never answered: no silent stale row
      out[static_cast<size_t>(h) * head_dim + d] = __ushort_as_bfloat16(0x7FC0);
  }
  end_call(state, epoch);
}

// One CTA.  Inbox: [2 slots][world][2][tokens] words, value f32 then index u32.  Greedy rule of the
// reference (strictly greater wins, equal values keep the lower index, NaN never wins, the scan
// starts from (-inf, 0)).
__global__ void __launch_bounds__(64)
argmax_peer_combine_kernel(const float *__restrict__ value, const uint32_t *__restrict__ index,
                           uint32_t *const *peer_inbox, uint32_t *const *peer_flags, uint32_t *state,
                           uint32_t *__restrict__ tokens, uint32_t world, uint32_t rank, uint32_t n_tokens) {
  const uint32_t epoch = begin_call(state);
  const size_t slot = static_cast<size_t>(epoch & 1u) * world * 2u * n_tokens;
  for (uint32_t t = threadIdx.x; t < n_tokens; t += blockDim.x) {
    const uint32_t v = __float_as_uint(value[t]), i = index[t];
    const size_t at = slot + static_cast<size_t>(rank) * 2u * n_tokens + t;
    for (uint32_t p = 0; p < world; ++p) {
      st_peer_u32(peer_inbox[p] + at, v);
      st_peer_u32(peer_inbox[p] + at + n_tokens, i);
    }
  }
  if (signal_and_wait(peer_flags, state, world, rank, epoch, 1, 0)) {
    const uint32_t *inbox = peer_inbox[rank] + slot;
    for (uint32_t t = threadIdx.x; t < n_tokens; t += blockDim.x) {
      float best = -INFINITY;
      uint32_t best_i = 0;
      uint32_t vs[kMaxWorld], is[kMaxWorld];
#pragma unroll
      for (uint32_t p = 0; p < kMaxWorld; ++p) {                // all loads first
        vs[p] = p < world ? ld_inbox_u32(inbox + static_cast<size_t>(p) * 2u * n_tokens + t) : 0xff800000u;
        is[p] = p < world ? ld_inbox_u32(inbox + static_cast<size_t>(p) * 2u * n_tokens + n_tokens + t) : 0u;
      }
#pragma unroll
      for (uint32_t p = 0; p < kMaxWorld; ++p) {
        const float v = __uint_as_float(vs[p]);
        if (p < world && (v > best || (v == best && is[p] < best_i))) {
          best = v;
          best_i = is[p];
        }
      }
      tokens[t] = best_i;
    }
  } else {
    for (uint32_t t = threadIdx.x; t < n_tokens; t += blockDim.x) tokens[t] = 0xFFFFFFFFu;   // no token has this id
  }
  end_call(state, epoch);
}

}  // namespace

// ---- CUDA IPC plumbing: lets the ranks of one node map each other's inboxes --------------------

extern "C" int qwen36_ipc_get_handle(qwen36_device_ptr_t ptr, void *handle_out_64_bytes) {
  if (ptr.ptr == 0 || handle_out_64_bytes == nullptr) return QWEN36_STATUS_NULL_POINTER;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, as_ptr<void>(ptr)) != cudaSuccess) return QWEN36_STATUS_CUDA_ERROR;
  memcpy(handle_out_64_bytes, &h, sizeof(h));
  return QWEN36_STATUS_SUCCESS;
}

extern "C" int qwen36_ipc_open_handle(const void *handle_64_bytes, qwen36_device_ptr_t *out) {
  if (handle_64_bytes == nullptr || out == nullptr) return QWEN36_STATUS_NULL_POINTER;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64_bytes, sizeof(h));
  void *p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return QWEN36_STATUS_CUDA_ERROR;
  out->ptr = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(p));
  return QWEN36_STATUS_SUCCESS;
}

extern "C" int qwen36_ipc_close_handle(qwen36_device_ptr_t ptr) {
  if (ptr.ptr == 0) return QWEN36_STATUS_NULL_POINTER;
  return q36::cuda_status(cudaIpcCloseMemHandle(as_ptr<void>(ptr)));
}

extern "C" size_t qwen36_attention_peer_inbox_bytes(size_t world, size_t q_heads, size_t head_dim) {
  return 2 * world * q_heads * ((head_dim + 2 + 3) / 4 * 4) * sizeof(float);
}

extern "C" size_t qwen36_argmax_peer_inbox_bytes(size_t world, size_t tokens) {
  return 2 * world * 2 * tokens * sizeof(uint32_t);
}

int q36::launch_attention_peer_merge(const float *part_o, const float *part_m, const float *part_l, uint32_t n_parts,
                                     qwen36_device_ptr_t peer_inbox, qwen36_device_ptr_t peer_flags,
                                     qwen36_device_ptr_t state, qwen36_device_ptr_t output_bf16, size_t world,
                                     size_t rank, size_t q_heads, size_t head_dim) {
  if (world == 0 || world > kMaxWorld || rank >= world || q_heads == 0 || head_dim == 0 || n_parts == 0 ||
      n_parts > static_cast<uint32_t>(q36::kMergeThreads) || part_o == nullptr || part_m == nullptr ||
      part_l == nullptr || peer_inbox.ptr == 0 || peer_flags.ptr == 0 || state.ptr == 0 || output_bf16.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  // programmatic stream serialisation: the CTAs take their seats while the kernel that writes the
  // partials is still running and wait for it on the device
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(q_heads));
  cfg.blockDim = dim3(q36::kMergeThreads);
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return q36::cuda_status(cudaLaunchKernelEx(
      &cfg, attention_peer_merge_kernel, part_o, part_m, part_l, n_parts, as_ptr<float *const>(peer_inbox),
      as_ptr<uint32_t *const>(peer_flags), as_ptr<uint32_t>(state), as_ptr<__nv_bfloat16>(output_bf16),
      static_cast<uint32_t>(world), static_cast<uint32_t>(rank), static_cast<uint32_t>(q_heads),
      static_cast<uint32_t>(head_dim)));
}

extern "C" int qwen36_attention_peer_merge(const qwen36_attention_peer_merge_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  return q36::launch_attention_peer_merge(as_ptr<const float>(spec->partial_acc_f32),
                                          as_ptr<const float>(spec->partial_max_f32),
                                          as_ptr<const float>(spec->partial_denom_f32), 1, spec->peer_inbox,
                                          spec->peer_flags, spec->state, spec->output_bf16, spec->world, spec->rank,
                                          spec->q_heads, spec->head_dim);
}

extern "C" int qwen36_argmax_peer_combine(const qwen36_argmax_peer_combine_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->world == 0 || spec->world > kMaxWorld || spec->rank >= spec->world || spec->tokens == 0 ||
      spec->best_value_f32.ptr == 0 || spec->best_index_u32.ptr == 0 || spec->peer_inbox.ptr == 0 ||
      spec->peer_flags.ptr == 0 || spec->state.ptr == 0 || spec->output_token_u32.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  argmax_peer_combine_kernel<<<1, 64, 0, q36::stream()>>>(
      as_ptr<const float>(spec->best_value_f32), as_ptr<const uint32_t>(spec->best_index_u32),
      as_ptr<uint32_t *const>(spec->peer_inbox), as_ptr<uint32_t *const>(spec->peer_flags),
      as_ptr<uint32_t>(spec->state), as_ptr<uint32_t>(spec->output_token_u32), static_cast<uint32_t>(spec->world),
      static_cast<uint32_t>(spec->rank), static_cast<uint32_t>(spec->tokens));
  return q36::launch_status();
}

// 1 when a peer never raised its flag within the wait limit (that call poisoned its output and wrote
// its number into state[2]).  Sticky until qwen36_peer_reset_error.
extern "C" int qwen36_peer_last_error(void) {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_peer_error, sizeof(v)) != cudaSuccess) return -1;
  return static_cast<int>(v);
}

extern "C" int qwen36_peer_reset_error(void) {
  const unsigned int v = 0;
  return q36::cuda_status(cudaMemcpyToSymbol(g_peer_error, &v, sizeof(v)));
}
