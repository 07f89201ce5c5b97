// Fused producers of NVFP4 activations for the decode path:
//   qwen36_rmsnorm_nvfp4_quantize : (x [+ residual]) -> RMSNorm * (1 + w) -> bf16 copy + NVFP4 codes + scales
//   qwen36_swiglu_nvfp4_quantize  : silu(gate) * up  -> NVFP4 codes + scales
// (reference: kernels-cuda/interpreter/opcodes/rmsnorm_nvfp4_quant.cuh:113-281,
//  swiglu_nvfp4_quant.cuh:13-75, entry points kernels-cuda/ops.cu:1007-1031,1500-1521).
//
// Both are single-vector, latency-bound launches that sit between two GEMVs of every decode
// layer.  The arithmetic follows the reference expression by expression, because the codes they
// emit must be the reference's: the sum of squares is taken as 256 strided partial sums met by a
// halving tree, the normaliser is rsqrtf, silu divides by 1 + expf(-g), the group scale and the
// codes use the shared NVFP4 codec.  What changes is the shape of the launch: the reference walks
// whole 16-value groups with one thread each (two passes of 256 threads for hidden = 5120, sixteen
// serial IEEE divisions per thread); here the vector is fetched once, by 1024 threads in one round
// trip, into shared memory as float32, two lanes share a group in the norm kernel and sixteen lanes
// share one in the SwiGLU kernel, 256 threads per CTA instead of 32.
// Both launch with programmatic stream serialisation: the CTA takes its seat (and the norm kernel
// fetches its norm weights, which are model state) while the kernel ahead drains, and lets the
// kernel behind (a GEMV that streams its weights before it needs this output) take its seats at once.
#include "common.cuh"
#include "kv_split.cuh"
#include "nvfp4_quant_group.cuh"

namespace {

using q36::as_ptr;

constexpr uint32_t kNormSumThreads = 256;   // partial sums of the reference's reduction (ops.cu:1017)
constexpr uint32_t kNormThreads = 1024;

__device__ __forceinline__ float group_scale_value(float amax, float global_scale) {
  return amax > 0.0f ? fmaxf(amax / (6.0f * global_scale), 1.0e-8f) : 1.0f;
}

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_nvfp4_quantize_kernel(const __nv_bfloat16 *__restrict__ input, const __nv_bfloat16 *__restrict__ weight,
                              const __nv_bfloat16 *__restrict__ residual, __nv_bfloat16 *__restrict__ residual_out,
                              __nv_bfloat16 *__restrict__ output_bf16, uint8_t *__restrict__ output_fp4,
                              uint8_t *__restrict__ output_scale, float *__restrict__ tensor_scale, size_t hidden,
                              float eps, float input_tensor_scale) {
  __shared__ float scratch[kNormSumThreads];
  __shared__ float total;
  extern __shared__ __align__(16) float value[];            // input (+ residual) as float32, read three times below
  // The norm weights of this thread's eight values (first pass of the quantise loop below) travel
  // with the input instead of after the reductions.
  float w_first[8];
  {
    const size_t start = (static_cast<size_t>(threadIdx.x) >> 1) * 16 + (threadIdx.x & 1u) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) w_first[i] = start + i < hidden ? __bfloat162float(weight[start + i]) : 0.0f;
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");               // input and residual come from the kernel ahead
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // ---- one round trip to L2: every thread fetches its elements at once -------------------------
  constexpr int kBatch = 8;                                  // 8192 elements per pass: loads issued before any use
  for (size_t base = 0; base < hidden; base += static_cast<size_t>(kBatch) * kNormThreads) {
    __nv_bfloat16 in_raw[kBatch], res_raw[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const size_t d = base + threadIdx.x + static_cast<size_t>(i) * kNormThreads;
      in_raw[i] = d < hidden ? input[d] : __float2bfloat16(0.0f);
      res_raw[i] = (d < hidden && residual != nullptr) ? residual[d] : __float2bfloat16(0.0f);
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const size_t d = base + threadIdx.x + static_cast<size_t>(i) * kNormThreads;
      if (d < hidden) {
        float v = __bfloat162float(in_raw[i]);
        if (residual != nullptr) v += __bfloat162float(res_raw[i]);
        value[d] = v;
        if (residual_out != nullptr) residual_out[d] = __float2bfloat16(v);
      }
    }
  }
  __syncthreads();
  // ---- sum of squares: thread t < 256 adds pairs t, t + 256, ... in that order ----------------
  if (threadIdx.x < kNormSumThreads) {
    float local_sum = 0.0f;
    const size_t pairs = hidden / 2;
    for (size_t p = threadIdx.x; p < pairs; p += kNormSumThreads) {
      const float a = value[2 * p], b = value[2 * p + 1];
      local_sum += a * a + b * b;
    }
    if ((hidden & 1u) != 0u && threadIdx.x == 0u) {
      const float v = value[hidden - 1];
      local_sum += v * v;
    }
    scratch[threadIdx.x] = local_sum;
  }
  __syncthreads();
  // The reference's halving tree over the 256 partials (s[t] += s[t + stride], stride = 128 ... 1),
  // same pairings in the same order, evaluated by one warp without block barriers: strides 128, 64
  // and 32 from shared memory, 16 ... 1 as shuffles.
  if (threadIdx.x < 32) {
    const uint32_t t = threadIdx.x;
    const float lo = (scratch[t] + scratch[t + 128]) + (scratch[t + 64] + scratch[t + 192]);
    const float hi = (scratch[t + 32] + scratch[t + 160]) + (scratch[t + 96] + scratch[t + 224]);
    float s32 = lo + hi;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s32 += __shfl_down_sync(0xffffffffu, s32, off);
    if (t == 0) total = s32;
  }
  __syncthreads();
  const float norm_scale = rsqrtf(total / static_cast<float>(hidden) + eps);
  const size_t groups = q36::div_ceil(hidden, 16);
  const size_t sf_inner = q36::round_up(groups, 4);
  const float global_scale = input_tensor_scale > 0.0f ? input_tensor_scale : 1.0f;

  // ---- normalise, quantise: two adjacent lanes per 16-value group, eight values each ----------
  const size_t half_groups = groups * 2;
  for (size_t hg0 = 0; hg0 < half_groups; hg0 += kNormThreads) {     // uniform trip count: shuffles below
    const size_t hg = hg0 + threadIdx.x;
    const bool live = hg < half_groups;
    const size_t group = hg >> 1, start = group * 16 + (hg & 1u) * 8;
    float weighted[8];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const size_t d = start + i;
      weighted[i] = 0.0f;
      if (live && d < hidden) {
        const float w = value[d] * norm_scale * (1.0f + (hg0 == 0 ? w_first[i] : __bfloat162float(weight[d])));
        weighted[i] = w;
        if (output_bf16 != nullptr) output_bf16[d] = __float2bfloat16(w);
        amax = fmaxf(amax, fabsf(w));
      }
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const uint32_t scale_code = q36::encode_ue4m3(group_scale_value(amax, global_scale));
    const float decoded_scale = fmaxf(q36::decode_e4m3(scale_code) * global_scale, 1.0e-8f);
    if (live && (hg & 1u) == 0u) output_scale[q36::sf_offset(group, 0, sf_inner)] = static_cast<uint8_t>(scale_code);
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const size_t d = start + i;
      if (live && d < hidden) {
        // (two encode_e2m1 calls in one: hardware conversion + the reference's tie and -0 rules)
        const uint32_t packed = d + 1 < hidden
                                    ? q36::encode_e2m1x2(weighted[i] / decoded_scale, weighted[i + 1] / decoded_scale)
                                    : q36::encode_e2m1(weighted[i] / decoded_scale);
        output_fp4[d / 2] = static_cast<uint8_t>(packed);
      }
    }
  }
  if (threadIdx.x == 0 && tensor_scale != nullptr) *tensor_scale = global_scale;
}

constexpr uint32_t kSwigluThreads = 256;

// One lane per value, sixteen lanes per group.
__global__ void __launch_bounds__(kSwigluThreads)
swiglu_nvfp4_quantize_kernel(const __nv_bfloat16 *__restrict__ gate, const __nv_bfloat16 *__restrict__ up,
                             uint8_t *__restrict__ output_fp4, uint8_t *__restrict__ output_scale,
                             float *__restrict__ tensor_scale, size_t values, float input_tensor_scale) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const float global_scale = input_tensor_scale > 0.0f ? input_tensor_scale : 1.0f;
  const size_t idx = static_cast<size_t>(blockIdx.x) * kSwigluThreads + threadIdx.x;
  const size_t group = idx >> 4;
  const size_t sf_inner = q36::round_up(q36::div_ceil(values, 16), 4);
  float y = 0.0f;
  if (idx < values) {
    const float g = __bfloat162float(gate[idx]);
    const float u = __bfloat162float(up[idx]);
    const float silu = g / (1.0f + expf(-g));
    y = silu * u;
  }
  float amax = fabsf(y);
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const uint32_t scale_code = q36::encode_ue4m3(group_scale_value(amax, global_scale));
  const float decoded_scale = fmaxf(q36::decode_e4m3(scale_code) * global_scale, 1.0e-8f);
  const uint32_t code = q36::encode_e2m1(y / decoded_scale);
  const uint32_t other = __shfl_down_sync(0xffffffffu, code, 1);
  if (idx < values) {
    if ((idx & 15u) == 0u) output_scale[q36::sf_offset(group, 0, sf_inner)] = static_cast<uint8_t>(scale_code);
    if ((idx & 1u) == 0u)
      output_fp4[idx / 2] = static_cast<uint8_t>(code | (idx + 1 < values ? other << 4 : 0u));
  }
  if (idx == 0 && tensor_scale != nullptr) *tensor_scale = global_scale;
}

// silu(gate) * up for a whole [rows, values] activation block -> NVFP4 codes + tiled scales, the
// prefill form of the producer above: the bf16 [rows, values] intermediate of the unfused chain
// (SwiGLU kernel, then qwen36_nvfp4_quantize_rows) is never written or read back.  Row r of the
// output is what swiglu_nvfp4_quantize_kernel gives for row r alone (same expressions in float32,
// no bf16 round trip), its scale bytes at the tiled position of (group, r).  Launch shape of the row
// quantiser: blockDim (64, 4), a thread owns one 16-group of a row, rows advance by the grid with
// the next row's 64 bytes already in flight.
__global__ void __launch_bounds__(256)
swiglu_nvfp4_quantize_rows_kernel(const __nv_bfloat16 *__restrict__ gate, const __nv_bfloat16 *__restrict__ up,
                                  uint8_t *__restrict__ out_fp4, uint8_t *__restrict__ out_sf,
                                  float *__restrict__ tensor_scale, uint32_t rows, uint32_t values, size_t stride,
                                  float input_tensor_scale) {
  const float g = input_tensor_scale > 0.0f ? input_tensor_scale : 1.0f;
  const float six_g = __fmul_rn(6.0f, g), rcp6 = __frcp_rn(six_g);
  const uint32_t groups = values >> 4, padded = (groups + 3u) & ~3u;
  const uint32_t group = blockIdx.x * 64u + threadIdx.x;
  const bool in_row = group < groups;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && threadIdx.y == 0 && tensor_scale != nullptr) *tensor_scale = g;

  const uint32_t row_step = gridDim.y * 4u;
  uint32_t row = blockIdx.y * 4u + threadIdx.y;
  uint4 ng0 = make_uint4(0u, 0u, 0u, 0u), ng1 = ng0, nu0 = ng0, nu1 = ng0;
  if (in_row && row < rows) {
    const size_t at = static_cast<size_t>(row) * stride + group * 16u;
    ng0 = __ldcs(reinterpret_cast<const uint4 *>(gate + at));
    ng1 = __ldcs(reinterpret_cast<const uint4 *>(gate + at) + 1);
    nu0 = __ldcs(reinterpret_cast<const uint4 *>(up + at));
    nu1 = __ldcs(reinterpret_cast<const uint4 *>(up + at) + 1);
  }
  for (; row < rows; row += row_step) {
    uint32_t sf_code = 0;
    const uint32_t gw[8] = {ng0.x, ng0.y, ng0.z, ng0.w, ng1.x, ng1.y, ng1.z, ng1.w};
    const uint32_t uw[8] = {nu0.x, nu0.y, nu0.z, nu0.w, nu1.x, nu1.y, nu1.z, nu1.w};
    if (in_row && row + row_step < rows) {
      const size_t at = static_cast<size_t>(row + row_step) * stride + group * 16u;
      ng0 = __ldcs(reinterpret_cast<const uint4 *>(gate + at));
      ng1 = __ldcs(reinterpret_cast<const uint4 *>(gate + at) + 1);
      nu0 = __ldcs(reinterpret_cast<const uint4 *>(up + at));
      nu1 = __ldcs(reinterpret_cast<const uint4 *>(up + at) + 1);
    }
    if (in_row) {
      float y[16];
      float amax = 0.0f;
      uint32_t any = 0u, smallest = 0xffffffffu;                  // smallest nonzero magnitude, as bits - 1
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float gv = __uint_as_float((i & 1) ? (gw[i >> 1] & 0xffff0000u) : (gw[i >> 1] << 16));
        const float uv = __uint_as_float((i & 1) ? (uw[i >> 1] & 0xffff0000u) : (uw[i >> 1] << 16));
        const float silu = gv / (1.0f + expf(-gv));
        y[i] = silu * uv;
        amax = fmaxf(amax, fabsf(y[i]));
        const uint32_t mag = __float_as_uint(y[i]) & 0x7fffffffu;
        any |= mag;
        smallest = min(smallest, mag - 1u);
      }
      uint32_t lo, hi;
      q36::nvfp4_quantize_group(y, amax, any != 0u, smallest < 0x0f800000u, g, six_g, rcp6, lo, hi, sf_code);
      *reinterpret_cast<uint2 *>(out_fp4 + (static_cast<size_t>(row) * (values >> 1) + group * 8u)) = make_uint2(lo, hi);
    }
    // the four scale bytes of a quad of groups form one word of the tiled layout (see q36::sf_offset)
    const uint32_t lane4 = threadIdx.x & 3u;
    uint32_t word = sf_code << (8u * lane4);
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if (in_row) {
      const size_t off = (static_cast<size_t>(group >> 2) + static_cast<size_t>(row >> 7) * (padded >> 2)) * 512u +
                         (row & 31u) * 16u + ((row >> 5) & 3u) * 4u + lane4;
      if ((group | 3u) < groups) {
        if (lane4 == 0u) *reinterpret_cast<uint32_t *>(out_sf + off) = word;
      } else {
        out_sf[off] = static_cast<uint8_t>(sf_code);
      }
    }
  }
}

}  // namespace

extern "C" int qwen36_swiglu_nvfp4_quantize_rows(const qwen36_swiglu_nvfp4_quantize_rows_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->rows == 0 || spec->intermediate == 0 || spec->gate_bf16.ptr == 0 || spec->up_bf16.ptr == 0 ||
      spec->output_fp4.ptr == 0 || spec->output_scale_e4m3.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  // whole groups, 16-byte loads, 8-byte code stores, 4-byte scale words
  if (spec->intermediate % 16 != 0 || spec->input_row_stride < spec->intermediate || spec->input_row_stride % 8 != 0 ||
      (spec->gate_bf16.ptr & 15u) != 0 || (spec->up_bf16.ptr & 15u) != 0 || (spec->output_fp4.ptr & 7u) != 0 ||
      (spec->output_scale_e4m3.ptr & 3u) != 0 || spec->rows >= (1ull << 31) || spec->intermediate >= (1ull << 31))
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const size_t padded = q36::round_up(spec->intermediate / 16, 4);
  const size_t gx = q36::div_ceil(padded, 64), row_chunks = q36::div_ceil(spec->rows, 4);
  const size_t want = q36::div_ceil(static_cast<size_t>(q36::sm_count_current_device()) * 24, gx);
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(row_chunks < want ? row_chunks : want));
  swiglu_nvfp4_quantize_rows_kernel<<<grid, dim3(64, 4), 0, q36::stream()>>>(
      as_ptr<const __nv_bfloat16>(spec->gate_bf16), as_ptr<const __nv_bfloat16>(spec->up_bf16),
      as_ptr<uint8_t>(spec->output_fp4), as_ptr<uint8_t>(spec->output_scale_e4m3),
      as_ptr<float>(spec->output_tensor_scale_f32), static_cast<uint32_t>(spec->rows),
      static_cast<uint32_t>(spec->intermediate), spec->input_row_stride, spec->input_tensor_scale_f32);
  return q36::launch_status();
}

extern "C" int qwen36_rmsnorm_nvfp4_quantize(const qwen36_rmsnorm_nvfp4_quantize_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->hidden == 0 || spec->input_bf16.ptr == 0 || spec->weight_bf16.ptr == 0 || spec->output_fp4.ptr == 0 ||
      spec->output_scale_e4m3.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const float eps = spec->eps == 0.0f ? 1.0e-6f : spec->eps;
  const size_t smem = spec->hidden * sizeof(float);
  if (smem > 200 * 1024) return QWEN36_STATUS_INVALID_ARGUMENT;
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(rmsnorm_nvfp4_quantize_kernel), 200 * 1024) != cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  return q36::cuda_status(q36::launch_after_previous(
      rmsnorm_nvfp4_quantize_kernel, dim3(1), dim3(kNormThreads), smem, q36::stream(),
      as_ptr<const __nv_bfloat16>(spec->input_bf16), as_ptr<const __nv_bfloat16>(spec->weight_bf16),
      as_ptr<const __nv_bfloat16>(spec->residual_bf16), as_ptr<__nv_bfloat16>(spec->residual_out_bf16),
      as_ptr<__nv_bfloat16>(spec->output_bf16), as_ptr<uint8_t>(spec->output_fp4),
      as_ptr<uint8_t>(spec->output_scale_e4m3), as_ptr<float>(spec->output_tensor_scale_f32), spec->hidden, eps,
      spec->input_tensor_scale_f32));
}

extern "C" int qwen36_swiglu_nvfp4_quantize(const qwen36_swiglu_nvfp4_quantize_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->intermediate == 0 || spec->gate_bf16.ptr == 0 || spec->up_bf16.ptr == 0 || spec->output_fp4.ptr == 0 ||
      spec->output_scale_e4m3.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const size_t padded = q36::round_up(spec->intermediate, 16);
  const unsigned blocks = static_cast<unsigned>(q36::div_ceil(padded, kSwigluThreads));
  return q36::cuda_status(q36::launch_after_previous(
      swiglu_nvfp4_quantize_kernel, dim3(blocks), dim3(kSwigluThreads), size_t{0}, q36::stream(),
      as_ptr<const __nv_bfloat16>(spec->gate_bf16), as_ptr<const __nv_bfloat16>(spec->up_bf16),
      as_ptr<uint8_t>(spec->output_fp4), as_ptr<uint8_t>(spec->output_scale_e4m3),
      as_ptr<float>(spec->output_tensor_scale_f32), spec->intermediate, spec->input_tensor_scale_f32));
}
