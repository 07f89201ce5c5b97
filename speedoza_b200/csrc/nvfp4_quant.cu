// NVFP4 activation quantisation, block-scale retiling and weight
// dequantisation.  All three are HBM-bound byte shuffles: one thread owns one
// 16-value group, four neighbouring lanes own the four groups of one scale
// word, loads and stores are 16/8/4-byte vectors.
//
// Rounding follows the reference bit for bit (kernels-cuda/ops.cu:81-139,
// 704-761): IEEE float32 division by the decoded scale, E2M1 ties toward zero,
// UE4M3 ties down.
#include "common.cuh"
#include "kv_split.cuh"
#include "nvfp4_quant_group.cuh"

#include <atomic>

namespace {

using q36::as_ptr;

constexpr int kThreads = 256;

// One thread per 16-group.  `quads` = ceil(groups / 4): the group index space
// of a row is padded to a multiple of four so that the lanes 4q..4q+3 always
// belong to one row and one 4-byte scale word.
// Index: uint32_t when rows * padded groups and every byte offset fit 32 bits (index arithmetic is a
// visible share of this kernel's instructions), size_t otherwise.
template <typename Index>
__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_kernel(const __nv_bfloat16 *__restrict__ in, uint8_t *__restrict__ out_fp4,
                      uint8_t *__restrict__ out_sf, float *__restrict__ tensor_scale, Index rows,
                      Index values, float input_tensor_scale) {
  asm volatile("griddepcontrol.wait;" ::: "memory");               // launched with programmatic stream serialisation
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const float g = input_tensor_scale > 0.0f ? input_tensor_scale : 1.0f;
  const Index groups = (values + 15) / 16;
  const Index padded = (groups + 3) / 4 * 4;
  const Index idx = static_cast<Index>(blockIdx.x) * kThreads + threadIdx.x;
  const Index row = idx / padded;
  const Index group = idx - row * padded;
  const bool valid = row < rows && group < groups;

  if (idx == 0 && tensor_scale != nullptr) *tensor_scale = g;

  uint32_t sf_code = 0;
  if (valid) {
    const Index start = group * 16;
    const __nv_bfloat16 *src = in + (row * values + start);
    const bool full = start + 16 <= values;
    float x[16];
    if (full && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
      const uint4 lo = __ldg(reinterpret_cast<const uint4 *>(src));
      const uint4 hi = __ldg(reinterpret_cast<const uint4 *>(src) + 1);
      const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x[2 * i] = __uint_as_float(w[i] << 16);
        x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        x[i] = start + i < values ? __bfloat162float(src[i]) : 0.0f;
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));

    const float sv = amax > 0.0f ? fmaxf(__fdiv_rn(amax, __fmul_rn(6.0f, g)), 1.0e-8f) : 1.0f;
    sf_code = q36::encode_ue4m3(sv);
    const float ds = fmaxf(__fmul_rn(q36::decode_e4m3(sf_code), g), 1.0e-8f);

    // Codes.  The reference divides by ds in IEEE float32 and compares against fixed thresholds.
    // Fast path: multiply by the correctly rounded reciprocal (quotient within 2 ulps of the IEEE
    // one) and let the hardware conversion round to E2M1; that gives the reference's code unless
    // the quotient lies within a few ulps of a rounding boundary (all seven boundaries have zero
    // low 21 mantissa bits, so one masked compare finds them, plus infinities and NaN) or is a
    // negative value so small that the IEEE quotient may underflow to -0 (which the reference
    // encodes as +0).  Those rare groups are redone with the IEEE division.  (+0 quotients also
    // match the masked compare, so a group that mixes zeros with other values takes the exact
    // route too; an all-zero group is answered directly.)
    uint32_t lo = 0, hi = 0;
    const float rcp = __frcp_rn(ds);
    uint32_t near_boundary = 0xffffffffu, tiny_negative = 0xffffffffu;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float q0 = __fmul_rn(x[2 * i], rcp), q1 = __fmul_rn(x[2 * i + 1], rcp);
      uint32_t byte;
      asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}"
          : "=r"(byte) : "f"(q1), "f"(q0));
      if (i < 4) lo |= byte << (8 * i); else hi |= byte << (8 * (i - 4));
      const uint32_t b0 = __float_as_uint(q0), b1 = __float_as_uint(q1);
      near_boundary = min(near_boundary, min((b0 + 4u) & 0x001ffff8u, (b1 + 4u) & 0x001ffff8u));
      tiny_negative = min(tiny_negative, min(b0 - 0x80000000u, b1 - 0x80000000u));
    }
    uint32_t any_bits = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) any_bits |= __float_as_uint(x[i]);
    if ((any_bits & 0x7fffffffu) == 0u) {
      lo = hi = 0;                                   // every value is +0 or -0 (padding): every code is +0
    } else if (near_boundary == 0u || tiny_negative < 0x0d800000u) {      // exact route
      lo = hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        lo |= q36::encode_e2m1x2(__fdiv_rn(x[2 * i], ds), __fdiv_rn(x[2 * i + 1], ds)) << (8 * i);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        hi |= q36::encode_e2m1x2(__fdiv_rn(x[8 + 2 * i], ds), __fdiv_rn(x[9 + 2 * i], ds)) << (8 * i);
    }

    uint8_t *dst = out_fp4 + (row * ((values + 1) / 2) + start / 2);
    if (full && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
      *reinterpret_cast<uint2 *>(dst) = make_uint2(lo, hi);
    } else {
      const uint64_t both = (static_cast<uint64_t>(hi) << 32) | lo;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (start + 2 * i < values) dst[i] = static_cast<uint8_t>(both >> (8 * i));
    }
  }

  // Gather the four scale bytes of the quad into one word.
  const unsigned lane4 = threadIdx.x & 3u;
  uint32_t word = sf_code << (8 * lane4);
  word |= __shfl_xor_sync(0xffffffffu, word, 1);
  word |= __shfl_xor_sync(0xffffffffu, word, 2);
  if (valid) {
    // tiled scale layout (see q36::sf_offset), in Index arithmetic
    const Index r128 = row % 128;
    const Index off = ((group / 4) + (row / 128) * (padded / 4)) * 512 + (r128 % 32) * 16 + (r128 / 32) * 4 + (group % 4);
    if ((group | 3) < groups) {          // the whole quad is real: one 4-byte store
      if (lane4 == 0) *reinterpret_cast<uint32_t *>(out_sf + off) = word;
    } else {
      out_sf[off] = static_cast<uint8_t>(sf_code);
    }
  }
}

// The same quantisation for the common layout (values % 16 == 0, aligned rows), built to be bound
// by HBM rather than by instruction issue: 64 x 4 threads, a thread owns one 16-group of one row
// (no division to find its row), rows advance by the grid; the group's scale arithmetic takes the
// branch-free route when the scale is a normal UE4M3 number:
//   * amax / (6 g) by reciprocal + two FMAs (the quotient is recomputed with the IEEE division when it
//     lies within two ulps of a UE4M3 rounding boundary, so the scale byte is always the reference's);
//   * UE4M3 encode = (bits + 0x7FFFF) >> 20 rebased (the +0x7FFFF carries into the exponent exactly as
//     the reference's mantissa overflow does), clamp at 0x7E; decode = code << 20 rebased;
//   * codes by multiplication with the correctly rounded reciprocal + the hardware e2m1x2 conversion;
//     the rare pairs on which that can differ from the reference's division + threshold chain are
//     found by one masked compare and patched in place (see the loop).
// Groups whose scale is subnormal, saturated or very large are done with the reference's own
// arithmetic (IEEE divisions, threshold chain).
__global__ void __launch_bounds__(256)
nvfp4_quantize_fast_kernel(const __nv_bfloat16 *__restrict__ in, uint8_t *__restrict__ out_fp4,
                           uint8_t *__restrict__ out_sf, float *__restrict__ tensor_scale, uint32_t rows,
                           uint32_t values, float input_tensor_scale) {
  const float g = input_tensor_scale > 0.0f ? input_tensor_scale : 1.0f;
  const float six_g = __fmul_rn(6.0f, g), rcp6 = __frcp_rn(six_g);
  const uint32_t groups = values >> 4, padded = (groups + 3u) & ~3u;
  const uint32_t group = blockIdx.x * 64u + threadIdx.x;
  const bool in_row = group < groups;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && threadIdx.y == 0 && tensor_scale != nullptr) *tensor_scale = g;

  // A thread walks several rows; the two 16-byte loads of the next row are issued before the current
  // row is worked on, so the arithmetic of one group hides the memory latency of the next.
  const uint32_t row_step = gridDim.y * 4u;
  uint32_t row = blockIdx.y * 4u + threadIdx.y;
  uint4 n0 = make_uint4(0u, 0u, 0u, 0u), n1 = n0;
  if (in_row && row < rows) {
    const uint4 *src = reinterpret_cast<const uint4 *>(in + (static_cast<size_t>(row) * values + group * 16u));
    n0 = __ldcs(src);
    n1 = __ldcs(src + 1);
  }
  for (; row < rows; row += row_step) {
    uint32_t sf_code = 0;
    const uint4 v0 = n0, v1 = n1;
    if (in_row && row + row_step < rows) {
      const uint4 *src = reinterpret_cast<const uint4 *>(in + (static_cast<size_t>(row + row_step) * values + group * 16u));
      n0 = __ldcs(src);
      n1 = __ldcs(src + 1);
    }
    if (in_row) {
      const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      float x[16];
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x[2 * i] = __uint_as_float(w[i] << 16);
        x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        amax = fmaxf(amax, fmaxf(fabsf(x[2 * i]), fabsf(x[2 * i + 1])));
      }
      uint32_t any = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) any |= w[i];
      uint32_t lo, hi;
      q36::nvfp4_quantize_group(x, amax, (any & 0x7fff7fffu) != 0u, false, g, six_g, rcp6, lo, hi, sf_code);
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

// Row-major [rows, inner_groups] scale bytes -> tiled layout.  One thread per
// 4-byte word of the OUTPUT, so that every byte of the tiled buffer (padding
// included, as zero) is written exactly once and no separate memset is needed.
__global__ void __launch_bounds__(kThreads)
nvfp4_retile_kernel(const uint8_t *__restrict__ in, uint32_t *__restrict__ out, size_t rows,
                    size_t inner_groups, size_t words) {
  const size_t w = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (w >= words) return;
  const size_t tiles_per_block = q36::round_up(inner_groups, 4) / 4;
  const size_t tile = w / 128, in_tile = w % 128;
  const size_t row = (tile / tiles_per_block) * 128 + (in_tile % 4) * 32 + in_tile / 4;
  const size_t g0 = (tile % tiles_per_block) * 4;
  uint32_t v = 0;
  if (row < rows) {
    const uint8_t *src = in + row * inner_groups + g0;
    if (g0 + 4 <= inner_groups && (reinterpret_cast<uintptr_t>(src) & 3u) == 0) {
      v = __ldg(reinterpret_cast<const uint32_t *>(src));
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (g0 + i < inner_groups) v |= static_cast<uint32_t>(__ldg(src + i)) << (8 * i);
    }
  }
  out[w] = v;
}

// One thread per 16-group: 8 weight bytes in, 16 floats out.
__global__ void __launch_bounds__(kThreads)
nvfp4_dequantize_kernel(const uint8_t *__restrict__ weight, const uint8_t *__restrict__ sf,
                        const float *__restrict__ tensor_scale, float *__restrict__ out,
                        size_t out_features, size_t in_features) {
  const size_t groups = q36::div_ceil(in_features, 16);
  const size_t idx = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (idx >= out_features * groups) return;
  const size_t row = idx / groups, group = idx % groups;
  const float global = tensor_scale == nullptr ? 1.0f : __ldg(tensor_scale);
  const float scale =
      __fmul_rn(q36::decode_e4m3(__ldg(sf + q36::sf_offset(group, row, q36::round_up(groups, 4)))), global);
  const uint8_t *w = weight + row * q36::div_ceil(in_features, 2) + group * 8;
  float *dst = out + row * in_features + group * 16;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const size_t col = group * 16 + i;
    if (col < in_features) {
      const uint32_t b = __ldg(w + i / 2);
      dst[i] = __fmul_rn(q36::e2m1_value((i & 1) ? (b >> 4) : b), scale);
    }
  }
}

std::atomic<int> g_quantize_path{0};      // test hook: 1 = always the general kernel

int launch_quantize(qwen36_device_ptr_t in, qwen36_device_ptr_t fp4, qwen36_device_ptr_t sf,
                    qwen36_device_ptr_t ts, size_t rows, size_t values, float its) {
  const size_t padded = q36::round_up(q36::div_ceil(values, 16), 4);
  if (values % 16 == 0 && values < (1ull << 31) && rows < (1ull << 31) && (in.ptr & 15u) == 0 && (fp4.ptr & 7u) == 0 &&
      (sf.ptr & 3u) == 0 && g_quantize_path.load() != 1) {
    // about three waves of eight 256-thread CTAs per SM; a CTA covers 64 groups of 4 rows per step
    const size_t gx = q36::div_ceil(padded, 64), row_chunks = q36::div_ceil(rows, 4);
    const size_t want = q36::div_ceil(static_cast<size_t>(q36::sm_count_current_device()) * 24, gx);
    const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(row_chunks < want ? row_chunks : want));
    nvfp4_quantize_fast_kernel<<<grid, dim3(64, 4), 0, q36::stream()>>>(
        as_ptr<const __nv_bfloat16>(in), as_ptr<uint8_t>(fp4), as_ptr<uint8_t>(sf), as_ptr<float>(ts),
        static_cast<uint32_t>(rows), static_cast<uint32_t>(values), its);
    return q36::launch_status();
  }
  const size_t total = rows * padded;
  const size_t blocks = q36::div_ceil(total, kThreads);
  if (blocks > 0x7fffffffull) return QWEN36_STATUS_INVALID_ARGUMENT;
  // 32-bit indices when the thread index space, the element offsets (rows * values) and the tiled
  // scale offsets all stay below 2^32
  const bool small = (rows + 128) * (values + 64) < (1ull << 32) && (blocks + 1) * kThreads < (1ull << 32);
  const dim3 grid(static_cast<unsigned>(blocks)), block(kThreads);
  if (small)
    return q36::cuda_status(q36::launch_after_previous(
        nvfp4_quantize_kernel<uint32_t>, grid, block, size_t{0}, q36::stream(), as_ptr<const __nv_bfloat16>(in),
        as_ptr<uint8_t>(fp4), as_ptr<uint8_t>(sf), as_ptr<float>(ts), static_cast<uint32_t>(rows),
        static_cast<uint32_t>(values), its));
  return q36::cuda_status(q36::launch_after_previous(
      nvfp4_quantize_kernel<size_t>, grid, block, size_t{0}, q36::stream(), as_ptr<const __nv_bfloat16>(in),
      as_ptr<uint8_t>(fp4), as_ptr<uint8_t>(sf), as_ptr<float>(ts), rows, values, its));
}

}  // namespace

// Test hook: 1 sends every shape through the general kernel, 0 restores the library's own routing.
extern "C" void qwen36_nvfp4_quantize_set_path(int path) { g_quantize_path.store(path); }

extern "C" int qwen36_nvfp4_quantize_bf16(const qwen36_nvfp4_quantize_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->values == 0 || spec->input_bf16.ptr == 0 || spec->output_fp4.ptr == 0 ||
      spec->output_scale_e4m3.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  return launch_quantize(spec->input_bf16, spec->output_fp4, spec->output_scale_e4m3,
                         spec->output_tensor_scale_f32, 1, spec->values, spec->input_tensor_scale_f32);
}

extern "C" int qwen36_nvfp4_quantize_rows(const qwen36_nvfp4_quantize_rows_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->rows == 0 || spec->values == 0 || spec->input_bf16.ptr == 0 || spec->output_fp4.ptr == 0 ||
      spec->output_scale_e4m3.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  return launch_quantize(spec->input_bf16, spec->output_fp4, spec->output_scale_e4m3,
                         spec->output_tensor_scale_f32, spec->rows, spec->values,
                         spec->input_tensor_scale_f32);
}

extern "C" int qwen36_nvfp4_retile_scales(const qwen36_nvfp4_retile_scales_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->rows == 0 || spec->inner_groups == 0 || spec->input_row_major_u8.ptr == 0 ||
      spec->output_tiled_u8.ptr == 0 || (spec->output_tiled_u8.ptr & 3u) != 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const size_t words = q36::sf_bytes(spec->inner_groups, spec->rows) / 4;
  nvfp4_retile_kernel<<<static_cast<unsigned>(q36::div_ceil(words, kThreads)), kThreads, 0, q36::stream()>>>(
      as_ptr<const uint8_t>(spec->input_row_major_u8), as_ptr<uint32_t>(spec->output_tiled_u8), spec->rows,
      spec->inner_groups, words);
  return q36::launch_status();
}

extern "C" int qwen36_nvfp4_dequantize(const qwen36_nvfp4_dequantize_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->out_features == 0 || spec->in_features == 0 || spec->weight_u8.ptr == 0 ||
      spec->block_scale_e4m3.ptr == 0 || spec->output_f32.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const size_t total = spec->out_features * q36::div_ceil(spec->in_features, 16);
  nvfp4_dequantize_kernel<<<static_cast<unsigned>(q36::div_ceil(total, kThreads)), kThreads, 0, q36::stream()>>>(
      as_ptr<const uint8_t>(spec->weight_u8), as_ptr<const uint8_t>(spec->block_scale_e4m3),
      as_ptr<const float>(spec->tensor_scale_f32), as_ptr<float>(spec->output_f32), spec->out_features,
      spec->in_features);
  return q36::launch_status();
}

extern "C" size_t qwen36_nvfp4_tiled_scale_bytes(size_t rows, size_t inner_groups) {
  return q36::sf_bytes(inner_groups, rows);
}

extern "C" int qwen36_nvfp4_tile_scales_host(const uint8_t *row_major, uint8_t *tiled, size_t rows,
                                             size_t inner_groups) {
  if (row_major == nullptr || tiled == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (rows == 0 || inner_groups == 0) return QWEN36_STATUS_INVALID_ARGUMENT;
  const size_t sf_inner = q36::round_up(inner_groups, 4);
  const size_t bytes = q36::sf_bytes(inner_groups, rows);
  for (size_t i = 0; i < bytes; ++i) tiled[i] = 0;
  for (size_t r = 0; r < rows; ++r)
    for (size_t g = 0; g < inner_groups; ++g)
      tiled[q36::sf_offset(g, r, sf_inner)] = row_major[r * inner_groups + g];
  return QWEN36_STATUS_SUCCESS;
}
