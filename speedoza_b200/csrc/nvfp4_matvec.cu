// W4A16 NVFP4 GEMV: y[row] = bf16( sum_g (sum_{i<16} x[16g+i] * e2m1(w)) * (ue4m3(sf[g,row]) * global) )
// (semantics of kernels-cuda/ops.cu:547-639 in the reference).
//
// HBM-bound weight streaming.  Work unit = a "row quad": rows r, r+32, r+64,
// r+96 of one 128-row block.  Those four rows share one 16-byte word per scale
// tile (4 rows x 4 groups), so a lane fetches its scales with ONE 16-byte load
// per 128 weights, and reuses every activation register four times.  Lanes of
// a warp stride along K with 16-byte weight loads (512 contiguous bytes per
// row per warp instruction); two iterations of loads stay in flight per lane.
// Nibbles are expanded by cvt.rn.f16x2.e2m1x2 (two weights per instruction);
// products accumulate in float32.
//
// The weight and scale loads of the first iteration are issued before
// griddepcontrol.wait, so under programmatic dependent launch they overlap
// the tail of the kernel that produces x.
#include "common.cuh"

#include <atomic>
#include <cuda_fp16.h>
#include <mutex>

namespace {

using q36::as_ptr;

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

// How activations are held in shared memory / multiplied:
//   0: float32, one fma.rn.f32x2 per weight pair (exact products).
//   1: float16 scaled by a power of two so that max|x| lands in [2^14, 2^15),
//      one mixed-precision fma.rn.f32.f16 per weight (exact products; values
//      below max|x| * 2^-38 flush, far below float32 accumulation error).
template <int MODE> struct XT;
template <> struct XT<0> { using type = float; };
template <> struct XT<1> { using type = __half; };

// 16-byte chunk swizzle of the activation buffer so that the eight lanes of a
// quarter warp, which read chunks that are a whole number of 128-byte rows
// apart, land on distinct bank groups.
template <int MODE> __device__ __forceinline__ uint32_t x_chunk(uint32_t lane_slot, uint32_t i) {
  if (MODE == 0) return lane_slot * 8u + (i ^ (lane_slot & 7u));             // 8 chunks per slot
  return lane_slot * 4u + (i ^ ((lane_slot >> 1) & 3u));                      // 4 chunks per slot
}

__device__ __forceinline__ void e2m1x8_to_h2(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}

// acc += w.lo * x.lo + w.hi * x.hi, float16 operands, float32 accumulate.
__device__ __forceinline__ void fma_mixed(float &acc, uint32_t w_h2, uint32_t x_h2) {
  asm("{\n\t.reg .f16 wl, wh, xl, xh;\n\t"
      "mov.b32 {wl, wh}, %1;\n\t"
      "mov.b32 {xl, xh}, %2;\n\t"
      "fma.rn.f32.f16 %0, wl, xl, %0;\n\t"
      "fma.rn.f32.f16 %0, wh, xh, %0;\n\t}"
      : "+f"(acc)
      : "r"(w_h2), "r"(x_h2));
}

__device__ __forceinline__ void fma_f32x2(float2 &acc, float2 a, float2 b) {
  unsigned long long c = *reinterpret_cast<unsigned long long *>(&acc);
  asm("fma.rn.f32x2 %0, %1, %2, %0;"
      : "+l"(c)
      : "l"(*reinterpret_cast<unsigned long long *>(&a)), "l"(*reinterpret_cast<unsigned long long *>(&b)));
  acc = *reinterpret_cast<float2 *>(&c);
}

struct Frag {
  uint4 w[4];   // 32 weights of each of the four rows
  uint4 s;      // scale bytes [row j][group c] at byte 4*j + c
};

template <int MODE, int KSPLIT>
__global__ void __launch_bounds__(kThreads)
nvfp4_matvec_kernel(const __nv_bfloat16 *__restrict__ x, const uint8_t *__restrict__ weight,
                    const uint8_t *__restrict__ sf, const float *__restrict__ tensor_scale,
                    __nv_bfloat16 *__restrict__ y, uint32_t K, uint32_t N) {
  using xt = typename XT<MODE>::type;
  extern __shared__ __align__(16) uint8_t smem[];
  float *lut = reinterpret_cast<float *>(smem);                 // 256 decoded scales * global
  float *red = lut + 256;                                       // kWarps * 4 partial sums
  uint32_t *amax_bits = reinterpret_cast<uint32_t *>(red + kWarps * 4);
  uint4 *xs = reinterpret_cast<uint4 *>(smem + 2048);           // activations, swizzled 16-byte chunks

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  constexpr uint32_t kQuadsPerCta = kWarps / KSPLIT;
  const uint32_t quad = blockIdx.x * kQuadsPerCta + warp / KSPLIT;
  const uint32_t ks = warp % KSPLIT;
  const uint32_t rb = quad >> 5, r = quad & 31u;                // 128-row block, row within sub-block
  const uint32_t row0 = rb * 128u + r;
  const uint32_t iters = (K + 1023u) / 1024u;
  const uint32_t tiles_per_block = (K / 16u + 3u) / 4u;
  const bool quad_valid = row0 < N;

  const uint8_t *wrow[4];
  bool rvalid[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    rvalid[j] = row0 + 32u * j < N;
    wrow[j] = weight + static_cast<size_t>(row0 + 32u * j) * (K / 2u);
  }
  const uint8_t *sfrow = sf + static_cast<size_t>(rb) * tiles_per_block * 512u + r * 16u;

  auto load = [&](Frag &f, uint32_t it) {
    const uint32_t col = lane * 32u + it * 1024u;
    if (quad_valid && col < K) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        f.w[j] = rvalid[j] ? __ldcs(reinterpret_cast<const uint4 *>(wrow[j] + col / 2u)) : make_uint4(0, 0, 0, 0);
      f.s = __ldcs(reinterpret_cast<const uint4 *>(sfrow + static_cast<size_t>(col / 64u) * 512u));
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) f.w[j] = make_uint4(0, 0, 0, 0);
      f.s = make_uint4(0, 0, 0, 0);
    }
  };

  // Scale table and first loads do not depend on the previous kernel.
  {
    const float global = tensor_scale == nullptr ? 1.0f : __ldg(tensor_scale);
    lut[threadIdx.x] = __fmul_rn(q36::decode_e4m3(threadIdx.x), global);
    if (threadIdx.x == 0) *amax_bits = 0u;
  }
  Frag cur, nxt;
  load(cur, ks);

  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // Stage x.  Slot = 32 consecutive activations (what one lane consumes per
  // iteration); K is a multiple of 32.
  int shift = 0;
  if (MODE == 1) {
    __syncthreads();
    uint32_t m = 0;
    for (uint32_t i = threadIdx.x; i < K / 2u; i += kThreads) {
      const uint32_t v = __ldcg(reinterpret_cast<const uint32_t *>(x) + i);
      m = max(m, max(v & 0x7fffu, (v >> 16) & 0x7fffu));
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if (lane == 0) atomicMax(amax_bits, m);
    __syncthreads();
    const uint32_t e = (*amax_bits >> 7) & 0xffu;
    shift = e == 255u ? 0 : (e < 15u ? 126 : 141 - static_cast<int>(e));
  }
  {
    const float up = __uint_as_float(static_cast<uint32_t>(127 + shift) << 23);
    const uint32_t slots = K / 32u;
    // one thread converts 8 activations (one 16-byte load) at a time
    for (uint32_t c = threadIdx.x; c < slots * 4u; c += kThreads) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(x) + c);   // L2 only: x may be fresh from the previous kernel
      const uint32_t slot = c >> 2, sub = c & 3u;
      const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
      float f[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(wv[i] << 16);
        f[2 * i + 1] = __uint_as_float(wv[i] & 0xffff0000u);
      }
      if (MODE == 0) {
        xs[x_chunk<0>(slot, sub * 2u)] = *reinterpret_cast<uint4 *>(&f[0]);
        xs[x_chunk<0>(slot, sub * 2u + 1u)] = *reinterpret_cast<uint4 *>(&f[4]);
      } else {
        __half2 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i] * up, f[2 * i + 1] * up);
        xs[x_chunk<1>(slot, sub)] = *reinterpret_cast<uint4 *>(h);
      }
    }
  }
  __syncthreads();

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t cbase = 2u * (lane & 1u);       // first of this lane's two groups inside its scale tile

  for (uint32_t it = ks; it < iters; it += KSPLIT) {
    if (it + KSPLIT < iters) load(nxt, it + KSPLIT);
    const uint32_t slot = lane + it * 32u;
    if (slot * 32u < K) {
      const uint32_t sw[4] = {cur.s.x, cur.s.y, cur.s.z, cur.s.w};
#pragma unroll
      for (int half = 0; half < 2; ++half) {          // the two 16-groups of this slot
        float local[4];
        if (MODE == 0) {
          float2 a2[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
          const uint4 xa = xs[x_chunk<0>(slot, half * 4u + 0u)], xb = xs[x_chunk<0>(slot, half * 4u + 1u)];
          const uint4 xc = xs[x_chunk<0>(slot, half * 4u + 2u)], xd = xs[x_chunk<0>(slot, half * 4u + 3u)];
          const float2 xv[8] = {{__uint_as_float(xa.x), __uint_as_float(xa.y)}, {__uint_as_float(xa.z), __uint_as_float(xa.w)},
                                {__uint_as_float(xb.x), __uint_as_float(xb.y)}, {__uint_as_float(xb.z), __uint_as_float(xb.w)},
                                {__uint_as_float(xc.x), __uint_as_float(xc.y)}, {__uint_as_float(xc.z), __uint_as_float(xc.w)},
                                {__uint_as_float(xd.x), __uint_as_float(xd.y)}, {__uint_as_float(xd.z), __uint_as_float(xd.w)}};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t w0 = half == 0 ? cur.w[j].x : cur.w[j].z;
            const uint32_t w1 = half == 0 ? cur.w[j].y : cur.w[j].w;
            uint32_t h[4];
            e2m1x8_to_h2(w0, h);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              fma_f32x2(a2[j], __half22float2(*reinterpret_cast<__half2 *>(&h[i])), xv[i]);
            e2m1x8_to_h2(w1, h);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              fma_f32x2(a2[j], __half22float2(*reinterpret_cast<__half2 *>(&h[i])), xv[4 + i]);
            local[j] = a2[j].x + a2[j].y;
          }
        } else {
          const uint4 xa = xs[x_chunk<1>(slot, half * 2u)], xb = xs[x_chunk<1>(slot, half * 2u + 1u)];
          const uint32_t xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t w0 = half == 0 ? cur.w[j].x : cur.w[j].z;
            const uint32_t w1 = half == 0 ? cur.w[j].y : cur.w[j].w;
            uint32_t h[4];
            float a = 0.f;
            e2m1x8_to_h2(w0, h);
#pragma unroll
            for (int i = 0; i < 4; ++i) fma_mixed(a, h[i], xv[i]);
            e2m1x8_to_h2(w1, h);
#pragma unroll
            for (int i = 0; i < 4; ++i) fma_mixed(a, h[i], xv[4 + i]);
            local[j] = a;
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t code = (sw[j] >> (8u * (cbase + half))) & 0xffu;
          acc[j] = fmaf(local[j], lut[code], acc[j]);
        }
      }
    }
    cur = nxt;
  }

#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
  }
  const float down = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
  if (KSPLIT == 1) {
    if (lane < 4 && quad_valid && row0 + 32u * lane < N) {
      const float v = lane == 0 ? acc[0] : lane == 1 ? acc[1] : lane == 2 ? acc[2] : acc[3];
      y[row0 + 32u * lane] = __float2bfloat16(v * down);
    }
  } else {
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) red[warp * 4 + j] = acc[j];
    }
    __syncthreads();
    if (ks == 0 && lane < 4 && quad_valid && row0 + 32u * lane < N) {
      float v = 0.f;
#pragma unroll
      for (int k2 = 0; k2 < KSPLIT; ++k2) v += red[(warp + k2) * 4 + lane];
      y[row0 + 32u * lane] = __float2bfloat16(v * down);
    }
  }
}

// Any shape, any alignment: one warp per row, byte loads.  Only taken when
// in_features is not a multiple of 32 or a pointer is not 16-byte aligned.
__global__ void __launch_bounds__(kThreads)
nvfp4_matvec_generic_kernel(const __nv_bfloat16 *__restrict__ x, const uint8_t *__restrict__ weight,
                            const uint8_t *__restrict__ sf, const float *__restrict__ tensor_scale,
                            __nv_bfloat16 *__restrict__ y, size_t K, size_t N) {
  const size_t row = static_cast<size_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  const unsigned lane = threadIdx.x & 31u;
  if (row >= N) return;
  const size_t packed = (K + 1) / 2, groups = (K + 15) / 16, sf_inner = q36::round_up(groups, 4);
  const float global = tensor_scale == nullptr ? 1.0f : __ldg(tensor_scale);
  float sum = 0.f;
  for (size_t g = lane; g < groups; g += 32) {
    const float scale = __fmul_rn(q36::decode_e4m3(__ldg(sf + q36::sf_offset(g, row, sf_inner))), global);
    float local = 0.f;
    for (int i = 0; i < 16; ++i) {
      const size_t col = g * 16 + i;
      if (col < K) {
        const uint32_t b = __ldg(weight + row * packed + col / 2);
        local = fmaf(__bfloat162float(x[col]), q36::e2m1_value((col & 1) ? (b >> 4) : b), local);
      }
    }
    sum = fmaf(local, scale, sum);
  }
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if (lane == 0) y[row] = __float2bfloat16(sum);
}

std::atomic<int> g_mode{1};

template <int MODE, int KSPLIT>
int launch_fast(const qwen36_nvfp4_matvec_spec_t *s) {
  const uint32_t K = static_cast<uint32_t>(s->in_features), N = static_cast<uint32_t>(s->out_features);
  const size_t smem = 2048 + static_cast<size_t>(K) * sizeof(typename XT<MODE>::type);
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(nvfp4_matvec_kernel<MODE, KSPLIT>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  });
  if (attr_err != cudaSuccess) return QWEN36_STATUS_CUDA_ERROR;
  const uint32_t quads = ((N + 127u) / 128u) * 32u;
  constexpr uint32_t per_cta = kWarps / KSPLIT;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((quads + per_cta - 1) / per_cta);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return q36::cuda_status(cudaLaunchKernelEx(
      &cfg, nvfp4_matvec_kernel<MODE, KSPLIT>, as_ptr<const __nv_bfloat16>(s->input_bf16),
      as_ptr<const uint8_t>(s->weight_u8), as_ptr<const uint8_t>(s->block_scale_e4m3),
      as_ptr<const float>(s->tensor_scale_f32), as_ptr<__nv_bfloat16>(s->output_bf16), K, N));
}

template <int MODE>
int launch_mode(const qwen36_nvfp4_matvec_spec_t *s) {
  // Aim for at least ~16 warps per SM on a 148-SM part: split K across the
  // warps of a CTA when there are few row quads.
  const size_t quads = q36::div_ceil(s->out_features, 128) * 32;
  const size_t iters = q36::div_ceil(s->in_features, 1024);
  int ksplit = 1;
  while (ksplit < 8 && quads * ksplit < 2368 && static_cast<size_t>(ksplit) * 2 <= iters) ksplit *= 2;
  switch (ksplit) {
    case 1: return launch_fast<MODE, 1>(s);
    case 2: return launch_fast<MODE, 2>(s);
    case 4: return launch_fast<MODE, 4>(s);
    default: return launch_fast<MODE, 8>(s);
  }
}

}  // namespace

// Test/bench hook: 0 = float32 activations + packed f32x2 FMA, 1 = scaled
// float16 activations + mixed-precision FMA (default).  Not part of the
// reference ABI.
extern "C" void qwen36_nvfp4_matvec_set_mode(int mode) { g_mode.store(mode == 0 ? 0 : 1); }

extern "C" int qwen36_nvfp4_matvec(const qwen36_nvfp4_matvec_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->out_features == 0 || spec->in_features == 0 || spec->input_bf16.ptr == 0 ||
      spec->weight_u8.ptr == 0 || spec->block_scale_e4m3.ptr == 0 || spec->output_bf16.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const bool fast = spec->in_features % 32 == 0 && spec->in_features <= 48 * 1024 &&
                    spec->out_features < (1u << 31) &&
                    ((spec->input_bf16.ptr | spec->weight_u8.ptr | spec->block_scale_e4m3.ptr) & 15u) == 0;
  if (!fast) {
    const size_t blocks = q36::div_ceil(spec->out_features, kWarps);
    nvfp4_matvec_generic_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, q36::stream()>>>(
        as_ptr<const __nv_bfloat16>(spec->input_bf16), as_ptr<const uint8_t>(spec->weight_u8),
        as_ptr<const uint8_t>(spec->block_scale_e4m3), as_ptr<const float>(spec->tensor_scale_f32),
        as_ptr<__nv_bfloat16>(spec->output_bf16), spec->in_features, spec->out_features);
    return q36::launch_status();
  }
  return g_mode.load() == 0 ? launch_mode<0>(spec) : launch_mode<1>(spec);
}
