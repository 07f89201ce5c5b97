// Pieces shared by the split-KV attention kernels that run both products on the tensor cores
// (int8, FP8 and BF16 caches, head size 256): the float16 MMA wrapper, the asynchronous-copy
// helpers of the shared-memory staged forms, and the CTA epilogue that merges the eight warps'
// running softmax states into one (m, l, o) partial per q head.
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace q36 {

constexpr int kSplitThreads = 256;
constexpr int kSplitWarps = kSplitThreads / 32;

// Launch with programmatic stream serialisation: the grid may take its seats while the previous
// kernel in the stream drains.  The kernel must execute griddepcontrol.wait before it touches
// anything an earlier kernel may have written (and before it overwrites anything one may still read).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_after_previous(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem_bytes,
                                         cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}


// One step of the online softmax for head g (the four lanes t = 0 .. 3 of a lane group hold its
// sixteen tokens): s_log2[i] are this lane's four scores in log2 units (-inf = masked).  Updates
// the running maximum and sum (identical on the four lanes), leaves the probabilities in p and
// returns the factor by which everything accumulated so far has to be scaled.
__device__ __forceinline__ float online_softmax_step(const float (&s_log2)[4], float (&p)[4], float &m_run,
                                                     float &l_run) {
  float tile_max = fmaxf(fmaxf(s_log2[0], s_log2[1]), fmaxf(s_log2[2], s_log2[3]));
  tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
  tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
  const float m_new = fmaxf(m_run, tile_max);
  const float corr = m_new == -INFINITY ? 1.f : exp2f(m_run - m_new);
  float p_sum = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    p[i] = s_log2[i] == -INFINITY ? 0.f : exp2f(s_log2[i] - m_new);
    p_sum += p[i];
  }
  p_sum += __shfl_xor_sync(0xffffffffu, p_sum, 1);
  p_sum += __shfl_xor_sync(0xffffffffu, p_sum, 2);
  l_run = l_run * corr + p_sum;
  m_run = m_new;
  return corr;
}

// Scales the running outputs by the heads' correction factors: lane (g, t) holds heads 2t and
// 2t + 1 in its accumulators, whose factors live on lanes 8t and 8t + 4.
__device__ __forceinline__ void rescale_outputs(float (&o)[2][8][4], float corr) {
  const uint32_t t = threadIdx.x & 3u;
  const float c_even = __shfl_sync(0xffffffffu, corr, 8 * t), c_odd = __shfl_sync(0xffffffffu, corr, 8 * t + 4);
  if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[h][j][0] *= c_even; o[h][j][1] *= c_odd; o[h][j][2] *= c_even; o[h][j][3] *= c_odd;
      }
  }
}

// Epilogue shared by the tensor-core split kernels: merges the eight warps' running softmax states
// (maxima in log2 units, outputs scaled by 1 / out_scale) and writes the CTA's partial.
// o[h][j][c]: head 2t + (c & 1), dim 16 (g + 8 h) + 2 j + (c >> 1).
constexpr uint32_t kEpiStride = 256 + 4;                          // row stride: heads land a quarter of the banks apart
template <int G>
__device__ __forceinline__ void split_epilogue(float (&o)[2][8][4], float m_run, float l_run, float out_scale,
                                               float (*s_m)[8], float (*s_l)[8], float (*s_o)[kEpiStride],
                                               float *__restrict__ part_o, float *__restrict__ part_m,
                                               float *__restrict__ part_l, uint32_t head0, uint32_t split,
                                               uint32_t n_splits) {
  constexpr uint32_t D = 256, DP = kEpiStride;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  // ---- merge the warps of the CTA: weights per head from the running maxima; the weighted outputs
  // meet in four shared-memory slices (warps 4..7 write, warps 0..3 add), then every thread sums
  // the four slices of its outputs.  A lane holds all sixteen dims of chunk g + 8 h for its two
  // heads (dims 2 j from c = e, 2 j + 1 from c = e + 2), so it moves them as four 16-byte vectors.
  if (t == 0 && g < G) { s_m[warp][g] = m_run; s_l[warp][g] = l_run; }
  __syncthreads();
  float wgt[2];                                                    // heads 2t, 2t + 1
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const uint32_t head = 2 * t + e;
    float M = -INFINITY;
    if (head < G)
      for (int w = 0; w < kSplitWarps; ++w) M = fmaxf(M, s_m[w][head]);
    const float mine = head < G ? s_m[warp][head] : -INFINITY;
    wgt[e] = mine == -INFINITY ? 0.f : exp2f(mine - M) * out_scale;
  }
  float (*slice)[DP] = &s_o[(warp & 3u) * G];
  for (int round = 0; round < 2; ++round) {
    if ((warp >> 2) == static_cast<uint32_t>(1 - round)) {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t head = 2 * t + e;
          if (head < G) {
            float4 *dst = reinterpret_cast<float4 *>(&slice[head][16 * (g + 8 * h)]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float a0 = o[h][2 * q][e], a1 = o[h][2 * q][e + 2], a2 = o[h][2 * q + 1][e], a3 = o[h][2 * q + 1][e + 2];
              if (round == 0) {
                dst[q] = make_float4(wgt[e] * a0, wgt[e] * a1, wgt[e] * a2, wgt[e] * a3);
              } else {
                const float4 p = dst[q];
                dst[q] = make_float4(fmaf(wgt[e], a0, p.x), fmaf(wgt[e], a1, p.y), fmaf(wgt[e], a2, p.z), fmaf(wgt[e], a3, p.w));
              }
            }
          }
        }
    }
    __syncthreads();
  }
  const bool vec_out = (reinterpret_cast<uintptr_t>(part_o) & 15u) == 0;
  for (uint32_t idx = threadIdx.x; idx < G * (D / 4); idx += kSplitThreads) {
    const uint32_t hd = idx / (D / 4), d = (idx % (D / 4)) * 4;
    const size_t slot = static_cast<size_t>(head0 + hd) * n_splits + split;
    const float4 s0 = *reinterpret_cast<const float4 *>(&s_o[hd][d]), s1 = *reinterpret_cast<const float4 *>(&s_o[G + hd][d]);
    const float4 s2 = *reinterpret_cast<const float4 *>(&s_o[2 * G + hd][d]), s3 = *reinterpret_cast<const float4 *>(&s_o[3 * G + hd][d]);
    const float4 r = make_float4((s0.x + s1.x) + (s2.x + s3.x), (s0.y + s1.y) + (s2.y + s3.y),
                                 (s0.z + s1.z) + (s2.z + s3.z), (s0.w + s1.w) + (s2.w + s3.w));
    float *out = part_o + slot * D + d;
    if (vec_out) {
      *reinterpret_cast<float4 *>(out) = r;
    } else {
      out[0] = r.x; out[1] = r.y; out[2] = r.z; out[3] = r.w;
    }
    if (d == 0) {
      float M = -INFINITY, den = 0.f;
      for (int w = 0; w < kSplitWarps; ++w) M = fmaxf(M, s_m[w][hd]);
      for (int w = 0; w < kSplitWarps; ++w)
        den = fmaf(s_m[w][hd] == -INFINITY ? 0.f : exp2f(s_m[w][hd] - M), s_l[w][hd], den);
      part_m[slot] = M * 0.6931471805599453f;
      part_l[slot] = den;
    }
  }
}

}  // namespace q36
