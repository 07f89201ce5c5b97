// Log-sum-exp merge of split-KV partials: the arithmetic shared by the single-GPU merge kernel and
// the cross-rank merge, so that every route produces the same bits.
//   M = max m_s,  w_s = (m_s == -inf ? 0 : exp(m_s - M)),  den = sum w_s l_s,  acc[d] = sum w_s o_s[d]
// (reference: kernels-cuda/attention.cu:1473-1554).  A block of 256 threads per q head.
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace q36 {

constexpr int kMergeThreads = 256;

// One part per thread (n_parts <= 256).  Leaves the weights in s_w[0 .. 255] and returns M and den
// to every thread.  s_red: 8 floats.  Contains block barriers: call from all threads.
__device__ __forceinline__ void lse_weights(const float *pm, const float *pl, uint32_t n_parts, float *s_w,
                                            float *s_red, float &M_out, float &den_out) {
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const float my_m = threadIdx.x < n_parts ? __ldcg(pm + threadIdx.x) : -INFINITY;
  const float my_l = threadIdx.x < n_parts ? __ldcg(pl + threadIdx.x) : 0.f;
  float M = my_m;
  for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
  if (lane == 0) s_red[warp] = M;
  __syncthreads();
  M = s_red[0];
  for (int w = 1; w < kMergeThreads / 32; ++w) M = fmaxf(M, s_red[w]);
  const float wgt = my_m == -INFINITY ? 0.f : __expf(my_m - M);
  s_w[threadIdx.x] = wgt;
  float den = wgt * my_l;
  for (int off = 16; off > 0; off >>= 1) den += __shfl_xor_sync(0xffffffffu, den, off);
  __syncthreads();
  if (lane == 0) s_red[warp] = den;
  __syncthreads();
  den = 0.f;
  for (int w = 0; w < kMergeThreads / 32; ++w) den += s_red[w];
  M_out = M;
  den_out = den;
}

// The first N parts' values of output dim d, fetched ahead of the weights (the loads then travel
// while lse_weights runs its reductions: with N >= n_parts the whole merge costs one round trip to
// L2 instead of one per batch).  Clamped indices: no branch, no out-of-range read.
template <int N>
__device__ __forceinline__ void lse_prefetch(const float *po, uint32_t n_parts, uint32_t head_dim, uint32_t d,
                                             float (&v)[N]) {
#pragma unroll
  for (uint32_t i = 0; i < static_cast<uint32_t>(N); ++i)
    v[i] = __ldcg(po + static_cast<size_t>(min(i, n_parts - 1)) * head_dim + d);
}

// sum over parts of s_w[s] * po[s * head_dim + d], in part order; `first` holds the values of parts
// 0 .. N - 1 from lse_prefetch, the rest is fetched sixteen loads at a time (a plain loop pays the L2
// latency once per part in its remainder iterations).
template <int N>
__device__ __forceinline__ float lse_accumulate(const float *po, const float *s_w, uint32_t n_parts,
                                                uint32_t head_dim, uint32_t d, const float (&first)[N]) {
  float acc = 0.f;
#pragma unroll
  for (uint32_t i = 0; i < static_cast<uint32_t>(N); ++i)
    if (i < n_parts) acc = fmaf(s_w[i], first[i], acc);
  for (uint32_t s0 = N; s0 < n_parts; s0 += 16) {
    float v[16];
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i)
      v[i] = __ldcg(po + static_cast<size_t>(min(s0 + i, n_parts - 1)) * head_dim + d);   // clamped: no branch
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i)
      if (s0 + i < n_parts) acc = fmaf(s_w[s0 + i], v[i], acc);
  }
  return acc;
}

__device__ __forceinline__ float lse_accumulate(const float *po, const float *s_w, uint32_t n_parts,
                                                uint32_t head_dim, uint32_t d) {
  float first[16];
  lse_prefetch(po, n_parts, head_dim, d, first);
  return lse_accumulate(po, s_w, n_parts, head_dim, d, first);
}

}  // namespace q36
