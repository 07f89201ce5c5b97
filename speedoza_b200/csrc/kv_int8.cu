// int8 per-vector KV cache: encode, split-KV decode attention, (m, l, o) merge.
//
// Cache layout (kernels-cuda/turboquant.cu:23-67 in the reference): int8
// [position, kv_heads, head_dim] for K and for V, float32 metadata
// [position, kv_heads, 2] = (k_scale, v_scale), scale = absmax / 127, code =
// clamp(round-to-nearest-even(v / scale), -127, 127), all-zero vector -> 0.
//
// Decode attention is HBM-bound on the cache read.  One CTA owns one kv head
// and one contiguous token range ("split"); it serves every q head of that kv
// head's group from the same K/V bytes, so the cache is read exactly once.  A
// warp takes a token, the 32 lanes take head_dim/32 dims each (coalesced 256-
// byte rows at head_dim 256), scores meet in a butterfly, the softmax is the
// online (running max) form.  Every split leaves an un-normalised partial
// (m, l, o) in caller scratch in the layout of the reference's split paths
// (kernels-cuda/attention.cu:1083-1094); a second kernel merges them.
#include "common.cuh"

#include <atomic>

#include <cuda_fp16.h>

#include <mutex>

#include "kv_split.cuh"
#include "lse_merge.cuh"
#include "peer_combine.cuh"

namespace {

// %globaltimer stamps (time, CTA, event) appended to a log for a timeline of a few calls; compiled in
// only with -DQ36_ATTN_TRACE.
#ifdef Q36_ATTN_TRACE
constexpr uint32_t kTraceEntries = 1u << 15;
__device__ unsigned long long g_attn_trace[kTraceEntries][2];
__device__ unsigned int g_attn_trace_n = 0;
#define Q36_ATRACE(cta_, ev)                                                        \
  do {                                                                             \
    if (threadIdx.x == 0) {                                                        \
      unsigned long long t_;                                                       \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                       \
      const unsigned int at_ = atomicAdd(&g_attn_trace_n, 1u);                     \
      if (at_ < kTraceEntries) { g_attn_trace[at_][0] = t_; g_attn_trace[at_][1] = (static_cast<unsigned long long>(cta_) << 8) | (ev); } \
    }                                                                              \
  } while (0)
#else
#define Q36_ATRACE(cta_, ev)
#endif

using q36::as_ptr;

constexpr int kThreads = 256;
static_assert(kThreads == q36::kMergeThreads, "merge block size");
constexpr int kWarps = kThreads / 32;
constexpr int kMaxSplits = 128;
constexpr int kMinTokensPerSplit = 256;

// ------------------------------------------------------------------ encode

__device__ __forceinline__ int quantize_s8(float v, float scale) {
  const float scaled = scale == 0.0f ? 0.0f : __fdiv_rn(v, scale);
  int r = __float2int_rn(scaled);          // round-to-nearest-even, as lrintf
  r = r > 127 ? 127 : r;
  return r < -127 ? -127 : r;
}

// One warp per (token, kv head, K|V) vector.
__global__ void __launch_bounds__(kThreads)
kv_encode_kernel(const __nv_bfloat16 *__restrict__ k, const __nv_bfloat16 *__restrict__ v,
                 int8_t *__restrict__ kq, int8_t *__restrict__ vq, float *__restrict__ meta, size_t position,
                 size_t tokens, size_t kv_heads, size_t head_dim) {
  asm volatile("griddepcontrol.wait;" ::: "memory");               // launched with programmatic stream serialisation
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const size_t vec = static_cast<size_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  const unsigned lane = threadIdx.x & 31u;
  if (vec >= tokens * kv_heads * 2) return;
  const size_t which = vec & 1, th = vec >> 1;          // th = token * kv_heads + head
  const __nv_bfloat16 *src = (which ? v : k) + th * head_dim;
  const size_t row = position * kv_heads + th;
  int8_t *dst = (which ? vq : kq) + row * head_dim;
  const bool vec8 = head_dim % 8 == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0 &&
                    (reinterpret_cast<uintptr_t>(dst) & 7u) == 0;
  float amax = 0.f;
  if (vec8) {
    for (size_t d = lane * 8; d < head_dim; d += 256) {
      const uint4 p = __ldcs(reinterpret_cast<const uint4 *>(src + d));
      const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
        amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w[i] << 16)), fabsf(__uint_as_float(w[i] & 0xffff0000u))));
    }
  } else {
    for (size_t d = lane; d < head_dim; d += 32) amax = fmaxf(amax, fabsf(__bfloat162float(src[d])));
  }
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const float scale = __fdiv_rn(amax, 127.0f);
  if (lane == 0) meta[row * 2 + which] = scale;
  if (vec8) {
    for (size_t d = lane * 8; d < head_dim; d += 256) {
      const uint4 p = __ldg(reinterpret_cast<const uint4 *>(src + d));   // second touch: L1/L2 hit
      const uint32_t w[4] = {p.x, p.y, p.z, p.w};
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        lo |= (quantize_s8(__uint_as_float(w[i] << 16), scale) & 0xff) << (16 * i);
        lo |= (quantize_s8(__uint_as_float(w[i] & 0xffff0000u), scale) & 0xff) << (16 * i + 8);
        hi |= (quantize_s8(__uint_as_float(w[2 + i] << 16), scale) & 0xff) << (16 * i);
        hi |= (quantize_s8(__uint_as_float(w[2 + i] & 0xffff0000u), scale) & 0xff) << (16 * i + 8);
      }
      *reinterpret_cast<uint2 *>(dst + d) = make_uint2(lo, hi);
    }
  } else {
    for (size_t d = lane; d < head_dim; d += 32)
      dst[d] = static_cast<int8_t>(quantize_s8(__bfloat162float(src[d]), scale));
  }
}

// The same encode for head_dim 256 and many vectors (prefill: tokens x kv_heads x 2 of them), built
// to run at the HBM rate: a warp walks vectors with a stride of the grid, a lane owns eight values
// (one 16-byte load, kept in registers for both passes) and the next vector's load is in flight
// while the current ones are worked on.  v / scale becomes v * (1 / scale) with the correctly rounded
// reciprocal: that product is within 2^-16 of the IEEE quotient (|quotient| <= 127), so it rounds to
// the same integer unless it lies within 2^-14 of a tie, and those values (and every vector whose
// maximum is zero, tiny, huge, infinite or a NaN) take the reference's division.
__device__ __forceinline__ void kv_encode_vector256(const uint4 &cur, unsigned lane, int8_t *__restrict__ dst,
                                                    float *__restrict__ meta_slot) {
  const uint32_t w[4] = {cur.x, cur.y, cur.z, cur.w};
  // max |x| on the bf16 bit patterns, two at a time (for finite values the order of magnitudes is the
  // order of their bits); a NaN shows up as a maximum above the infinity pattern
  uint32_t m2 = __vmaxu2(__vmaxu2(w[0] & 0x7fff7fffu, w[1] & 0x7fff7fffu), __vmaxu2(w[2] & 0x7fff7fffu, w[3] & 0x7fff7fffu));
  const uint32_t mx = __reduce_max_sync(0xffffffffu, max(m2 & 0xffffu, m2 >> 16));
  float x[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
  uint32_t b[8];
  float scale;
  bool redo = !(mx >= 0x0100u && mx <= 0x7e00u);                    // warp-uniform: amax finite, in [2^-124, 2^125), no NaN
  if (!redo) {
    // amax / 127, correctly rounded, from the rounded reciprocal and two FMAs (127 is far from an
    // all-ones significand and the quotient is a normal number here, so the correction is exact)
    const float amax = __uint_as_float(mx << 16);
    constexpr float kR127 = 0x1.020408p-7f;                         // RN(1 / 127)
    const float s0 = __fmul_rn(amax, kR127);
    scale = fmaf(fmaf(-s0, 127.0f, amax), kR127, s0);
    // Round to nearest even by adding 1.5 * 2^23 (no conversion instructions: they run at a fraction
    // of the FP32 rate): |q| <= 127 (1 + 2^-23) because |x| <= amax, so the sum's low mantissa bits
    // are the integer in two's complement and its low byte is the code, already within +-127.
    const float rcp = __frcp_rn(scale);
    constexpr float kMagic = 12582912.0f;
    float worst = 0.f;                                              // largest distance of a product from its integer
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float q = __fmul_rn(x[i], rcp);
      const float t = __fadd_rn(q, kMagic);
      b[i] = __float_as_uint(t);
      worst = fmaxf(worst, fabsf(__fsub_rn(q, __fsub_rn(t, kMagic))));
    }
    redo = worst > 0.5f - 0x1p-14f;                                 // some product too close to a tie: this lane's eight again, exactly
    if (redo) {
#pragma unroll
      for (int i = 0; i < 8; ++i) b[i] = static_cast<uint32_t>(quantize_s8(x[i], scale));
    }
  } else {
    // zero, tiny, huge, infinite or NaN-bearing vectors: the reference's own arithmetic
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    scale = __fdiv_rn(amax, 127.0f);
#pragma unroll
    for (int i = 0; i < 8; ++i) b[i] = static_cast<uint32_t>(quantize_s8(x[i], scale));
  }
  if (lane == 0) *meta_slot = scale;
  const uint32_t lo = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
  const uint32_t hi = __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410);
  *reinterpret_cast<uint2 *>(dst + lane * 8u) = make_uint2(lo, hi);
}

// The grid holds an even number of warps, so a warp stays with K or with V for its whole walk and
// its source, destination and scale pointers advance by constants.
__global__ void __launch_bounds__(kThreads)
kv_encode_rows256_kernel(const __nv_bfloat16 *__restrict__ k, const __nv_bfloat16 *__restrict__ v,
                         int8_t *__restrict__ kq, int8_t *__restrict__ vq, float *__restrict__ meta, size_t position,
                         size_t vecs, size_t kv_heads) {
  constexpr size_t D = 256;
  const unsigned lane = threadIdx.x & 31u;
  const size_t step = static_cast<size_t>(gridDim.x) * kWarps;     // even
  size_t vec = static_cast<size_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  const size_t which = vec & 1, th0 = vec >> 1, th_step = step >> 1;
  const uint4 *src = reinterpret_cast<const uint4 *>((which ? v : k) + th0 * D) + lane;
  int8_t *dst = (which ? vq : kq) + (position * kv_heads + th0) * D;
  float *slot = meta + (position * kv_heads + th0) * 2 + which;
  const size_t src_step = th_step * (D / 8);                        // in 16-byte units
  // two vectors per turn, the next two already requested: two 16-byte loads per lane always in flight
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 n0 = vec < vecs ? __ldcs(src) : zero, n1 = vec + step < vecs ? __ldcs(src + src_step) : zero;
  for (; vec < vecs; vec += 2 * step) {
    const uint4 c0 = n0, c1 = n1;
    src += 2 * src_step;
    n0 = vec + 2 * step < vecs ? __ldcs(src) : zero;
    n1 = vec + 3 * step < vecs ? __ldcs(src + src_step) : zero;
    kv_encode_vector256(c0, lane, dst, slot);
    if (vec + step < vecs) kv_encode_vector256(c1, lane, dst + th_step * D, slot + th_step * 2);
    dst += 2 * th_step * D;
    slot += 4 * th_step;
  }
}

// --------------------------------------------------------------- attention

// 4 signed bytes -> 4 floats without integer-to-float conversions: flip the
// sign bit (value + 128 as unsigned), splice each byte under the exponent of
// 2^23 with a byte permute, subtract 2^23 + 128.
__device__ __forceinline__ void s8x4_to_f32(uint32_t w, float (&f)[4]) {
  const uint32_t u = w ^ 0x80808080u;
  f[0] = __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7440)) - 8388736.0f;
  f[1] = __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7441)) - 8388736.0f;
  f[2] = __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7442)) - 8388736.0f;
  f[3] = __uint_as_float(__byte_perm(u, 0x4b000000u, 0x7443)) - 8388736.0f;
}

// G = q heads per kv head handled together, DPL = dims per lane
// (head_dim = 32 * DPL exactly when VEC, else head_dim <= 32 * DPL).
// Grid (kv head groups, n_splits).  Partials: part_o [q_heads, n_splits, D],
// part_m / part_l [q_heads, n_splits].
template <int G, int DPL, bool VEC>
__global__ void __launch_bounds__(kThreads)
kv_attention_split_kernel(const __nv_bfloat16 *__restrict__ q, const int8_t *__restrict__ kq,
                          const int8_t *__restrict__ vq, const float *__restrict__ meta,
                          float *__restrict__ part_o, float *__restrict__ part_m, float *__restrict__ part_l,
                          size_t t_begin, size_t t_end, uint32_t kv_heads, uint32_t q_per_kv,
                          uint32_t head_dim, uint32_t n_splits) {
  __shared__ float s_m[kWarps][G], s_l[kWarps][G];
  __shared__ float s_o[G][32 * DPL];

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t head0 = blockIdx.x * G;                 // first q head of this CTA
  const uint32_t kvh = head0 / q_per_kv;
  const uint32_t split = blockIdx.y;
  const size_t total = t_end - t_begin;
  const size_t per_split = q36::div_ceil(total, n_splits);
  const size_t s_begin = t_begin + min(total, per_split * split);
  const size_t s_end = t_begin + min(total, per_split * (split + 1));
  const float sm_scale = rsqrtf(static_cast<float>(head_dim)) * 1.4426950408889634f;   // * log2(e)

  float qv[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const uint32_t d = lane * DPL + i;
      qv[g][i] = d < head_dim ? __bfloat162float(q[static_cast<size_t>(head0 + g) * head_dim + d]) : 0.f;
    }

  float m[G], l[G], o[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[g][i] = 0.f;
  }

  for (size_t t = s_begin + warp; t < s_end; t += kWarps) {
    const size_t row = t * kv_heads + kvh;
    const float2 sc = __ldg(reinterpret_cast<const float2 *>(meta) + row);
    float kf[DPL], vf[DPL];
    if constexpr (VEC && DPL == 8) {
      const uint2 kw = __ldcs(reinterpret_cast<const uint2 *>(kq + row * head_dim) + lane);
      const uint2 vw = __ldcs(reinterpret_cast<const uint2 *>(vq + row * head_dim) + lane);
      float t4[4];
      s8x4_to_f32(kw.x, t4); kf[0] = t4[0]; kf[1] = t4[1]; kf[2] = t4[2]; kf[3] = t4[3];
      s8x4_to_f32(kw.y, t4); kf[4] = t4[0]; kf[5] = t4[1]; kf[6] = t4[2]; kf[7] = t4[3];
      s8x4_to_f32(vw.x, t4); vf[0] = t4[0]; vf[1] = t4[1]; vf[2] = t4[2]; vf[3] = t4[3];
      s8x4_to_f32(vw.y, t4); vf[4] = t4[0]; vf[5] = t4[1]; vf[6] = t4[2]; vf[7] = t4[3];
    } else if constexpr (VEC && DPL == 4) {
      float t4[4];
      s8x4_to_f32(__ldcs(reinterpret_cast<const uint32_t *>(kq + row * head_dim) + lane), t4);
      kf[0] = t4[0]; kf[1] = t4[1]; kf[2] = t4[2]; kf[3] = t4[3];
      s8x4_to_f32(__ldcs(reinterpret_cast<const uint32_t *>(vq + row * head_dim) + lane), t4);
      vf[0] = t4[0]; vf[1] = t4[1]; vf[2] = t4[2]; vf[3] = t4[3];
    } else {
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const uint32_t d = lane * DPL + i;
        kf[i] = d < head_dim ? static_cast<float>(kq[row * head_dim + d]) : 0.f;
        vf[i] = d < head_dim ? static_cast<float>(vq[row * head_dim + d]) : 0.f;
      }
    }
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float a = 0.f;
#pragma unroll
      for (int i = 0; i < DPL; ++i) a = fmaf(qv[g][i], kf[i], a);
      s[g] = a;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], off);
    const float kscale = sc.x * sm_scale;     // score in log2 units
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float sg = s[g] * kscale;
      if (sg > m[g]) {                         // warp-uniform: every lane holds the same score
        const float corr = exp2f(m[g] - sg);   // 0 on the first token (m = -inf)
        l[g] *= corr;
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[g][i] *= corr;
        m[g] = sg;
      }
      const float p = exp2f(sg - m[g]);
      l[g] += p;
      const float pv = p * sc.y;
#pragma unroll
      for (int i = 0; i < DPL; ++i) o[g][i] = fmaf(pv, vf[i], o[g][i]);
    }
  }

  // Merge the warps of the CTA: bring every warp to the common maximum, then
  // add the warps' accumulators into shared memory one warp per round (a
  // fixed order, so results do not depend on scheduling).
  if (lane == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
  }
  __syncthreads();
  float wgt[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float M = -INFINITY;
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w][g]);
    wgt[g] = m[g] == -INFINITY ? 0.f : exp2f(m[g] - M);
  }
  for (int w = 0; w < kWarps; ++w) {
    if (warp == w) {
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          float *dst = &s_o[g][lane * DPL + i];
          *dst = w == 0 ? wgt[g] * o[g][i] : fmaf(wgt[g], o[g][i], *dst);
        }
    }
    __syncthreads();
  }
  for (uint32_t idx = threadIdx.x; idx < G * head_dim; idx += kThreads) {
    const uint32_t g = idx / head_dim, d = idx % head_dim;
    const size_t slot = static_cast<size_t>(head0 + g) * n_splits + split;
    part_o[slot * head_dim + d] = s_o[g][d];
    if (d == 0) {
      float M = -INFINITY, den = 0.f;
      for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w][g]);
      for (int w = 0; w < kWarps; ++w)
        den = fmaf(s_m[w][g] == -INFINITY ? 0.f : exp2f(s_m[w][g] - M), s_l[w][g], den);
      part_m[slot] = M * 0.6931471805599453f;      // back to natural-log units
      part_l[slot] = den;
    }
  }
}

// Fast path for head_dim 256: same grid and outputs as kv_attention_split_kernel, but a warp
// handles FOUR consecutive tokens per iteration.  All loads of the next four tokens are issued
// before the current four are consumed (register prefetch).  The 4 x G partial scores of a lane
// are summed across the warp with a transpose-reduce (31 shuffles for up to 32 values, after which
// lane 8 t + h holds the score of token t, head h) instead of one 5-step butterfly per score; the
// online softmax runs once per four tokens, with the per-head state living on lane h.
template <int G>
__global__ void __launch_bounds__(kThreads)
kv_attention_fast_kernel(const __nv_bfloat16 *__restrict__ q, const int8_t *__restrict__ kq,
                         const int8_t *__restrict__ vq, const float *__restrict__ meta,
                         float *__restrict__ part_o, float *__restrict__ part_m, float *__restrict__ part_l,
                         size_t t_begin, size_t t_end, uint32_t kv_heads, uint32_t q_per_kv, uint32_t n_splits) {
  constexpr uint32_t D = 256;
  __shared__ float s_m[kWarps][8], s_l[kWarps][8];
  __shared__ float s_o[G][D];

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t head0 = blockIdx.x * G;
  const uint32_t kvh = head0 / q_per_kv;
  const uint32_t split = blockIdx.y;
  const size_t total = t_end - t_begin;
  const size_t per_split = q36::div_ceil(total, n_splits);
  const size_t s_begin = t_begin + min(total, per_split * split);
  const size_t s_end = t_begin + min(total, per_split * (split + 1));
  const float sm_scale = 0.0625f * 1.4426950408889634f;        // rsqrt(256) * log2(e)

  float qv[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint4 p = __ldg(reinterpret_cast<const uint4 *>(q + static_cast<size_t>(head0 + g) * D) + lane);
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      qv[g][2 * i] = __uint_as_float(w[i] << 16);
      qv[g][2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  float o[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i) o[g][i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;          // state of head (lane & 7), identical on its 4 lanes

  struct Batch { uint2 k[4], v[4]; float2 sc[4]; };
  auto load = [&](Batch &b, size_t t0) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const size_t tok = t0 + t;
      if (tok < s_end) {
        const size_t row = tok * kv_heads + kvh;
        b.k[t] = __ldcs(reinterpret_cast<const uint2 *>(kq + row * D) + lane);
        b.v[t] = __ldcs(reinterpret_cast<const uint2 *>(vq + row * D) + lane);
        b.sc[t] = __ldg(reinterpret_cast<const float2 *>(meta) + row);
      } else {
        b.k[t] = make_uint2(0x0, 0x0); b.v[t] = make_uint2(0, 0); b.sc[t] = make_float2(0.f, 0.f);
      }
    }
  };

  const size_t stride = static_cast<size_t>(kWarps) * 4;
  Batch cur, nxt;
  size_t t0 = s_begin + static_cast<size_t>(warp) * 4;
  if (t0 < s_end) load(cur, t0);
  for (; t0 < s_end; t0 += stride) {
    if (t0 + stride < s_end) load(nxt, t0 + stride);
    // ---- partial scores: v[8 t + g] = sum over this lane's 8 dims of q[g] * k[t]
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = 0.f;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float kf[8], t4[4];
      s8x4_to_f32(cur.k[t].x, t4); kf[0] = t4[0]; kf[1] = t4[1]; kf[2] = t4[2]; kf[3] = t4[3];
      s8x4_to_f32(cur.k[t].y, t4); kf[4] = t4[0]; kf[5] = t4[1]; kf[6] = t4[2]; kf[7] = t4[3];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) a = fmaf(qv[g][i], kf[i], a);
        v[8 * t + g] = a;
      }
    }
    // ---- transpose-reduce: afterwards v[0] on lane L is the warp total of value index L
#pragma unroll
    for (int width = 16; width >= 1; width >>= 1) {
      const bool upper = (lane & width) != 0;
#pragma unroll
      for (int i = 0; i < width; ++i) {
        const float send = upper ? v[i] : v[i + width];
        const float keep = upper ? v[i + width] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, width);
      }
    }
    // ---- online softmax for (token = lane >> 3, head = lane & 7)
    const uint32_t tl = lane >> 3;
    const bool valid = (lane & 7u) < G && t0 + tl < s_end;
    const float kscale = tl == 0 ? cur.sc[0].x : tl == 1 ? cur.sc[1].x : tl == 2 ? cur.sc[2].x : cur.sc[3].x;
    const float s_log2 = valid ? v[0] * kscale * sm_scale : -INFINITY;
    float tile_max = fmaxf(s_log2, __shfl_xor_sync(0xffffffffu, s_log2, 8));
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 16));
    const float m_new = fmaxf(m_run, tile_max);
    const float corr = m_new == -INFINITY ? 1.f : exp2f(m_run - m_new);      // exp2(-inf) = 0 on first use
    const float p = valid ? exp2f(s_log2 - m_new) : 0.f;
    float p_sum = p + __shfl_xor_sync(0xffffffffu, p, 8);
    p_sum += __shfl_xor_sync(0xffffffffu, p_sum, 16);
    l_run = l_run * corr + p_sum;
    m_run = m_new;
    // ---- P V: every lane needs corr[g] and p[t][g]
    float vf[4][8];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float t4[4];
      s8x4_to_f32(cur.v[t].x, t4); vf[t][0] = t4[0]; vf[t][1] = t4[1]; vf[t][2] = t4[2]; vf[t][3] = t4[3];
      s8x4_to_f32(cur.v[t].y, t4); vf[t][4] = t4[0]; vf[t][5] = t4[1]; vf[t][6] = t4[2]; vf[t][7] = t4[3];
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float cg = __shfl_sync(0xffffffffu, corr, g);
      if (cg != 1.f) {                      // warp-uniform
#pragma unroll
        for (int i = 0; i < 8; ++i) o[g][i] *= cg;
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float pv = __shfl_sync(0xffffffffu, p, 8 * t + g) * cur.sc[t].y;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[g][i] = fmaf(pv, vf[t][i], o[g][i]);
      }
    }
    cur = nxt;
  }

  // ---- merge the warps of the CTA (same scheme as the general kernel)
  if (lane < G) { s_m[warp][lane] = m_run; s_l[warp][lane] = l_run; }
  __syncthreads();
  float wgt[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float M = -INFINITY;
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w][g]);
    const float mine = s_m[warp][g];
    wgt[g] = mine == -INFINITY ? 0.f : exp2f(mine - M);
  }
  for (int w = 0; w < kWarps; ++w) {
    if (warp == w) {
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float *dst = &s_o[g][lane * 8 + i];
          *dst = w == 0 ? wgt[g] * o[g][i] : fmaf(wgt[g], o[g][i], *dst);
        }
    }
    __syncthreads();
  }
  for (uint32_t idx = threadIdx.x; idx < G * D; idx += kThreads) {
    const uint32_t g = idx / D, d = idx % D;
    const size_t slot = static_cast<size_t>(head0 + g) * n_splits + split;
    part_o[slot * D + d] = s_o[g][d];
    if (d == 0) {
      float M = -INFINITY, den = 0.f;
      for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w][g]);
      for (int w = 0; w < kWarps; ++w)
        den = fmaf(s_m[w][g] == -INFINITY ? 0.f : exp2f(s_m[w][g] - M), s_l[w][g], den);
      part_m[slot] = M * 0.6931471805599453f;
      part_l[slot] = den;
    }
  }
}

// Merge n_parts partials per q head.  FINAL: write bf16 output (sum w*o /
// sum w*l, 0 when the denominator is 0).  !FINAL: write one combined partial.
template <bool FINAL>
__global__ void __launch_bounds__(kThreads)
kv_merge_kernel(const float *__restrict__ part_o, const float *__restrict__ part_m,
                const float *__restrict__ part_l, uint32_t n_parts, uint32_t head_dim,
                __nv_bfloat16 *__restrict__ out, float *__restrict__ out_o, float *__restrict__ out_m,
                float *__restrict__ out_l) {
  __shared__ float s_w[kThreads];        // weight of every part (n_parts <= kThreads)
  __shared__ float s_red[kWarps];
  const size_t qh = blockIdx.x;
  const float *pm = part_m + qh * n_parts, *pl = part_l + qh * n_parts;
  const float *po = part_o + qh * n_parts * head_dim;
  // launched with programmatic stream serialisation after the split kernel: the CTAs are resident
  // by the time the partials are complete (a no-op after an ordinary launch)
  Q36_ATRACE(1000u + blockIdx.x, 0);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  Q36_ATRACE(1000u + blockIdx.x, 1);
  // the outputs of the first 48 parts (one CTA per SM and kv head gives 37) travel with the (m, l)
  // pairs: one round trip to L2 for the whole merge
  float first[48];
  if (threadIdx.x < head_dim) q36::lse_prefetch(po, n_parts, head_dim, threadIdx.x, first);
  float M, den;
  q36::lse_weights(pm, pl, n_parts, s_w, s_red, M, den);
  Q36_ATRACE(1000u + blockIdx.x, 2);
  for (uint32_t d = threadIdx.x; d < head_dim; d += kThreads) {
    const float acc = d == threadIdx.x ? q36::lse_accumulate(po, s_w, n_parts, head_dim, d, first)
                                       : q36::lse_accumulate(po, s_w, n_parts, head_dim, d);
    if (FINAL) out[qh * head_dim + d] = __float2bfloat16(den > 0.f ? __fdiv_rn(acc, den) : 0.f);
    else out_o[qh * head_dim + d] = acc;
  }
  if (!FINAL && threadIdx.x == 0) { out_m[qh] = M; out_l[qh] = den; }
  Q36_ATRACE(1000u + blockIdx.x, 3);
}

template <bool FINAL>
int launch_merge_after_splits(unsigned q_heads, const float *o, const float *m, const float *l, uint32_t n_parts,
                              uint32_t head_dim, __nv_bfloat16 *out, float *out_o, float *out_m, float *out_l) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(q_heads);
  cfg.blockDim = dim3(kThreads);
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return q36::cuda_status(cudaLaunchKernelEx(&cfg, kv_merge_kernel<FINAL>, o, m, l, n_parts, head_dim, out, out_o,
                                             out_m, out_l));
}

struct Scratch { float *o, *m, *l; };
std::atomic<int> g_use_fast_attention{3};            // 3 tensor-core form fed through shared memory, 2 tensor-core form fed from registers, 1 SIMT fast path, 0 general kernel

// Scratch for qwen36_turboquant_attention_static: lives in the library image, so every GPU that
// loads the library holds these 4 MiB until the process exits.  Sized for
// q_heads * (head_dim + 2) <= kStaticHeadFloats (e.g. 32 heads of 256 dims).
constexpr size_t kStaticHeadFloats = 32 * (256 + 2);
constexpr size_t kStaticScratchFloats = kMaxSplits * kStaticHeadFloats;
static __device__ __align__(256) float g_static_attention_scratch[kStaticScratchFloats];

size_t scratch_bytes(size_t q_heads, size_t head_dim) {
  return q_heads * kMaxSplits * (head_dim + 2) * sizeof(float);
}

Scratch carve(float *base, size_t q_heads, size_t head_dim) {
  return {base, base + q_heads * kMaxSplits * head_dim, base + q_heads * kMaxSplits * (head_dim + 1)};
}

std::atomic<int> g_force_splits{0};                  // test hook: > 0 overrides the split count

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    cached[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
  }
  return cached[dev];
}

// one_wave: the kernel runs one CTA per SM (the tensor-core form: a CTA's start-up and merge cost
// about as much as 1500 tokens, and nothing overlaps them), so the grid is one CTA per SM or less.
uint32_t pick_splits(size_t tokens, size_t ctas_per_split, bool one_wave) {
  if (g_force_splits > 0) { const int f = g_force_splits.load(); return static_cast<uint32_t>(f > static_cast<int>(kMaxSplits) ? static_cast<int>(kMaxSplits) : f); }
  // otherwise fill ~2 CTAs per SM; at least kMinTokensPerSplit tokens each
  const size_t sms = static_cast<size_t>(sm_count());
  size_t want = one_wave ? sms / ctas_per_split : q36::div_ceil(2 * sms, ctas_per_split);
  size_t cap = q36::div_ceil(tokens, kMinTokensPerSplit);
  size_t n = want < cap ? want : cap;
  if (n < 1) n = 1;
  if (n > kMaxSplits) n = kMaxSplits;
  return static_cast<uint32_t>(n);
}

// ---- tensor-core form (head_dim 256, up to 8 q heads per kv head) ---------------------------
//
// The SIMT kernels above convert and multiply every int8 element once per q head and end up
// issue-bound long before HBM is.  Here both products run on the tensor cores as
// mma.sync.m16n8k16 with float16 operands and float32 accumulation; int8 -> float16 is exact
// (0x6400 | (byte ^ 0x80) is 1024 + 128 + value; one packed subtraction removes the bias), q is
// rounded to float16, probabilities to float16 after scaling by v_scale * 1024.
//
// A warp owns 16 tokens at a time (two blocks of eight).  Lane (g = lane / 4, t = lane % 4):
//   S = Q K^T : A = Q (row g = q head g, rows >= G are zero), B = K^T with token g of the block as
//       its column; the contraction index is permuted so that a lane's operands are the sixteen
//       consecutive bytes it loads: step 4 j + i covers dims 64 j + 16 t + 4 i .. + 3.
//       The accumulator leaves lane (g, t) with head g's scores of tokens 2t, 2t + 1 of the block.
//   O^T = V^T P^T : those four scores (two blocks) are exactly the B fragment of the second
//       product (column = head g, contraction slots 2t, 2t+1, 2t+8, 2t+9 = this lane's tokens),
//       so probabilities never leave their registers.  A = V^T: a lane loads sixteen dims
//       (16 (g + 8 h) ..) of its four tokens and pairs bytes of neighbouring tokens; mma (h, j)
//       has dim 16 (g + 8 h) + 2 j in row g and the next dim in row g + 8.  Its accumulator holds
//       heads 2t, 2t + 1 of those two dims.
using q36::mma_f16;
// (lo byte of x, lo byte of y) as int8 -> float16x2; x and y already XORed with 0x80 per byte.
template <int BYTE>
__device__ __forceinline__ uint32_t s8pair_to_h2(uint32_t x, uint32_t y) {
  const uint32_t sel = BYTE | ((4 + BYTE) << 4);                  // byte0 = x.b[BYTE], byte1 = y.b[BYTE]
  const uint32_t two = __byte_perm(x, y, sel);                    // bytes: x.b, y.b, -, -
  const uint32_t spread = __byte_perm(two, 0x64646464u, 0x5140);   // x.b, 0x64, y.b, 0x64
  const __half2 biased = *reinterpret_cast<const __half2 *>(&spread);
  const __half2 r = __hsub2(biased, __half2half2(__ushort_as_half(0x6480)));   // - (1024 + 128)
  return *reinterpret_cast<const uint32_t *>(&r);
}
// bytes (2 * PAIR, 2 * PAIR + 1) of one word as int8 -> float16x2 of (value + 1152): the bias is
// taken out of the finished dot product instead (1152 * sum of the other operand), which saves a
// packed subtraction per pair
template <int PAIR>
__device__ __forceinline__ uint32_t s8x2_to_h2_biased(uint32_t x) {
  return __byte_perm(x, 0x64646464u, PAIR == 0 ? 0x5140 : 0x7362);
}

template <int G>
__global__ void __launch_bounds__(kThreads, 1)
kv_attention_mma_kernel(const __nv_bfloat16 *__restrict__ q, const int8_t *__restrict__ kq,
                        const int8_t *__restrict__ vq, const float *__restrict__ meta,
                        float *__restrict__ part_o, float *__restrict__ part_m, float *__restrict__ part_l,
                        size_t t_begin, size_t t_end, uint32_t kv_heads, uint32_t q_per_kv, uint32_t n_splits) {
  constexpr uint32_t D = 256;
  constexpr float kPScale = 1024.0f;                              // keeps p * v_scale out of the float16 subnormals
  __shared__ float s_m[kWarps][8], s_l[kWarps][8];
  __shared__ __align__(16) float s_o[4 * G][q36::kEpiStride];

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  const uint32_t head0 = blockIdx.x * G;
  const uint32_t kvh = head0 / q_per_kv;
  const uint32_t split = blockIdx.y;
  const size_t total = t_end - t_begin;
  // whole rounds of 8 warps x 16 tokens per split, so that every warp runs the same number of groups
  const size_t per_split = q36::round_up(q36::div_ceil(total, n_splits), static_cast<size_t>(kWarps) * 16);
  const size_t s_begin = t_begin + min(total, per_split * split);
  const size_t s_end = t_begin + min(total, per_split * (split + 1));
  const float sm_scale = 0.0625f * 1.4426950408889634f;           // rsqrt(256) * log2(e)

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the merge may take its seats early

  __shared__ uint2 s_q[16][32];
  float q_bias = 0.f;
  float o[2][8][4];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[h][j][c] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;                           // head g, identical on its four lanes

  // tokens of lane t inside a 16-token group: 2t, 2t + 1, 8 + 2t, 9 + 2t
  struct KBuf { uint4 k[2][4]; };
  struct VBuf { uint4 v[4][2]; float2 sc[4]; };
  auto load_k = [&](KBuf &b, size_t t0) {
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const size_t tok = t0 + 8 * blk + g;
      if (tok < s_end) {
        const uint4 *src = reinterpret_cast<const uint4 *>(kq + (tok * kv_heads + kvh) * D) + t;
#pragma unroll
        for (int j = 0; j < 4; ++j) b.k[blk][j] = __ldcs(src + 4 * j);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) b.k[blk][j] = make_uint4(0, 0, 0, 0);
      }
    }
  };
  auto load_v = [&](VBuf &b, size_t t0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const size_t tok = t0 + 2 * t + (i & 1) + 8 * (i >> 1);
      if (tok < s_end) {
        const size_t row = tok * kv_heads + kvh;
        const uint4 *src = reinterpret_cast<const uint4 *>(vq + row * D) + g;
        b.v[i][0] = __ldcs(src);
        b.v[i][1] = __ldcs(src + 8);
        b.sc[i] = __ldg(reinterpret_cast<const float2 *>(meta) + row);
      } else {
        b.v[i][0] = b.v[i][1] = make_uint4(0, 0, 0, 0);
        b.sc[i] = make_float2(0.f, 0.f);
      }
    }
  };
  // S = Q K^T for the two 8-token blocks of a group: four independent accumulator chains (two
  // blocks x even / odd steps); out = this lane's scores of tokens 2t, 2t+1, 8+2t, 9+2t
  auto scores = [&](const KBuf &b, float (&out)[4]) {
    float acc[2][2][4];
#pragma unroll
    for (int blk = 0; blk < 2; ++blk)
#pragma unroll
      for (int par = 0; par < 2; ++par)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[blk][par][c] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t w[2][4];
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        w[blk][0] = b.k[blk][j].x ^ 0x80808080u; w[blk][1] = b.k[blk][j].y ^ 0x80808080u;
        w[blk][2] = b.k[blk][j].z ^ 0x80808080u; w[blk][3] = b.k[blk][j].w ^ 0x80808080u;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint2 qf = s_q[4 * j + i][lane];
#pragma unroll
        for (int blk = 0; blk < 2; ++blk)
          mma_f16(acc[blk][i & 1], qf.x, 0u, qf.y, 0u, s8x2_to_h2_biased<0>(w[blk][i]), s8x2_to_h2_biased<1>(w[blk][i]));
      }
    }
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      out[2 * blk] = (acc[blk][0][0] + acc[blk][1][0]) - q_bias;
      out[2 * blk + 1] = (acc[blk][0][1] + acc[blk][1][1]) - q_bias;
    }
  };

  // Software pipeline over this warp's groups: while the probabilities of group n multiply V, the
  // scores of group n + 1 are already being formed (independent tensor-core work), K of group
  // n + 2 and V of group n + 1 are in flight.
  const size_t stride = static_cast<size_t>(kWarps) * 16;
  KBuf k_now, k_next;               // K of group n + 1 (scored during iteration n), K of group n + 2
  VBuf v_now, v_next;               // V and scales of group n, of group n + 1
  float sc_[4] = {0.f, 0.f, 0.f, 0.f}, sc_next[4];
  size_t t0 = s_begin + static_cast<size_t>(warp) * 16;
  if (t0 < s_end) {                                  // first loads fly while q is staged
    load_k(k_next, t0);
    load_v(v_now, t0);
    load_k(k_now, t0 + stride);                      // past-the-end groups load zeros
  }

  // Q fragments (the same for every warp, so they live in shared memory): step s = 4 j + i covers
  // dims 64 j + 16 t + 4 i .. + 3 of head g
  if (warp == 0) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 raw0 = make_uint4(0, 0, 0, 0), raw1 = make_uint4(0, 0, 0, 0);
    if (g < G) {
      const uint4 *src = reinterpret_cast<const uint4 *>(q + static_cast<size_t>(head0 + g) * D + 64 * j + 16 * t);
      raw0 = __ldg(src);
      raw1 = __ldg(src + 1);
    }
    const uint32_t w[8] = {raw0.x, raw0.y, raw0.z, raw0.w, raw1.x, raw1.y, raw1.z, raw1.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t pair = w[2 * i + half];                    // two bf16: dims 4 i + 2 half, + 1
        const __half2 h = __floats2half2_rn(__uint_as_float(pair << 16), __uint_as_float(pair & 0xffff0000u));
        reinterpret_cast<uint32_t *>(&s_q[4 * j + i][lane])[half] = *reinterpret_cast<const uint32_t *>(&h);
      }
    }
  }
  }
  __syncthreads();

  // 1152 * (sum of head g's float16 q): the K operand carries that bias on every element
#pragma unroll
  for (int s16 = 0; s16 < 16; ++s16) {
    const uint2 qf = s_q[s16][lane];
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&qf.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&qf.y));
    q_bias += (a.x + a.y) + (b.x + b.y);
  }
  q_bias += __shfl_xor_sync(0xffffffffu, q_bias, 1);
  q_bias += __shfl_xor_sync(0xffffffffu, q_bias, 2);
  q_bias *= 1152.0f;

  if (t0 < s_end) scores(k_next, sc_);
  for (; t0 < s_end; t0 += stride) {
    load_k(k_next, t0 + 2 * stride);
    load_v(v_next, t0 + stride);
    // ---- online softmax, head g: this lane's four tokens, then the four lanes of the head
    float s_log2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const size_t tok = t0 + 2 * t + (i & 1) + 8 * (i >> 1);
      s_log2[i] = (g < G && tok < s_end) ? sc_[i] * v_now.sc[i].x * sm_scale : -INFINITY;
    }
    float p[4];
    const float corr = q36::online_softmax_step(s_log2, p, m_run, l_run);
    const __half2 pb0 = __floats2half2_rn(p[0] * v_now.sc[0].y * kPScale, p[1] * v_now.sc[1].y * kPScale);
    const __half2 pb1 = __floats2half2_rn(p[2] * v_now.sc[2].y * kPScale, p[3] * v_now.sc[3].y * kPScale);
    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(&pb0), b1 = *reinterpret_cast<const uint32_t *>(&pb1);
    // ---- scores of the next group (nothing below depends on them)
    scores(k_now, sc_next);
    // ---- rescale the running output: this lane's accumulators belong to heads 2t and 2t + 1
    q36::rescale_outputs(o, corr);
    // ---- O^T += V^T P^T
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t va[4] = {v_now.v[0][h].x ^ 0x80808080u, v_now.v[0][h].y ^ 0x80808080u, v_now.v[0][h].z ^ 0x80808080u, v_now.v[0][h].w ^ 0x80808080u};
      const uint32_t vb[4] = {v_now.v[1][h].x ^ 0x80808080u, v_now.v[1][h].y ^ 0x80808080u, v_now.v[1][h].z ^ 0x80808080u, v_now.v[1][h].w ^ 0x80808080u};
      const uint32_t vc[4] = {v_now.v[2][h].x ^ 0x80808080u, v_now.v[2][h].y ^ 0x80808080u, v_now.v[2][h].z ^ 0x80808080u, v_now.v[2][h].w ^ 0x80808080u};
      const uint32_t vd[4] = {v_now.v[3][h].x ^ 0x80808080u, v_now.v[3][h].y ^ 0x80808080u, v_now.v[3][h].z ^ 0x80808080u, v_now.v[3][h].w ^ 0x80808080u};
#pragma unroll
      for (int w = 0; w < 4; ++w) {                                // word w holds dims 4 w .. 4 w + 3 of the chunk
        mma_f16(o[h][2 * w], s8pair_to_h2<0>(va[w], vb[w]), s8pair_to_h2<1>(va[w], vb[w]),
                s8pair_to_h2<0>(vc[w], vd[w]), s8pair_to_h2<1>(vc[w], vd[w]), b0, b1);
        mma_f16(o[h][2 * w + 1], s8pair_to_h2<2>(va[w], vb[w]), s8pair_to_h2<3>(va[w], vb[w]),
                s8pair_to_h2<2>(vc[w], vd[w]), s8pair_to_h2<3>(vc[w], vd[w]), b0, b1);
      }
    }
    k_now = k_next;
    v_now = v_next;
#pragma unroll
    for (int i = 0; i < 4; ++i) sc_[i] = sc_next[i];
  }

  q36::split_epilogue<G>(o, m_run, l_run, 1.0f / kPScale, s_m, s_l, s_o, part_o, part_m, part_l, head0, split, n_splits);
}

// ---- tensor-core form fed through shared memory.  Same products and fragment plan as
// kv_attention_mma_kernel, but K, V and the per-token scales travel global -> shared memory with
// asynchronous copies (cp.async) into a private three-stage ring per warp, so that the bytes in
// flight (two stages = 16 KB per warp, 128 KB per SM) do not have to fit in registers.  A stage
// holds the K rows, the V rows and the (k_scale, v_scale) pairs of a 16-token group; 16-byte chunks
// are XOR-swizzled on the way in so that the fragment reads are free of bank conflicts: K chunk c
// of row r sits at c ^ 4 (r & 1), V chunk c of row r at c ^ 2 ((r / 2) & 3).  No block barrier
// inside the loop: a warp waits for its own copies (wait_group + __syncwarp).
constexpr int kStages = 3;
constexpr uint32_t kTileBytes = 16 * 256;                         // 16 tokens x 256 bytes
constexpr uint32_t kStageBytes = 2 * kTileBytes + 16 * 8;         // K tile, V tile, 16 scale pairs
constexpr uint32_t kRingBytes = kWarps * kStages * kStageBytes;   // 195 KB
constexpr uint32_t kStagedSmemBytes = kRingBytes + 16 * 32 * 8 + 2 * kWarps * 8 * 4;

template <int G>
__global__ void __launch_bounds__(kThreads, 1)
kv_attention_staged_kernel(const __nv_bfloat16 *__restrict__ q, const int8_t *__restrict__ kq,
                           const int8_t *__restrict__ vq, const float *__restrict__ meta,
                           float *__restrict__ part_o, float *__restrict__ part_m, float *__restrict__ part_l,
                           size_t t_begin, size_t t_end, uint32_t kv_heads, uint32_t q_per_kv, uint32_t n_splits) {
  constexpr uint32_t D = 256;
  constexpr float kPScale = 1024.0f;                              // keeps p * v_scale out of the float16 subnormals
  extern __shared__ __align__(128) uint8_t smem[];
  // ring | q fragments | per-warp maxima and sums; the epilogue's output slices reuse the ring
  uint2 (*s_q)[32] = reinterpret_cast<uint2 (*)[32]>(smem + kRingBytes);
  float (*s_m)[8] = reinterpret_cast<float (*)[8]>(smem + kRingBytes + 16 * 32 * 8);
  float (*s_l)[8] = s_m + kWarps;
  float (*s_o)[q36::kEpiStride] = reinterpret_cast<float (*)[q36::kEpiStride]>(smem);

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  const uint32_t head0 = blockIdx.x * G;
  const uint32_t kvh = head0 / q_per_kv;
  const uint32_t split = blockIdx.y;
  const size_t total = t_end - t_begin;
  const size_t per_split = q36::round_up(q36::div_ceil(total, n_splits), static_cast<size_t>(kWarps) * 16);
  const size_t s_begin = t_begin + min(total, per_split * split);
  const size_t s_end = t_begin + min(total, per_split * (split + 1));
  const float sm_scale = 0.0625f * 1.4426950408889634f;           // rsqrt(256) * log2(e)
  // launched with programmatic stream serialisation: seated while the previous kernel drains, but
  // nothing is read or written before that kernel (the producer of q, of the newest cache row, or
  // the reader of the partial buffers) has completed
  const uint32_t cta_flat = blockIdx.y * gridDim.x + blockIdx.x;
  (void)cta_flat;
  Q36_ATRACE(cta_flat, 0);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  Q36_ATRACE(cta_flat, 1);

  const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + warp * (kStages * kStageBytes);
  const size_t stride = static_cast<size_t>(kWarps) * 16;
  size_t t0 = s_begin + static_cast<size_t>(warp) * 16;
  // one stage: lane copies chunk (lane & 15) of rows (lane >> 4) + 2 r, r = 0 .. 7, of K and of V,
  // lanes 0 .. 15 the scale pair of row `lane`; rows past the end of the split are zero-filled
  // (source size 0, address kept inside the cache)
  const uint32_t chunk = lane & 15u, row0 = lane >> 4;
  auto issue = [&](uint32_t stage, size_t tg) {
    const uint32_t base = ring + stage * kStageBytes;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const uint32_t row = row0 + 2u * r;
      const size_t tok = tg + row;
      const bool valid = tok < s_end;
      const size_t off = ((valid ? tok : s_begin) * kv_heads + kvh) * D + chunk * 16u;
      const uint32_t bytes = valid ? 16u : 0u;
      q36::cp_async_16(base + row * 256u + ((chunk ^ ((row & 1u) << 2)) << 4), kq + off, bytes);
      q36::cp_async_16(base + kTileBytes + row * 256u + ((chunk ^ (((row >> 1) & 3u) << 1)) << 4), vq + off, bytes);
    }
    if (lane < 16u) {
      const size_t tok = tg + lane;
      const bool valid = tok < s_end;
      const float *src = meta + ((valid ? tok : s_begin) * kv_heads + kvh) * 2;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(base + 2 * kTileBytes + lane * 8u), "l"(src),
                   "r"(valid ? 8u : 0u) : "memory");
    }
    q36::cp_async_commit();
  };
  if (t0 < s_end) {
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue(s, t0 + s * stride);
  }

  // Q fragments (float16): step 4 j + i covers dims 64 j + 16 t + 4 i .. + 3 of head g
  if (warp == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 raw0 = make_uint4(0, 0, 0, 0), raw1 = make_uint4(0, 0, 0, 0);
      if (g < G) {
        const uint4 *src = reinterpret_cast<const uint4 *>(q + static_cast<size_t>(head0 + g) * D + 64 * j + 16 * t);
        raw0 = __ldg(src);
        raw1 = __ldg(src + 1);
      }
      const uint32_t w[8] = {raw0.x, raw0.y, raw0.z, raw0.w, raw1.x, raw1.y, raw1.z, raw1.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const uint32_t pair = w[2 * i + half];
          const __half2 h = __floats2half2_rn(__uint_as_float(pair << 16), __uint_as_float(pair & 0xffff0000u));
          reinterpret_cast<uint32_t *>(&s_q[4 * j + i][lane])[half] = *reinterpret_cast<const uint32_t *>(&h);
        }
      }
    }
  }
  __syncthreads();
  Q36_ATRACE(cta_flat, 2);
  // 1152 * (sum of head g's float16 q): the K operand carries that bias on every element
  float q_bias = 0.f;
#pragma unroll
  for (int s16 = 0; s16 < 16; ++s16) {
    const uint2 qf = s_q[s16][lane];
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&qf.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&qf.y));
    q_bias += (a.x + a.y) + (b.x + b.y);
  }
  q_bias += __shfl_xor_sync(0xffffffffu, q_bias, 1);
  q_bias += __shfl_xor_sync(0xffffffffu, q_bias, 2);
  q_bias *= 1152.0f;

  float o[2][8][4];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[h][j][c] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  uint32_t stage = 0;
  for (; t0 < s_end; t0 += stride) {
    issue(stage == 0 ? kStages - 1 : stage - 1, t0 + (kStages - 1) * stride);   // refill the stage read last time
    q36::cp_async_wait<kStages - 1>();
    if (t0 == s_begin) Q36_ATRACE(cta_flat, 3);
    __syncwarp();
    const uint32_t kt = ring + stage * kStageBytes, vt = kt + kTileBytes, mt = vt + kTileBytes;
    // ---- S = Q K^T: four independent accumulator chains (two blocks x even / odd steps)
    float sc_[4];
    {
      float acc[2][2][4];
#pragma unroll
      for (int blk = 0; blk < 2; ++blk)
#pragma unroll
        for (int par = 0; par < 2; ++par)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[blk][par][c] = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w[2][4];
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          const uint4 kw = q36::lds128(kt + (8u * blk + g) * 256u + (((t + 4u * j) ^ ((g & 1u) << 2)) << 4));
          w[blk][0] = kw.x ^ 0x80808080u; w[blk][1] = kw.y ^ 0x80808080u;
          w[blk][2] = kw.z ^ 0x80808080u; w[blk][3] = kw.w ^ 0x80808080u;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint2 qf = s_q[4 * j + i][lane];
#pragma unroll
          for (int blk = 0; blk < 2; ++blk)
            mma_f16(acc[blk][i & 1], qf.x, 0u, qf.y, 0u, s8x2_to_h2_biased<0>(w[blk][i]), s8x2_to_h2_biased<1>(w[blk][i]));
        }
      }
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        sc_[2 * blk] = (acc[blk][0][0] + acc[blk][1][0]) - q_bias;
        sc_[2 * blk + 1] = (acc[blk][0][1] + acc[blk][1][1]) - q_bias;
      }
    }
    // ---- online softmax, head g: this lane's four tokens, then the four lanes of the head
    float2 scl[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t row = 2u * t + (i & 1) + 8u * (i >> 1);
      asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(scl[i].x), "=f"(scl[i].y) : "r"(mt + row * 8u));
    }
    float s_log2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const size_t tok = t0 + 2 * t + (i & 1) + 8 * (i >> 1);
      s_log2[i] = (g < G && tok < s_end) ? sc_[i] * scl[i].x * sm_scale : -INFINITY;
    }
    float p[4];
    const float corr = q36::online_softmax_step(s_log2, p, m_run, l_run);
    const __half2 pb0 = __floats2half2_rn(p[0] * scl[0].y * kPScale, p[1] * scl[1].y * kPScale);
    const __half2 pb1 = __floats2half2_rn(p[2] * scl[2].y * kPScale, p[3] * scl[3].y * kPScale);
    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(&pb0), b1 = *reinterpret_cast<const uint32_t *>(&pb1);
    // ---- rescale the running output: this lane's accumulators belong to heads 2t and 2t + 1
    q36::rescale_outputs(o, corr);
    // ---- O^T += V^T P^T: rows 2t, 2t + 1, 2t + 8, 2t + 9 of the V tile, chunk g + 8 h
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint4 x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        x[i] = q36::lds128(vt + (2u * t + (i & 1) + 8u * (i >> 1)) * 256u + (((g + 8u * h) ^ (t << 1)) << 4));
      const uint32_t va[4] = {x[0].x ^ 0x80808080u, x[0].y ^ 0x80808080u, x[0].z ^ 0x80808080u, x[0].w ^ 0x80808080u};
      const uint32_t vb[4] = {x[1].x ^ 0x80808080u, x[1].y ^ 0x80808080u, x[1].z ^ 0x80808080u, x[1].w ^ 0x80808080u};
      const uint32_t vc[4] = {x[2].x ^ 0x80808080u, x[2].y ^ 0x80808080u, x[2].z ^ 0x80808080u, x[2].w ^ 0x80808080u};
      const uint32_t vd[4] = {x[3].x ^ 0x80808080u, x[3].y ^ 0x80808080u, x[3].z ^ 0x80808080u, x[3].w ^ 0x80808080u};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        mma_f16(o[h][2 * w], s8pair_to_h2<0>(va[w], vb[w]), s8pair_to_h2<1>(va[w], vb[w]),
                s8pair_to_h2<0>(vc[w], vd[w]), s8pair_to_h2<1>(vc[w], vd[w]), b0, b1);
        mma_f16(o[h][2 * w + 1], s8pair_to_h2<2>(va[w], vb[w]), s8pair_to_h2<3>(va[w], vb[w]),
                s8pair_to_h2<2>(vc[w], vd[w]), s8pair_to_h2<3>(vc[w], vd[w]), b0, b1);
      }
    }
    __syncwarp();                                    // every lane is done with this stage before it is refilled
    stage = stage + 1 == kStages ? 0 : stage + 1;
  }
  Q36_ATRACE(cta_flat, 4);
  q36::cp_async_wait<0>();
  __syncthreads();                                   // the ring becomes the epilogue's slices
  Q36_ATRACE(cta_flat, 5);
  q36::split_epilogue<G>(o, m_run, l_run, 1.0f / kPScale, s_m, s_l, s_o, part_o, part_m, part_l, head0, split, n_splits);
  Q36_ATRACE(cta_flat, 6);
}

template <int G>
int launch_split_g(const __nv_bfloat16 *q, const int8_t *kq, const int8_t *vq, const float *meta, Scratch sc,
                   size_t t_begin, size_t t_end, const qwen36_attention_shape_t &sh, uint32_t q_per_kv,
                   uint32_t n_splits) {
  const dim3 grid(static_cast<unsigned>(sh.q_heads / G), n_splits);
  const uint32_t D = static_cast<uint32_t>(sh.head_dim), KV = static_cast<uint32_t>(sh.kv_heads);
  const bool aligned = ((reinterpret_cast<uintptr_t>(kq) | reinterpret_cast<uintptr_t>(vq)) & 7u) == 0;
#define Q36_GO(DPL, VEC)                                                                              \
  kv_attention_split_kernel<G, DPL, VEC><<<grid, kThreads, 0, q36::stream()>>>(                        \
      q, kq, vq, meta, sc.o, sc.m, sc.l, t_begin, t_end, KV, q_per_kv, D, n_splits)
  if (D == 256 && G <= 8 && g_use_fast_attention == 3 &&
      ((reinterpret_cast<uintptr_t>(kq) | reinterpret_cast<uintptr_t>(vq) | reinterpret_cast<uintptr_t>(q)) & 15u) == 0 &&
      (reinterpret_cast<uintptr_t>(meta) & 7u) == 0) {
    if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(kv_attention_staged_kernel<G>),
                                 static_cast<int>(kStagedSmemBytes)) != cudaSuccess)
      return QWEN36_STATUS_CUDA_ERROR;
    return q36::cuda_status(q36::launch_after_previous(kv_attention_staged_kernel<G>, grid, dim3(kThreads),
                                                       kStagedSmemBytes, q36::stream(), q, kq, vq, meta, sc.o, sc.m,
                                                       sc.l, t_begin, t_end, KV, q_per_kv, n_splits));
  }
  if (D == 256 && G <= 8 && g_use_fast_attention >= 2 &&
      ((reinterpret_cast<uintptr_t>(kq) | reinterpret_cast<uintptr_t>(vq) | reinterpret_cast<uintptr_t>(q)) & 15u) == 0) {
    kv_attention_mma_kernel<G><<<grid, kThreads, 0, q36::stream()>>>(q, kq, vq, meta, sc.o, sc.m, sc.l, t_begin,
                                                                      t_end, KV, q_per_kv, n_splits);
    return q36::launch_status();
  }
  if (D == 256 && aligned && (reinterpret_cast<uintptr_t>(q) & 15u) == 0 && g_use_fast_attention) {
    kv_attention_fast_kernel<G><<<grid, kThreads, 0, q36::stream()>>>(q, kq, vq, meta, sc.o, sc.m, sc.l, t_begin,
                                                                       t_end, KV, q_per_kv, n_splits);
    return q36::launch_status();
  }
  if (D == 256 && aligned) Q36_GO(8, true);
  else if (D == 128 && aligned) Q36_GO(4, true);
  else if (D == 64) Q36_GO(2, true);
  else if (D <= 64) Q36_GO(2, false);
  else if (D <= 128) Q36_GO(4, false);
  else Q36_GO(8, false);
#undef Q36_GO
  return q36::launch_status();
}

// Runs the split kernel over [t_begin, t_end) and returns the number of
// splits used (0 on error, with *status set).
uint32_t run_splits(qwen36_device_ptr_t q, qwen36_device_ptr_t kq, qwen36_device_ptr_t vq,
                    qwen36_device_ptr_t meta, Scratch sc, size_t t_begin, size_t t_end,
                    const qwen36_attention_shape_t &sh, int *status) {
  const uint32_t q_per_kv = static_cast<uint32_t>(sh.q_heads / sh.kv_heads);
  const int G = (q_per_kv == 1 || q_per_kv == 2 || q_per_kv == 4 || q_per_kv == 6 || q_per_kv == 8)
                    ? static_cast<int>(q_per_kv) : 1;
  const size_t tokens = t_end > t_begin ? t_end - t_begin : 0;
  const __nv_bfloat16 *qp = as_ptr<const __nv_bfloat16>(q);
  const int8_t *kp = as_ptr<const int8_t>(kq), *vp = as_ptr<const int8_t>(vq);
  const bool tensor_core_form = sh.head_dim == 256 && g_use_fast_attention >= 2 &&
      ((reinterpret_cast<uintptr_t>(kp) | reinterpret_cast<uintptr_t>(vp) | reinterpret_cast<uintptr_t>(qp)) & 15u) == 0;
  const uint32_t n_splits = pick_splits(tokens, sh.q_heads / G, tensor_core_form);
  const float *mp = as_ptr<const float>(meta);
  const size_t tb = t_begin, te = t_begin + tokens;
  switch (G) {
    case 2: *status = launch_split_g<2>(qp, kp, vp, mp, sc, tb, te, sh, q_per_kv, n_splits); break;
    case 4: *status = launch_split_g<4>(qp, kp, vp, mp, sc, tb, te, sh, q_per_kv, n_splits); break;
    case 6: *status = launch_split_g<6>(qp, kp, vp, mp, sc, tb, te, sh, q_per_kv, n_splits); break;
    case 8: *status = launch_split_g<8>(qp, kp, vp, mp, sc, tb, te, sh, q_per_kv, n_splits); break;
    default: *status = launch_split_g<1>(qp, kp, vp, mp, sc, tb, te, sh, q_per_kv, n_splits); break;
  }
  return *status == QWEN36_STATUS_SUCCESS ? n_splits : 0;
}

bool shape_ok(const qwen36_attention_shape_t &sh) {
  return sh.q_heads != 0 && sh.kv_heads != 0 && sh.head_dim != 0 && sh.q_heads % sh.kv_heads == 0;
}

}  // namespace

extern "C" int qwen36_turboquant_encode_kv_rows(const qwen36_turboquant_encode_rows_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->k_bf16.ptr == 0 || spec->v_bf16.ptr == 0 || spec->k_quantized_i8.ptr == 0 ||
      spec->v_quantized_i8.ptr == 0 || spec->metadata_f32.ptr == 0 || spec->shape.kv_heads == 0 ||
      spec->shape.head_dim == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  if (spec->tokens == 0) return QWEN36_STATUS_SUCCESS;
  const size_t vecs = spec->tokens * spec->shape.kv_heads * 2;
  if (spec->shape.head_dim == 256 && vecs >= 4096 &&
      ((spec->k_bf16.ptr | spec->v_bf16.ptr) & 15u) == 0 && ((spec->k_quantized_i8.ptr | spec->v_quantized_i8.ptr) & 7u) == 0) {
    // one wave: every block must be resident at once, or the strided walk leaves the late blocks a tail of their own
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kv_encode_rows256_kernel, kThreads, 0) != cudaSuccess || per_sm < 1)
      per_sm = 4;
    const size_t blocks = std::min(q36::div_ceil(vecs, static_cast<size_t>(kWarps)),
                                   static_cast<size_t>(sm_count()) * static_cast<size_t>(per_sm));
    kv_encode_rows256_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, q36::stream()>>>(
        as_ptr<const __nv_bfloat16>(spec->k_bf16), as_ptr<const __nv_bfloat16>(spec->v_bf16),
        as_ptr<int8_t>(spec->k_quantized_i8), as_ptr<int8_t>(spec->v_quantized_i8),
        as_ptr<float>(spec->metadata_f32), spec->position, vecs, spec->shape.kv_heads);
    return q36::launch_status();
  }
  return q36::cuda_status(q36::launch_after_previous(
      kv_encode_kernel, dim3(static_cast<unsigned>(q36::div_ceil(vecs, kWarps))), dim3(kThreads), size_t{0}, q36::stream(),
      as_ptr<const __nv_bfloat16>(spec->k_bf16), as_ptr<const __nv_bfloat16>(spec->v_bf16),
      as_ptr<int8_t>(spec->k_quantized_i8), as_ptr<int8_t>(spec->v_quantized_i8),
      as_ptr<float>(spec->metadata_f32), spec->position, spec->tokens, spec->shape.kv_heads,
      spec->shape.head_dim));
}

extern "C" int qwen36_turboquant_encode_kv(const qwen36_turboquant_encode_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  qwen36_turboquant_encode_rows_spec_t rows{};
  rows.position = spec->position;
  rows.tokens = 1;
  rows.k_bf16 = spec->k_bf16;
  rows.v_bf16 = spec->v_bf16;
  rows.k_quantized_i8 = spec->k_quantized_i8;
  rows.v_quantized_i8 = spec->v_quantized_i8;
  rows.metadata_f32 = spec->metadata_f32;
  rows.shape = spec->shape;
  return qwen36_turboquant_encode_kv_rows(&rows);
}

// Test hook: 0 routes head_dim 256 through the general kernel instead of the 4-token fast path.
extern "C" void qwen36_turboquant_attention_set_fast(int mode) { g_use_fast_attention = mode < 0 ? 0 : (mode > 3 ? 3 : mode); }

// Test hook: n > 0 fixes the number of KV splits, 0 restores the heuristic.
extern "C" void qwen36_turboquant_attention_force_splits(int n) { g_force_splits = n < 0 ? 0 : n; }

extern "C" size_t qwen36_turboquant_attention_workspace_bytes(size_t q_heads, size_t head_dim) {
  return scratch_bytes(q_heads, head_dim);
}

extern "C" int qwen36_turboquant_attention(const qwen36_turboquant_attention_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->q_bf16.ptr == 0 || spec->k_quantized_i8.ptr == 0 || spec->v_quantized_i8.ptr == 0 ||
      spec->metadata_f32.ptr == 0 || spec->output_bf16.ptr == 0 || !shape_ok(spec->shape))
    return QWEN36_STATUS_INVALID_ARGUMENT;
  if (spec->shape.head_dim > 256) return QWEN36_STATUS_NOT_IMPLEMENTED;
  if (spec->workspace.ptr == 0 || (spec->workspace.ptr & 15u) != 0 ||
      spec->workspace_bytes < scratch_bytes(spec->shape.q_heads, spec->shape.head_dim))
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const Scratch sc = carve(as_ptr<float>(spec->workspace), spec->shape.q_heads, spec->shape.head_dim);
  int status = QWEN36_STATUS_SUCCESS;
  const uint32_t n = run_splits(spec->q_bf16, spec->k_quantized_i8, spec->v_quantized_i8, spec->metadata_f32,
                                sc, 0, spec->position + 1, spec->shape, &status);
  if (n == 0) return status;
  return launch_merge_after_splits<true>(static_cast<unsigned>(spec->shape.q_heads),
      sc.o, sc.m, sc.l, n, static_cast<uint32_t>(spec->shape.head_dim), as_ptr<__nv_bfloat16>(spec->output_bf16),
      nullptr, nullptr, nullptr);
}

// Attention over this rank's token range and the cross-rank merge, two launches: the split kernel,
// then one kernel that merges the splits, pushes the result to the peers and merges theirs.
extern "C" int qwen36_turboquant_attention_peer(const qwen36_turboquant_attention_peer_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->q_bf16.ptr == 0 || spec->k_quantized_i8.ptr == 0 || spec->v_quantized_i8.ptr == 0 ||
      spec->metadata_f32.ptr == 0 || spec->output_bf16.ptr == 0 || !shape_ok(spec->shape) ||
      spec->t_end < spec->t_begin)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  if (spec->shape.head_dim > 256) return QWEN36_STATUS_NOT_IMPLEMENTED;
  if (spec->workspace.ptr == 0 || (spec->workspace.ptr & 15u) != 0 ||
      spec->workspace_bytes < scratch_bytes(spec->shape.q_heads, spec->shape.head_dim))
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const Scratch sc = carve(as_ptr<float>(spec->workspace), spec->shape.q_heads, spec->shape.head_dim);
  int status = QWEN36_STATUS_SUCCESS;
  const uint32_t n = run_splits(spec->q_bf16, spec->k_quantized_i8, spec->v_quantized_i8, spec->metadata_f32,
                                sc, spec->t_begin, spec->t_end, spec->shape, &status);
  if (n == 0) return status;
  return q36::launch_attention_peer_merge(sc.o, sc.m, sc.l, n, spec->peer_inbox, spec->peer_flags, spec->state,
                                          spec->output_bf16, spec->world, spec->rank, spec->shape.q_heads,
                                          spec->shape.head_dim);
}

extern "C" int qwen36_turboquant_attention_partial(const qwen36_turboquant_attention_partial_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->q_bf16.ptr == 0 || spec->k_quantized_i8.ptr == 0 || spec->v_quantized_i8.ptr == 0 ||
      spec->metadata_f32.ptr == 0 || spec->partial_acc_f32.ptr == 0 || spec->partial_max_f32.ptr == 0 ||
      spec->partial_denom_f32.ptr == 0 || !shape_ok(spec->shape) || spec->t_end < spec->t_begin)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  if (spec->shape.head_dim > 256) return QWEN36_STATUS_NOT_IMPLEMENTED;
  if (spec->workspace.ptr == 0 || (spec->workspace.ptr & 15u) != 0 ||
      spec->workspace_bytes < scratch_bytes(spec->shape.q_heads, spec->shape.head_dim))
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const Scratch sc = carve(as_ptr<float>(spec->workspace), spec->shape.q_heads, spec->shape.head_dim);
  int status = QWEN36_STATUS_SUCCESS;
  const uint32_t n = run_splits(spec->q_bf16, spec->k_quantized_i8, spec->v_quantized_i8, spec->metadata_f32,
                                sc, spec->t_begin, spec->t_end, spec->shape, &status);
  if (n == 0) return status;
  return launch_merge_after_splits<false>(static_cast<unsigned>(spec->shape.q_heads),
      sc.o, sc.m, sc.l, n, static_cast<uint32_t>(spec->shape.head_dim), nullptr,
      as_ptr<float>(spec->partial_acc_f32), as_ptr<float>(spec->partial_max_f32),
      as_ptr<float>(spec->partial_denom_f32));
}

// Device address of g_static_attention_scratch on the current device, looked up once per
// device.  In host code the array's name is only a handle for cudaGetSymbolAddress, never a
// pointer a kernel could use.
static float *static_scratch_for_current_device(int *status) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static float *ptrs[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *status = QWEN36_STATUS_CUDA_ERROR;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    float *p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_attention_scratch) != cudaSuccess || p == nullptr) {
      *status = QWEN36_STATUS_CUDA_ERROR;
      return nullptr;
    }
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

extern "C" size_t qwen36_turboquant_attention_static_max_head_floats(void) { return kStaticHeadFloats; }

extern "C" int qwen36_turboquant_attention_static(const qwen36_turboquant_attention_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->q_bf16.ptr == 0 || spec->k_quantized_i8.ptr == 0 || spec->v_quantized_i8.ptr == 0 ||
      spec->metadata_f32.ptr == 0 || spec->output_bf16.ptr == 0 || !shape_ok(spec->shape))
    return QWEN36_STATUS_INVALID_ARGUMENT;
  if (spec->shape.head_dim > 256) return QWEN36_STATUS_NOT_IMPLEMENTED;
  // the built-in scratch has a fixed size: larger shapes must use qwen36_turboquant_attention
  if (spec->shape.q_heads * (spec->shape.head_dim + 2) > kStaticHeadFloats) return QWEN36_STATUS_INVALID_ARGUMENT;
  int status = QWEN36_STATUS_SUCCESS;
  float *base = static_scratch_for_current_device(&status);
  if (base == nullptr) return status;
  const Scratch sc = carve(base, spec->shape.q_heads, spec->shape.head_dim);
  const uint32_t n = run_splits(spec->q_bf16, spec->k_quantized_i8, spec->v_quantized_i8, spec->metadata_f32,
                                sc, 0, spec->position + 1, spec->shape, &status);
  if (n == 0) return status;
  return launch_merge_after_splits<true>(static_cast<unsigned>(spec->shape.q_heads),
      sc.o, sc.m, sc.l, n, static_cast<uint32_t>(spec->shape.head_dim), as_ptr<__nv_bfloat16>(spec->output_bf16),
      nullptr, nullptr, nullptr);
}

extern "C" int qwen36_attention_merge_partials(const qwen36_attention_merge_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->q_heads == 0 || spec->head_dim == 0 || spec->n_parts == 0 || spec->n_parts > kThreads ||
      spec->partial_acc_f32.ptr == 0 ||
      spec->partial_max_f32.ptr == 0 || spec->partial_denom_f32.ptr == 0 || spec->output_bf16.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  kv_merge_kernel<true><<<static_cast<unsigned>(spec->q_heads), kThreads, 0, q36::stream()>>>(
      as_ptr<const float>(spec->partial_acc_f32), as_ptr<const float>(spec->partial_max_f32),
      as_ptr<const float>(spec->partial_denom_f32), static_cast<uint32_t>(spec->n_parts),
      static_cast<uint32_t>(spec->head_dim), as_ptr<__nv_bfloat16>(spec->output_bf16), nullptr, nullptr, nullptr);
  return q36::launch_status();
}

#ifdef Q36_ATTN_TRACE
// Copies the stamp log (32768 entries of {time ns, cta << 8 | event}) to `dst`, returns the number of
// entries written since the last read (or -1) and rewinds the log.
extern "C" int qwen36_attention_trace_read(void *dst) {
  unsigned int n = 0;
  const unsigned int zero = 0;
  if (cudaMemcpyFromSymbol(&n, g_attn_trace_n, sizeof(n)) != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(dst, g_attn_trace, sizeof(g_attn_trace)) != cudaSuccess) return -1;
  if (cudaMemcpyToSymbol(g_attn_trace_n, &zero, sizeof(zero)) != cudaSuccess) return -1;
  return static_cast<int>(n < kTraceEntries ? n : kTraceEntries);
}
#endif
