// lm_head: FP8 E4M3 weight with one float scale per row.
//   quantise (one-off), W8A16 GEMV for n <= 16 tokens, greedy argmax over bf16
//   logits, and the GEMV fused with the argmax (no logits written).
//
// The GEMV is HBM-bound (1.27 GB of weight per call at vocab 248320).  Each
// warp streams whole rows with 16-byte loads, 512 contiguous bytes per warp
// instruction, R rows and two K-steps in flight.  It keeps the reference's
// float32 summation order (kernels-cuda/lm_head_fp8.cu:122-194): lane l adds
// the products of bytes 16*l + 512*j .. +15 in ascending order with fused
// multiply-adds, the lanes meet in a 16,8,4,2,1 xor butterfly, then the row
// scale is applied and the value rounded to bf16.  Every product is exact in
// float32 (4-bit x 8-bit significands), so the logits are bit-identical to the
// reference's and the greedy argmax picks the same token.
#include "common.cuh"
#include "kv_split.cuh"

#include <atomic>

#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <mutex>

namespace cg = cooperative_groups;

namespace {

using q36::as_ptr;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// ---------------------------------------------------------------- quantise

// One CTA per row: amax, scale = amax/448 (1 for an all-zero row), then
// saturating round-to-nearest-even cast of w * (1/scale)
// (kernels-cuda/lm_head_fp8.cu:37-80).
__global__ void __launch_bounds__(kThreads)
lm_head_quantize_kernel(const __nv_bfloat16 *__restrict__ w, uint8_t *__restrict__ q,
                        float *__restrict__ scales, size_t rows, size_t cols) {
  __shared__ float warp_amax[kWarps];
  __shared__ float s_scale;
  const size_t row = blockIdx.x;
  const __nv_bfloat16 *src = w + row * cols;
  float amax = 0.f;
  for (size_t c = threadIdx.x; c < cols; c += kThreads) amax = fmaxf(amax, fabsf(__bfloat162float(src[c])));
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) warp_amax[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < kWarps; ++i) m = fmaxf(m, warp_amax[i]);
    s_scale = m > 0.f ? __fdiv_rn(m, 448.0f) : 1.0f;
    scales[row] = s_scale;
  }
  __syncthreads();
  const float inv = __fdiv_rn(1.0f, s_scale);
  for (size_t c = threadIdx.x; c < cols; c += kThreads) {
    const __nv_fp8_e4m3 v(__fmul_rn(__bfloat162float(src[c]), inv));
    q[row * cols + c] = reinterpret_cast<const uint8_t &>(v);
  }
}

// -------------------------------------------------------------------- GEMV

__device__ __forceinline__ bool better(float cand, uint32_t cand_idx, float cur, uint32_t cur_idx) {
  return cand > cur || (cand == cur && cand_idx < cur_idx);   // kernels-cuda/ops.cu:19-23
}

// two E4M3 bytes (low 16 bits of `pair`) -> two floats, exact
__device__ __forceinline__ float2 e4m3x2_to_f32(uint32_t pair) {
  uint32_t h2;
  asm("{\n\t.reg .b16 p;\n\tcvt.u16.u32 p, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, p;\n\t}" : "=r"(h2) : "r"(pair));
  return __half22float2(*reinterpret_cast<__half2 *>(&h2));
}

// Rows a warp carries at once: more rows keep more 16-byte loads in flight and share every
// activation load; bounded by registers (rows x tokens accumulators).  With float32 staging the
// CTAs are larger (fewer warps per SM), so each warp carries twice as many rows.
template <int N, bool XF32> struct RowsPerWarp {
  static constexpr int value = N == 1 ? 4 : (XF32 ? (N <= 4 ? 4 : 2) : (N <= 4 ? 2 : 1));
};

// x lives in shared memory as bf16, 16-byte chunks, chunk c stored at
// c ^ ((c >> 3) & 1) so that a quarter warp (chunks 2l+i, l = 0..7) hits eight
// distinct bank groups.
__device__ __forceinline__ uint32_t xswz(uint32_t chunk) { return chunk ^ ((chunk >> 3) & 1u); }

// Tail of the fused variant: per-warp winners -> CTA winner -> `partials`; the last CTA to finish
// (ticket counter) merges them, writes the tokens and re-zeroes the ticket.
template <int N>
__device__ __forceinline__ void fused_argmax_tail(const float (&best)[N], const uint32_t (&best_idx)[N], uint32_t warp,
                                                  uint32_t lane, float2 *__restrict__ partials, unsigned *__restrict__ ticket,
                                                  uint32_t *__restrict__ out_tokens, float *__restrict__ out_best) {
    __shared__ float s_val[kWarps][N];
    __shared__ uint32_t s_idx[kWarps][N];
    __shared__ bool s_last;
    if (lane == 0) {
#pragma unroll
      for (int t = 0; t < N; ++t) { s_val[warp][t] = best[t]; s_idx[warp][t] = best_idx[t]; }
    }
    __syncthreads();
    if (threadIdx.x < N) {
      float bv = s_val[0][threadIdx.x];
      uint32_t bi = s_idx[0][threadIdx.x];
      for (int w = 1; w < kWarps; ++w)
        if (better(s_val[w][threadIdx.x], s_idx[w][threadIdx.x], bv, bi)) { bv = s_val[w][threadIdx.x]; bi = s_idx[w][threadIdx.x]; }
      partials[static_cast<size_t>(blockIdx.x) * N + threadIdx.x] = make_float2(bv, __uint_as_float(bi));
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (s_last) {
      __threadfence();
      // Every thread takes the CTAs b = thread, thread + 256, ... of every token (all loads of a
      // thread are independent: one round trip), then the winners meet by shuffles and through the
      // same shared arrays.  `better` is a total order (value, then lower index), so the order in
      // which candidates meet does not change the winner.
      float bv[N];
      uint32_t bi[N];
#pragma unroll
      for (int t = 0; t < N; ++t) { bv[t] = -INFINITY; bi[t] = 0u; }   // what a scan that nothing beats returns
      for (uint32_t b = threadIdx.x; b < gridDim.x; b += kThreads) {
#pragma unroll
        for (int t = 0; t < N; ++t) {
          const float2 p = __ldcg(partials + static_cast<size_t>(b) * N + t);
          const uint32_t pi = __float_as_uint(p.y);
          if (better(p.x, pi, bv[t], bi[t])) { bv[t] = p.x; bi[t] = pi; }
        }
      }
#pragma unroll
      for (int t = 0; t < N; ++t) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, bv[t], off);
          const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi[t], off);
          if (better(ov, oi, bv[t], bi[t])) { bv[t] = ov; bi[t] = oi; }
        }
        if (lane == 0) { s_val[warp][t] = bv[t]; s_idx[warp][t] = bi[t]; }
      }
      __syncthreads();
      if (threadIdx.x < N) {
        float fv = s_val[0][threadIdx.x];
        uint32_t fi = s_idx[0][threadIdx.x];
        for (int w = 1; w < kWarps; ++w)
          if (better(s_val[w][threadIdx.x], s_idx[w][threadIdx.x], fv, fi)) { fv = s_val[w][threadIdx.x]; fi = s_idx[w][threadIdx.x]; }
        out_tokens[threadIdx.x] = fi;
        if (out_best != nullptr) out_best[threadIdx.x] = fv;
      }
      if (threadIdx.x == 0) *ticket = 0u;      // ready for the next call
    }
}

// FUSED = false: writes y[t * rows + row] (bf16).
// FUSED = true : keeps the running (value, index) of the bf16-rounded logits
//   per token; per-CTA winners go to `partials`, the last CTA to finish (ticket
//   counter) merges them, writes the tokens and re-zeroes the ticket.
// XF32: the activations are staged as float32 (16-byte chunks, XOR-swizzled so that the eight
// lanes of a quarter warp, 64 bytes apart, hit distinct bank groups) instead of bf16.  With
// several tokens and only one or two rows per warp the bf16 -> f32 unpack would otherwise cost as
// many instructions as the FMAs themselves.
__device__ __forceinline__ uint32_t xswz32(uint32_t chunk) { return chunk ^ ((chunk >> 3) & 7u); }

// Can token t's activations go through the float16 route below without changing a bit of the
// result?  Yes when they are all finite, the largest magnitude lies within 2^-100 .. 2^100 (no
// float32 overflow or subnormal in either computation) and every nonzero value lies within 2^28 of
// the largest (so that, times the power of two that lifts the largest into [2^14, 2^15), every
// value is a normal float16: a bf16 value has 8 significant bits, a float16 has 11).  Every CTA
// evaluates this on the same data and reaches the same verdict.  max_e[t] = biased exponent of the
// token's largest magnitude (0 for an all-zero token).
template <int N>
__device__ __forceinline__ bool x_fits_f16(const __nv_bfloat16 *__restrict__ x, uint32_t cols, uint32_t (&max_e)[N]) {
  __shared__ uint32_t s_max[N], s_min[N], s_bad;
  if (threadIdx.x < N) { s_max[threadIdx.x] = 0u; s_min[threadIdx.x] = 255u; }
  if (threadIdx.x == 0) s_bad = 0u;
  __syncthreads();
  const uint32_t chunks_per_tok = cols / 8u;
  for (uint32_t t = 0; t < static_cast<uint32_t>(N); ++t) {
    uint32_t mx = 0u, mn = 255u, bad = 0u;
    for (uint32_t c = threadIdx.x; c < chunks_per_tok; c += kThreads) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(x) + t * chunks_per_tok + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t bits = (w[i] >> (16 * h)) & 0x7fffu;
          const uint32_t e = bits >> 7;
          if (bits != 0u) {
            if (e == 0u || e == 255u) bad = 1u;                // bf16 subnormal, infinity or NaN
            mx = max(mx, e);
            mn = min(mn, e);
          }
        }
      }
    }
    mx = __reduce_max_sync(0xffffffffu, mx);
    mn = __reduce_min_sync(0xffffffffu, mn);
    bad = __reduce_or_sync(0xffffffffu, bad);
    if ((threadIdx.x & 31u) == 0u) {
      atomicMax(&s_max[t], mx);
      atomicMin(&s_min[t], mn);
      if (bad) atomicOr(&s_bad, 1u);
    }
  }
  __syncthreads();
  bool fit = s_bad == 0u;
#pragma unroll
  for (int t = 0; t < N; ++t) {
    max_e[t] = s_max[t];
    if (s_max[t] != 0u) fit = fit && s_max[t] >= 27u && s_max[t] <= 227u && s_max[t] - s_min[t] <= 28u;
  }
  return fit;
}

// UNFIT_ONLY: the launch that follows a float16-route launch on the same inputs; it returns at
// once when that one did the work.
template <int N, bool FUSED, bool XF32, bool UNFIT_ONLY = false>
__global__ void __launch_bounds__(kThreads)
lm_head_gemv_kernel(const uint8_t *__restrict__ weight, const float *__restrict__ row_scales,
                    const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ y, size_t rows,
                    uint32_t cols, uint32_t row_offset, uint32_t *__restrict__ out_tokens,
                    float *__restrict__ out_best, float2 *__restrict__ partials,
                    unsigned *__restrict__ ticket) {
  constexpr int R = RowsPerWarp<N, XF32>::value;
  extern __shared__ __align__(16) uint8_t smem[];
  uint4 *xs = reinterpret_cast<uint4 *>(smem);        // N * cols bf16, swizzled chunks
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t chunks_per_tok = cols / 8u;
  if constexpr (UNFIT_ONLY) {
    uint32_t unused[N];
    if (x_fits_f16<N>(x, cols, unused)) return;
  }

  if constexpr (XF32) {
    for (uint32_t c = threadIdx.x; c < N * chunks_per_tok; c += kThreads) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(x) + c);
      xs[xswz32(2u * c)] = make_uint4(v.x << 16, v.x & 0xffff0000u, v.y << 16, v.y & 0xffff0000u);
      xs[xswz32(2u * c + 1u)] = make_uint4(v.z << 16, v.z & 0xffff0000u, v.w << 16, v.w & 0xffff0000u);
    }
  } else {
    for (uint32_t c = threadIdx.x; c < N * chunks_per_tok; c += kThreads)
      xs[xswz(c)] = __ldcg(reinterpret_cast<const uint4 *>(x) + c);
  }
  __syncthreads();

  float best[N];
  uint32_t best_idx[N];
#pragma unroll
  for (int t = 0; t < N; ++t) { best[t] = -INFINITY; best_idx[t] = 0u; }

  const size_t warps_total = static_cast<size_t>(gridDim.x) * kWarps;
  const uint32_t steps = cols / 512u;            // full 512-byte K-steps; the reference loop
                                                 // (kk + 15 < cols) also covers a ragged last
                                                 // step for lanes whose 16 bytes still fit
  const bool tail = lane * 16u + steps * 512u + 15u < cols;

  for (size_t row0 = (static_cast<size_t>(blockIdx.x) * kWarps + warp) * R; row0 < rows;
       row0 += warps_total * R) {
    const int r_count = static_cast<int>(min(static_cast<size_t>(R), rows - row0));
    float acc[R][N];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < N; ++t) acc[r][t] = 0.f;

    const uint8_t *w0 = weight + row0 * cols + lane * 16u;
    uint4 cur[R], nxt[R];
    auto load = [&](uint4 (&dst)[R], uint32_t step) {
#pragma unroll
      for (int r = 0; r < R; ++r)
        dst[r] = r < r_count ? __ldcs(reinterpret_cast<const uint4 *>(w0 + static_cast<size_t>(r) * cols + step * 512u))
                             : make_uint4(0, 0, 0, 0);
    };
    const uint32_t my_steps = steps + (tail ? 1u : 0u);
    if (my_steps > 0) load(cur, 0);
    for (uint32_t s = 0; s < my_steps; ++s) {
      if (s + 1 < my_steps) load(nxt, s + 1);
      const uint32_t chunk0 = (lane * 16u + s * 512u) / 8u;        // first of two x chunks
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float wf[R][8];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const uint32_t w_lo = half == 0 ? cur[r].x : cur[r].z;
          const uint32_t w_hi = half == 0 ? cur[r].y : cur[r].w;
          const float2 f0 = e4m3x2_to_f32(w_lo), f1 = e4m3x2_to_f32(w_lo >> 16);
          const float2 f2 = e4m3x2_to_f32(w_hi), f3 = e4m3x2_to_f32(w_hi >> 16);
          wf[r][0] = f0.x; wf[r][1] = f0.y; wf[r][2] = f1.x; wf[r][3] = f1.y;
          wf[r][4] = f2.x; wf[r][5] = f2.y; wf[r][6] = f3.x; wf[r][7] = f3.y;
        }
#pragma unroll
        for (int t = 0; t < N; ++t) {
          float xv[8];
          if constexpr (XF32) {
            const uint32_t c32 = 2u * (t * chunks_per_tok + chunk0 + half);
            const uint4 xa = xs[xswz32(c32)], xb = xs[xswz32(c32 + 1u)];
            xv[0] = __uint_as_float(xa.x); xv[1] = __uint_as_float(xa.y); xv[2] = __uint_as_float(xa.z); xv[3] = __uint_as_float(xa.w);
            xv[4] = __uint_as_float(xb.x); xv[5] = __uint_as_float(xb.y); xv[6] = __uint_as_float(xb.z); xv[7] = __uint_as_float(xb.w);
          } else {
            const uint4 xc = xs[xswz(t * chunks_per_tok + chunk0 + half)];
            const uint32_t xw[4] = {xc.x, xc.y, xc.z, xc.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              xv[2 * i] = __uint_as_float(xw[i] << 16);
              xv[2 * i + 1] = __uint_as_float(xw[i] & 0xffff0000u);
            }
          }
#pragma unroll
          for (int r = 0; r < R; ++r)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[r][t] = fmaf(wf[r][i], xv[i], acc[r][t]);
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) cur[r] = nxt[r];
    }

#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (r >= r_count) break;
      const float scale = __ldg(row_scales + row0 + r);
#pragma unroll
      for (int t = 0; t < N; ++t) {
        float v = acc[r][t];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        const __nv_bfloat16 logit = __float2bfloat16(__fmul_rn(v, scale));
        if (!FUSED) {
          if (lane == 0) y[static_cast<size_t>(t) * rows + row0 + r] = logit;
        } else {
          const float lv = __bfloat162float(logit);
          const uint32_t idx = static_cast<uint32_t>(row0 + r) + row_offset;
          if (better(lv, idx, best[t], best_idx[t])) { best[t] = lv; best_idx[t] = idx; }
        }
      }
    }
  }

  if (FUSED) fused_argmax_tail<N>(best, best_idx, warp, lane, partials, ticket, out_tokens, out_best);
}

// Float16 route for 2..8 tokens.  The reference's sum for (row, token) is a float32 FMA chain per
// lane over exact products e4m3 x bf16.  Here the token's activations are staged as float16 times
// a power of two (exact, see x_fits_f16), the weights are expanded to float16 by the hardware
// conversion (exact) and the chain runs on the mixed-precision fma.rn.f32.f16: the same products,
// the same order, every partial sum the reference's times that power of two, which is divided out
// at the end.  Per weight that is one conversion slot and one FMA per token, against a conversion,
// an unpack and an FMA per token on the float32 route, and the staged vector is half the size.
// A warp carries four rows (every activation load from shared memory serves all four).  Its weights
// do not wait in registers: every lane copies its own 16 bytes of each row with cp.async into a ring
// that belongs to the warp (a stage = four rows x 512 bytes) and reads them back when their turn
// comes, so several steps are in flight without costing a register, and the ring runs on across
// row groups (no cold start every ten steps).  With one step ahead in registers a warp could not
// finish a step faster than one loaded-memory latency, which is what held the float32 route at
// 3.3 TB/s at a few tokens.  A lane only ever reads what it copied itself, so nothing but its own
// cp.async.wait_group orders the ring.
constexpr int kF16Rows = 4;
constexpr uint32_t kF16StageBytes = kF16Rows * 512u;
template <int N> struct F16Ring { static constexpr int kStages = N <= 4 ? 4 : (N <= 6 ? 3 : 2); };
template <int N, bool FUSED>
__global__ void __launch_bounds__(kThreads, 2)
lm_head_gemv_f16_kernel(const uint8_t *__restrict__ weight, const float *__restrict__ row_scales,
                        const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ y, size_t rows,
                        uint32_t cols, uint32_t row_offset, uint32_t *__restrict__ out_tokens,
                        float *__restrict__ out_best, float2 *__restrict__ partials,
                        unsigned *__restrict__ ticket) {
  constexpr int R = kF16Rows;
  constexpr int S = F16Ring<N>::kStages;
  extern __shared__ __align__(16) uint8_t smem[];
  uint4 *xs = reinterpret_cast<uint4 *>(smem);        // N * cols float16, swizzled 16-byte chunks
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t chunks_per_tok = cols / 8u;
  uint32_t max_e[N];
  if (!x_fits_f16<N>(x, cols, max_e)) return;         // the float32 route, launched next, does the work
  float unscale[N];
#pragma unroll
  for (int t = 0; t < N; ++t) {
    const uint32_t e = max_e[t];
    const float up = e == 0u ? 1.0f : __uint_as_float((268u - e) << 23);       // 2^(141 - e)
    unscale[t] = e == 0u ? 1.0f : __uint_as_float((e - 14u) << 23);            // 2^(e - 141)
    for (uint32_t c = threadIdx.x; c < chunks_per_tok; c += kThreads) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(x) + t * chunks_per_tok + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      __half2 h[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        h[i] = __floats2half2_rn(__uint_as_float(w[i] << 16) * up, __uint_as_float(w[i] & 0xffff0000u) * up);
      xs[xswz(t * chunks_per_tok + c)] = *reinterpret_cast<uint4 *>(h);
    }
  }
  __syncthreads();

  float best[N];
  uint32_t best_idx[N];
#pragma unroll
  for (int t = 0; t < N; ++t) { best[t] = -INFINITY; best_idx[t] = 0u; }

  const size_t warps_total = static_cast<size_t>(gridDim.x) * kWarps;
  const uint32_t steps = cols / 512u;                             // this route takes cols % 512 == 0 only
  const size_t first_row = (static_cast<size_t>(blockIdx.x) * kWarps + warp) * R;
  const uint32_t groups = first_row < rows ? static_cast<uint32_t>((rows - first_row + warps_total * R - 1) / (warps_total * R)) : 0u;
  const uint32_t total = groups * steps;                          // (row group, step) pairs of this warp, in order
  const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + static_cast<uint32_t>(N) * cols * 2u + warp * (S * kF16StageBytes) + lane * 16u;
  // stage q of the warp's sequence: rows past the end are zero-filled (source size 0)
  auto issue = [&](uint32_t q) {
    if (q < total) {
      const uint32_t grp = q / steps, step = q - grp * steps;
      const size_t row0 = first_row + static_cast<size_t>(grp) * warps_total * R;
      const uint32_t dst = ring + (q % S) * kF16StageBytes;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const bool in = row0 + r < rows;
        q36::cp_async_16(dst + r * 512u, weight + (in ? (row0 + r) * cols + step * 512u + lane * 16u : 0u), in ? 16u : 0u);
      }
    }
    q36::cp_async_commit();                                       // one group per stage, empty or not
  };
#pragma unroll
  for (int a = 0; a < S - 1; ++a) issue(a);
  uint32_t q = 0;
  for (uint32_t grp = 0; grp < groups; ++grp) {
    const size_t row0 = first_row + static_cast<size_t>(grp) * warps_total * R;
    const int r_count = static_cast<int>(min(static_cast<size_t>(R), rows - row0));
    float acc[R][N];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < N; ++t) acc[r][t] = 0.f;
    auto multiply = [&](const uint4 (&cur)[R], uint32_t s) {
      const uint32_t chunk0 = (lane * 16u + s * 512u) / 8u;        // first of two x chunks
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t wh[R][4];                                          // eight weights of each row as four f16x2
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const uint32_t w_lo = half == 0 ? cur[r].x : cur[r].z;
          const uint32_t w_hi = half == 0 ? cur[r].y : cur[r].w;
          asm("{\n\t.reg .b16 a, b, c, d;\n\tmov.b32 {a, b}, %4;\n\tmov.b32 {c, d}, %5;\n\t"
              "cvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t"
              "cvt.rn.f16x2.e4m3x2 %2, c;\n\tcvt.rn.f16x2.e4m3x2 %3, d;\n\t}"
              : "=r"(wh[r][0]), "=r"(wh[r][1]), "=r"(wh[r][2]), "=r"(wh[r][3]) : "r"(w_lo), "r"(w_hi));
        }
#pragma unroll
        for (int t = 0; t < N; ++t) {
          const uint4 xc = xs[xswz(t * chunks_per_tok + chunk0 + half)];
          const uint32_t xw[4] = {xc.x, xc.y, xc.z, xc.w};
#pragma unroll
          for (int r = 0; r < R; ++r)
#pragma unroll
            for (int i = 0; i < 4; ++i)
              asm("{\n\t.reg .f16 wl, wu, xl, xu;\n\tmov.b32 {wl, wu}, %1;\n\tmov.b32 {xl, xu}, %2;\n\t"
                  "fma.rn.f32.f16 %0, wl, xl, %0;\n\tfma.rn.f32.f16 %0, wu, xu, %0;\n\t}"
                  : "+f"(acc[r][t]) : "r"(wh[r][i]), "r"(xw[i]));
        }
      }
    };
    for (uint32_t step = 0; step < steps; ++step, ++q) {
      q36::cp_async_wait<S - 2>();                                // stage q has landed (this lane's own copies)
      uint4 cur[R];
#pragma unroll
      for (int r = 0; r < R; ++r) cur[r] = q36::lds128(ring + (q % S) * kF16StageBytes + r * 512u);
      issue(q + S - 1);                                           // into the slot that was read one step ago
      multiply(cur, step);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (r >= r_count) break;
      const float scale = __ldg(row_scales + row0 + r);
#pragma unroll
      for (int t = 0; t < N; ++t) {
        float v = acc[r][t];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        const __nv_bfloat16 logit = __float2bfloat16(__fmul_rn(v * unscale[t], scale));
        if (!FUSED) {
          if (lane == 0) y[static_cast<size_t>(t) * rows + row0 + r] = logit;
        } else {
          const float lv = __bfloat162float(logit);
          const uint32_t idx = static_cast<uint32_t>(row0 + r) + row_offset;
          if (better(lv, idx, best[t], best_idx[t])) { best[t] = lv; best_idx[t] = idx; }
        }
      }
    }
  }
  if (FUSED) fused_argmax_tail<N>(best, best_idx, warp, lane, partials, ticket, out_tokens, out_best);
}

// ------------------------------------------------------------------ argmax

constexpr int kArgmaxCluster = 8;
constexpr int kArgmaxThreads = 512;

// One cluster of 8 CTAs per logits row.  Each thread scans 8 bf16 logits per
// 16-byte load; CTA winners meet in the shared memory of cluster rank 0
// (distributed shared memory), which writes the token.  Greedy rule of
// kernels-cuda/ops.cu:299-427: score = logit / temperature (1.0 when <= 0),
// strictly greater wins, ties keep the lower index, the scan starts from
// (-inf, 0) so NaN never wins.
__global__ void __launch_bounds__(kArgmaxThreads)
argmax_rows_kernel(const __nv_bfloat16 *__restrict__ logits, uint32_t *__restrict__ out,
                   uint32_t *__restrict__ mirror_last, size_t rows, size_t vocab, float temperature) {
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float s_val[kArgmaxThreads / 32];
  __shared__ uint32_t s_idx[kArgmaxThreads / 32];
  __shared__ float c_val[kArgmaxCluster];
  __shared__ uint32_t c_idx[kArgmaxCluster];

  const size_t row = blockIdx.x / kArgmaxCluster;
  const uint32_t rank = cluster.block_rank();
  const __nv_bfloat16 *l = logits + row * vocab;
  const float temp = temperature > 0.f ? temperature : 1.0f;
  const bool divide = temp != 1.0f;

  float bv = -INFINITY;
  uint32_t bi = 0u;
  auto consider = [&](float raw, uint32_t idx) {
    const float s = divide ? __fdiv_rn(raw, temp) : raw;
    if (better(s, idx, bv, bi)) { bv = s; bi = idx; }
  };
  // head elements until 16-byte alignment, then vector body, then tail
  const uintptr_t addr = reinterpret_cast<uintptr_t>(l);
  const size_t head = min(vocab, static_cast<size_t>(((16 - (addr & 15)) & 15) / 2));
  const size_t vec = (vocab - head) / 8;
  const uint32_t tid = rank * kArgmaxThreads + threadIdx.x;
  const uint32_t nthreads = kArgmaxCluster * kArgmaxThreads;
  if (tid < head) consider(__bfloat162float(l[tid]), tid);
  const uint4 *lv = reinterpret_cast<const uint4 *>(l + head);
  for (size_t v = tid; v < vec; v += nthreads) {
    const uint4 p = __ldcs(lv + v);
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
    const uint32_t base = static_cast<uint32_t>(head + v * 8);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      consider(__uint_as_float(w[i] << 16), base + 2 * i);
      consider(__uint_as_float(w[i] & 0xffff0000u), base + 2 * i + 1);
    }
  }
  for (size_t i = head + vec * 8 + tid; i < vocab; i += nthreads) consider(__bfloat162float(l[i]), static_cast<uint32_t>(i));

  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = bv; s_idx[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kArgmaxThreads / 32; ++w)
      if (better(s_val[w], s_idx[w], bv, bi)) { bv = s_val[w]; bi = s_idx[w]; }
    float *dst_v = cluster.map_shared_rank(c_val, 0);
    uint32_t *dst_i = cluster.map_shared_rank(c_idx, 0);
    dst_v[rank] = bv;
    dst_i[rank] = bi;
  }
  cluster.sync();
  if (rank == 0 && threadIdx.x == 0) {
    bv = c_val[0]; bi = c_idx[0];
    for (int r = 1; r < kArgmaxCluster; ++r)
      if (better(c_val[r], c_idx[r], bv, bi)) { bv = c_val[r]; bi = c_idx[r]; }
    out[row] = bi;
    if (mirror_last != nullptr && row + 1 == rows) *mirror_last = bi;
  }
}

int launch_argmax(const __nv_bfloat16 *logits, uint32_t *out, uint32_t *mirror, size_t rows, size_t vocab,
                  float temperature) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(rows * kArgmaxCluster));
  cfg.blockDim = dim3(kArgmaxThreads);
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kArgmaxCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return q36::cuda_status(cudaLaunchKernelEx(&cfg, argmax_rows_kernel, logits, out, mirror, rows, vocab, temperature));
}

int sm_count() { return q36::sm_count_current_device(); }

// Bytes of activation staging: float32 for 2..8 tokens while that fits, bf16 otherwise.
bool stage_f32(size_t n, size_t cols) { return n >= 2 && n <= 8 && n * cols * 4 <= 200 * 1024; }
size_t stage_bytes(size_t n, size_t cols) { return n * cols * (stage_f32(n, cols) ? 4 : 2); }

template <int N, bool FUSED, bool XF32>
int launch_gemv_x(const uint8_t *w, const float *scales, const __nv_bfloat16 *x, __nv_bfloat16 *y, size_t rows,
                  size_t cols, uint32_t row_offset, uint32_t *tokens, float *best, float2 *partials,
                  unsigned *ticket, unsigned grid) {
  const size_t smem = static_cast<size_t>(N) * cols * (XF32 ? 4 : 2);
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(lm_head_gemv_kernel<N, FUSED, XF32>), 200 * 1024) != cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  lm_head_gemv_kernel<N, FUSED, XF32><<<grid, kThreads, smem, q36::stream()>>>(
      w, scales, x, y, rows, static_cast<uint32_t>(cols), row_offset, tokens, best, partials, ticket);
  return q36::launch_status();
}

std::atomic<int> g_gemv_route{0};      // test hook: 1 = never take the float16 route

template <int N, bool FUSED>
int launch_gemv_n(const uint8_t *w, const float *scales, const __nv_bfloat16 *x, __nv_bfloat16 *y, size_t rows,
                  size_t cols, uint32_t row_offset, uint32_t *tokens, float *best, float2 *partials,
                  unsigned *ticket, unsigned grid) {
  if constexpr (N >= 2 && N <= 8) {
    if (stage_f32(N, cols)) {
      // (2..8 tokens gain 7-40 % on the float16 route, fused or not: two tokens 352 -> 260 us; one token is
      // faster on the bf16-staged kernel below, 206 against 212 us; the fused four-token instance, at the
      // 128-register limit, only since the last CTA's merge of the winners stopped being a serial scan)
      if (g_gemv_route.load() == 0 && cols % 512 == 0) {
        // float16 route first; the float32 route right behind it runs only for activations the
        // float16 route declines (both decide on the same data, on the device, so nothing is read back)
        const size_t smem16 = static_cast<size_t>(N) * cols * 2 + static_cast<size_t>(kWarps) * F16Ring<N>::kStages * kF16StageBytes;
        if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(lm_head_gemv_f16_kernel<N, FUSED>), 200 * 1024) != cudaSuccess)
          return QWEN36_STATUS_CUDA_ERROR;
        const size_t need = q36::div_ceil(rows, static_cast<size_t>(kWarps) * kF16Rows);
        const size_t cap = static_cast<size_t>(sm_count()) * 2;
        lm_head_gemv_f16_kernel<N, FUSED><<<static_cast<unsigned>(need < cap ? need : cap), kThreads, smem16, q36::stream()>>>(
            w, scales, x, y, rows, static_cast<uint32_t>(cols), row_offset, tokens, best, partials, ticket);
        if (q36::launch_status() != QWEN36_STATUS_SUCCESS) return QWEN36_STATUS_CUDA_ERROR;
        const size_t smem = static_cast<size_t>(N) * cols * 4;
        if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(lm_head_gemv_kernel<N, FUSED, true, true>), 200 * 1024) != cudaSuccess)
          return QWEN36_STATUS_CUDA_ERROR;
        lm_head_gemv_kernel<N, FUSED, true, true><<<grid, kThreads, smem, q36::stream()>>>(
            w, scales, x, y, rows, static_cast<uint32_t>(cols), row_offset, tokens, best, partials, ticket);
        return q36::launch_status();
      }
      return launch_gemv_x<N, FUSED, true>(w, scales, x, y, rows, cols, row_offset, tokens, best, partials, ticket, grid);
    }
  }
  return launch_gemv_x<N, FUSED, false>(w, scales, x, y, rows, cols, row_offset, tokens, best, partials, ticket, grid);
}

template <bool FUSED>
int launch_gemv(size_t n, const uint8_t *w, const float *scales, const __nv_bfloat16 *x, __nv_bfloat16 *y,
                size_t rows, size_t cols, uint32_t row_offset, uint32_t *tokens, float *best, float2 *partials,
                unsigned *ticket, unsigned grid) {
#define Q36_CASE(NN) \
  case NN: return launch_gemv_n<NN, FUSED>(w, scales, x, y, rows, cols, row_offset, tokens, best, partials, ticket, grid);
  switch (n) {
    Q36_CASE(1) Q36_CASE(2) Q36_CASE(3) Q36_CASE(4) Q36_CASE(5) Q36_CASE(6) Q36_CASE(7) Q36_CASE(8)
    Q36_CASE(9) Q36_CASE(10) Q36_CASE(11) Q36_CASE(12) Q36_CASE(13) Q36_CASE(14) Q36_CASE(15) Q36_CASE(16)
    default: return QWEN36_STATUS_INVALID_ARGUMENT;
  }
#undef Q36_CASE
}

// Persistent grid: enough CTAs to fill the GPU, never more than there is work.
unsigned gemv_grid(size_t rows, size_t n, size_t cols) {
  const bool f32 = stage_f32(n, cols);
  const int r = n == 1 ? 4 : (f32 ? (n <= 4 ? 4 : 2) : (n <= 4 ? 2 : 1));
  const size_t need = q36::div_ceil(rows, static_cast<size_t>(kWarps) * r);
  const size_t smem = stage_bytes(n, cols);
  const size_t per_sm = smem > 100 * 1024 ? 1 : (smem > 48 * 1024 ? 2 : 4);
  const size_t cap = static_cast<size_t>(sm_count()) * per_sm;
  return static_cast<unsigned>(need < cap ? need : cap);
}

constexpr size_t kChunkTokens = 8;      // tokens per launch: the float16 route's limit

bool gemv_args_ok(size_t rows, size_t cols, size_t n, uint64_t w, uint64_t s, uint64_t x) {
  // cols % 16: kernels-cuda/lm_head_fp8.cu:594; 16-byte aligned operands for
  // the vector loads (row starts inherit it from cols % 16).
  return rows != 0 && cols != 0 && n != 0 && n <= QWEN36_LM_HEAD_FP8_MAX_N && cols % 16 == 0 && w != 0 &&
         s != 0 && x != 0 && ((w | x) & 15u) == 0 && n * cols * 2 <= 200 * 1024;
}

}  // namespace

extern "C" int qwen36_lm_head_fp8_quantize(const qwen36_lm_head_fp8_quantize_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->rows == 0 || spec->cols == 0 || spec->weight_bf16.ptr == 0 || spec->weight_e4m3.ptr == 0 ||
      spec->row_scales_f32.ptr == 0 || spec->rows > 0x7fffffffull)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  lm_head_quantize_kernel<<<static_cast<unsigned>(spec->rows), kThreads, 0, q36::stream()>>>(
      as_ptr<const __nv_bfloat16>(spec->weight_bf16), as_ptr<uint8_t>(spec->weight_e4m3),
      as_ptr<float>(spec->row_scales_f32), spec->rows, spec->cols);
  return q36::launch_status();
}

extern "C" int qwen36_lm_head_fp8_gemv(const qwen36_lm_head_fp8_gemv_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->output_bf16.ptr == 0 ||
      !gemv_args_ok(spec->rows, spec->cols, spec->n, spec->weight_e4m3.ptr, spec->row_scales_f32.ptr,
                    spec->input_bf16.ptr))
    return QWEN36_STATUS_INVALID_ARGUMENT;
  // More than eight tokens go out as launches of at most eight (the float16 route): 9 tokens cost
  // 552 + 206 us that way against 1264 us in one pass of the many-token kernel, 16 cost 1105 against 2425.
  for (size_t t0 = 0; t0 < spec->n; t0 += kChunkTokens) {
    const size_t nt = spec->n - t0 < kChunkTokens ? spec->n - t0 : kChunkTokens;
    const int rc = launch_gemv<false>(nt, as_ptr<const uint8_t>(spec->weight_e4m3), as_ptr<const float>(spec->row_scales_f32),
                                      as_ptr<const __nv_bfloat16>(spec->input_bf16) + t0 * spec->cols,
                                      as_ptr<__nv_bfloat16>(spec->output_bf16) + t0 * spec->rows, spec->rows, spec->cols, 0u,
                                      nullptr, nullptr, nullptr, nullptr, gemv_grid(spec->rows, nt, spec->cols));
    if (rc != QWEN36_STATUS_SUCCESS) return rc;
  }
  return QWEN36_STATUS_SUCCESS;
}

extern "C" size_t qwen36_lm_head_fp8_argmax_workspace_bytes(size_t rows, size_t n) {
  (void)rows;
  // ticket word (padded to 16 bytes) + one (value, index) pair per CTA per token
  return 16 + static_cast<size_t>(148 * 4) * 8 * (n == 0 ? 1 : n);
}

extern "C" int qwen36_lm_head_fp8_gemv_argmax(const qwen36_lm_head_fp8_argmax_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->output_token_u32.ptr == 0 || spec->workspace.ptr == 0 || (spec->workspace.ptr & 15u) != 0 ||
      !gemv_args_ok(spec->rows, spec->cols, spec->n, spec->weight_e4m3.ptr, spec->row_scales_f32.ptr,
                    spec->input_bf16.ptr))
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const size_t slots = (spec->workspace_bytes < 16 ? 0 : spec->workspace_bytes - 16) / (8 * spec->n);
  if (slots == 0) return QWEN36_STATUS_INVALID_ARGUMENT;
  // launches of at most eight tokens, as above; they follow one another on the stream, so they share
  // the ticket (it is back at zero when a launch ends) and the winners' slots
  for (size_t t0 = 0; t0 < spec->n; t0 += kChunkTokens) {
    const size_t nt = spec->n - t0 < kChunkTokens ? spec->n - t0 : kChunkTokens;
    unsigned grid = gemv_grid(spec->rows, nt, spec->cols);
    if (grid > slots) grid = static_cast<unsigned>(slots);
    float *best = as_ptr<float>(spec->best_value_f32);
    const int rc = launch_gemv<true>(nt, as_ptr<const uint8_t>(spec->weight_e4m3), as_ptr<const float>(spec->row_scales_f32),
                                     as_ptr<const __nv_bfloat16>(spec->input_bf16) + t0 * spec->cols, nullptr, spec->rows,
                                     spec->cols, spec->row_offset, as_ptr<uint32_t>(spec->output_token_u32) + t0,
                                     best == nullptr ? nullptr : best + t0,
                                     reinterpret_cast<float2 *>(static_cast<uintptr_t>(spec->workspace.ptr + 16)),
                                     as_ptr<unsigned>(spec->workspace), grid);
    if (rc != QWEN36_STATUS_SUCCESS) return rc;
  }
  return QWEN36_STATUS_SUCCESS;
}

extern "C" int qwen36_sample(const qwen36_sampling_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->vocab_size == 0 || spec->logits_bf16.ptr == 0 || spec->output_token_u32.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  return launch_argmax(as_ptr<const __nv_bfloat16>(spec->logits_bf16), as_ptr<uint32_t>(spec->output_token_u32),
                       as_ptr<uint32_t>(spec->mirror_output_token_u32), 1, spec->vocab_size, spec->temperature);
}

extern "C" int qwen36_sample_rows(const qwen36_sampling_rows_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->rows == 0 || spec->vocab_size == 0 || spec->logits_bf16.ptr == 0 || spec->output_token_u32.ptr == 0 ||
      spec->rows > (1u << 24))
    return QWEN36_STATUS_INVALID_ARGUMENT;
  return launch_argmax(as_ptr<const __nv_bfloat16>(spec->logits_bf16), as_ptr<uint32_t>(spec->output_token_u32),
                       as_ptr<uint32_t>(spec->mirror_last_output_token_u32), spec->rows, spec->vocab_size,
                       spec->temperature);
}

// Test hook: 1 keeps 2..8-token calls on the float32-staged kernel alone, 0 restores the default
// (float16 route with the float32 route behind it).
extern "C" void qwen36_lm_head_fp8_gemv_set_route(int route) { g_gemv_route.store(route != 0 ? 1 : 0); }
