// Exact-argmax guards of the FP8 lm_head (two-stage greedy decode):
//   qwen36_lm_head_top2_margin     : per row top-1 token + "top1 - top2 >= eps" verdict over bf16 logits
//   qwen36_lm_head_top8_rescore    : top-8 block winners rescored against the bf16 weight in float64
//   qwen36_bf16_matvec_argmax_rows : predicated full bf16 lm_head + argmax for the rows whose guard failed
// (reference: kernels-cuda/lm_head_fp8.cu:203-494,528-590 and kernels-cuda/ops.cu:19-37,453-515,1104-1153).
//
// The verdicts are defined by the reference's arithmetic, which these kernels keep: the 240-block
// strided partition of the vocabulary whose block winners are the top-8 candidates, float64 lane
// partials met by a shuffle-down tree for the rescore, float32 lane-strided partials met by the
// same tree for the bf16 matvec, the (ordered float, 0xffffffff - token) key for its argmax.
// What changes is how the bytes move: the scan reads 16 bytes per lane, and the bf16 lm_head makes
// ONE pass over the 2.5 GB weight for all rows that still need it (the reference re-reads the
// weight once per row), with the activations staged as float32 in shared memory.
#include "common.cuh"
#include "kv_split.cuh"

#include <math.h>

namespace {

using q36::as_ptr;

constexpr uint32_t kBlocks = QWEN36_LM_HEAD_TOP2_BLOCKS;     // vocabulary partition of the scan
constexpr uint32_t kThreads = 256;
constexpr uint32_t kNoToken = 0xffffffffu;

struct Top2 {
  float v1, v2;
  uint32_t i1;
};
struct WsEntry {      // 16 bytes per (row, block): the reference's workspace layout
  float v1, v2;
  uint32_t i1, pad;
};

// Keeps the best value (lowest index among equals) and the second-best value of the multiset.
__device__ __forceinline__ void consider(Top2 &t, float v, uint32_t i) {
  if (v > t.v1 || (v == t.v1 && i < t.i1)) {
    t.v2 = t.v1;
    t.v1 = v;
    t.i1 = i;
  } else if (v > t.v2) {
    t.v2 = v;
  }
}
__device__ __forceinline__ void merge(Top2 &t, const Top2 &o) {
  if (o.v1 > t.v1 || (o.v1 == t.v1 && o.i1 < t.i1)) {
    t.v2 = fmaxf(t.v1, o.v2);
    t.v1 = o.v1;
    t.i1 = o.i1;
  } else {
    t.v2 = fmaxf(t.v2, o.v1);
  }
}
__device__ __forceinline__ Top2 warp_merge(Top2 mine) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    Top2 other;
    other.v1 = __shfl_down_sync(0xffffffffu, mine.v1, off);
    other.v2 = __shfl_down_sync(0xffffffffu, mine.v2, off);
    other.i1 = __shfl_down_sync(0xffffffffu, mine.i1, off);
    merge(mine, other);
  }
  return mine;
}
// Result valid in thread 0.
__device__ __forceinline__ Top2 block_merge(Top2 mine, Top2 *warp_smem) {
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  mine = warp_merge(mine);
  if (lane == 0) warp_smem[warp] = mine;
  __syncthreads();
  if (warp == 0) {
    mine = lane < kThreads / 32 ? warp_smem[lane] : Top2{-INFINITY, -INFINITY, kNoToken};
    mine = warp_merge(mine);
  }
  return mine;
}

// Block b of a row owns the 256-token chunks b, b + 240, b + 480, ... (the reference's thread
// striding, kernels-cuda/lm_head_fp8.cu:283-301).  Here one warp takes a chunk at a time and a lane
// reads eight consecutive logits with one 16-byte load.
__global__ void __launch_bounds__(kThreads)
top2_scan_kernel(const __nv_bfloat16 *__restrict__ logits, WsEntry *__restrict__ ws, size_t vocab) {
  asm volatile("griddepcontrol.wait;" ::: "memory");               // launched with programmatic stream serialisation
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ Top2 warp_smem[kThreads / 32];
  const size_t row = blockIdx.y;
  const __nv_bfloat16 *row_logits = logits + row * vocab;
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const bool vec = (reinterpret_cast<uintptr_t>(row_logits) & 15u) == 0;
  Top2 mine{-INFINITY, -INFINITY, kNoToken};
  for (size_t chunk = blockIdx.x + static_cast<size_t>(warp) * kBlocks; chunk * 256 < vocab;
       chunk += static_cast<size_t>(kBlocks) * (kThreads / 32)) {
    const size_t base = chunk * 256 + lane * 8u;
    if (vec && base + 8 <= vocab) {
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(row_logits + base));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        consider(mine, __uint_as_float(w[i] << 16), static_cast<uint32_t>(base + 2 * i));
        consider(mine, __uint_as_float(w[i] & 0xffff0000u), static_cast<uint32_t>(base + 2 * i + 1));
      }
    } else {
      for (uint32_t i = 0; i < 8 && base + i < vocab; ++i)
        consider(mine, __bfloat162float(row_logits[base + i]), static_cast<uint32_t>(base + i));
    }
  }
  mine = block_merge(mine, warp_smem);
  if (threadIdx.x == 0) ws[row * kBlocks + blockIdx.x] = WsEntry{mine.v1, mine.v2, mine.i1, 0u};
}

__global__ void __launch_bounds__(kThreads)
top2_verdict_kernel(const WsEntry *__restrict__ ws, uint32_t *__restrict__ tokens, uint32_t *__restrict__ flags,
                    uint32_t *__restrict__ mirror_last, uint32_t *__restrict__ fallback_count, size_t rows, float eps) {
  asm volatile("griddepcontrol.wait;" ::: "memory");               // launched with programmatic stream serialisation
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ Top2 warp_smem[kThreads / 32];
  const size_t row = blockIdx.x;
  Top2 mine{-INFINITY, -INFINITY, kNoToken};
  for (uint32_t b = threadIdx.x; b < kBlocks; b += kThreads) {
    const WsEntry e = ws[row * kBlocks + b];
    merge(mine, Top2{e.v1, e.v2, e.i1});
  }
  mine = block_merge(mine, warp_smem);
  if (threadIdx.x == 0) {
    const bool ok = (mine.v1 - mine.v2) >= eps;
    tokens[row] = mine.i1;
    flags[row] = ok ? 1u : 0u;
    if (mirror_last != nullptr && row + 1 == rows) *mirror_last = mine.i1;
    if (!ok && fallback_count != nullptr) atomicAdd(fallback_count, 1u);
  }
}

constexpr int kCandidates = 8;

// One CTA per row (kernels-cuda/lm_head_fp8.cu:338-494): the eight best block winners are the
// candidates, everything else is bounded by B = max(ninth winner, best block runner-up); warp w
// recomputes candidate w's logit from the bf16 weight in float64; the verdict is
// best >= B + eps.
__global__ void __launch_bounds__(kThreads)
top8_rescore_kernel(const WsEntry *__restrict__ ws, const __nv_bfloat16 *__restrict__ weight,
                    const __nv_bfloat16 *__restrict__ input, uint32_t *__restrict__ tokens,
                    uint32_t *__restrict__ flags, uint32_t *__restrict__ mirror_last,
                    uint32_t *__restrict__ fallback_count, size_t rows, size_t vocab, size_t cols, float eps,
                    uint32_t staged) {
  // staged: a cluster of eight CTAs serves a row.  Every CTA repeats the (cheap, deterministic)
  // extraction; CTA r then recomputes candidate r alone, one warp with the float64 units of an SM to
  // itself, and leaves its sum in the first CTA's shared memory, which gives the verdict.  The sum is
  // a chain of cols / 32 dependent float64 multiply-adds per lane in the reference's order (about
  // 4 us at 5120 columns), which no layout shortens.  The activation row and the candidate's weight
  // row travel into shared memory by cp.async (all of a row's copies in flight at once; the row's
  // address is only known after the extraction) and the sum reads them from there.
  extern __shared__ __align__(16) uint8_t rows_smem[];               // [2][cols] bf16 when staged
  __shared__ float winner_v[kBlocks];
  __shared__ uint32_t winner_i[kBlocks];
  __shared__ float warp_max_v2[kThreads / 32];
  __shared__ uint32_t cand_i[kCandidates];
  __shared__ float ninth_v;
  __shared__ double rescored[kCandidates];
  uint32_t rank = 0;
  if (staged) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const size_t row = staged ? blockIdx.x / kCandidates : blockIdx.x;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  asm volatile("griddepcontrol.wait;" ::: "memory");               // launched with programmatic stream serialisation
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (staged) {
    const __nv_bfloat16 *x_row = input + row * cols;
    for (size_t c = static_cast<size_t>(threadIdx.x) * 8; c < cols; c += static_cast<size_t>(kThreads) * 8)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(rows_smem + c * 2))),
                   "l"(x_row + c) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  float max_v2 = -INFINITY;
  for (uint32_t b = threadIdx.x; b < kBlocks; b += kThreads) {
    const WsEntry e = ws[row * kBlocks + b];
    winner_v[b] = e.v1;
    winner_i[b] = e.i1;
    max_v2 = fmaxf(max_v2, e.v2);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) max_v2 = fmaxf(max_v2, __shfl_down_sync(0xffffffffu, max_v2, off));
  if (lane == 0) warp_max_v2[warp] = max_v2;
  __syncthreads();

  if (warp == 0) {
    // Nine extractions of the maximum (ties toward the smaller token; -inf and NaN are never taken,
    // as in the reference's scan).  Every block winner becomes a 64-bit key, value bits made monotonic
    // on top and the complemented token below, eight keys per lane in registers; an extraction is
    // a local maximum and two warp reductions, and the owner clears its key.
    constexpr uint32_t kPerLane = (kBlocks + 31) / 32;
    uint32_t key_hi[kPerLane], key_lo[kPerLane];
#pragma unroll
    for (uint32_t i = 0; i < kPerLane; ++i) {
      const uint32_t b = lane + 32u * i;
      key_hi[i] = 0u;
      key_lo[i] = 0u;
      if (b < kBlocks) {
        const float v = winner_v[b];
        const uint32_t bits = __float_as_uint(v);
        if (v == v && v != -INFINITY) {
          key_hi[i] = (bits & 0x80000000u) != 0u ? ~bits : (bits | 0x80000000u);
          key_lo[i] = ~winner_i[b];
        }
      }
    }
    for (int k = 0; k <= kCandidates; ++k) {
      uint32_t hi = 0u, lo = 0u;
#pragma unroll
      for (uint32_t i = 0; i < kPerLane; ++i)
        if (key_hi[i] > hi || (key_hi[i] == hi && key_lo[i] > lo)) { hi = key_hi[i]; lo = key_lo[i]; }
      const uint32_t top_hi = __reduce_max_sync(0xffffffffu, hi);
      const uint32_t top_lo = __reduce_max_sync(0xffffffffu, hi == top_hi ? lo : 0u);
      if (top_hi != 0u) {
#pragma unroll
        for (uint32_t i = 0; i < kPerLane; ++i)
          if (key_hi[i] == top_hi && key_lo[i] == top_lo) key_hi[i] = key_lo[i] = 0u;     // tokens are unique: one owner
      }
      if (lane == 0) {
        if (k < kCandidates) {
          cand_i[k] = top_hi == 0u ? kNoToken : ~top_lo;
        } else {
          ninth_v = top_hi == 0u ? -INFINITY
                                 : __uint_as_float((top_hi & 0x80000000u) != 0u ? (top_hi & 0x7fffffffu) : ~top_hi);
        }
      }
    }
  }
  if (staged) asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  if (staged ? warp == 0u : warp < kCandidates) {
    const uint32_t which = staged ? rank : warp;                    // the candidate this warp recomputes
    const uint32_t cand = cand_i[which];
    double sum = 0.0;
    if (staged && cand != kNoToken && static_cast<size_t>(cand) < vocab) {
      const __nv_bfloat16 *w_row = weight + static_cast<size_t>(cand) * cols;
      const __nv_bfloat16 *xs = reinterpret_cast<const __nv_bfloat16 *>(rows_smem);
      __nv_bfloat16 *wsm = reinterpret_cast<__nv_bfloat16 *>(rows_smem) + cols;
      for (size_t c = static_cast<size_t>(lane) * 8; c < cols; c += 256)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(wsm + c))),
                     "l"(w_row + c) : "memory");
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncwarp();
      // bf16 -> float64 on the integer units where the value is zero or a normal number (sign, exponent
      // rebased by 896, seven fraction bits on top of the 52): the conversion instructions share the
      // float64 pipe, which a single warp cannot afford twice per product
      const uint16_t *wb = reinterpret_cast<const uint16_t *>(wsm), *xb = reinterpret_cast<const uint16_t *>(xs);
      auto widen = [](uint32_t b) -> double {
        const uint32_t mag = b & 0x7fffu, e = mag >> 7;
        if (e - 1u < 254u || mag == 0u) {
          const uint32_t hi = ((b & 0x8000u) << 16) | (mag == 0u ? 0u : (mag << 13) + 0x38000000u);
          return __hiloint2double(static_cast<int>(hi), 0);
        }
        return static_cast<double>(__uint_as_float(b << 16));       // subnormal, infinity, NaN
      };
      for (size_t c = lane; c < cols; c += 32u) sum += widen(wb[c]) * widen(xb[c]);
    } else if (cand != kNoToken && static_cast<size_t>(cand) < vocab) {
      const __nv_bfloat16 *w_row = weight + static_cast<size_t>(cand) * cols;
      const __nv_bfloat16 *x_row = input + row * cols;
      // Same elements per lane, same order of additions as a plain strided loop; the loads of eighty
      // steps go out together (a plain loop pays one round trip to memory every few steps, and the
      // row's address is only known here).
      constexpr uint32_t kBatch = 80;
      for (size_t c0 = lane; c0 < cols; c0 += 32u * kBatch) {
        __nv_bfloat16 wv[kBatch], xv[kBatch];
#pragma unroll
        for (uint32_t i = 0; i < kBatch; ++i) {
          const size_t c = c0 + 32u * i;
          wv[i] = c < cols ? w_row[c] : __float2bfloat16(0.0f);
          xv[i] = c < cols ? x_row[c] : __float2bfloat16(0.0f);
        }
#pragma unroll
        for (uint32_t i = 0; i < kBatch; ++i)
          if (c0 + 32u * i < cols)
            sum += static_cast<double>(__bfloat162float(wv[i])) * static_cast<double>(__bfloat162float(xv[i]));
      }
    } else {
      sum = -INFINITY;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, off);
    if (lane == 0) {
      const double mine = cand == kNoToken ? -INFINITY : sum;
      if (staged) {
        uint32_t remote;                                              // rescored[which] of the cluster's first CTA
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote)
                     : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(&rescored[which]))), "r"(0u));
        asm volatile("st.shared::cluster.f64 [%0], %1;" ::"r"(remote), "d"(mine) : "memory");
      } else {
        rescored[which] = mine;
      }
    }
  }
  if (staged) {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (rank != 0u) return;
  } else {
    __syncthreads();
  }

  if (threadIdx.x == 0) {
    double best = -INFINITY;
    uint32_t best_token = 0;
    for (int k = 0; k < kCandidates; ++k) {
      const double v = rescored[k];
      const uint32_t tok = cand_i[k];
      if (tok != kNoToken && (v > best || (v == best && tok < best_token))) {
        best = v;
        best_token = tok;
      }
    }
    float bound = ninth_v;
    for (uint32_t w = 0; w < kThreads / 32; ++w) bound = fmaxf(bound, warp_max_v2[w]);
    const bool ok = best >= static_cast<double>(bound) + static_cast<double>(eps);
    tokens[row] = best_token;
    flags[row] = ok ? 1u : 0u;
    if (mirror_last != nullptr && row + 1 == rows) *mirror_last = best_token;
    if (!ok && fallback_count != nullptr) atomicAdd(fallback_count, 1u);
  }
}

// ---- predicated bf16 lm_head + argmax -------------------------------------------------------

constexpr int kMaxActive = 8;          // rows handled per pass over the weight
// Vocabulary rows a warp carries at once and column steps per software-pipeline batch.  Few rows
// for a single token (small register footprint, many resident warps), more rows when several
// tokens share every weight load.
template <int N> struct ArgmaxShape {
  static constexpr int kVocab = N == 1 ? 1 : (N <= 4 ? 4 : 8);
  static constexpr int kSteps = N == 1 ? 16 : 4;
};

__device__ __forceinline__ unsigned long long argmax_key(float score, uint32_t token) {
  if (!isfinite(score)) return 0ull;
  const uint32_t bits = __float_as_uint(score);
  const uint32_t ordered = (bits & 0x80000000u) != 0u ? ~bits : (bits ^ 0x80000000u);
  return (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - token);
}

// One pass over the weight for up to N rows that still need the bf16 answer.  Lane l accumulates
// columns l, l + 32, ... in float32 in that order and the lanes meet in a shuffle-down tree: the
// logit of every (row, token) pair has the reference's bits (kernels-cuda/ops.cu:474-487).
template <int N>
__global__ void __launch_bounds__(kThreads)
bf16_argmax_kernel(const __nv_bfloat16 *__restrict__ input, const __nv_bfloat16 *__restrict__ weight,
                   unsigned long long *__restrict__ best_keys, const uint32_t *__restrict__ skip_flags,
                   size_t rows, size_t row_base, size_t out_features, uint32_t in_features) {
  extern __shared__ __align__(16) float xs[];                // [N][in_features]
  __shared__ int active_row[N];
  __shared__ int n_active;
  if (threadIdx.x == 0) {
    int n = 0;
    for (size_t r = row_base; r < rows && n < N; ++r)
      if (skip_flags == nullptr || skip_flags[r] == 0u) active_row[n++] = static_cast<int>(r - row_base);
    // rows beyond the N-th active one belong to the next pass: they are found again from row_base + last + 1
    n_active = n;
  }
  __syncthreads();
  const int n_act = n_active;
  if (n_act == 0) return;
  for (int t = 0; t < n_act; ++t) {
    const __nv_bfloat16 *x_row = input + (row_base + active_row[t]) * in_features;
    for (uint32_t c = threadIdx.x; c < in_features; c += kThreads) xs[t * in_features + c] = __bfloat162float(x_row[c]);
  }
  __syncthreads();

  constexpr int kVocabPerWarp = ArgmaxShape<N>::kVocab;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const size_t warps_total = static_cast<size_t>(gridDim.x) * (kThreads / 32);
  unsigned long long best[N];
#pragma unroll
  for (int t = 0; t < N; ++t) best[t] = 0ull;

  for (size_t v0 = (static_cast<size_t>(blockIdx.x) * (kThreads / 32) + warp) * kVocabPerWarp; v0 < out_features;
       v0 += warps_total * kVocabPerWarp) {
    float acc[kVocabPerWarp][N];
#pragma unroll
    for (int r = 0; r < kVocabPerWarp; ++r)
#pragma unroll
      for (int t = 0; t < N; ++t) acc[r][t] = 0.f;
    const unsigned short *w0 = reinterpret_cast<const unsigned short *>(weight) + v0 * in_features;
    // Column steps of 32 (lane l owns column l of each step), software-pipelined kSteps at a time:
    // the 2-byte loads of the next batch are in flight while the current one is multiplied.
    constexpr int kSteps = ArgmaxShape<N>::kSteps;
    const uint32_t steps = (in_features + 31u) / 32u;
    unsigned short cur[kSteps][kVocabPerWarp], nxt[kSteps][kVocabPerWarp];
    auto load_batch = [&](unsigned short (&dst)[kSteps][kVocabPerWarp], uint32_t s0) {
#pragma unroll
      for (int u = 0; u < kSteps; ++u) {
        const uint32_t col = (s0 + u) * 32u + lane;
#pragma unroll
        for (int r = 0; r < kVocabPerWarp; ++r)
          dst[u][r] = (col < in_features && v0 + r < out_features)
                          ? __ldcs(w0 + static_cast<size_t>(r) * in_features + col) : static_cast<unsigned short>(0);
      }
    };
    load_batch(cur, 0);
    for (uint32_t s0 = 0; s0 < steps; s0 += kSteps) {
      if (s0 + kSteps < steps) load_batch(nxt, s0 + kSteps);
#pragma unroll
      for (int u = 0; u < kSteps; ++u) {
        const uint32_t col = (s0 + u) * 32u + lane;
        if (col < in_features) {                            // no padding terms: the sums keep the reference's bits
#pragma unroll
          for (int t = 0; t < N; ++t) {
            const float x = xs[t * in_features + col];
#pragma unroll
            for (int r = 0; r < kVocabPerWarp; ++r)
              acc[r][t] = fmaf(x, __uint_as_float(static_cast<uint32_t>(cur[u][r]) << 16), acc[r][t]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kSteps; ++u)
#pragma unroll
        for (int r = 0; r < kVocabPerWarp; ++r) cur[u][r] = nxt[u][r];
    }
#pragma unroll
    for (int r = 0; r < kVocabPerWarp; ++r) {
      if (v0 + r >= out_features) break;
#pragma unroll
      for (int t = 0; t < N; ++t) {
        float s = acc[r][t];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
        const unsigned long long key = argmax_key(s, static_cast<uint32_t>(v0 + r));
        if (key > best[t]) best[t] = key;
      }
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int t = 0; t < N; ++t)
      if (t < n_act && best[t] != 0ull) atomicMax(best_keys + row_base + active_row[t], best[t]);
  }
}

// Same sums, faster bytes: for in_features % 256 == 0 and 16-byte aligned rows.  A warp fetches
// 256 columns of a vocabulary row with one 16-byte load per lane, parks them in a warp-private
// shared-memory tile, and every lane then picks up ITS columns (lane, lane + 32, ...) as 2-byte
// shared-memory reads, so lane l still adds columns l, l + 32, l + 64, ... in that order.
constexpr int kFastRows = 4;           // vocabulary rows per warp

template <int N>
__global__ void __launch_bounds__(kThreads)
bf16_argmax_fast_kernel(const __nv_bfloat16 *__restrict__ input, const __nv_bfloat16 *__restrict__ weight,
                        unsigned long long *__restrict__ best_keys, const uint32_t *__restrict__ skip_flags,
                        size_t rows, size_t row_base, size_t out_features, uint32_t in_features) {
  extern __shared__ __align__(16) float xs_raw[];
  float *xs = xs_raw;                                                    // [N][in_features]
  uint4 *tiles = reinterpret_cast<uint4 *>(xs_raw + static_cast<size_t>(N) * in_features);   // [warps][kFastRows][32]
  __shared__ int active_row[N];
  __shared__ int n_active;
  if (threadIdx.x == 0) {
    int n = 0;
    for (size_t r = row_base; r < rows && n < N; ++r)
      if (skip_flags == nullptr || skip_flags[r] == 0u) active_row[n++] = static_cast<int>(r - row_base);
    n_active = n;
  }
  __syncthreads();
  const int n_act = n_active;
  if (n_act == 0) return;
  for (int t = 0; t < n_act; ++t) {
    const __nv_bfloat16 *x_row = input + (row_base + active_row[t]) * in_features;
    for (uint32_t c = threadIdx.x; c < in_features; c += kThreads) xs[t * in_features + c] = __bfloat162float(x_row[c]);
  }
  __syncthreads();

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  uint4 *tile = tiles + warp * (kFastRows * 32);
  const unsigned short *tile16 = reinterpret_cast<const unsigned short *>(tile);
  const size_t warps_total = static_cast<size_t>(gridDim.x) * (kThreads / 32);
  const uint32_t chunks = in_features / 256u;
  unsigned long long best[N];
#pragma unroll
  for (int t = 0; t < N; ++t) best[t] = 0ull;

  for (size_t v0 = (static_cast<size_t>(blockIdx.x) * (kThreads / 32) + warp) * kFastRows; v0 < out_features;
       v0 += warps_total * kFastRows) {
    float acc[kFastRows][N];
#pragma unroll
    for (int r = 0; r < kFastRows; ++r)
#pragma unroll
      for (int t = 0; t < N; ++t) acc[r][t] = 0.f;
    const uint4 *w0 = reinterpret_cast<const uint4 *>(weight + v0 * in_features) + lane;
    const size_t row_stride = in_features / 8u;                         // uint4 per vocabulary row
    uint4 cur[kFastRows], nxt[kFastRows];
    auto load_chunk = [&](uint4 (&dst)[kFastRows], uint32_t c) {
#pragma unroll
      for (int r = 0; r < kFastRows; ++r)
        dst[r] = v0 + r < out_features ? __ldcs(w0 + static_cast<size_t>(r) * row_stride + c * 32u) : make_uint4(0, 0, 0, 0);
    };
    load_chunk(cur, 0);
    for (uint32_t c = 0; c < chunks; ++c) {
      if (c + 1 < chunks) load_chunk(nxt, c + 1);
      __syncwarp();                                                      // the previous chunk's reads are done
#pragma unroll
      for (int r = 0; r < kFastRows; ++r) tile[r * 32 + lane] = cur[r];
      __syncwarp();
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const uint32_t col = c * 256u + m * 32u + lane;
        float w[kFastRows];
#pragma unroll
        for (int r = 0; r < kFastRows; ++r)
          w[r] = __uint_as_float(static_cast<uint32_t>(tile16[r * 256 + m * 32 + lane]) << 16);
#pragma unroll
        for (int t = 0; t < N; ++t) {
          const float x = xs[t * in_features + col];
#pragma unroll
          for (int r = 0; r < kFastRows; ++r) acc[r][t] = fmaf(x, w[r], acc[r][t]);
        }
      }
#pragma unroll
      for (int r = 0; r < kFastRows; ++r) cur[r] = nxt[r];
    }
#pragma unroll
    for (int r = 0; r < kFastRows; ++r) {
      if (v0 + r >= out_features) break;
#pragma unroll
      for (int t = 0; t < N; ++t) {
        float sum = acc[r][t];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, off);
        const unsigned long long key = argmax_key(sum, static_cast<uint32_t>(v0 + r));
        if (key > best[t]) best[t] = key;
      }
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int t = 0; t < N; ++t)
      if (t < n_act && best[t] != 0ull) atomicMax(best_keys + row_base + active_row[t], best[t]);
  }
}

__global__ void bf16_argmax_finalize_kernel(const unsigned long long *__restrict__ best_keys,
                                            uint32_t *__restrict__ tokens, uint32_t *__restrict__ mirror_last,
                                            const uint32_t *__restrict__ skip_flags, size_t rows) {
  const size_t row = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  if (skip_flags != nullptr && skip_flags[row] != 0u) return;      // the stage-1 token stands
  const unsigned long long key = best_keys[row];
  const uint32_t token = key == 0ull ? 0u : 0xffffffffu - static_cast<uint32_t>(key & 0xffffffffull);
  tokens[row] = token;
  if (mirror_last != nullptr && row + 1 == rows) *mirror_last = token;
}

int sm_count() { return q36::sm_count_current_device(); }

template <int N>
int launch_bf16_argmax_fast(const qwen36_bf16_matvec_argmax_rows_spec_t *s, size_t row_base) {
  const size_t smem = static_cast<size_t>(N) * s->in_features * sizeof(float) + (kThreads / 32) * kFastRows * 512;
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(bf16_argmax_fast_kernel<N>), 220 * 1024) != cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  const size_t need = q36::div_ceil(s->out_features, static_cast<size_t>(kThreads / 32) * kFastRows);
  const size_t per_sm = smem > 100 * 1024 ? 1 : (smem > 70 * 1024 ? 2 : (smem > 52 * 1024 ? 3 : (smem > 40 * 1024 ? 4 : 5)));
  const size_t cap = static_cast<size_t>(sm_count()) * per_sm;
  bf16_argmax_fast_kernel<N><<<static_cast<unsigned>(need < cap ? need : cap), kThreads, smem, q36::stream()>>>(
      as_ptr<const __nv_bfloat16>(s->input_bf16), as_ptr<const __nv_bfloat16>(s->weight_bf16),
      as_ptr<unsigned long long>(s->workspace), as_ptr<const uint32_t>(s->skip_flags_u32), s->rows, row_base,
      s->out_features, static_cast<uint32_t>(s->in_features));
  return q36::launch_status();
}

template <int N>
int launch_bf16_argmax(const qwen36_bf16_matvec_argmax_rows_spec_t *s, size_t row_base) {
  if (s->in_features % 256 == 0 && (s->weight_bf16.ptr & 15u) == 0) return launch_bf16_argmax_fast<N>(s, row_base);
  const size_t smem = static_cast<size_t>(N) * s->in_features * sizeof(float);
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(bf16_argmax_kernel<N>), 200 * 1024) != cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  const size_t need = q36::div_ceil(s->out_features, static_cast<size_t>(kThreads / 32) * ArgmaxShape<N>::kVocab);
  const size_t per_sm = smem > 100 * 1024 ? 1 : (smem > 48 * 1024 ? 2 : (smem > 24 * 1024 ? 4 : 8));
  const size_t cap = static_cast<size_t>(sm_count()) * per_sm;
  bf16_argmax_kernel<N><<<static_cast<unsigned>(need < cap ? need : cap), kThreads, smem, q36::stream()>>>(
      as_ptr<const __nv_bfloat16>(s->input_bf16), as_ptr<const __nv_bfloat16>(s->weight_bf16),
      as_ptr<unsigned long long>(s->workspace), as_ptr<const uint32_t>(s->skip_flags_u32), s->rows, row_base,
      s->out_features, static_cast<uint32_t>(s->in_features));
  return q36::launch_status();
}

bool guard_args_ok(size_t rows, size_t vocab, uint64_t logits, uint64_t tokens, uint64_t flags, uint64_t ws,
                   size_t ws_bytes) {
  return rows != 0 && vocab != 0 && logits != 0 && tokens != 0 && flags != 0 && ws != 0 &&
         ws_bytes >= rows * kBlocks * sizeof(WsEntry) && rows <= 65535 && vocab <= 0xffffffffull;
}

}  // namespace

extern "C" int qwen36_lm_head_top2_margin(const qwen36_lm_head_top2_margin_spec_t *spec) {
  if (spec == nullptr || !guard_args_ok(spec->rows, spec->vocab, spec->logits_bf16.ptr, spec->tokens_u32.ptr,
                                        spec->flags_u32.ptr, spec->workspace.ptr, spec->workspace_bytes))
    return QWEN36_STATUS_INVALID_ARGUMENT;                  // also for a null spec, as the reference does
  if (q36::launch_after_previous(top2_scan_kernel, dim3(kBlocks, static_cast<unsigned>(spec->rows)), dim3(kThreads), size_t{0},
                                 q36::stream(), as_ptr<const __nv_bfloat16>(spec->logits_bf16),
                                 as_ptr<WsEntry>(spec->workspace), spec->vocab) != cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  return q36::cuda_status(q36::launch_after_previous(
      top2_verdict_kernel, dim3(static_cast<unsigned>(spec->rows)), dim3(kThreads), size_t{0}, q36::stream(),
      as_ptr<const WsEntry>(spec->workspace), as_ptr<uint32_t>(spec->tokens_u32), as_ptr<uint32_t>(spec->flags_u32),
      as_ptr<uint32_t>(spec->mirror_last_token_u32), as_ptr<uint32_t>(spec->fallback_count_u32), spec->rows, spec->eps));
}

extern "C" int qwen36_lm_head_top8_rescore(const qwen36_lm_head_top8_rescore_spec_t *spec) {
  if (spec == nullptr || spec->cols == 0 || spec->weight_bf16.ptr == 0 || spec->input_bf16.ptr == 0 ||
      !guard_args_ok(spec->rows, spec->vocab, spec->logits_bf16.ptr, spec->tokens_u32.ptr, spec->flags_u32.ptr,
                     spec->workspace.ptr, spec->workspace_bytes))
    return QWEN36_STATUS_INVALID_ARGUMENT;
  if (q36::launch_after_previous(top2_scan_kernel, dim3(kBlocks, static_cast<unsigned>(spec->rows)), dim3(kThreads), size_t{0},
                                 q36::stream(), as_ptr<const __nv_bfloat16>(spec->logits_bf16),
                                 as_ptr<WsEntry>(spec->workspace), spec->vocab) != cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  // a cluster of eight CTAs per row, rows through shared memory, when they are made of whole 16-byte
  // pieces and two of them fit
  const size_t stage_bytes = 2 * spec->cols * sizeof(__nv_bfloat16);
  const bool staged = spec->cols % 8 == 0 && ((spec->weight_bf16.ptr | spec->input_bf16.ptr) & 15u) == 0 &&
                      stage_bytes <= 200 * 1024 && spec->rows <= (1u << 24) &&
                      q36::ensure_dynamic_smem(reinterpret_cast<const void *>(top8_rescore_kernel), 200 * 1024) == cudaSuccess;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(spec->rows) * (staged ? kCandidates : 1));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = staged ? stage_bytes : 0;
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = staged ? kCandidates : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return q36::cuda_status(cudaLaunchKernelEx(
      &cfg, top8_rescore_kernel, as_ptr<const WsEntry>(spec->workspace), as_ptr<const __nv_bfloat16>(spec->weight_bf16),
      as_ptr<const __nv_bfloat16>(spec->input_bf16), as_ptr<uint32_t>(spec->tokens_u32), as_ptr<uint32_t>(spec->flags_u32),
      as_ptr<uint32_t>(spec->mirror_last_token_u32), as_ptr<uint32_t>(spec->fallback_count_u32),
      static_cast<size_t>(spec->rows), static_cast<size_t>(spec->vocab), static_cast<size_t>(spec->cols), spec->eps,
      staged ? 1u : 0u));
}

extern "C" int qwen36_bf16_matvec_argmax_rows(const qwen36_bf16_matvec_argmax_rows_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->rows == 0 || spec->out_features == 0 || spec->in_features == 0 || spec->input_bf16.ptr == 0 ||
      spec->weight_bf16.ptr == 0 || spec->output_token_u32.ptr == 0 || spec->workspace.ptr == 0 ||
      spec->workspace_bytes < spec->rows * sizeof(unsigned long long) || spec->out_features > 0xffffffffull ||
      spec->in_features * sizeof(float) > 200 * 1024)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  if (cudaMemsetAsync(as_ptr<void>(spec->workspace), 0, spec->rows * sizeof(unsigned long long), q36::stream()) !=
      cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  // Rows per pass: as many as the float32 staging of their activations allows (at most eight).
  // Every pass skips flagged rows itself, so a pass over rows that are all flagged reads nothing.
  size_t per_pass = (200 * 1024) / (spec->in_features * sizeof(float));
  if (per_pass > kMaxActive) per_pass = kMaxActive;
  if (per_pass > spec->rows) per_pass = spec->rows;
  for (size_t base = 0; base < spec->rows; base += per_pass) {
    // the window [base, base + per_pass) holds at most per_pass active rows
    qwen36_bf16_matvec_argmax_rows_spec_t window = *spec;
    window.rows = base + per_pass < spec->rows ? base + per_pass : spec->rows;
    int rc;
    switch (per_pass) {
      case 1: rc = launch_bf16_argmax<1>(&window, base); break;
      case 2: rc = launch_bf16_argmax<2>(&window, base); break;
      case 3: rc = launch_bf16_argmax<3>(&window, base); break;
      case 4: rc = launch_bf16_argmax<4>(&window, base); break;
      case 5: rc = launch_bf16_argmax<5>(&window, base); break;
      case 6: rc = launch_bf16_argmax<6>(&window, base); break;
      case 7: rc = launch_bf16_argmax<7>(&window, base); break;
      default: rc = launch_bf16_argmax<8>(&window, base); break;
    }
    if (rc != QWEN36_STATUS_SUCCESS) return rc;
  }
  const unsigned blocks = static_cast<unsigned>(q36::div_ceil(spec->rows, static_cast<size_t>(128)));
  bf16_argmax_finalize_kernel<<<blocks, 128, 0, q36::stream()>>>(
      as_ptr<const unsigned long long>(spec->workspace), as_ptr<uint32_t>(spec->output_token_u32),
      as_ptr<uint32_t>(spec->mirror_last_output_token_u32), as_ptr<const uint32_t>(spec->skip_flags_u32), spec->rows);
  return q36::launch_status();
}
