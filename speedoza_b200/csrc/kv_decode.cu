// Decode attention over a BF16 or FP8 (E4M3) KV cache with the cache-append side effect:
// qwen36_attention_decode of the reference ABI (kernels-cuda/attention.cu:2716-2876; kernels
// attention.cu:842-1000, 1225-1471, 1473-1554 and attention_decode_tiled.cu:159-357).
//
//   out[qh] = softmax_t( q[qh] . K[t, kvh] / sqrt(head_dim) ) V[t, kvh],  t = 0 .. position
//   rows t < position come from the cache (bf16, or E4M3 bytes without a scale), row t == position
//   is the not-yet-cached k_new / v_new in bf16; afterwards cache row `position` holds k_new /
//   v_new (copied for BF16, encoded with the reference's round-half-up E4M3 encoder for FP8).
//
// Launch shape (B200): with the caller's partial buffers, the cached rows [0, position) are cut
// into one split per SM (kv head x split CTAs); every CTA serves all q heads of its kv head from
// one read of K / V and writes a partial (m, l, o) per head.  Head size 256 with 1 / 2 / 4 / 6 / 8
// q heads per kv head runs both products on the tensor cores (one kernel per cache type, below);
// every other shape takes a general kernel (a CTA per q head and split).  One merge kernel (a CTA
// per q head, launched with programmatic stream serialisation) combines the partials, adds the
// current token in float32, writes the bf16 output and appends the row to the cache.  Without
// partial buffers one CTA per q head walks the whole context and finishes the head itself.  The
// position may live on the device (position_device_i32), so no grid depends on it: a captured
// graph stays valid while the context grows.  TurboQuant3 / 3.5 caches are not part of this
// library.
#include "common.cuh"

#include <atomic>

#include <math.h>

#include <mutex>

#include "kv_split.cuh"
#include "lse_merge.cuh"

namespace {

using q36::as_ptr;
using q36::cp_async_16;
using q36::cp_async_commit;
using q36::cp_async_wait;
using q36::kEpiStride;
using q36::lds128;
using q36::mma_f16;
using q36::split_epilogue;

constexpr int kThreads = 256;
static_assert(kThreads == q36::kMergeThreads && kThreads == q36::kSplitThreads, "block size");
constexpr int kWarps = kThreads / 32;
constexpr int kMaxSplits = 256;              // the merge handles one partial per thread
constexpr uint32_t kMinTokensPerSplit = 256;
constexpr int kKvBf16 = 0, kKvFp8 = 1;

std::atomic<int> g_decode_mode{1};                       // test hook: 0 = general kernel only, 1 = tensor-core forms where they apply
std::atomic<int> g_decode_force_splits{0};               // test hook: > 0 overrides the split count

// E4M3 byte -> float as the reference reads its cache (attention.cu:101-116): 0x7F / 0xFF are +-448.
__device__ __forceinline__ float kv_e4m3_to_f32(uint32_t code) {
  const uint32_t e = (code >> 3) & 15u, m = code & 7u;
  float v;
  if (e == 0u) v = static_cast<float>(m) * 0x1p-9f;
  else if (e == 15u && m == 7u) v = 448.0f;
  else v = __uint_as_float(((e + 120u) << 23) | (m << 20));
  return (code & 0x80u) ? -v : v;
}

// float -> E4M3 byte of the cache append (attention.cu:118-160): the magnitude is rounded half UP,
// |v| >= 448 saturates to 0x7E, zero and non-finite values give 0.  The reference forms
// floorf((frac * 2 - 1) * 8 + 0.5) from frexpf; on the bit pattern that is "add half a step of the
// 3-bit mantissa and truncate" (every intermediate value is exact in float32).
__device__ __forceinline__ uint32_t kv_f32_to_e4m3(float value) {
  const uint32_t bits = __float_as_uint(value);
  const uint32_t abs_bits = bits & 0x7fffffffu;
  if (abs_bits == 0u || abs_bits >= 0x7f800000u) return 0u;
  const uint32_t sign = (bits >> 24) & 0x80u;
  const float a = __uint_as_float(abs_bits);
  if (a >= 448.0f) return sign | 0x7eu;
  uint32_t code;
  if (a < 0x1p-6f) {
    if (a >= (7.0f * 0x1p-9f + 0x1p-6f) * 0.5f) code = 0x08u;
    else {
      const int m = static_cast<int>(floorf(__fadd_rn(__fmul_rn(a, 512.0f), 0.5f)));
      code = m <= 0 ? 0u : static_cast<uint32_t>(m);
    }
  } else {
    uint32_t e = (abs_bits >> 23) - 120u;                       // exponent field: a = 1.m * 2^(e - 7)
    uint32_t m = ((abs_bits & 0x007fffffu) + 0x00080000u) >> 20;
    if (m >= 8u) { m = 0u; ++e; }
    if (e >= 15u) { e = 15u; if (m > 6u) m = 6u; }
    code = (e << 3) | m;
  }
  return sign | code;
}

__device__ __forceinline__ size_t read_position(size_t scalar, const int32_t *device) {
  return device != nullptr ? static_cast<size_t>(max(__ldg(device), 0)) : scalar;
}

// Tokens [begin, end) of one split of the cached rows [0, position).
__device__ __forceinline__ void split_range(size_t position, uint32_t n_splits, uint32_t split, size_t &begin,
                                            size_t &end) {
  size_t per = q36::round_up(q36::div_ceil(position, n_splits), static_cast<size_t>(kWarps) * 16);
  if (per < kMinTokensPerSplit) per = kMinTokensPerSplit;
  begin = min(position, per * split);
  end = min(position, per * (split + 1));
}

template <bool FP8>
__device__ __forceinline__ float cache_value(const void *cache, size_t index) {
  if (FP8) return kv_e4m3_to_f32(__ldg(static_cast<const uint8_t *>(cache) + index));
  return q36::bf16_bits_to_f32(__ldg(static_cast<const uint16_t *>(cache) + index));
}

// Adds the current token (k_new / v_new: bf16, not yet in the cache) to a head's merged state
// (acc = this thread's dim of sum w o, M, den), writes the bf16 output, and lets the first q head
// of every kv group append the row to the cache at `position`.  One dim per thread; contains a
// block barrier.  s_red: kWarps floats nobody else is using.
template <bool FP8>
__device__ __forceinline__ void finish_head(float acc, float M, float den, const __nv_bfloat16 *__restrict__ q,
                                            const __nv_bfloat16 *__restrict__ k_new,
                                            const __nv_bfloat16 *__restrict__ v_new, void *cache_k, void *cache_v,
                                            __nv_bfloat16 *__restrict__ out, size_t position, uint32_t qh,
                                            uint32_t kv_heads, uint32_t q_per_kv, uint32_t head_dim, float *s_red) {
  const uint32_t d = threadIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const bool active = d < head_dim;
  const uint32_t kvh = qh / q_per_kv;
  const __nv_bfloat16 kb = active ? k_new[static_cast<size_t>(kvh) * head_dim + d] : __float2bfloat16(0.f);
  const __nv_bfloat16 vb = active ? v_new[static_cast<size_t>(kvh) * head_dim + d] : __float2bfloat16(0.f);
  const float qv = active ? __bfloat162float(q[static_cast<size_t>(qh) * head_dim + d]) : 0.f;
  float dot = qv * __bfloat162float(kb);
  for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
  if (lane == 0) s_red[warp] = dot;
  __syncthreads();
  dot = 0.f;
  for (int w = 0; w < kWarps; ++w) dot += s_red[w];
  const float s = dot * rsqrtf(static_cast<float>(head_dim));
  const float m_new = fmaxf(M, s);
  const float c_old = M == -INFINITY ? 0.f : __expf(M - m_new);
  const float p = __expf(s - m_new);
  if (!active) return;
  const float o = __fdiv_rn(fmaf(p, __bfloat162float(vb), acc * c_old), fmaf(den, c_old, p));
  out[static_cast<size_t>(qh) * head_dim + d] = __float2bfloat16(o);
  if (qh % q_per_kv == 0) {
    const size_t off = (position * kv_heads + kvh) * head_dim + d;
    if (FP8) {
      static_cast<uint8_t *>(cache_k)[off] = static_cast<uint8_t>(kv_f32_to_e4m3(__bfloat162float(kb)));
      static_cast<uint8_t *>(cache_v)[off] = static_cast<uint8_t>(kv_f32_to_e4m3(__bfloat162float(vb)));
    } else {
      static_cast<__nv_bfloat16 *>(cache_k)[off] = kb;
      static_cast<__nv_bfloat16 *>(cache_v)[off] = vb;
    }
  }
}

// ---- general kernel: any head_dim <= 256, any grouping.  One CTA per (q head, split); a warp
// takes every eighth token, lane l holds dims l, l + 32, ...; the eight warps' running softmax
// states meet in shared memory at the end.  DIRECT (no partial buffers): one CTA per q head walks
// the whole context, then adds the current token, writes the output and appends the cache row.
template <bool FP8, bool DIRECT>
__global__ void __launch_bounds__(kThreads)
decode_split_general_kernel(const __nv_bfloat16 *__restrict__ q, const __nv_bfloat16 *__restrict__ k_new,
                            const __nv_bfloat16 *__restrict__ v_new, void *cache_k, void *cache_v,
                            float *__restrict__ part_o, float *__restrict__ part_m, float *__restrict__ part_l,
                            __nv_bfloat16 *__restrict__ out, size_t position_scalar,
                            const int32_t *__restrict__ position_device, uint32_t kv_heads, uint32_t q_per_kv,
                            uint32_t head_dim, uint32_t n_splits) {
  __shared__ float s_m[kWarps], s_l[kWarps];
  __shared__ float s_o[kWarps][256];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t qh = blockIdx.x, split = blockIdx.y, kvh = qh / q_per_kv;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const size_t position = read_position(position_scalar, position_device);
  size_t s_begin, s_end;
  split_range(position, n_splits, split, s_begin, s_end);
  const float scale = rsqrtf(static_cast<float>(head_dim));

  float qv[8], acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t d = lane + 32u * j;
    qv[j] = d < head_dim ? __bfloat162float(q[static_cast<size_t>(qh) * head_dim + d]) : 0.f;
    acc[j] = 0.f;
  }
  float m_run = -INFINITY, l_run = 0.f;
  for (size_t t = s_begin + warp; t < s_end; t += kWarps) {
    const size_t base = (t * kv_heads + kvh) * head_dim;
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t d = lane + 32u * j;
      if (d < head_dim) dot = fmaf(qv[j], cache_value<FP8>(cache_k, base + d), dot);
    }
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    const float s = dot * scale;
    const float m_new = fmaxf(m_run, s);
    const float corr = m_run == -INFINITY ? 0.f : __expf(m_run - m_new);
    const float p = __expf(s - m_new);
    l_run = l_run * corr + p;
    m_run = m_new;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t d = lane + 32u * j;
      if (d < head_dim) acc[j] = fmaf(p, cache_value<FP8>(cache_v, base + d), acc[j] * corr);
    }
  }
  if (lane == 0) { s_m[warp] = m_run; s_l[warp] = l_run; }
#pragma unroll
  for (int j = 0; j < 8; ++j) s_o[warp][lane + 32 * j] = acc[j];
  __syncthreads();
  float M = -INFINITY;
  for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w]);
  if (DIRECT) {
    __shared__ float s_red[kWarps];
    float o = 0.f, den = 0.f;
    for (int w = 0; w < kWarps; ++w) {
      const float wgt = s_m[w] == -INFINITY ? 0.f : __expf(s_m[w] - M);
      o = fmaf(wgt, s_o[w][threadIdx.x], o);
      den = fmaf(wgt, s_l[w], den);
    }
    finish_head<FP8>(o, M, den, q, k_new, v_new, cache_k, cache_v, out, position, qh, kv_heads, q_per_kv, head_dim,
                     s_red);
    return;
  }
  const size_t slot = static_cast<size_t>(qh) * n_splits + split;
  for (uint32_t d = threadIdx.x; d < head_dim; d += kThreads) {
    float o = 0.f;
    for (int w = 0; w < kWarps; ++w) o = fmaf(s_m[w] == -INFINITY ? 0.f : __expf(s_m[w] - M), s_o[w][d], o);
    part_o[slot * head_dim + d] = o;
  }
  if (threadIdx.x == 0) {
    float den = 0.f;
    for (int w = 0; w < kWarps; ++w) den = fmaf(s_m[w] == -INFINITY ? 0.f : __expf(s_m[w] - M), s_l[w], den);
    part_m[slot] = M;
    part_l[slot] = den;
  }
}

// ---- merge of the split partials + current token + cache append: one CTA per q head.
template <bool FP8>
__global__ void __launch_bounds__(kThreads)
decode_merge_append_kernel(const float *__restrict__ part_o, const float *__restrict__ part_m,
                           const float *__restrict__ part_l, uint32_t n_parts, const __nv_bfloat16 *__restrict__ q,
                           const __nv_bfloat16 *__restrict__ k_new, const __nv_bfloat16 *__restrict__ v_new,
                           void *cache_k, void *cache_v, __nv_bfloat16 *__restrict__ out, size_t position_scalar,
                           const int32_t *__restrict__ position_device, uint32_t kv_heads, uint32_t q_per_kv,
                           uint32_t head_dim) {
  __shared__ float s_w[kThreads];
  __shared__ float s_red[kWarps];
  const uint32_t qh = blockIdx.x;
  const size_t position = read_position(position_scalar, position_device);
  // launched with programmatic stream serialisation after the split kernel: resident by the time
  // the partials are complete (a no-op after an ordinary launch)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const float *po = part_o + static_cast<size_t>(qh) * n_parts * head_dim;
  const uint32_t d = min(threadIdx.x, head_dim - 1);              // idle threads fetch a valid address
  float first[48];                                                // one CTA per SM and kv head gives 37 parts
  q36::lse_prefetch(po, n_parts, head_dim, d, first);             // in flight while the weights are formed
  float M, den;
  q36::lse_weights(part_m + static_cast<size_t>(qh) * n_parts, part_l + static_cast<size_t>(qh) * n_parts, n_parts,
                   s_w, s_red, M, den);
  const float acc = threadIdx.x < head_dim ? q36::lse_accumulate(po, s_w, n_parts, head_dim, d, first) : 0.f;
  __syncthreads();                                                // s_red is reused below
  finish_head<FP8>(acc, M, den, q, k_new, v_new, cache_k, cache_v, out, position, qh, kv_heads, q_per_kv, head_dim,
                   s_red);
}

// ---- tensor-core form for the FP8 cache (head_dim 256, G <= 8 q heads per kv head).
//
// Both products run as mma.sync.m16n8k16 with float16 operands and float32 accumulation: E4M3 ->
// float16 is exact (cvt.rn.f16x2.e4m3x2), q is rounded to float16, probabilities to float16 after
// scaling by kPScale.  Fragment plan, lane (g = lane / 4, t = lane % 4), a warp owns 16 tokens at
// a time:
//   S = Q K^T : A = Q (row g = q head g, rows >= G zero), B = K^T with token g of an 8-token block
//       as its column; the contraction index is permuted so that a lane's operands are sixteen
//       consecutive bytes of a row: step 4 j + i covers dims 64 j + 16 t + 4 i .. + 3.
//       The accumulator leaves lane (g, t) with head g's scores of tokens 2t, 2t + 1 of the block.
//   O^T = V^T P^T : those scores are exactly the B fragment of the second product (column =
//       head g, contraction slots 2t, 2t+1, 2t+8, 2t+9 = this lane's tokens), so probabilities
//       stay in registers.  A = V^T: a lane reads dims 16 (g + 8 h) .. + 15 of its four tokens and
//       pairs bytes of neighbouring tokens; mma (h, j) has dim 16 (g + 8 h) + 2 j in row g and the
//       next dim in row g + 8; its accumulator holds heads 2t, 2t + 1 of those two dims.
// four E4M3 bytes -> two float16x2 (bytes 0, 1 and bytes 2, 3)
__device__ __forceinline__ void e4m3x4_to_h2x2(uint32_t w, uint32_t &lo, uint32_t &hi) {
  asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
      : "=r"(lo), "=r"(hi) : "r"(w));
}
// 0x7F -> 0x7E and 0xFF -> 0xFE in every byte (a byte whose low seven bits are all ones loses bit 0)
__device__ __forceinline__ uint32_t e4m3_nan_to_448(uint32_t w) {
  const uint32_t t = (w & 0x7f7f7f7fu) + 0x01010101u;
  return w ^ ((t >> 7) & 0x01010101u);
}
__device__ __forceinline__ uint4 e4m3_nan_to_448(uint4 v) {
  return make_uint4(e4m3_nan_to_448(v.x), e4m3_nan_to_448(v.y), e4m3_nan_to_448(v.z), e4m3_nan_to_448(v.w));
}

// K / V travel global -> shared memory with 16-byte asynchronous copies (cp.async) into a private
// three-stage ring per warp, so the
// bytes in flight (two stages = 16 KB per warp, 128 KB per SM) no longer have to fit in
// registers.  A stage holds the K and the V rows of a 16-token group (256 bytes each); 16-byte
// chunks are XOR-swizzled on the way in so that the fragment reads are free of bank conflicts:
// K chunk c of row r sits at c ^ 4 (r & 1), V chunk c of row r at c ^ 2 ((r / 2) & 3).  No block
// barrier inside the loop: a warp waits for its own copies (wait_group + __syncwarp).
// The reference reads the bytes 0x7F / 0xFF as +-448 (what 0x7E / 0xFE decode to) where the
// hardware conversion gives NaN.  The cache append never writes them, so they are handled out of
// line: the fast pass converts bytes as they are; a NaN anywhere in the CTA's result sends the CTA through a
// second pass that rewrites those bytes first (template flag FIX).
constexpr int kStages = 3;
constexpr uint32_t kTileBytes = 16 * 256;                         // 16 tokens x 256 bytes
constexpr uint32_t kStageBytes = 2 * kTileBytes;                  // K tile + V tile
constexpr uint32_t kRingBytes = kWarps * kStages * kStageBytes;   // 192 KB
constexpr uint32_t kStagedSmemBytes = kRingBytes + 16 * 32 * 8 + 2 * kWarps * 8 * 4;

// One stage of the ring: lane copies chunk (lane & 15) of rows (lane >> 4) + 2 r, r = 0 .. 7, of K
// and of V; rows past the end of the split are zero-filled (source size 0, address kept inside the
// cache).  Ends with a commit: one group per stage.
__device__ __forceinline__ void fp8_stage_issue(uint32_t base, size_t tg, size_t s_begin, size_t s_end,
                                                const uint8_t *__restrict__ cache_k,
                                                const uint8_t *__restrict__ cache_v, uint32_t kv_heads,
                                                uint32_t kvh) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t chunk = lane & 15u, row0 = lane >> 4;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const uint32_t row = row0 + 2u * r;
    const size_t tok = tg + row;
    const bool valid = tok < s_end;
    const size_t off = ((valid ? tok : s_begin) * kv_heads + kvh) * 256u + chunk * 16u;
    const uint32_t bytes = valid ? 16u : 0u;
    cp_async_16(base + row * 256u + ((chunk ^ ((row & 1u) << 2)) << 4), cache_k + off, bytes);
    cp_async_16(base + kTileBytes + row * 256u + ((chunk ^ (((row >> 1) & 3u) << 1)) << 4), cache_v + off, bytes);
  }
  cp_async_commit();
}

template <int G, bool FIX>
__device__ __forceinline__ void fp8_staged_pass(float (&o)[2][8][4], float &m_run, float &l_run,
                                                const uint8_t *__restrict__ cache_k,
                                                const uint8_t *__restrict__ cache_v, uint32_t ring /* this warp's */,
                                                const uint2 (*s_q)[32], size_t s_begin, size_t s_end,
                                                uint32_t kv_heads, uint32_t kvh, bool primed) {
  constexpr float kPScale = 64.0f;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  const float sm_scale = 0.0625f * 1.4426950408889634f;           // rsqrt(256) * log2(e)
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[h][j][c] = 0.f;
  m_run = -INFINITY;
  l_run = 0.f;
  const size_t stride = static_cast<size_t>(kWarps) * 16;
  size_t t0 = s_begin + static_cast<size_t>(warp) * 16;
  if (t0 >= s_end) return;

  auto issue = [&](uint32_t stage, size_t tg) {
    fp8_stage_issue(ring + stage * kStageBytes, tg, s_begin, s_end, cache_k, cache_v, kv_heads, kvh);
  };
  if (!primed) {
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue(s, t0 + s * stride);
  }

  uint32_t stage = 0;
  for (; t0 < s_end; t0 += stride) {
    issue(stage == 0 ? kStages - 1 : stage - 1, t0 + (kStages - 1) * stride);   // refill the stage read last time
    cp_async_wait<kStages - 1>();
    __syncwarp();
    const uint32_t kt = ring + stage * kStageBytes, vt = kt + kTileBytes;
    // ---- S = Q K^T
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
          uint4 kw = lds128(kt + (8u * blk + g) * 256u + (((t + 4u * j) ^ ((g & 1u) << 2)) << 4));
          if (FIX) kw = e4m3_nan_to_448(kw);
          w[blk][0] = kw.x; w[blk][1] = kw.y; w[blk][2] = kw.z; w[blk][3] = kw.w;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint2 qf = s_q[4 * j + i][lane];
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            uint32_t b0, b1;
            e4m3x4_to_h2x2(w[blk][i], b0, b1);
            mma_f16(acc[blk][i & 1], qf.x, 0u, qf.y, 0u, b0, b1);
          }
        }
      }
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        sc_[2 * blk] = acc[blk][0][0] + acc[blk][1][0];
        sc_[2 * blk + 1] = acc[blk][0][1] + acc[blk][1][1];
      }
    }
    // ---- online softmax, head g: this lane's four tokens, then the four lanes of the head
    float s_log2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const size_t tok = t0 + 2 * t + (i & 1) + 8 * (i >> 1);
      s_log2[i] = (g < G && tok < s_end) ? sc_[i] * sm_scale : -INFINITY;
    }
    float p[4];
    const float corr = q36::online_softmax_step(s_log2, p, m_run, l_run);
    const __half2 pb0 = __floats2half2_rn(p[0] * kPScale, p[1] * kPScale);
    const __half2 pb1 = __floats2half2_rn(p[2] * kPScale, p[3] * kPScale);
    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(&pb0), b1 = *reinterpret_cast<const uint32_t *>(&pb1);
    q36::rescale_outputs(o, corr);
    // ---- O^T += V^T P^T: rows 2t, 2t + 1, 2t + 8, 2t + 9 of the V tile, chunk g + 8 h
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint4 x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[i] = lds128(vt + (2u * t + (i & 1) + 8u * (i >> 1)) * 256u + (((g + 8u * h) ^ (t << 1)) << 4));
        if (FIX) x[i] = e4m3_nan_to_448(x[i]);
      }
      const uint32_t va[4] = {x[0].x, x[0].y, x[0].z, x[0].w}, vb[4] = {x[1].x, x[1].y, x[1].z, x[1].w};
      const uint32_t vc[4] = {x[2].x, x[2].y, x[2].z, x[2].w}, vd[4] = {x[3].x, x[3].y, x[3].z, x[3].w};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint32_t ab0, ab1, ab2, ab3, cd0, cd1, cd2, cd3;
        e4m3x4_to_h2x2(__byte_perm(va[w], vb[w], 0x5140), ab0, ab1);
        e4m3x4_to_h2x2(__byte_perm(va[w], vb[w], 0x7362), ab2, ab3);
        e4m3x4_to_h2x2(__byte_perm(vc[w], vd[w], 0x5140), cd0, cd1);
        e4m3x4_to_h2x2(__byte_perm(vc[w], vd[w], 0x7362), cd2, cd3);
        mma_f16(o[h][2 * w], ab0, ab1, cd0, cd1, b0, b1);
        mma_f16(o[h][2 * w + 1], ab2, ab3, cd2, cd3, b0, b1);
      }
    }
    __syncwarp();                                    // every lane is done with this stage before it is refilled
    stage = stage + 1 == kStages ? 0 : stage + 1;
  }
  cp_async_wait<0>();
}

template <int G>
__global__ void __launch_bounds__(kThreads, 1)
decode_split_fp8_staged_kernel(const __nv_bfloat16 *__restrict__ q, const uint8_t *__restrict__ cache_k,
                               const uint8_t *__restrict__ cache_v, float *__restrict__ part_o,
                               float *__restrict__ part_m, float *__restrict__ part_l, size_t position_scalar,
                               const int32_t *__restrict__ position_device, uint32_t kv_heads, uint32_t q_per_kv,
                               uint32_t n_splits) {
  constexpr uint32_t D = 256;
  extern __shared__ __align__(128) uint8_t smem[];
  // ring | q fragments | per-warp maxima and sums; the epilogue's output slices reuse the ring
  uint2 (*s_q)[32] = reinterpret_cast<uint2 (*)[32]>(smem + kRingBytes);
  float (*s_m)[8] = reinterpret_cast<float (*)[8]>(smem + kRingBytes + 16 * 32 * 8);
  float (*s_l)[8] = s_m + kWarps;
  float (*s_o)[kEpiStride] = reinterpret_cast<float (*)[kEpiStride]>(smem);

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  const uint32_t head0 = blockIdx.x * G;
  const uint32_t kvh = head0 / q_per_kv;
  const uint32_t split = blockIdx.y;
  asm volatile("griddepcontrol.wait;" ::: "memory");       // seated early; nothing is touched before the previous kernel is done
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const size_t position = read_position(position_scalar, position_device);
  size_t s_begin, s_end;
  split_range(position, n_splits, split, s_begin, s_end);

  // the first two stages of this warp's ring fly while q is staged
  const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + warp * (kStages * kStageBytes);
  {
    const size_t first = s_begin + static_cast<size_t>(warp) * 16;
    if (first < s_end) {
#pragma unroll
      for (int st = 0; st < kStages - 1; ++st)
        fp8_stage_issue(ring + st * kStageBytes, first + st * (static_cast<size_t>(kWarps) * 16), s_begin, s_end, cache_k,
                        cache_v, kv_heads, kvh);
    }
  }
  // Q fragments: step 4 j + i covers dims 64 j + 16 t + 4 i .. + 3 of head g, as float16
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

  float o[2][8][4];
  float m_run, l_run;
  fp8_staged_pass<G, false>(o, m_run, l_run, cache_k, cache_v, ring, s_q, s_begin, s_end, kv_heads, kvh, true);
  float probe = l_run;                                            // NaN anywhere in this thread's state?
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j) probe += (o[h][j][0] + o[h][j][1]) + (o[h][j][2] + o[h][j][3]);
  if (__syncthreads_or(probe != probe))
    fp8_staged_pass<G, true>(o, m_run, l_run, cache_k, cache_v, ring, s_q, s_begin, s_end, kv_heads, kvh, false);
  __syncthreads();                                                // the ring becomes the epilogue's slices
  split_epilogue<G>(o, m_run, l_run, 1.0f / 64.0f, s_m, s_l, s_o, part_o, part_m, part_l, head0, split, n_splits);
}

// ---- tensor-core form for the BF16 cache (head_dim 256, G <= 8 q heads per kv head).
//
// Same fragment plan as the FP8 kernel with bfloat16 operands (mma.sync.m16n8k16 bf16, float32
// accumulation): q and K enter exactly as stored, probabilities are rounded to bfloat16.  A row is
// 512 bytes, so a lane's sixteen-byte loads hold eight dims: step 2 j + i of S = Q K^T covers dims
// 32 j + 8 t + 4 i .. + 3, and for O^T = V^T P^T a lane loads dims 16 (g + 8 h) .. + 15 of its four
// tokens as two loads per token, pairing the halves of neighbouring tokens' words.  K and V of a
// 16-token group take 128 registers, so there is one buffer of each; it is refilled for the next
// group as soon as the product that reads it has been issued.
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <int G>
__global__ void __launch_bounds__(kThreads, 1)
decode_split_bf16_mma_kernel(const __nv_bfloat16 *__restrict__ q, const __nv_bfloat16 *__restrict__ cache_k,
                             const __nv_bfloat16 *__restrict__ cache_v, float *__restrict__ part_o,
                             float *__restrict__ part_m, float *__restrict__ part_l, size_t position_scalar,
                             const int32_t *__restrict__ position_device, uint32_t kv_heads, uint32_t q_per_kv,
                             uint32_t n_splits) {
  constexpr uint32_t D = 256;
  __shared__ float s_m[kWarps][8], s_l[kWarps][8];
  __shared__ __align__(16) float s_o[4 * G][kEpiStride];
  __shared__ uint2 s_q[16][32];

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t g = lane >> 2, t = lane & 3u;
  const uint32_t head0 = blockIdx.x * G;
  const uint32_t kvh = head0 / q_per_kv;
  const uint32_t split = blockIdx.y;
  asm volatile("griddepcontrol.wait;" ::: "memory");       // seated early; nothing is touched before the previous kernel is done
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const size_t position = read_position(position_scalar, position_device);
  size_t s_begin, s_end;
  split_range(position, n_splits, split, s_begin, s_end);
  const float sm_scale = 0.0625f * 1.4426950408889634f;           // rsqrt(256) * log2(e)

  float o[2][8][4];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[h][j][c] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  struct KBuf { uint4 k[2][8]; };
  struct VBuf { uint4 v[4][2][2]; };
  auto load_k = [&](KBuf &b, size_t t0) {
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const size_t tok = t0 + 8 * blk + g;
      if (tok < s_end) {
        const uint4 *src = reinterpret_cast<const uint4 *>(cache_k + (tok * kv_heads + kvh) * D) + t;
#pragma unroll
        for (int j = 0; j < 8; ++j) b.k[blk][j] = __ldcs(src + 4 * j);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) b.k[blk][j] = make_uint4(0, 0, 0, 0);
      }
    }
  };
  auto load_v = [&](VBuf &b, size_t t0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const size_t tok = t0 + 2 * t + (i & 1) + 8 * (i >> 1);
      if (tok < s_end) {
        const uint4 *src = reinterpret_cast<const uint4 *>(cache_v + (tok * kv_heads + kvh) * D) + 2 * g;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          b.v[i][h][0] = __ldcs(src + 16 * h);
          b.v[i][h][1] = __ldcs(src + 16 * h + 1);
        }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) b.v[i][h][0] = b.v[i][h][1] = make_uint4(0, 0, 0, 0);
      }
    }
  };

  const size_t stride = static_cast<size_t>(kWarps) * 16;
  KBuf kb;
  VBuf vb;
  size_t t0 = s_begin + static_cast<size_t>(warp) * 16;
  if (t0 < s_end) {                                  // first loads fly while q is staged
    load_k(kb, t0);
    load_v(vb, t0);
  }
  // Q fragments, the same for every warp: step 2 j + i holds words 2 i, 2 i + 1 of the sixteen
  // bytes at dims 32 j + 8 t of head g
  if (warp == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (g < G) raw = __ldg(reinterpret_cast<const uint4 *>(q + static_cast<size_t>(head0 + g) * D) + t + 4 * j);
      s_q[2 * j][lane] = make_uint2(raw.x, raw.y);
      s_q[2 * j + 1][lane] = make_uint2(raw.z, raw.w);
    }
  }
  __syncthreads();

  for (; t0 < s_end; t0 += stride) {
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
      for (int j = 0; j < 8; ++j) {
        const uint2 q0 = s_q[2 * j][lane], q1 = s_q[2 * j + 1][lane];
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          mma_bf16(acc[blk][0], q0.x, 0u, q0.y, 0u, kb.k[blk][j].x, kb.k[blk][j].y);
          mma_bf16(acc[blk][1], q1.x, 0u, q1.y, 0u, kb.k[blk][j].z, kb.k[blk][j].w);
        }
      }
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        sc_[2 * blk] = acc[blk][0][0] + acc[blk][1][0];
        sc_[2 * blk + 1] = acc[blk][0][1] + acc[blk][1][1];
      }
    }
    load_k(kb, t0 + stride);                         // refill for the next group (zeros past the end)
    // ---- online softmax, head g: this lane's four tokens, then the four lanes of the head
    float s_log2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const size_t tok = t0 + 2 * t + (i & 1) + 8 * (i >> 1);
      s_log2[i] = (g < G && tok < s_end) ? sc_[i] * sm_scale : -INFINITY;
    }
    float p[4];
    const float corr = q36::online_softmax_step(s_log2, p, m_run, l_run);
    const uint32_t b0 = pack_bf16x2(p[0], p[1]), b1 = pack_bf16x2(p[2], p[3]);
    q36::rescale_outputs(o, corr);
    // ---- O^T += V^T P^T: word w of a token's 32 bytes holds dims 2 w, 2 w + 1
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint4 xa = vb.v[0][h][half], xb = vb.v[1][h][half], xc = vb.v[2][h][half], xd = vb.v[3][h][half];
        const uint32_t va[4] = {xa.x, xa.y, xa.z, xa.w}, vb_[4] = {xb.x, xb.y, xb.z, xb.w};
        const uint32_t vc[4] = {xc.x, xc.y, xc.z, xc.w}, vd[4] = {xd.x, xd.y, xd.z, xd.w};
#pragma unroll
        for (int w = 0; w < 4; ++w)
          mma_bf16(o[h][4 * half + w], __byte_perm(va[w], vb_[w], 0x5410), __byte_perm(va[w], vb_[w], 0x7632),
                   __byte_perm(vc[w], vd[w], 0x5410), __byte_perm(vc[w], vd[w], 0x7632), b0, b1);
      }
    }
    load_v(vb, t0 + stride);
  }
  split_epilogue<G>(o, m_run, l_run, 1.0f, s_m, s_l, s_o, part_o, part_m, part_l, head0, split, n_splits);
}

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

struct Args {
  const __nv_bfloat16 *q, *k_new, *v_new;
  void *cache_k, *cache_v;
  float *part_o, *part_m, *part_l;
  __nv_bfloat16 *out;
  size_t position;
  const int32_t *position_device;
  uint32_t q_heads, kv_heads, q_per_kv, head_dim;
};

template <bool FP8>
int launch_direct(const Args &a) {
  decode_split_general_kernel<FP8, true><<<dim3(a.q_heads, 1), kThreads, 0, q36::stream()>>>(
      a.q, a.k_new, a.v_new, a.cache_k, a.cache_v, nullptr, nullptr, nullptr, a.out, a.position, a.position_device,
      a.kv_heads, a.q_per_kv, a.head_dim, 1u);
  return q36::launch_status();
}

template <int G>
int launch_fp8_staged(const Args &a, uint32_t n_splits) {
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(decode_split_fp8_staged_kernel<G>),
                               static_cast<int>(kStagedSmemBytes)) != cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  return q36::cuda_status(q36::launch_after_previous(
      decode_split_fp8_staged_kernel<G>, dim3(a.q_heads / G, n_splits), dim3(kThreads), kStagedSmemBytes, q36::stream(),
      a.q, static_cast<const uint8_t *>(a.cache_k), static_cast<const uint8_t *>(a.cache_v), a.part_o, a.part_m,
      a.part_l, a.position, a.position_device, a.kv_heads, a.q_per_kv, n_splits));
}

template <int G>
int launch_bf16_mma(const Args &a, uint32_t n_splits) {
  return q36::cuda_status(q36::launch_after_previous(
      decode_split_bf16_mma_kernel<G>, dim3(a.q_heads / G, n_splits), dim3(kThreads), 0, q36::stream(), a.q,
      static_cast<const __nv_bfloat16 *>(a.cache_k), static_cast<const __nv_bfloat16 *>(a.cache_v), a.part_o,
      a.part_m, a.part_l, a.position, a.position_device, a.kv_heads, a.q_per_kv, n_splits));
}

template <bool FP8>
int launch_merge(const Args &a, uint32_t n_parts) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(a.q_heads);
  cfg.blockDim = dim3(kThreads);
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return q36::cuda_status(cudaLaunchKernelEx(
      &cfg, decode_merge_append_kernel<FP8>, static_cast<const float *>(a.part_o),
      static_cast<const float *>(a.part_m), static_cast<const float *>(a.part_l), n_parts, a.q, a.k_new, a.v_new,
      a.cache_k, a.cache_v, a.out, a.position, a.position_device, a.kv_heads, a.q_per_kv, a.head_dim));
}

// How many splits to launch: one CTA per SM for the tensor-core form (a CTA's start-up and merge
// cost about as much as 1500 tokens), about two per SM for the general kernel; never more than
// the caller's buffers hold, than the merge handles, or (when the position is known on the host)
// than there are 256-token pieces.  With a device-side position the count cannot follow the
// position, so that a captured launch stays valid: later splits are then empty and cost nothing.
uint32_t pick_splits(const Args &a, size_t caller_splits, size_t ctas_per_split, bool one_wave) {
  const size_t sms = static_cast<size_t>(sm_count());
  size_t n = one_wave ? sms / ctas_per_split : q36::div_ceil(2 * sms, ctas_per_split);
  if (g_decode_force_splits > 0) n = static_cast<size_t>(g_decode_force_splits.load());
  else if (a.position_device == nullptr) {
    const size_t cap = q36::div_ceil(a.position, kMinTokensPerSplit);
    if (n > cap) n = cap;
  }
  if (n > caller_splits) n = caller_splits;
  if (n > kMaxSplits) n = kMaxSplits;
  if (n < 1) n = 1;
  return static_cast<uint32_t>(n);
}

template <bool FP8>
int run_split_path(const Args &a, size_t caller_splits) {
  const bool aligned16 = ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.cache_k) |
                           reinterpret_cast<uintptr_t>(a.cache_v)) & 15u) == 0;
  const bool grouped = a.q_per_kv == 1 || a.q_per_kv == 2 || a.q_per_kv == 4 || a.q_per_kv == 6 || a.q_per_kv == 8;
  int status;
  uint32_t n;
  if (g_decode_mode >= 1 && a.head_dim == 256 && aligned16 && grouped) {
    n = pick_splits(a, caller_splits, a.kv_heads, true);
#define Q36_DECODE_GO(G) status = FP8 ? launch_fp8_staged<G>(a, n) : launch_bf16_mma<G>(a, n)
    switch (a.q_per_kv) {
      case 1: Q36_DECODE_GO(1); break;
      case 2: Q36_DECODE_GO(2); break;
      case 4: Q36_DECODE_GO(4); break;
      case 6: Q36_DECODE_GO(6); break;
      default: Q36_DECODE_GO(8); break;
    }
#undef Q36_DECODE_GO
  } else {
    n = pick_splits(a, caller_splits, a.q_heads, false);
    decode_split_general_kernel<FP8, false><<<dim3(a.q_heads, n), kThreads, 0, q36::stream()>>>(
        a.q, a.k_new, a.v_new, a.cache_k, a.cache_v, a.part_o, a.part_m, a.part_l, a.out, a.position,
        a.position_device, a.kv_heads, a.q_per_kv, a.head_dim, n);
    status = q36::launch_status();
  }
  if (status != QWEN36_STATUS_SUCCESS) return status;
  return launch_merge<FP8>(a, n);
}

}  // namespace

extern "C" void qwen36_attention_decode_set_mode(int mode) { g_decode_mode = mode != 0 ? 1 : 0; }
extern "C" void qwen36_attention_decode_force_splits(int n) { g_decode_force_splits = n < 0 ? 0 : n; }

extern "C" int qwen36_attention_decode(const qwen36_attention_decode_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  const qwen36_attention_shape_t &sh = spec->shape;
  // the reference's checks (kernels-cuda/attention.cu:2720-2734)
  if (spec->q_bf16.ptr == 0 || spec->k_bf16.ptr == 0 || spec->v_bf16.ptr == 0 || spec->kv_cache_k.ptr == 0 ||
      spec->kv_cache_v.ptr == 0 || spec->output_bf16.ptr == 0 || sh.q_heads == 0 || sh.kv_heads == 0 ||
      sh.head_dim == 0 || sh.head_dim > 256 || sh.q_heads % sh.kv_heads != 0 || spec->kv_cache_dtype < 0 ||
      spec->kv_cache_dtype > 3 || (spec->kv_cache_dtype >= 2 && spec->kv_cache_metadata.ptr == 0))
    return QWEN36_STATUS_INVALID_ARGUMENT;
  if (spec->kv_cache_dtype >= 2) return QWEN36_STATUS_NOT_IMPLEMENTED;   // TurboQuant3 / 3.5 caches
  Args a;
  a.q = as_ptr<const __nv_bfloat16>(spec->q_bf16);
  a.k_new = as_ptr<const __nv_bfloat16>(spec->k_bf16);
  a.v_new = as_ptr<const __nv_bfloat16>(spec->v_bf16);
  a.cache_k = as_ptr<void>(spec->kv_cache_k);
  a.cache_v = as_ptr<void>(spec->kv_cache_v);
  a.part_o = as_ptr<float>(spec->partial_acc_f32);
  a.part_m = as_ptr<float>(spec->partial_max_f32);
  a.part_l = as_ptr<float>(spec->partial_denom_f32);
  a.out = as_ptr<__nv_bfloat16>(spec->output_bf16);
  a.position = spec->position;
  a.position_device = as_ptr<const int32_t>(spec->position_device_i32);
  a.q_heads = static_cast<uint32_t>(sh.q_heads);
  a.kv_heads = static_cast<uint32_t>(sh.kv_heads);
  a.q_per_kv = static_cast<uint32_t>(sh.q_heads / sh.kv_heads);
  a.head_dim = static_cast<uint32_t>(sh.head_dim);
  const bool fp8 = spec->kv_cache_dtype == kKvFp8;
  const bool partials = a.part_o != nullptr && a.part_m != nullptr && a.part_l != nullptr;
  if (partials && spec->decode_n_splits >= 2) {
    if (spec->split_timesteps_per_block != 0 && spec->split_timesteps_per_block < 64)
      return QWEN36_STATUS_INVALID_ARGUMENT;                       // attention.cu:2752-2754
    return fp8 ? run_split_path<true>(a, spec->decode_n_splits) : run_split_path<false>(a, spec->decode_n_splits);
  }
  return fp8 ? launch_direct<true>(a) : launch_direct<false>(a);
}
