// Split-KV attention of a SHORT query chunk over a LONG BF16 / FP8 (E4M3) cache, on the tensor cores:
//   * qwen36_attention_flash_splitk_prefill_bf16(spec, n_splits): the speculative-verify step,
//     q <= 32 tokens x q_heads against cache rows [0, start + tokens) with a causal mask inside the
//     chunk (row i sees rows <= start + i); replaces kernels-cuda/attention_flash_splitk.cu:96-420,
//     504-600 (partition, partial layout and reduce of that file are kept, see below);
//   * qwen36_attention_decode_split_tiled(spec, n_splits, timesteps): one decode token with the
//     reference's fixed-size splits, partials only, plus the cache append by the split that owns
//     the position; replaces kernels-cuda/attention_decode_tiled.cu:159-357,370-403.
//
// One kernel serves both.  A CTA = (kv head, chunk of up to 64 (token, q head) rows, split): the
// rows of ALL q heads that share the kv head ride in one CTA, so K / V are read once per kv head
// (the reference launches one CTA per q head and reads them q_per_kv times).  A warp owns a 16-row
// tile of those rows and a slice of the timesteps of every 64-row K / V tile (see the kernel):
// S = Q K^T and O += P V as mma.sync.m16n8k16 with float32 accumulation, online softmax in
// registers (a row lives in the four lanes of a quad), probabilities rounded to the operand type
// before P V as in the reference, l accumulated from the unrounded values.  K / V tiles travel
// through a cp.async ring and sit in shared memory in 16-byte chunks XOR-swizzled by row, which
// makes every ldmatrix conflict-free.  A BF16 cache multiplies in bf16; an FP8 cache is expanded
// E4M3 -> f16 (exact) and multiplies in f16 with q rounded to f16 (11 significant bits, q needs 8).
//
// Partial contract (what the reduce and the reference's callers see):
//   acc[((token * q_heads + qh) * n_splits + split) * head_dim + d]  unnormalised, float32
//   m / l[(token * q_heads + qh) * n_splits + split]                 max of scaled scores / denominator
//   empty split = (-inf, 0, 0)
// Verify: the 64-row K iterations [0, ceil((start + tokens) / 64)) are dealt evenly, in order, to
// the splits (attention_flash_splitk.cu:139-149).  Decode: split s = timesteps [s * block, (s + 1)
// * block) cut at position + 1; timestep == position is the not yet cached k_bf16 / v_bf16 row.
#include "common.cuh"

#include <cuda_fp16.h>
#include <math.h>
#include <mutex>

namespace {

using q36::as_ptr;

constexpr uint32_t kD = 256;                 // head_dim
constexpr uint32_t kTile = 64;               // KV rows per iteration
constexpr uint32_t kRowBytes = kD * 2;       // one row of 2-byte elements
constexpr uint32_t kStages = 3;              // K / V tiles in flight (cp.async ring)
constexpr uint32_t kMergeStride = kD + 8;    // floats per row of the warps' meeting area

// Shared memory of a CTA with MT 16-row tiles of (token, q head) rows:
//   Q (16 MT rows) | FP8 only: K and V of the current tile expanded to f16 | ring of kStages tiles in
//   the cache's own format (K then V; bf16 rows are stored chunk-swizzled, ready for ldmatrix).
// After the loop the area behind Q is reused for the warps' (m, l, o).
template <bool FP8, int MT>
struct Layout {
  static constexpr uint32_t kRows = 16u * MT;
  static constexpr uint32_t kQBytes = kRows * kRowBytes;
  static constexpr uint32_t kWorkBytes = FP8 ? 2u * kTile * kRowBytes : 0u;
  static constexpr uint32_t kCacheRowBytes = FP8 ? kD : kRowBytes;
  static constexpr uint32_t kStageBytes = 2u * kTile * kCacheRowBytes;
  static constexpr uint32_t kSmemBytes = kQBytes + kWorkBytes + kStages * kStageBytes;
  static_assert(kSmemBytes <= 227u * 1024u, "shared memory budget");
};

struct Params {
  const __nv_bfloat16 *q;                    // [tokens, q_heads, 256]
  const void *cache_k, *cache_v;             // [rows, kv_heads, 256] bf16 or e4m3 bytes
  const __nv_bfloat16 *k_new, *v_new;        // decode: [kv_heads, 256], the row at `position`
  float *pacc, *pmax, *pden;
  const int32_t *pos_device;
  uint32_t pos_scalar, tokens, q_heads, kv_heads, n_splits, split_block;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// 16 bytes global -> shared without passing through registers; src_bytes == 0 writes zeros.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool F16>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (F16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool F16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (F16) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
  }
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// 16 E4M3 bytes -> 16 float16 (two 16-byte chunks).  0x7F / 0xFF are NaN to the hardware conversion
// and +-448 to the reference's reader (attention_flash_splitk.cu:54-72): they are stepped down to
// 0x7E / 0xFE (= +-448) first.
__device__ __forceinline__ void e4m3x16_to_f16(const uint4 &in, uint4 &lo, uint4 &hi) {
  const uint32_t w[4] = {in.x, in.y, in.z, in.w};
  uint32_t h[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t v = w[i] - (__vcmpeq4(w[i] & 0x7f7f7f7fu, 0x7f7f7f7fu) & 0x01010101u);
    asm("{\n\t.reg .b16 p, q;\n\tmov.b32 {p, q}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, p;\n\tcvt.rn.f16x2.e4m3x2 %1, q;\n\t}"
        : "=r"(h[2 * i]), "=r"(h[2 * i + 1]) : "r"(v));
  }
  lo = make_uint4(h[0], h[1], h[2], h[3]);
  hi = make_uint4(h[4], h[5], h[6], h[7]);
}

// bf16 row (as eight 16-byte chunks per 64 values) -> f16, for q and for the decode step's new row.
__device__ __forceinline__ uint4 bf16x8_to_f16(const uint4 &in) {
  const uint32_t w[4] = {in.x, in.y, in.z, in.w};
  uint32_t h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 v = __floats2half2_rn(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
    h[i] = *reinterpret_cast<const uint32_t *>(&v);
  }
  return make_uint4(h[0], h[1], h[2], h[3]);
}

// The reference's E4M3 writer of the cache append (attention_decode_tiled.cu:62-117): magnitude
// rounded half up, saturation at 0x7E, zero and non-finite values give 0.
__device__ __forceinline__ uint8_t encode_e4m3_append(float v) {
  if (!(fabsf(v) <= 3.0e38f) || v == 0.0f) return 0;
  const bool negative = v < 0.0f;
  const float a = fabsf(v);
  uint32_t code;
  if (a >= 448.0f) {
    code = 0x7e;
  } else if (a < 0x1p-6f) {
    const int m = static_cast<int>(floorf(a * 512.0f + 0.5f));
    code = m >= 8 ? 0x08u : static_cast<uint32_t>(m);
  } else {
    int e = 0;
    const float frac = frexpf(a, &e);
    int m = static_cast<int>(floorf((frac * 2.0f - 1.0f) * 8.0f + 0.5f));
    int ef = e + 6;
    if (m >= 8) { m = 0; ef += 1; }
    if (ef >= 15) { ef = 15; m = min(m, 6); }
    code = static_cast<uint32_t>((ef << 3) | m);
  }
  return static_cast<uint8_t>((negative ? 0x80u : 0u) | code);
}

// FP8: the cache holds E4M3 bytes and the product runs in f16; otherwise bf16 throughout.
// DECODE: one token, timestep == position comes from k_new / v_new, the owning split appends it.
// MT: 16-row tiles of (token, q head) rows per CTA.  The NW warps form MT x TH: warp w works on row
// tile w % MT and on the timesteps [th * 64 / TH, (th + 1) * 64 / TH) of every 64-row KV tile, th =
// w / MT, with an online-softmax state of its own; the TH states of a row meet once, after the loop.
// So 4 query tokens x 6 heads (24 rows, MT = 2) or a decode token (6 rows, MT = 1) keep every
// tensor core busy on rows that exist, instead of three warps out of four multiplying padding.
// K / V tiles arrive through a three-deep cp.async ring, two tiles ahead of the one being multiplied.
template <bool FP8, bool DECODE, int MT, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
attention_splitk_tc_kernel(const Params p) {
  using L = Layout<FP8, MT>;
  constexpr uint32_t NT = NW * 32u, TH = NW / MT, W = kTile / TH;               // timesteps per warp per tile
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t *sq = smem, *work = smem + L::kQBytes, *ring = work + L::kWorkBytes;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t gid = lane >> 2, tig = lane & 3u;
  const uint32_t mt = warp % MT, th = warp / MT;
  const uint32_t kvh = blockIdx.x, chunk = blockIdx.y, split = blockIdx.z;
  const uint32_t q_per_kv = p.q_heads / p.kv_heads;
  const uint32_t m_rows = p.tokens * q_per_kv;                       // rows of this kv head
  const uint32_t start = p.pos_device != nullptr ? static_cast<uint32_t>(*p.pos_device) : p.pos_scalar;

  // KV range of this split
  uint32_t t0, t1;
  if (DECODE) {
    t0 = split * p.split_block;
    t1 = min(t0 + p.split_block, start + 1u);
  } else {
    const uint32_t visible = start + p.tokens;                        // rows [0, visible)
    const uint32_t iters = (visible - 1u + kTile) / kTile;
    const uint32_t per = (iters + p.n_splits - 1u) / p.n_splits;
    t0 = min(split * per, iters) * kTile;
    t1 = min(min((split + 1u) * per, iters) * kTile, visible);
  }
  const uint32_t n_tiles = t1 > t0 ? (t1 - t0 + kTile - 1u) / kTile : 0u;

  // this lane's two rows: (token, q head) pairs, token-major
  const uint32_t row_lo = chunk * L::kRows + mt * 16u + gid, row_hi = row_lo + 8u;
  const bool ok_lo = row_lo < m_rows, ok_hi = row_hi < m_rows;
  const bool warp_has_rows = chunk * L::kRows + mt * 16u < m_rows;
  const uint32_t tok_lo = row_lo / q_per_kv, tok_hi = row_hi / q_per_kv;
  // last visible timestep of each row (inclusive)
  const uint32_t lim_lo = DECODE ? start : start + tok_lo, lim_hi = DECODE ? start : start + tok_hi;

  // ---- tile `idx` of the split -> ring slot idx % kStages, in the cache's format.  Rows at or past t1
  // arrive as zeros; the decode step's own row comes from k_new / v_new (directly for a bf16 cache,
  // at the expansion for an FP8 cache).
  const uint8_t *ck = static_cast<const uint8_t *>(p.cache_k), *cv = static_cast<const uint8_t *>(p.cache_v);
  auto load_tile = [&](uint32_t idx) {
    const uint32_t base = t0 + idx * kTile;
    const uint32_t dst = smem_u32(ring + (idx % kStages) * L::kStageBytes);
    constexpr uint32_t kChunks = L::kCacheRowBytes / 16u;             // 16-byte chunks per row: 16 or 32
    if (base + kTile <= t1 && !(DECODE && start < base + kTile)) {
      // whole tile of cache rows: a thread's copies differ by a fixed stride (its chunk, and the
      // row's swizzle, stay the same from one of its rows to the next)
      constexpr uint32_t kRowStep = NT / kChunks;                     // rows between two copies of a thread: 8 or 16 (4 / 8 with four warps)
      const uint32_t r0 = threadIdx.x / kChunks, c = threadIdx.x % kChunks;
      const size_t off = (static_cast<size_t>(base + r0) * p.kv_heads + kvh) * L::kCacheRowBytes + c * 16u;
      const size_t step = static_cast<size_t>(kRowStep) * p.kv_heads * L::kCacheRowBytes;
      const uint8_t *ks = ck + off, *vs = cv + off;
#pragma unroll
      for (uint32_t n = 0; n < kTile / kRowStep; ++n) {
        const uint32_t r = r0 + n * kRowStep;
        const uint32_t at = dst + (FP8 ? r * kD + c * 16u : r * kRowBytes + ((c ^ (r & 7u)) << 4));
        cp_async16(at, ks, 16u);
        cp_async16(at + kTile * L::kCacheRowBytes, vs, 16u);
        ks += step;
        vs += step;
      }
      return;
    }
#pragma unroll 4
    for (uint32_t i = threadIdx.x; i < kTile * kChunks; i += NT) {
      const uint32_t r = i / kChunks, c = i % kChunks, t = base + r;
      const size_t off = (static_cast<size_t>(t) * p.kv_heads + kvh) * L::kCacheRowBytes + c * 16u;
      const uint8_t *ks = ck + off, *vs = cv + off;
      uint32_t bytes = t < t1 ? 16u : 0u;
      if (DECODE && t == start) {
        if (FP8) {
          bytes = 0u;
        } else {
          ks = reinterpret_cast<const uint8_t *>(p.k_new + kvh * kD) + c * 16u;
          vs = reinterpret_cast<const uint8_t *>(p.v_new + kvh * kD) + c * 16u;
        }
      }
      if (bytes == 0u) { ks = ck; vs = cv; }
      const uint32_t at = FP8 ? r * kD + c * 16u : r * kRowBytes + ((c ^ (r & 7u)) << 4);
      cp_async16(dst + at, ks, bytes);
      cp_async16(dst + kTile * L::kCacheRowBytes + at, vs, bytes);
    }
  };
  for (uint32_t s = 0; s + 1u < kStages; ++s) {
    if (s < n_tiles) load_tile(s);
    cp_async_commit();
  }

  // ---- stage Q: chunk c of row r at chunk c ^ (r & 7)
  for (uint32_t i = threadIdx.x; i < L::kRows * 32u; i += NT) {
    const uint32_t r = i >> 5, c = i & 31u, row = chunk * L::kRows + r;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < m_rows) {
      const uint32_t tok = row / q_per_kv, qh = kvh * q_per_kv + row % q_per_kv;
      v = __ldg(reinterpret_cast<const uint4 *>(p.q + (static_cast<size_t>(tok) * p.q_heads + qh) * kD) + c);
      if (FP8) v = bf16x8_to_f16(v);
    }
    *reinterpret_cast<uint4 *>(sq + r * kRowBytes + ((c ^ (r & 7u)) << 4)) = v;
  }

  float o[32][4];
#pragma unroll
  for (int j = 0; j < 32; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  constexpr float kScaleLog2 = 0.0625f * 1.4426950408889634f;        // rsqrt(256) * log2(e)

  for (uint32_t it = 0; it < n_tiles; ++it) {
    const uint32_t base = t0 + it * kTile;
    cp_async_wait<kStages - 2>();                                     // this thread's part of tile `it` has landed
    __syncthreads();                                                  // everybody's has; tile it - 1 is consumed (and Q staged)
    if (it + kStages - 1u < n_tiles) load_tile(it + kStages - 1u);    // into the slot tile it - 1 left
    cp_async_commit();
    const uint8_t *slot = ring + (it % kStages) * L::kStageBytes;
    const uint8_t *sk = slot, *sv = slot + kTile * L::kCacheRowBytes;
    if (FP8) {
      // ---- expand E4M3 -> f16 into the work tile (chunk-swizzled rows of 512 bytes)
      uint8_t *wk = work, *wv = work + kTile * kRowBytes;
#pragma unroll 2
      for (uint32_t i = threadIdx.x; i < kTile * 16u; i += NT) {
        const uint32_t r = i >> 4, c = i & 15u, t = base + r;
        uint4 klo, khi, vlo, vhi;
        if (DECODE && t == start && t < t1) {
          klo = bf16x8_to_f16(__ldg(reinterpret_cast<const uint4 *>(p.k_new + kvh * kD) + 2u * c));
          khi = bf16x8_to_f16(__ldg(reinterpret_cast<const uint4 *>(p.k_new + kvh * kD) + 2u * c + 1u));
          vlo = bf16x8_to_f16(__ldg(reinterpret_cast<const uint4 *>(p.v_new + kvh * kD) + 2u * c));
          vhi = bf16x8_to_f16(__ldg(reinterpret_cast<const uint4 *>(p.v_new + kvh * kD) + 2u * c + 1u));
        } else {
          e4m3x16_to_f16(*reinterpret_cast<const uint4 *>(sk + r * kD + c * 16u), klo, khi);
          e4m3x16_to_f16(*reinterpret_cast<const uint4 *>(sv + r * kD + c * 16u), vlo, vhi);
        }
        // A 16-byte store is served eight lanes at a time: lanes c and c + 4 of such a group own chunk
        // pairs that fall on the same banks, so the upper four store their odd chunk first.
        const uint32_t sw = r & 7u, flip = (c >> 2) & 1u;
        const uint32_t first = ((2u * c + flip) ^ sw) << 4, second = ((2u * c + 1u - flip) ^ sw) << 4;
        *reinterpret_cast<uint4 *>(wk + r * kRowBytes + first) = flip ? khi : klo;
        *reinterpret_cast<uint4 *>(wv + r * kRowBytes + first) = flip ? vhi : vlo;
        *reinterpret_cast<uint4 *>(wk + r * kRowBytes + second) = flip ? klo : khi;
        *reinterpret_cast<uint4 *>(wv + r * kRowBytes + second) = flip ? vlo : vhi;
      }
      __syncthreads();
      sk = wk;
      sv = wv;
    }
    const uint32_t tw = base + th * W;                                // first timestep of this warp's slice
    if (!warp_has_rows || tw >= t1) continue;                         // padding rows / nothing visible: no work (warp-uniform)

    // ---- S = Q K^T for this warp's 16 rows x W timesteps
    // two accumulators per 8-timestep tile (even / odd k-steps): twice as many independent MMA chains
    float s[W / 8][4], s2[W / 8][4];
#pragma unroll
    for (uint32_t j = 0; j < W / 8u; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      s2[j][0] = s2[j][1] = s2[j][2] = s2[j][3] = 0.f;
    }
    const uint32_t q_row = mt * 16u + (lane & 15u);
    const uint32_t q_addr = smem_u32(sq) + q_row * kRowBytes, q_sw = q_row & 7u;
#pragma unroll 4
    for (uint32_t kk = 0; kk < 16u; kk += 2u) {
#pragma unroll
      for (uint32_t par = 0; par < 2u; ++par) {
        uint32_t a[4];
        ldmatrix_x4(a, q_addr + (((2u * (kk + par) + (lane >> 4)) ^ q_sw) << 4));
#pragma unroll
        for (uint32_t jp = 0; jp < W / 16u; ++jp) {                   // two 8-timestep tiles per load
          const uint32_t n_row = th * W + 16u * jp + 8u * (lane >> 4) + (lane & 7u);
          uint32_t b[4];
          ldmatrix_x4(b, smem_u32(sk) + n_row * kRowBytes + (((2u * (kk + par) + ((lane >> 3) & 1u)) ^ (n_row & 7u)) << 4));
          mma16816<FP8>(par == 0u ? s[2 * jp] : s2[2 * jp], a, b[0], b[1]);
          mma16816<FP8>(par == 0u ? s[2 * jp + 1] : s2[2 * jp + 1], a, b[2], b[3]);
        }
      }
    }
#pragma unroll
    for (uint32_t j = 0; j < W / 8u; ++j) {
      s[j][0] += s2[j][0]; s[j][1] += s2[j][1]; s[j][2] += s2[j][2]; s[j][3] += s2[j][3];
    }

    // ---- mask + online softmax (row gid: c0, c1 ; row gid + 8: c2, c3).  A slice that ends at or
    // before `start` and before t1 is visible to every row that exists: nothing to mask (padding
    // rows hold zero queries, their finite scores go nowhere).
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
    const bool all_visible = tw + W <= t1 && tw + W <= start + 1u;
#pragma unroll
    for (uint32_t j = 0; j < W / 8u; ++j) {
#pragma unroll
      for (uint32_t e = 0; e < 2u; ++e) {
        if (!all_visible) {
          const uint32_t t = tw + 8u * j + 2u * tig + e;
          if (!(ok_lo && t <= lim_lo && t < t1)) s[j][e] = -INFINITY;
          if (!(ok_hi && t <= lim_hi && t < t1)) s[j][2 + e] = -INFINITY;
        }
        mx_lo = fmaxf(mx_lo, s[j][e]);
        mx_hi = fmaxf(mx_hi, s[j][2 + e]);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    // all arithmetic on raw (unscaled) scores; exp2 with the scale folded in
    const float al_lo = m_lo == -INFINITY ? 0.f : exp2f((m_lo - mn_lo) * kScaleLog2);
    const float al_hi = m_hi == -INFINITY ? 0.f : exp2f((m_hi - mn_hi) * kScaleLog2);
    const float ref_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t pa[W / 16][4];                                          // P as A fragments, k-steps of 16 timesteps
#pragma unroll
    for (uint32_t j = 0; j < W / 8u; ++j) {
      const float p0 = exp2f((s[j][0] - ref_lo) * kScaleLog2), p1 = exp2f((s[j][1] - ref_lo) * kScaleLog2);
      const float p2 = exp2f((s[j][2] - ref_hi) * kScaleLog2), p3 = exp2f((s[j][3] - ref_hi) * kScaleLog2);
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      pa[j >> 1][(j & 1u) * 2u] = pack2<FP8>(p0, p1);
      pa[j >> 1][(j & 1u) * 2u + 1u] = pack2<FP8>(p2, p3);
    }
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    l_lo = l_lo * al_lo + sum_lo;
    l_hi = l_hi * al_hi + sum_hi;
    if (__any_sync(0xffffffffu, mn_lo != m_lo || mn_hi != m_hi)) {    // a running maximum moved (rare after the first tiles)
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        o[j][0] *= al_lo; o[j][1] *= al_lo;
        o[j][2] *= al_hi; o[j][3] *= al_hi;
      }
    }
    m_lo = mn_lo;
    m_hi = mn_hi;

    // ---- O += P V: k = timestep (steps of 16), n = head dimension (32 tiles of 8)
#pragma unroll
    for (uint32_t ks = 0; ks < W / 16u; ++ks) {
      const uint32_t v_row = th * W + 16u * ks + 8u * ((lane >> 3) & 1u) + (lane & 7u);
      const uint32_t v_addr = smem_u32(sv) + v_row * kRowBytes, v_sw = v_row & 7u;
#pragma unroll
      for (uint32_t jd = 0; jd < 32u; jd += 2u) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, v_addr + (((jd + (lane >> 4)) ^ v_sw) << 4));
        mma16816<FP8>(o[jd], pa[ks], b[0], b[1]);
        mma16816<FP8>(o[jd + 1], pa[ks], b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();

  // ---- partials: unnormalised O, m in scaled units, l
  if (TH == 1u) {
    if (ok_lo || ok_hi) {
      const uint32_t qh_lo = kvh * q_per_kv + row_lo % q_per_kv, qh_hi = kvh * q_per_kv + row_hi % q_per_kv;
      const size_t idx_lo = (static_cast<size_t>(tok_lo) * p.q_heads + qh_lo) * p.n_splits + split;
      const size_t idx_hi = (static_cast<size_t>(tok_hi) * p.q_heads + qh_hi) * p.n_splits + split;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (ok_lo) *reinterpret_cast<float2 *>(p.pacc + idx_lo * kD + 8 * j + 2 * tig) = make_float2(o[j][0], o[j][1]);
        if (ok_hi) *reinterpret_cast<float2 *>(p.pacc + idx_hi * kD + 8 * j + 2 * tig) = make_float2(o[j][2], o[j][3]);
      }
      if (tig == 0u) {
        if (ok_lo) { p.pmax[idx_lo] = m_lo == -INFINITY ? -INFINITY : m_lo * 0.0625f; p.pden[idx_lo] = l_lo; }
        if (ok_hi) { p.pmax[idx_hi] = m_hi == -INFINITY ? -INFINITY : m_hi * 0.0625f; p.pden[idx_hi] = l_hi; }
      }
    }
  } else {
    // the TH states of a row meet in shared memory (the ring is free now), in slice order
    float *so = reinterpret_cast<float *>(work);                      // [TH][16 MT][kMergeStride]
    float *sm = so + TH * L::kRows * kMergeStride, *sl = sm + TH * L::kRows;
    static_assert((TH * L::kRows * (kMergeStride + 2u)) * 4u <= L::kWorkBytes + kStages * L::kStageBytes, "meeting area");
    __syncthreads();
    const uint32_t r_lo = th * L::kRows + mt * 16u + gid, r_hi = r_lo + 8u;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      *reinterpret_cast<float2 *>(so + r_lo * kMergeStride + 8 * j + 2 * tig) = make_float2(o[j][0], o[j][1]);
      *reinterpret_cast<float2 *>(so + r_hi * kMergeStride + 8 * j + 2 * tig) = make_float2(o[j][2], o[j][3]);
    }
    if (tig == 0u) {
      sm[r_lo] = m_lo; sl[r_lo] = l_lo;
      sm[r_hi] = m_hi; sl[r_hi] = l_hi;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < L::kRows * (kD / 4u); i += NT) {
      const uint32_t r = i / (kD / 4u), d = (i % (kD / 4u)) * 4u, row = chunk * L::kRows + r;
      if (row >= m_rows) continue;
      float M = -INFINITY;
#pragma unroll
      for (uint32_t h = 0; h < TH; ++h) M = fmaxf(M, sm[h * L::kRows + r]);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      float den = 0.f;
#pragma unroll
      for (uint32_t h = 0; h < TH; ++h) {
        const float mh = sm[h * L::kRows + r];
        const float w = mh == -INFINITY ? 0.f : exp2f((mh - M) * kScaleLog2);
        const float4 v = *reinterpret_cast<const float4 *>(so + (h * L::kRows + r) * kMergeStride + d);
        acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y);
        acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
        den = fmaf(w, sl[h * L::kRows + r], den);
      }
      const uint32_t tok = row / q_per_kv, qh = kvh * q_per_kv + row % q_per_kv;
      const size_t idx = (static_cast<size_t>(tok) * p.q_heads + qh) * p.n_splits + split;
      *reinterpret_cast<float4 *>(p.pacc + idx * kD + d) = acc;
      if (d == 0u) { p.pmax[idx] = M == -INFINITY ? -INFINITY : M * 0.0625f; p.pden[idx] = den; }
    }
  }

  // ---- decode: the split that owns `position` appends the new row to the cache
  if (DECODE && chunk == 0u && t0 <= start && start < t1) {
    for (uint32_t d = threadIdx.x; d < kD; d += NT) {
      const size_t off = (static_cast<size_t>(start) * p.kv_heads + kvh) * kD + d;
      const __nv_bfloat16 kn = p.k_new[kvh * kD + d], vn = p.v_new[kvh * kD + d];
      if (FP8) {
        static_cast<uint8_t *>(const_cast<void *>(p.cache_k))[off] = encode_e4m3_append(__bfloat162float(kn));
        static_cast<uint8_t *>(const_cast<void *>(p.cache_v))[off] = encode_e4m3_append(__bfloat162float(vn));
      } else {
        static_cast<__nv_bfloat16 *>(const_cast<void *>(p.cache_k))[off] = kn;
        static_cast<__nv_bfloat16 *>(const_cast<void *>(p.cache_v))[off] = vn;
      }
    }
  }
}

// Log-sum-exp merge of the splits (attention_flash_splitk.cu:375-420): one CTA per (token, q head),
// one thread per head dimension; every thread forms the weights itself (n_splits is small).
__global__ void __launch_bounds__(kD)
attention_splitk_reduce_kernel(const float *__restrict__ pacc, const float *__restrict__ pmax,
                               const float *__restrict__ pden, __nv_bfloat16 *__restrict__ out, uint32_t n_splits) {
  const size_t flat = blockIdx.x;
  const uint32_t d = threadIdx.x;
  float m = -INFINITY;
  for (uint32_t s = 0; s < n_splits; ++s) m = fmaxf(m, pmax[flat * n_splits + s]);
  float dn = 0.f, acc = 0.f;
  for (uint32_t s0 = 0; s0 < n_splits; s0 += 16u) {                  // sixteen loads in flight, sums in split order
    float v[16];
#pragma unroll
    for (uint32_t i = 0; i < 16u; ++i) v[i] = __ldcg(pacc + (flat * n_splits + min(s0 + i, n_splits - 1u)) * kD + d);
#pragma unroll
    for (uint32_t i = 0; i < 16u; ++i) {
      if (s0 + i < n_splits) {
        const float pm = pmax[flat * n_splits + s0 + i];
        const float w = pm == -INFINITY ? 0.f : expf(pm - m);
        dn = fmaf(pden[flat * n_splits + s0 + i], w, dn);
        acc = fmaf(v[i], w, acc);
      }
    }
  }
  out[flat * kD + d] = __float2bfloat16(dn > 0.f ? acc / dn : 0.f);
}

// Grow-on-demand scratch for callers that pass no partial buffers (the reference keeps the same kind
// of process-wide scratch, attention_flash_splitk.cu:424-500).  Growing allocates, which a stream
// capture in progress forbids: the entry then declines with NOT_IMPLEMENTED, as the reference does.
struct Scratch {
  float *acc = nullptr, *mx = nullptr, *dn = nullptr;
  size_t rows = 0;                            // capacity in (token, head, split) rows
  int device = -1;
};
std::mutex g_scratch_mu;
Scratch g_scratch;

int reserve_scratch(size_t rows, float **acc, float **mx, float **dn) {
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return QWEN36_STATUS_CUDA_ERROR;
  if (g_scratch.device != dev || rows > g_scratch.rows) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(q36::stream(), &st) == cudaSuccess && st != cudaStreamCaptureStatusNone)
      return QWEN36_STATUS_NOT_IMPLEMENTED;
    if (g_scratch.device == dev) { cudaFree(g_scratch.acc); cudaFree(g_scratch.mx); cudaFree(g_scratch.dn); }
    g_scratch = Scratch{};
    float *a = nullptr, *m = nullptr, *d = nullptr;
    if (cudaMalloc(&a, rows * kD * sizeof(float)) != cudaSuccess || cudaMalloc(&m, rows * sizeof(float)) != cudaSuccess ||
        cudaMalloc(&d, rows * sizeof(float)) != cudaSuccess) {
      cudaFree(a); cudaFree(m); cudaFree(d);
      (void)cudaGetLastError();
      return QWEN36_STATUS_CUDA_ERROR;
    }
    g_scratch.acc = a; g_scratch.mx = m; g_scratch.dn = d;
    g_scratch.rows = rows;
    g_scratch.device = dev;
  }
  *acc = g_scratch.acc; *mx = g_scratch.mx; *dn = g_scratch.dn;
  return QWEN36_STATUS_SUCCESS;
}

template <bool FP8, bool DECODE, int MT, int NW>
int launch_mt(const Params &p, uint32_t chunks) {
  using L = Layout<FP8, MT>;
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(attention_splitk_tc_kernel<FP8, DECODE, MT, NW>),
                               static_cast<int>(L::kSmemBytes)) != cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  const dim3 grid(p.kv_heads, chunks, p.n_splits);
  attention_splitk_tc_kernel<FP8, DECODE, MT, NW><<<grid, NW * 32, L::kSmemBytes, q36::stream()>>>(p);
  return q36::launch_status();
}

// Rows of one kv head (tokens x q heads per kv head) decide the CTA's shape: up to 16 rows, one row
// tile and four timestep slices; up to 32, two and two; more, four row tiles per CTA and as many
// CTAs (blockIdx.y) as that takes.
template <bool FP8, bool DECODE>
int launch(const Params &p) {
  const uint32_t m_rows = p.tokens * (p.q_heads / p.kv_heads);
  if (m_rows <= 16u) return launch_mt<FP8, DECODE, 1, 4>(p, 1);
  if (m_rows <= 32u) return launch_mt<FP8, DECODE, 2, 8>(p, 1);
  return launch_mt<FP8, DECODE, 4, 8>(p, (m_rows + 63u) / 64u);
}

}  // namespace

extern "C" int qwen36_attention_flash_splitk_prefill_bf16(const qwen36_attention_prefill_spec_t *spec, int n_splits) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  // argument rules of kernels-cuda/attention_flash_splitk.cu:509-520
  if (spec->tokens == 0 || spec->tokens > 32 || spec->q_bf16.ptr == 0 || spec->kv_cache_k.ptr == 0 ||
      spec->kv_cache_v.ptr == 0 || spec->output_bf16.ptr == 0 || spec->shape.head_dim != kD ||
      spec->shape.q_heads == 0 || spec->shape.kv_heads == 0 || spec->shape.q_heads % spec->shape.kv_heads != 0 ||
      (spec->kv_cache_dtype != 0 && spec->kv_cache_dtype != 1) || n_splits < 1)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  if (spec->start_position + spec->tokens >= (1ull << 31) || spec->shape.q_heads > 65535 || n_splits > 65535)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  Params p{};
  p.q = as_ptr<const __nv_bfloat16>(spec->q_bf16);
  p.cache_k = as_ptr<const void>(spec->kv_cache_k);
  p.cache_v = as_ptr<const void>(spec->kv_cache_v);
  p.pos_device = as_ptr<const int32_t>(spec->start_position_device_i32);
  p.pos_scalar = static_cast<uint32_t>(spec->start_position);
  p.tokens = static_cast<uint32_t>(spec->tokens);
  p.q_heads = static_cast<uint32_t>(spec->shape.q_heads);
  p.kv_heads = static_cast<uint32_t>(spec->shape.kv_heads);
  p.n_splits = static_cast<uint32_t>(n_splits);
  const size_t rows = spec->tokens * spec->shape.q_heads * static_cast<size_t>(n_splits);
  if (spec->partial_acc_f32.ptr != 0 && spec->partial_max_f32.ptr != 0 && spec->partial_denom_f32.ptr != 0) {
    p.pacc = as_ptr<float>(spec->partial_acc_f32);
    p.pmax = as_ptr<float>(spec->partial_max_f32);
    p.pden = as_ptr<float>(spec->partial_denom_f32);
  } else {
    const int rc = reserve_scratch(rows, &p.pacc, &p.pmax, &p.pden);
    if (rc != QWEN36_STATUS_SUCCESS) return rc;
  }
  const int rc = spec->kv_cache_dtype == 1 ? launch<true, false>(p) : launch<false, false>(p);
  if (rc != QWEN36_STATUS_SUCCESS) return rc;
  attention_splitk_reduce_kernel<<<static_cast<unsigned>(spec->tokens * spec->shape.q_heads), kD, 0, q36::stream()>>>(
      p.pacc, p.pmax, p.pden, as_ptr<__nv_bfloat16>(spec->output_bf16), p.n_splits);
  return q36::launch_status();
}

extern "C" int qwen36_attention_decode_split_tiled(const qwen36_attention_decode_spec_t *spec, int n_splits,
                                                   int split_timesteps_per_block) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  // shapes the reference's entry takes (attention_decode_tiled.cu:376-388); everything else declines
  if (spec->shape.head_dim != kD || (spec->kv_cache_dtype != 0 && spec->kv_cache_dtype != 1) ||
      spec->shape.kv_heads == 0 || spec->shape.q_heads % spec->shape.kv_heads != 0 ||
      spec->shape.q_heads / spec->shape.kv_heads > 8 || spec->shape.q_heads / spec->shape.kv_heads < 2 || n_splits < 1 ||
      split_timesteps_per_block < 8 || split_timesteps_per_block % 8 != 0)
    return QWEN36_STATUS_NOT_IMPLEMENTED;
  if (spec->q_bf16.ptr == 0 || spec->k_bf16.ptr == 0 || spec->v_bf16.ptr == 0 || spec->kv_cache_k.ptr == 0 ||
      spec->kv_cache_v.ptr == 0 || spec->partial_acc_f32.ptr == 0 || spec->partial_max_f32.ptr == 0 ||
      spec->partial_denom_f32.ptr == 0 || spec->position >= (1ull << 31) || n_splits > 65535)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  Params p{};
  p.q = as_ptr<const __nv_bfloat16>(spec->q_bf16);
  p.k_new = as_ptr<const __nv_bfloat16>(spec->k_bf16);
  p.v_new = as_ptr<const __nv_bfloat16>(spec->v_bf16);
  p.cache_k = as_ptr<const void>(spec->kv_cache_k);
  p.cache_v = as_ptr<const void>(spec->kv_cache_v);
  p.pacc = as_ptr<float>(spec->partial_acc_f32);
  p.pmax = as_ptr<float>(spec->partial_max_f32);
  p.pden = as_ptr<float>(spec->partial_denom_f32);
  p.pos_device = as_ptr<const int32_t>(spec->position_device_i32);
  p.pos_scalar = static_cast<uint32_t>(spec->position);
  p.tokens = 1;
  p.q_heads = static_cast<uint32_t>(spec->shape.q_heads);
  p.kv_heads = static_cast<uint32_t>(spec->shape.kv_heads);
  p.n_splits = static_cast<uint32_t>(n_splits);
  p.split_block = static_cast<uint32_t>(split_timesteps_per_block);
  return spec->kv_cache_dtype == 1 ? launch<true, true>(p) : launch<false, true>(p);
}
