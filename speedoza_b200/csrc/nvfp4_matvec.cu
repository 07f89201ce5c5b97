// W4A16 NVFP4 GEMV: y[row] = bf16( sum_g (sum_{i<16} x[16g+i] * e2m1(w)) * (ue4m3(sf[g,row]) * global) )
// (semantics of kernels-cuda/ops.cu:547-639 in the reference).
//
// Entry points qwen36_nvfp4_matvec / qwen36_nvfp4_matvec_group.  Shapes with out_features % 128
// == 0 and in_features % 256 == 0 go to the tensor-core GEMV (nvfp4_gemv_mma.cu); this file holds
// the SIMT pipeline that takes the other 32-column-aligned shapes, and the generic kernel.
//
// SIMT pipeline: HBM-bound weight streaming.  Persistent CTAs; a producer warp drives the TMA
// engine (tiled TMA boxes when out_features % 128 == 0, else one cp.async.bulk per row segment;
// mbarrier ring of 72 KB per CTA), so the bytes in flight do not depend on occupancy or
// registers.  Eight consumer warps each own a "row quad": rows r, r+32, r+64,
// r+96 of one 128-row block.  Those four rows share one 16-byte word per scale
// tile (4 rows x 4 groups), so a lane fetches its scales with ONE 16-byte
// shared-memory load per 128 weights and reuses every activation register four
// times.  Lanes stride along K (32 columns each per stage).  Nibbles are
// expanded by cvt.rn.f16x2.e2m1x2 (two weights per instruction); products
// accumulate in float32; the lanes of a warp meet in a butterfly once per row.
//
// Weights and scales are streamed before griddepcontrol.wait, so under
// programmatic dependent launch the ring fills while the kernel that produces
// x is still finishing.
#include "common.cuh"
#include "nvfp4_gemv_mma.cuh"

#include <atomic>
#include <cuda.h>
#include <cuda_fp16.h>
#include <mutex>

namespace {

using q36::as_ptr;

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

// 16-byte chunk swizzle of the activation buffer (float16, four chunks per 32-value slot) so
// that the eight lanes of a quarter warp, which read chunks 64 bytes apart, land on distinct
// bank groups.
__device__ __forceinline__ uint32_t x_chunk(uint32_t slot, uint32_t i) {
  return slot * 4u + (i ^ ((slot >> 1) & 3u));
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

__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// even += w.lo * x.lo ; odd += w.hi * x.hi : float16 operands, float32 accumulate, products exact.
__device__ __forceinline__ void fma_mixed_eo(float &even, float &odd, uint32_t w_h2, uint32_t x_h2) {
  asm("{\n\t.reg .f16 wl, wh, xl, xh;\n\t"
      "mov.b32 {wl, wh}, %2;\n\t"
      "mov.b32 {xl, xh}, %3;\n\t"
      "fma.rn.f32.f16 %0, wl, xl, %0;\n\t"
      "fma.rn.f32.f16 %1, wh, xh, %1;\n\t}"
      : "+f"(even), "+f"(odd)
      : "r"(w_h2), "r"(x_h2));
}

// ---- shared-memory ring fed by the TMA engine --------------------------------------------
//
// QUADS (8, 4, 2 or 1) row quads form a work unit: rows r0 + q + 32 j of one 128-row block,
// q < QUADS, j < 4.  Consumer warp w serves quad w % QUADS and K-part w / QUADS: with fewer
// quads per unit the eight warps split K between them (stage s of a unit belongs to K-part
// s % KPARTS), so small matrices still spread over every SM.  One pipeline stage = 1024
// columns of a unit:
//   weights  [j][q][512 B]        : ONE 4-D tiled TMA box over the view
//                                   [N/128][4][32][K/2 bytes] of the weight matrix
//   scales   [16 tiles][QUADS*16 B]: ONE 3-D box over the view [N/128][tiles][512 B] of the tiled
//                                   scale buffer (128-byte swizzle when QUADS == 8, so that the
//                                   16 tiles a warp reads land on different banks)
// The producer warp's elected lane issues both copies against the stage's "full" mbarrier; the
// QUADS warps that read a stage release it through its "empty" mbarrier.  CTAs are persistent:
// unit = blockIdx.x, += gridDim.x, and the stream of stages runs across unit borders.  The ring
// always holds 72 KB (32 / QUADS stages); a 54 KB ring measured 17 % slower on the decode sweep.
// When N is not a multiple of 128 the tiled views would reach past the allocation, so that
// (rare) case feeds the same ring (QUADS = 8) with one cp.async.bulk per row segment instead.
constexpr uint32_t kSegBytes = 512;                         // 1024 columns of one row
constexpr uint32_t kRingStagesX8 = 4;                                // stages of the QUADS = 8 ring
constexpr uint32_t kRingBytes = kRingStagesX8 * 8u * (4u * kSegBytes + 256u);   // 73728
constexpr uint32_t kHeaderBytes = 2048;
constexpr uint32_t kSpinLimit = 1u << 24;

__device__ unsigned int g_matvec_error = 0;                 // set when a bounded wait gives up


__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: gives up after kSpinLimit polls, records it and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  atomicExch(&g_matvec_error, 1u);
  return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, uint32_t c0, uint32_t c1, uint32_t c2,
                                            uint32_t c3, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint32_t c0, uint32_t c1, uint32_t c2,
                                            uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// TMAP: stages are filled by tiled TMA through the two tensor maps (N % 128 == 0); otherwise
// (QUADS == 8 only) by per-row cp.async.bulk copies.
template <int QUADS, bool TMAP>
__global__ void __launch_bounds__(kThreads + 32)
nvfp4_matvec_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_sf,
                    const __nv_bfloat16 *__restrict__ x, const uint8_t *__restrict__ weight,
                    const uint8_t *__restrict__ sf, const float *__restrict__ tensor_scale,
                    __nv_bfloat16 *__restrict__ y, uint32_t K, uint32_t N) {
  constexpr uint32_t kStages = kRingStagesX8 * 8u / QUADS;  // 4, 8, 16, 32
  constexpr uint32_t KPARTS = kWarps / QUADS;               // warps that split K of one quad
  constexpr uint32_t kStageW = QUADS * 4u * kSegBytes;
  constexpr uint32_t kSfRow = QUADS * 16u;                  // bytes of one scale tile kept per stage
  constexpr uint32_t kStageBytes = kStageW + 16u * kSfRow;
  constexpr uint32_t kUnitsPerBlock = 32u / QUADS;
  static_assert(kStages * kStageBytes == kRingBytes, "ring size");

  extern __shared__ __align__(128) uint8_t smem_raw[];
  // the swizzled scale boxes need 1024-byte aligned stages
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float *lut = reinterpret_cast<float *>(smem);                          // 256 decoded scales * global
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + 1024);            // kStages (<= 32)
  uint64_t *empty = full + 32;
  float *red = reinterpret_cast<float *>(smem + 1024 + 512 + 16);        // [2][kWarps][4] K-part sums
  uint8_t *ring = smem + kHeaderBytes;
  uint4 *xs = reinterpret_cast<uint4 *>(ring + kRingBytes);              // activations, swizzled chunks
  float *xscale = reinterpret_cast<float *>(ring + kRingBytes + K * 2u); // inverse scale of every 32-value slot

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t iters = (K + 1023u) / 1024u;
  const uint32_t tiles_per_block = (K / 16u + 3u) / 4u;
  const uint32_t units = ((N + 127u) / 128u) * kUnitsPerBlock;
  const uint32_t row_bytes = K / 2u;

  if (warp == kWarps) {
    // The producer warp owns the barriers: it initialises them (one stage per lane), signals the
    // consumers through a named barrier it does not wait on, and starts streaming at once.
    if (lane < kStages) { mbar_init(&full[lane], 1); mbar_init(&empty[lane], QUADS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("bar.arrive 2, %0;" ::"n"(kThreads + 32) : "memory");   // does not block: see the consumers' bar.sync 2
  } else {
    const float global = tensor_scale == nullptr ? 1.0f : __ldg(tensor_scale);
    lut[threadIdx.x] = __fmul_rn(q36::decode_e4m3(threadIdx.x), global);
  }

  if (warp == kWarps) {
    // ------------------------------------------------------------------ producer warp
    // Weights and scales do not depend on the kernel that produced x: stream right away.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t g = 0;                                          // running stage number
    if (TMAP) {
      if (lane == 0) {
        for (uint32_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
          const uint32_t rb = unit / kUnitsPerBlock, r0 = (unit % kUnitsPerBlock) * QUADS;
          for (uint32_t it = 0; it < iters; ++it, ++g) {
            const uint32_t stage = g % kStages, phase = (g / kStages) & 1u;
            if (!mbar_wait(&empty[stage], phase ^ 1u)) return;
            uint8_t *dst = ring + stage * kStageBytes;
            mbar_expect_tx(&full[stage], kStageBytes);      // whole boxes; out-of-range columns arrive as zeros
            tma_load_4d(dst, &map_w, it * 128u, r0, 0u, rb, &full[stage]);
            tma_load_3d(dst + kStageW, &map_sf, r0 * 4u, it * 16u, rb, &full[stage]);
          }
        }
      }
      return;
    }
    const uint32_t j = lane >> 3, w = lane & 7u;            // QUADS == 8 here
    for (uint32_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
      const uint32_t rb = unit >> 2, r0 = (unit & 3u) * 8u;
      const uint32_t row = rb * 128u + r0 + w + 32u * j;
      const bool row_ok = row < N;
      const uint32_t rows_ok = __popc(__ballot_sync(0xffffffffu, row_ok));
      const uint8_t *wsrc = weight + static_cast<size_t>(row) * row_bytes;
      const uint8_t *ssrc = sf + static_cast<size_t>(rb) * tiles_per_block * 512u + r0 * 16u;
      for (uint32_t it = 0; it < iters; ++it, ++g) {
        const uint32_t stage = g % kStages, phase = (g / kStages) & 1u;
        if (!mbar_wait(&empty[stage], phase ^ 1u)) return;
        const uint32_t seg = min(kSegBytes, row_bytes - it * kSegBytes);
        const uint32_t tiles = min(16u, tiles_per_block - it * 16u);
        uint8_t *dst = ring + stage * kStageBytes;
        if (lane == 0) mbar_expect_tx(&full[stage], rows_ok * seg + tiles * 128u);
        __syncwarp();
        if (row_ok) bulk_g2s(dst + lane * kSegBytes, wsrc + it * kSegBytes, seg, &full[stage]);
        if (lane < tiles)
          bulk_g2s(dst + kStageW + lane * 128u, ssrc + static_cast<size_t>(it * 16u + lane) * 512u, 128u, &full[stage]);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // Stage x once per CTA as float16.  Every 32-value slot (what one lane consumes per stage) is
  // scaled by its own power of two that brings the slot's max|x| into [2^14, 2^15): every
  // product e2m1 * x is then exact in the mixed-precision FMA, values below the slot maximum
  // times 2^-38 flush (far below the float32 accumulation error), and no pass over the whole
  // vector is needed to find a common scale.  The inverse scale of each slot is kept beside it
  // and folded into the block scale.  This sits between the end of the producing kernel and the
  // first FMA, so it is kept short: every 16-byte L2 read of a pass is issued before the first
  // conversion (one round trip to L2), and warps past the end of x skip the conversion.
  constexpr uint32_t kBatch = 9;                             // 18432 values per pass: one pass for every decode shape
  const uint32_t n_chunks = K / 8u;
  const uint32_t warp_chunk0 = threadIdx.x & ~31u;           // first chunk of this warp inside a batch row
  for (uint32_t base = 0; base < n_chunks; base += kBatch * kThreads) {
    uint4 xr[kBatch];
#pragma unroll
    for (uint32_t i = 0; i < kBatch; ++i) {
      const uint32_t c = base + threadIdx.x + i * kThreads;
      xr[i] = c < n_chunks ? __ldcg(reinterpret_cast<const uint4 *>(x) + c)   // L2 only: x may be fresh
                           : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (uint32_t i = 0; i < kBatch; ++i) {
      if (base + warp_chunk0 + i * kThreads >= n_chunks) break;   // whole warp past the end (n_chunks % 4 == 0)
      const uint32_t c = base + threadIdx.x + i * kThreads;      // four consecutive lanes share a slot
      const uint32_t wv[4] = {xr[i].x, xr[i].y, xr[i].z, xr[i].w};
      uint32_t m2 = max_u16x2(max_u16x2(wv[0] & 0x7fff7fffu, wv[1] & 0x7fff7fffu),
                              max_u16x2(wv[2] & 0x7fff7fffu, wv[3] & 0x7fff7fffu));
      m2 = max_u16x2(m2, __shfl_xor_sync(0xffffffffu, m2, 1));
      m2 = max_u16x2(m2, __shfl_xor_sync(0xffffffffu, m2, 2));
      const uint32_t mx = max(m2 & 0xffffu, m2 >> 16);
      const uint32_t e = (mx >> 7) & 0xffu;
      const int shift = e == 255u ? 0 : (e < 15u ? 126 : 141 - static_cast<int>(e));
      if (c < n_chunks) {
        const float up = __uint_as_float(static_cast<uint32_t>(127 + shift) << 23);
        __half2 h[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
          h[q] = __floats2half2_rn(__uint_as_float(wv[q] << 16) * up, __uint_as_float(wv[q] & 0xffff0000u) * up);
        xs[x_chunk(c >> 2, c & 3u)] = *reinterpret_cast<uint4 *>(h);
        if ((c & 3u) == 0u) xscale[c >> 2] = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
      }
    }
  }
  // Meets the producer's arrival (barriers initialised) and publishes x and the scale table.
  asm volatile("bar.sync 2, %0;" ::"n"(kThreads + 32) : "memory");

  const uint32_t quad = warp % QUADS, kpart = warp / QUADS;
  const uint32_t rot0 = (16u * (lane & 1u) + 30u) & 31u;   // rotation that brings this lane's first scale byte to bits [9:2]
  uint32_t g0 = 0;                               // stage number of the current unit's first stage
  uint32_t flip = 0;
  bool dead = false;

  for (uint32_t unit = blockIdx.x; unit < units; unit += gridDim.x, g0 += iters, flip ^= 1u) {
    const uint32_t row0 = (unit / kUnitsPerBlock) * 128u + (unit % kUnitsPerBlock) * QUADS + quad;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (uint32_t it = kpart; it < iters; it += KPARTS) {
      const uint32_t g = g0 + it;
      const uint32_t stage = g % kStages, phase = (g / kStages) & 1u;
      // A wait that gives up (never seen in practice) only stops the arithmetic: the warp keeps
      // walking its stages and barriers so that nobody else is left waiting for it.
      if (!dead && !mbar_wait(&full[stage], phase)) dead = true;
      const uint8_t *st = ring + stage * kStageBytes;
      const uint32_t slot = lane + it * 32u;
      if (!dead && slot * 32u < K) {
        uint4 wq[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wq[j] = *reinterpret_cast<const uint4 *>(st + (j * QUADS + quad) * kSegBytes + lane * 16u);
        const uint32_t tile = lane >> 1;
        const uint32_t sf_chunk = (TMAP && QUADS == 8) ? (quad ^ (tile & 7u)) : quad;   // 128-byte swizzle of the TMA box
        const uint4 sq = *reinterpret_cast<const uint4 *>(st + kStageW + tile * kSfRow + sf_chunk * 16u);
        const uint32_t sw[4] = {sq.x, sq.y, sq.z, sq.w};
        const float slot_inv = xscale[slot];
#pragma unroll
        for (int half = 0; half < 2; ++half) {          // the two 16-groups of this slot
          // The mixed-precision FMA has a long latency, so every row keeps two accumulators
          // (even / odd column) and the four rows advance together: eight independent chains.
          const uint4 xa = xs[x_chunk(slot, half * 2u)], xb = xs[x_chunk(slot, half * 2u + 1u)];
          const uint32_t xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
          uint32_t h[4][8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t t[4];
            e2m1x8_to_h2(half == 0 ? wq[j].x : wq[j].z, t);
            h[j][0] = t[0]; h[j][1] = t[1]; h[j][2] = t[2]; h[j][3] = t[3];
            e2m1x8_to_h2(half == 0 ? wq[j].y : wq[j].w, t);
            h[j][4] = t[0]; h[j][5] = t[1]; h[j][6] = t[2]; h[j][7] = t[3];
          }
          float ae[4] = {0.f, 0.f, 0.f, 0.f}, ao[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) fma_mixed_eo(ae[j], ao[j], h[j][i], xv[i]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t off = __funnelshift_r(sw[j], sw[j], rot0 + 8u * half) & 0x3fcu;    // 4 * scale byte
            acc[j] = fmaf(ae[j] + ao[j], *reinterpret_cast<const float *>(reinterpret_cast<const uint8_t *>(lut) + off) * slot_inv, acc[j]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
    }
    if (KPARTS == 1) {
      if (lane < 4 && row0 + 32u * lane < N) {
        const float v = lane == 0 ? acc[0] : lane == 1 ? acc[1] : lane == 2 ? acc[2] : acc[3];
        y[row0 + 32u * lane] = __float2bfloat16(v);
      }
    } else {
      // K-parts of a quad meet in shared memory (two buffers alternate between units) and are
      // added in a fixed order.
      float *buf = red + flip * (kWarps * 4u);
      if (lane < 4) buf[warp * 4u + lane] = lane == 0 ? acc[0] : lane == 1 ? acc[1] : lane == 2 ? acc[2] : acc[3];
      asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
      if (kpart == 0 && lane < 4 && row0 + 32u * lane < N) {
        float v = 0.f;
#pragma unroll
        for (uint32_t kp = 0; kp < KPARTS; ++kp) v += buf[(kp * QUADS + quad) * 4u + lane];
        y[row0 + 32u * lane] = __float2bfloat16(v);
      }
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

std::atomic<int> g_force_quads{0};
int sm_count() { return q36::sm_count_current_device(); }

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link against libcuda).
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

bool make_maps(const qwen36_nvfp4_matvec_spec_t *s, uint32_t quads, CUtensorMap *map_w, CUtensorMap *map_sf) {
  EncodeFn enc = encode_fn();
  if (enc == nullptr) return false;
  const uint64_t K = s->in_features, N = s->out_features;
  const uint64_t row_bytes = K / 2, blocks = N / 128, tiles = (K / 16 + 3) / 4;
  const cuuint32_t ones[4] = {1, 1, 1, 1};
  {   // weights as uint32 [blocks][4][32][K/8]
    const cuuint64_t dims[4] = {K / 8, 32, 4, blocks};
    const cuuint64_t strides[3] = {row_bytes, 32 * row_bytes, 128 * row_bytes};
    const cuuint32_t box[4] = {128, quads, 4, 1};
    if (enc(map_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, reinterpret_cast<void *>(s->weight_u8.ptr), dims, strides, box,
            ones, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  {   // scales as uint32 [blocks][tiles][128]
    const cuuint64_t dims[3] = {128, tiles, blocks};
    const cuuint64_t strides[2] = {512, tiles * 512};
    const cuuint32_t box[3] = {quads * 4, 16, 1};
    if (enc(map_sf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, reinterpret_cast<void *>(s->block_scale_e4m3.ptr), dims,
            strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
            quads == 8 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  return true;
}

template <int QUADS, bool TMAP>
int launch_kernel(const qwen36_nvfp4_matvec_spec_t *s, const CUtensorMap &map_w, const CUtensorMap &map_sf) {
  const uint32_t K = static_cast<uint32_t>(s->in_features), N = static_cast<uint32_t>(s->out_features);
  const size_t smem = 1024 + kHeaderBytes + kRingBytes + static_cast<size_t>(K) * 2 + static_cast<size_t>(K) / 8;
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(nvfp4_matvec_kernel<QUADS, TMAP>), 227 * 1024) != cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  const uint32_t units = ((N + 127u) / 128u) * (32u / QUADS);
  const uint32_t cap = static_cast<uint32_t>(sm_count()) * 2u;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(units < cap ? units : cap);
  cfg.blockDim = dim3(kThreads + 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return q36::cuda_status(cudaLaunchKernelEx(
      &cfg, nvfp4_matvec_kernel<QUADS, TMAP>, map_w, map_sf, as_ptr<const __nv_bfloat16>(s->input_bf16),
      as_ptr<const uint8_t>(s->weight_u8), as_ptr<const uint8_t>(s->block_scale_e4m3),
      as_ptr<const float>(s->tensor_scale_f32), as_ptr<__nv_bfloat16>(s->output_bf16), K, N
      ));
}

int launch_fast(const qwen36_nvfp4_matvec_spec_t *s) {
  CUtensorMap map_w{}, map_sf{};
  if (s->out_features % 128 != 0) return launch_kernel<8, false>(s, map_w, map_sf);
  // Unit size (QUADS row quads per unit, 8 / QUADS K-parts).  Coarse units have the least
  // per-unit overhead; finer ones are only worth it when coarse units cannot give every SM two
  // CTAs or leave the last round-robin pass mostly empty.
  const uint32_t blocks = static_cast<uint32_t>(s->out_features / 128);
  const uint32_t iters = static_cast<uint32_t>((s->in_features + 1023) / 1024);
  const uint32_t ctas = 2u * static_cast<uint32_t>(sm_count());
  uint32_t quads = 8;
  const int forced = g_force_quads.load();
  if (forced == 1 || forced == 2 || forced == 4 || forced == 8) {
    quads = static_cast<uint32_t>(forced);
  } else {
    // measured on B200: halve the unit while the coarser one cannot give every SM two CTAs
    // for at least ~1.5 rounds
    while (quads > 2 && 8u / (quads / 2u) <= iters && blocks * (32u / quads) < ctas + ctas / 2u) quads /= 2;
  }
  if (8u / quads > iters) quads = 8;
  if (!make_maps(s, quads, &map_w, &map_sf)) return launch_kernel<8, false>(s, map_w, map_sf);
  switch (quads) {
    case 8: return launch_kernel<8, true>(s, map_w, map_sf);
    case 4: return launch_kernel<4, true>(s, map_w, map_sf);
    case 2: return launch_kernel<2, true>(s, map_w, map_sf);
    default: return launch_kernel<1, true>(s, map_w, map_sf);
  }
}

}  // namespace

// Test hook: a unit size of 1, 2, 4 or 8 row quads sends every 32-column-aligned shape through the
// SIMT pipeline with that unit size; anything else restores the library's own routing.
extern "C" void qwen36_nvfp4_matvec_force_quads(int quads) { g_force_quads.store(quads); }

// 1 when a bounded wait inside the GEMV pipeline ever gave up (a stage never arrived); the
// kernel then returns without finishing its rows.  Reads device memory: synchronises.
extern "C" int qwen36_nvfp4_matvec_last_error(void) {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_matvec_error, sizeof(v)) != cudaSuccess) return -1;
  return static_cast<int>(v);
}

extern "C" int qwen36_nvfp4_matvec(const qwen36_nvfp4_matvec_spec_t *spec) {
  if (spec == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (spec->out_features == 0 || spec->in_features == 0 || spec->input_bf16.ptr == 0 ||
      spec->weight_u8.ptr == 0 || spec->block_scale_e4m3.ptr == 0 || spec->output_bf16.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  const bool fast = spec->in_features % 32 == 0 && spec->in_features <= 32 * 1024 &&
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
  const int forced = g_force_quads.load();
  if (!(forced == 1 || forced == 2 || forced == 4 || forced == 8)) {
    const int rc = q36::nvfp4_gemv_mma_bf16(spec, 1);
    if (rc != QWEN36_STATUS_NOT_IMPLEMENTED) return rc;
  }
  return launch_fast(spec);
}

extern "C" int qwen36_nvfp4_matvec_group(const qwen36_nvfp4_matvec_spec_t *specs, size_t count) {
  if (specs == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (count == 0 || count > 4) return QWEN36_STATUS_INVALID_ARGUMENT;
  for (size_t i = 0; i < count; ++i) {
    const qwen36_nvfp4_matvec_spec_t &s = specs[i];
    if (s.out_features == 0 || s.in_features == 0 || s.input_bf16.ptr == 0 || s.weight_u8.ptr == 0 ||
        s.block_scale_e4m3.ptr == 0 || s.output_bf16.ptr == 0 || s.in_features != specs[0].in_features ||
        s.input_bf16.ptr != specs[0].input_bf16.ptr)
      return QWEN36_STATUS_INVALID_ARGUMENT;
  }
  const int rc = q36::nvfp4_gemv_mma_bf16(specs, count);
  if (rc != QWEN36_STATUS_NOT_IMPLEMENTED) return rc;
  for (size_t i = 0; i < count; ++i) {            // shapes the one-launch kernel declines: one call each
    const int one = qwen36_nvfp4_matvec(&specs[i]);
    if (one != QWEN36_STATUS_SUCCESS) return one;
  }
  return QWEN36_STATUS_SUCCESS;
}

namespace {
bool peer_spec_ok(const qwen36_nvfp4_matvec_peer_spec_t *p) {
  return p->world >= 1 && p->world <= 8 && p->rank < p->world && p->slots >= 1 && p->slots <= 1024 &&
         p->out_slot < p->slots && (p->in_slot == QWEN36_PEER_INPUT_LOCAL || p->in_slot < p->slots) &&
         p->peer_arena.ptr != 0 && p->state.ptr != 0;
}
}  // namespace

extern "C" int qwen36_nvfp4_matvec_peer(const qwen36_nvfp4_matvec_spec_t *specs, size_t count,
                                        const qwen36_nvfp4_matvec_peer_spec_t *peer) {
  if (specs == nullptr || peer == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (count == 0 || count > 4 || !peer_spec_ok(peer)) return QWEN36_STATUS_INVALID_ARGUMENT;
  for (size_t i = 0; i < count; ++i) {
    const qwen36_nvfp4_matvec_spec_t &s = specs[i];
    if (s.out_features == 0 || s.in_features == 0 || s.input_bf16.ptr == 0 || s.weight_u8.ptr == 0 ||
        s.block_scale_e4m3.ptr == 0 || s.in_features != specs[0].in_features ||
        s.input_bf16.ptr != specs[0].input_bf16.ptr || peer->row_offset[i] % 8 != 0 ||
        peer->output_offset_bytes[i] % 16 != 0)
      return QWEN36_STATUS_INVALID_ARGUMENT;
  }
  return q36::nvfp4_gemv_mma_bf16_peer(specs, count, peer);
}

extern "C" int qwen36_nvfp4_matvec_peer_collect(const qwen36_nvfp4_matvec_peer_spec_t *peer, size_t slot,
                                                qwen36_device_ptr_t cells, size_t n, qwen36_device_ptr_t output_bf16) {
  if (peer == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (!peer_spec_ok(peer) || slot >= peer->slots || n == 0 || n % 4 != 0 || cells.ptr == 0 || cells.ptr % 16 != 0 ||
      output_bf16.ptr == 0 || output_bf16.ptr % 8 != 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  return q36::nvfp4_gemv_peer_collect(peer, slot, 0, n, cells, output_bf16);
}
