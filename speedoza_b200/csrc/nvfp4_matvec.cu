// W4A16 NVFP4 GEMV: y[row] = bf16( sum_g (sum_{i<16} x[16g+i] * e2m1(w)) * (ue4m3(sf[g,row]) * global) )
// (semantics of kernels-cuda/ops.cu:547-639 in the reference).
//
// HBM-bound weight streaming.  Persistent CTAs; a producer warp drives the TMA
// engine (descriptor-free cp.async.bulk row segments, mbarrier ring of four
// 18 KB stages per CTA), so the bytes in flight do not depend on occupancy or
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

#include <atomic>
#include <cuda.h>
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

// ---- shared-memory ring fed by the TMA engine --------------------------------------------
//
// Work unit = 32 rows of one 128-row block: rows r0 + w + 32 j for consumer warp w = 0..7 and
// j = 0..3 (r0 in {0, 8, 16, 24}).  One pipeline stage = 1024 columns of a unit:
//   weights  [j][w][512 B]      16 KB : ONE 4-D tiled TMA box over the view
//                                       [N/128][4][32][K/2 bytes] of the weight matrix
//   scales   [16 tiles][128 B]   2 KB : ONE 3-D box (128-byte swizzle, so that the 16 tiles a
//                                       warp reads land on different banks) over the view
//                                       [N/128][tiles][512 B] of the tiled scale buffer
// The producer warp's elected lane issues both copies against the stage's "full" mbarrier; the
// eight consumer warps release a stage through its "empty" mbarrier.  CTAs are persistent:
// unit = blockIdx.x, += gridDim.x, and the stream of stages runs across unit borders.
// When N is not a multiple of 128 the tiled views would reach past the allocation, so that
// (rare) case feeds the same ring with one cp.async.bulk per row segment instead.
constexpr int kStages = 4;
constexpr uint32_t kSegBytes = 512;                         // 1024 columns of one row
constexpr uint32_t kStageW = 32 * kSegBytes;                // 16384
constexpr uint32_t kStageBytes = kStageW + 2048;            // 18432, a multiple of 1024
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

// TMAP: stages are filled by tiled TMA through the two tensor maps (N % 128 == 0); otherwise by
// per-row cp.async.bulk copies (scales then sit unswizzled).
template <int MODE, bool TMAP>
__global__ void __launch_bounds__(kThreads + 32)
nvfp4_matvec_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_sf,
                    const __nv_bfloat16 *__restrict__ x, const uint8_t *__restrict__ weight,
                    const uint8_t *__restrict__ sf, const float *__restrict__ tensor_scale,
                    __nv_bfloat16 *__restrict__ y, uint32_t K, uint32_t N) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  // the swizzled scale boxes need 1024-byte aligned stages
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float *lut = reinterpret_cast<float *>(smem);                          // 256 decoded scales * global
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + 1024);            // kStages
  uint64_t *empty = full + kStages;                                      // kStages
  uint32_t *amax_bits = reinterpret_cast<uint32_t *>(smem + 1024 + 128);
  uint8_t *ring = smem + kHeaderBytes;
  uint4 *xs = reinterpret_cast<uint4 *>(ring + kStages * kStageBytes);   // activations, swizzled chunks

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t iters = (K + 1023u) / 1024u;
  const uint32_t tiles_per_block = (K / 16u + 3u) / 4u;
  const uint32_t units = ((N + 127u) / 128u) * 4u;
  const uint32_t row_bytes = K / 2u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kWarps); }
    *amax_bits = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 256) {
    const float global = tensor_scale == nullptr ? 1.0f : __ldg(tensor_scale);
    lut[threadIdx.x] = __fmul_rn(q36::decode_e4m3(threadIdx.x), global);
  }
  __syncthreads();

  if (warp == kWarps) {
    // ------------------------------------------------------------------ producer warp
    // Weights and scales do not depend on the kernel that produced x: stream right away.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t stage = 0, phase = 0;
    if (TMAP) {
      if (lane == 0) {
        for (uint32_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
          const uint32_t rb = unit >> 2, r0 = (unit & 3u) * 8u;
          for (uint32_t it = 0; it < iters; ++it) {
            if (!mbar_wait(&empty[stage], phase ^ 1u)) return;
            uint8_t *dst = ring + stage * kStageBytes;
            mbar_expect_tx(&full[stage], kStageBytes);      // whole boxes, out-of-range columns arrive as zeros
            tma_load_4d(dst, &map_w, it * 128u, r0, 0u, rb, &full[stage]);
            tma_load_3d(dst + kStageW, &map_sf, r0 * 4u, it * 16u, rb, &full[stage]);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
      }
      return;
    }
    const uint32_t j = lane >> 3, w = lane & 7u;
    for (uint32_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
      const uint32_t rb = unit >> 2, r0 = (unit & 3u) * 8u;
      const uint32_t row = rb * 128u + r0 + w + 32u * j;
      const bool row_ok = row < N;
      const uint32_t rows_ok = __popc(__ballot_sync(0xffffffffu, row_ok));
      const uint8_t *wsrc = weight + static_cast<size_t>(row) * row_bytes;
      const uint8_t *ssrc = sf + static_cast<size_t>(rb) * tiles_per_block * 512u + r0 * 16u;
      for (uint32_t it = 0; it < iters; ++it) {
        if (!mbar_wait(&empty[stage], phase ^ 1u)) return;
        const uint32_t seg = min(kSegBytes, row_bytes - it * kSegBytes);
        const uint32_t tiles = min(16u, tiles_per_block - it * 16u);
        uint8_t *dst = ring + stage * kStageBytes;
        if (lane == 0) mbar_expect_tx(&full[stage], rows_ok * seg + tiles * 128u);
        __syncwarp();
        if (row_ok) bulk_g2s(dst + lane * kSegBytes, wsrc + it * kSegBytes, seg, &full[stage]);
        if (lane < tiles)
          bulk_g2s(dst + kStageW + lane * 128u, ssrc + static_cast<size_t>(it * 16u + lane) * 512u, 128u, &full[stage]);
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // Stage x once per CTA.  Slot = 32 consecutive activations (one lane, one iteration).
  int shift = 0;
  if (MODE == 1) {
    uint32_t m = 0;
    for (uint32_t i = threadIdx.x; i < K / 2u; i += kThreads) {
      const uint32_t v = __ldcg(reinterpret_cast<const uint32_t *>(x) + i);
      m = max(m, max(v & 0x7fffu, (v >> 16) & 0x7fffu));
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if (lane == 0) atomicMax(amax_bits, m);
    asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
    const uint32_t e = (*amax_bits >> 7) & 0xffu;
    shift = e == 255u ? 0 : (e < 15u ? 126 : 141 - static_cast<int>(e));
  }
  {
    const float up = __uint_as_float(static_cast<uint32_t>(127 + shift) << 23);
    const uint32_t slots = K / 32u;
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
  asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");

  const float down = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
  const uint32_t cbase = 2u * (lane & 1u);       // first of this lane's two groups inside its scale tile
  uint32_t stage = 0, phase = 0;

  for (uint32_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
    const uint32_t row0 = (unit >> 2) * 128u + (unit & 3u) * 8u + warp;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (uint32_t it = 0; it < iters; ++it) {
      if (!mbar_wait(&full[stage], phase)) return;
      const uint8_t *st = ring + stage * kStageBytes;
      const uint32_t slot = lane + it * 32u;
      if (slot * 32u < K) {
        uint4 wq[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wq[j] = *reinterpret_cast<const uint4 *>(st + (j * 8u + warp) * kSegBytes + lane * 16u);
        const uint32_t tile = lane >> 1;
        const uint32_t sf_chunk = TMAP ? (warp ^ (tile & 7u)) : warp;      // 128-byte swizzle of the TMA box
        const uint4 sq = *reinterpret_cast<const uint4 *>(st + kStageW + tile * 128u + sf_chunk * 16u);
        const uint32_t sw[4] = {sq.x, sq.y, sq.z, sq.w};
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
              const uint32_t w0 = half == 0 ? wq[j].x : wq[j].z;
              const uint32_t w1 = half == 0 ? wq[j].y : wq[j].w;
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
              const uint32_t w0 = half == 0 ? wq[j].x : wq[j].z;
              const uint32_t w1 = half == 0 ? wq[j].y : wq[j].w;
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
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
      if (++stage == kStages) { stage = 0; phase ^= 1u; }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
    }
    if (lane < 4 && row0 + 32u * lane < N) {
      const float v = lane == 0 ? acc[0] : lane == 1 ? acc[1] : lane == 2 ? acc[2] : acc[3];
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

int g_sms = 0;
int sm_count() {
  if (g_sms == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      return 148;
    g_sms = n;
  }
  return g_sms;
}

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

bool make_maps(const qwen36_nvfp4_matvec_spec_t *s, CUtensorMap *map_w, CUtensorMap *map_sf) {
  EncodeFn enc = encode_fn();
  if (enc == nullptr) return false;
  const uint64_t K = s->in_features, N = s->out_features;
  const uint64_t row_bytes = K / 2, blocks = N / 128, tiles = (K / 16 + 3) / 4;
  const cuuint32_t ones[4] = {1, 1, 1, 1};
  {   // weights as uint32 [blocks][4][32][K/8]
    const cuuint64_t dims[4] = {K / 8, 32, 4, blocks};
    const cuuint64_t strides[3] = {row_bytes, 32 * row_bytes, 128 * row_bytes};
    const cuuint32_t box[4] = {128, 8, 4, 1};
    if (enc(map_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, reinterpret_cast<void *>(s->weight_u8.ptr), dims, strides, box,
            ones, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  {   // scales as uint32 [blocks][tiles][128]
    const cuuint64_t dims[3] = {128, tiles, blocks};
    const cuuint64_t strides[2] = {512, tiles * 512};
    const cuuint32_t box[3] = {32, 16, 1};
    if (enc(map_sf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, reinterpret_cast<void *>(s->block_scale_e4m3.ptr), dims,
            strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  return true;
}

template <int MODE, bool TMAP>
int launch_kernel(const qwen36_nvfp4_matvec_spec_t *s, const CUtensorMap &map_w, const CUtensorMap &map_sf) {
  const uint32_t K = static_cast<uint32_t>(s->in_features), N = static_cast<uint32_t>(s->out_features);
  const size_t smem = 1024 + kHeaderBytes + static_cast<size_t>(kStages) * kStageBytes +
                      static_cast<size_t>(K) * sizeof(typename XT<MODE>::type);
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(nvfp4_matvec_kernel<MODE, TMAP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    227 * 1024);
  });
  if (attr_err != cudaSuccess) return QWEN36_STATUS_CUDA_ERROR;
  const uint32_t units = ((N + 127u) / 128u) * 4u;
  const uint32_t per_sm = smem <= 112 * 1024 ? 2u : 1u;
  const uint32_t cap = static_cast<uint32_t>(sm_count()) * per_sm;
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
      &cfg, nvfp4_matvec_kernel<MODE, TMAP>, map_w, map_sf, as_ptr<const __nv_bfloat16>(s->input_bf16),
      as_ptr<const uint8_t>(s->weight_u8), as_ptr<const uint8_t>(s->block_scale_e4m3),
      as_ptr<const float>(s->tensor_scale_f32), as_ptr<__nv_bfloat16>(s->output_bf16), K, N));
}

template <int MODE>
int launch_mode(const qwen36_nvfp4_matvec_spec_t *s) {
  CUtensorMap map_w{}, map_sf{};
  if (s->out_features % 128 == 0 && make_maps(s, &map_w, &map_sf)) return launch_kernel<MODE, true>(s, map_w, map_sf);
  return launch_kernel<MODE, false>(s, map_w, map_sf);
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
  return g_mode.load() == 0 ? launch_mode<0>(spec) : launch_mode<1>(spec);
}
