// W4A4 NVFP4 product on the 5th-generation tensor cores:
//   c[token][row] = bf16( alpha * sum_k e2m1(a[row,k]) * ue4m3(sfa) * e2m1(b[token,k]) * ue4m3(sfb) )
// tcgen05.mma kind::mxf4nvf4 with 16-element block scales, accumulators in TMEM.
//
// Tile: 128 weight rows (MMA M, TMEM lanes) x BN tokens (MMA N, TMEM columns) x 256 K per
// pipeline stage (four K=64 MMAs).  Per stage the TMA engine brings
//   A  : 128 rows x 128 bytes of packed weights      (2-D tiled TMA, 128-byte swizzle)
//   B  : BN tokens x 128 bytes of packed activations (2-D tiled TMA, 128-byte swizzle)
//   SFA: 2 KB  = four 512-byte scale tiles of the 128-row block   (1-D bulk copy)
//   SFB: 2 KB per 128 tokens                                      (1-D bulk copy)
// The 512-byte scale tile of the caller's layout (32 x 16 bytes: row r at (r%32)*16 + (r/32)*4)
// is exactly the shared-memory image that tcgen05.cp 32x128b.warpx4 turns into the TMEM
// scale operand, so scales go HBM -> smem -> TMEM without being touched by a thread.
//
// Warp roles (384 threads): warp 0 = TMA producer, warp 1 = TMEM allocator + MMA issuer, warp 2 =
// scale copier (tcgen05.cp shared memory -> TMEM), warps 4..11 = epilogue (TMEM -> registers ->
// alpha, bf16 -> global; a 256-token tile is drained by all eight, two per 32-lane quarter, so that
// no warp has to hold more than 64 packed registers: the accumulator is handed back to the MMA warp
// only when the drain is over, so a drain that spills registers stalls the tensor pipe; narrower
// tiles use warps 4..7 only).  CTAs are persistent over
// (row block, token block) tiles; with two accumulator stages the epilogue of one tile overlaps
// the MMAs of the next.  This single-CTA form uses no cluster; the CTA-pair and split-K forms
// further down do.  No multicast loads anywhere: every CTA loads its own tiles.
//
// Every mbarrier wait is bounded; a wait that gives up sets g_gemm_error, and all roles fall
// through to the common exit where TMEM is released.
#include "nvfp4_gemm_tc.cuh"

#include <atomic>
#include <cuda.h>
#include <mutex>
#include <tuple>
#include <vector>

namespace q36 {
namespace {

constexpr uint32_t kThreads = 384;            // 12 warps: 0 TMA, 1 MMA, 2 scale copier, 3 idle, 4..11 epilogue
constexpr uint32_t kWarpCopier = 2;
constexpr uint32_t kWarpEpilogue = 4;         // first epilogue warp; warp w drains TMEM lanes [32 (w % 4), +32)
constexpr uint32_t kBM = 128;
constexpr uint32_t kBKBytes = 128;            // 256 fp4 values
constexpr uint32_t kSpinLimit = 1u << 26;
#ifndef Q36_GEMM_AHEAD
#define Q36_GEMM_AHEAD 0
#endif
constexpr uint32_t kAhead = Q36_GEMM_AHEAD;   // weight stages asked of L2 ahead of the shared-memory ring

__device__ unsigned int g_gemm_error = 0;

// %globaltimer stamps of one CTA's pipeline events, per stage; compiled in only with -DQ36_GEMM_TRACE.
#ifdef Q36_GEMM_TRACE
constexpr uint32_t kTraceStages = 512, kTraceEvents = 8;
__device__ unsigned long long g_gemm_trace[kTraceStages][kTraceEvents];
#define Q36_GTRACE(g_, ev)                                                              \
  do {                                                                                  \
    if (blockIdx.x == 0 && (g_) < kTraceStages) {                                       \
      unsigned long long t_;                                                            \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                            \
      g_gemm_trace[(g_)][ev] = t_;                                                      \
    }                                                                                   \
  } while (0)
#define Q36_GTRACE1(g_, ev)                                                             \
  do {                                                                                  \
    if (blockIdx.x == 1 && (g_) < kTraceStages) {                                       \
      unsigned long long t_;                                                            \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                            \
      g_gemm_trace[(g_)][7 - (ev)] = t_;                                                \
    }                                                                                   \
  } while (0)
#else
#define Q36_GTRACE(g_, ev)
#define Q36_GTRACE1(g_, ev)
#endif
std::atomic<int> g_force_bn{0};
std::atomic<int> g_force_split{0};

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
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  atomicExch(&g_gemm_error, 1u);
  return false;
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint32_t c0, uint32_t c1, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
// L2 prefetch of a tile (no shared memory): the producer asks for the weight tile it will load a
// few stages later, so that the load that fills shared memory hits L2 instead of waiting on HBM.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap *map, uint32_t c0, uint32_t c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor, K-major operand tile with 128-byte swizzle: rows of 128 bytes,
// 8-row groups 1024 bytes apart.  Bits: [0,14) start >> 4, [16,30) leading offset >> 4 (unused
// for swizzled K-major, set to 1), [32,46) stride offset >> 4 = 64, [46,48) version = 1,
// [61,64) layout = 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t desc_sw128(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Descriptor of one 512-byte scale tile for tcgen05.cp: no swizzle, 8 rows x 16 bytes per core
// matrix, core matrices 128 bytes apart.
__device__ __forceinline__ uint64_t desc_sf(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4) | (8ull << 32) | (1ull << 46);
}

__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void mma_mxf4nvf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}

template <uint32_t BN> struct Cfg {
  static constexpr uint32_t kSfbTiles = (BN + 127) / 128;              // 512-byte scale tiles per K=64 for B
  static constexpr uint32_t kBRows = BN < 8 ? 8 : BN;
  static constexpr uint32_t kABytes = kBM * kBKBytes;                  // 16384
  static constexpr uint32_t kBBytes = ((kBRows * kBKBytes + 1023) / 1024) * 1024;
  static constexpr uint32_t kSfaBytes = 2048;
  static constexpr uint32_t kSfbBytes = 2048 * kSfbTiles;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr uint32_t kStages = BN >= 256 ? 4 : (BN >= 128 ? 5 : 6);
  static constexpr uint32_t kAccStages = BN >= 256 ? 1 : 2;
  static constexpr uint32_t kEpiWarps = BN >= 256 ? 8 : 4;             // warps that drain one accumulator
  static constexpr uint32_t kEpiCols = BN >= 256 ? BN / 2 : BN;        // columns per epilogue warp
  static constexpr uint32_t kAccCols = BN < 32 ? 32 : BN;              // columns reserved per accumulator stage
  static constexpr uint32_t kSfCols = 16 + 16 * kSfbTiles;             // per smem stage: SFA 4x4, SFB 4x4 per 128 tokens
  static constexpr uint32_t kTmemUsed = kAccStages * kAccCols + kStages * kSfCols;
  static constexpr uint32_t kTmemCols = kTmemUsed <= 32 ? 32 : kTmemUsed <= 64 ? 64 : kTmemUsed <= 128 ? 128
                                        : kTmemUsed <= 256 ? 256 : 512;
  static_assert(kTmemUsed <= 512, "TMEM budget");
  static constexpr uint32_t kSmemBytes = 1024 /*align slack*/ + 1024 /*barriers*/ + kStages * kStageBytes;
  static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((kBRows >> 3) << 17) | ((kBM >> 4) << 24);
};

// Tiles are numbered with the token block fastest: the CTAs that run at the same time cover a few
// weight row blocks times all token blocks, so every weight tile is fetched from HBM once (its
// other readers hit L2) and the much smaller activation matrix stays L2-resident.
template <uint32_t BN>
__global__ void __launch_bounds__(kThreads, 1)
nvfp4_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const uint8_t *__restrict__ a_sf, const uint8_t *__restrict__ b_sf,
                     __nv_bfloat16 *__restrict__ c, uint32_t m, uint32_t n, uint32_t k, float alpha) {
  using C = Cfg<BN>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);                   // [kStages]
  uint64_t *empty = full + 8;                                            // [kStages]
  uint64_t *sf_full = empty + 8;                                         // [kStages] scales are in TMEM
  uint64_t *sf_landed = sf_full + 8;                                     // [kStages] scale tiles are in shared memory
  uint64_t *acc_full = sf_landed + 8;                                    // [kAccStages]
  uint64_t *acc_empty = acc_full + 2;                                    // [kAccStages]
  uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
  uint8_t *stages = smem + 1024;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t m_blocks = m / kBM, n_blocks = (n + BN - 1) / BN;
  const uint32_t tiles = m_blocks * n_blocks;
  const uint32_t k_blocks = k / 256u;
  const uint32_t sf_tiles_per_block = k / 64u;                           // 512-byte tiles per 128 rows
  const uint32_t sf_tok_blocks = (n + 127u) / 128u;                      // 128-token scale blocks that exist

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < C::kStages; ++s) {
      mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&sf_full[s], 1); mbar_init(&sf_landed[s], 1);
    }
    for (uint32_t s = 0; s < C::kAccStages; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], C::kEpiWarps); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_base_slot;
  const uint32_t tmem_sf = tmem_base + C::kAccStages * C::kAccCols;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t g = 0;
      bool dead = false;
      uint32_t pf_tile = blockIdx.x, pf_kb = 0;
      auto prefetch_one = [&]() {
        if (pf_tile >= tiles) return;
        tma_prefetch_2d(&map_a, pf_kb * kBKBytes, (pf_tile / n_blocks) * kBM);
        if (++pf_kb == k_blocks) { pf_kb = 0; pf_tile += gridDim.x; }
      };
      for (uint32_t i = 0; i < kAhead; ++i) prefetch_one();
      for (uint32_t tile = blockIdx.x; tile < tiles && !dead; tile += gridDim.x) {
        const uint32_t nb = tile % n_blocks, mb = tile / n_blocks;
        for (uint32_t kb = 0; kb < k_blocks; ++kb, ++g) {
          if (kAhead != 0u) prefetch_one();
          const uint32_t s = g % C::kStages, ph = (g / C::kStages) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u)) { dead = true; break; }
          Q36_GTRACE(g, 0);
          uint8_t *st = stages + s * C::kStageBytes;
          // scale tiles of token blocks past the end of the activation tensor do not exist in
          // the caller's buffer: they are skipped (their columns are never stored)
          uint32_t sfb_tiles = 0;
#pragma unroll
          for (uint32_t t = 0; t < C::kSfbTiles; ++t)
            if ((static_cast<size_t>(nb) * BN) / 128u + t < sf_tok_blocks) ++sfb_tiles;
          // The (small) scale tiles go first and on a barrier of their own: the copier warp moves them
          // into TMEM while the operand tiles are still on their way.
          mbar_expect_tx(&sf_landed[s], C::kSfaBytes + sfb_tiles * 2048u);
          bulk_g2s(st + C::kABytes + C::kBBytes, a_sf + (static_cast<size_t>(mb) * sf_tiles_per_block + kb * 4u) * 512u,
                   2048u, &sf_landed[s]);
#pragma unroll
          for (uint32_t t = 0; t < C::kSfbTiles; ++t) {
            const size_t tok_block = (static_cast<size_t>(nb) * BN) / 128u + t;
            if (tok_block < sf_tok_blocks)
              bulk_g2s(st + C::kABytes + C::kBBytes + C::kSfaBytes + t * 2048u,
                       b_sf + (tok_block * sf_tiles_per_block + kb * 4u) * 512u, 2048u, &sf_landed[s]);
          }
          mbar_expect_tx(&full[s], C::kABytes + C::kBRows * kBKBytes);
          tma_load_2d(st, &map_a, kb * kBKBytes, mb * kBM, &full[s]);
          tma_load_2d(st + C::kABytes, &map_b, kb * kBKBytes, nb * BN, &full[s]);
          Q36_GTRACE(g, 1);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t g = 0, t_local = 0;
      bool dead = false;
      for (uint32_t tile = blockIdx.x; tile < tiles && !dead; tile += gridDim.x, ++t_local) {
        const uint32_t as = t_local % C::kAccStages, aph = (t_local / C::kAccStages) & 1u;
        if (!mbar_wait(&acc_empty[as], aph ^ 1u)) { dead = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + as * C::kAccCols;
        for (uint32_t kb = 0; kb < k_blocks; ++kb, ++g) {
          const uint32_t s = g % C::kStages, ph = (g / C::kStages) & 1u;
          const uint32_t st = smem_u32(stages + s * C::kStageBytes);
          const uint32_t sfa_t = tmem_sf + s * C::kSfCols, sfb_t = sfa_t + 16u;
          if (!mbar_wait(&full[s], ph)) { dead = true; break; }
          Q36_GTRACE(g, 4);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (!mbar_wait(&sf_full[s], ph)) { dead = true; break; }     // the copier warp has put this stage's scales in TMEM
          Q36_GTRACE(g, 5);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk)
            mma_mxf4nvf4(d_tmem, desc_sw128(st + kk * 32u), desc_sw128(st + C::kABytes + kk * 32u), C::kIdesc,
                         sfa_t + kk * 4u, sfb_t + kk * C::kSfbTiles * 4u, (kb | kk) != 0u);
          mma_commit(&empty[s]);                 // frees the smem stage once these MMAs have read it
          Q36_GTRACE(g, 6);
        }
        if (!dead) mma_commit(&acc_full[as]);    // accumulator complete
      }
    }
  } else if (warp == kWarpCopier) {
    // ---------------------------------------------------------------- scale copier
    // Moves each stage's scale tiles shared memory -> TMEM from its own instruction stream, so that
    // the copies of stage s+1 can run while the MMAs of stage s execute.
    if (lane == 0) {
      uint32_t g = 0;
      bool dead = false;
      for (uint32_t tile = blockIdx.x; tile < tiles && !dead; tile += gridDim.x) {
        for (uint32_t kb = 0; kb < k_blocks; ++kb, ++g) {
          const uint32_t s = g % C::kStages, ph = (g / C::kStages) & 1u;
          if (!mbar_wait(&sf_landed[s], ph)) { dead = true; break; }
          Q36_GTRACE(g, 2);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t st = smem_u32(stages + s * C::kStageBytes);
          const uint32_t sfa_t = tmem_sf + s * C::kSfCols, sfb_t = sfa_t + 16u;
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk) {
            tmem_cp_sf(sfa_t + kk * 4u, desc_sf(st + C::kABytes + C::kBBytes + kk * 512u));
#pragma unroll
            for (uint32_t t = 0; t < C::kSfbTiles; ++t)
              tmem_cp_sf(sfb_t + (kk * C::kSfbTiles + t) * 4u,
                         desc_sf(st + C::kABytes + C::kBBytes + C::kSfaBytes + t * 2048u + kk * 512u));
          }
          mma_commit(&sf_full[s]);
          Q36_GTRACE(g, 3);
        }
      }
    }
  } else if (warp >= kWarpEpilogue && warp < kWarpEpilogue + C::kEpiWarps) {
    // ---------------------------------------------------------------- epilogue warps
    const uint32_t quarter = warp & 3u;           // TMEM lanes [32*quarter, +32) are this warp's
    const uint32_t col0 = ((warp - kWarpEpilogue) >> 2) * C::kEpiCols;   // first accumulator column of this warp
    uint32_t t_local = 0;
    bool dead = false;
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t_local) {
      const uint32_t nb = tile % n_blocks, mb = tile / n_blocks;
      const uint32_t as = t_local % C::kAccStages, aph = (t_local / C::kAccStages) & 1u;
      if (!dead && !mbar_wait(&acc_full[as], aph)) dead = true;
      if (dead) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t row = mb * kBM + quarter * 32u + lane;           // feature index
      const uint32_t taddr = tmem_base + as * C::kAccCols + col0 + ((quarter * 32u) << 16);
      const uint32_t tok0 = nb * BN + col0;
      if constexpr (BN >= 32) {
        // Drain the accumulator first: every 32-column slice is scaled, rounded to bf16 and kept
        // as packed pairs (tokens 2j, 2j+1 of this lane's feature), the TMEM stage is handed
        // back to the MMA warp, and only then do the (slow) global stores run, overlapped with
        // the next tile's MMAs even when there is a single accumulator stage.
        uint32_t packed[C::kEpiCols / 2];
#pragma unroll
        for (uint32_t c0 = 0; c0 < C::kEpiCols; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (uint32_t j = 0; j < 32; j += 2) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha);
            packed[(c0 + j) / 2] = *reinterpret_cast<const uint32_t *>(&v);
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[as]);
        // Lane pairs swap halves so that the even lane holds features (f, f+1) of token 2j and the
        // odd lane those of token 2j+1: 4-byte stores, 64 contiguous bytes per token per warp.
        const bool odd = (lane & 1u) != 0u;
        __nv_bfloat16 *crow = c + (row & ~1u);
#pragma unroll
        for (uint32_t j = 0; j < C::kEpiCols / 2; ++j) {
          const uint32_t got = __shfl_xor_sync(0xffffffffu, packed[j], 1);
          // even: (mine.lo, got.lo) = token 2j ; odd: (got.hi, mine.hi) = token 2j+1
          const uint32_t v = odd ? __byte_perm(got, packed[j], 0x7632) : __byte_perm(packed[j], got, 0x5410);
          const uint32_t tok = tok0 + 2u * j + (odd ? 1u : 0u);
          if (tok < n) *reinterpret_cast<uint32_t *>(crow + static_cast<size_t>(tok) * m) = v;
        }
        continue;
      } else {
        uint32_t r[8];
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < C::kBRows; c0 += 8) {
          tmem_ld8(taddr + c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j) {
            const uint32_t tok = tok0 + c0 + j;
            if (tok < n) c[static_cast<size_t>(tok) * m + row] = __float2bfloat16(__uint_as_float(r[j]) * alpha);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[as]);
    }
  }

  // Common exit: everyone meets, then the allocating warp releases TMEM.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::kTmemCols) : "memory");
  }
}

// ============================================================================================
// CTA-pair form (tcgen05 cta_group::2) for large token counts: two CTAs of a cluster share one
// 256-row x 256-token tile.  Each CTA stages its own 128 weight rows and only HALF of the
// activation tile (128 tokens); the pair's MMAs read both halves, so the L2 -> shared-memory
// traffic per CTA drops from 54 KB to 38 KB per 256 K, and five stages fit instead of four.
// The even CTA of the pair ("leader") owns the full / scale / accumulator-free barriers and
// issues every tcgen05.cp and tcgen05.mma for both CTAs; tcgen05.commit fans the "stage free"
// and "accumulator ready" signals out to both.  Both CTAs run a TMA producer (signalling the
// leader's barrier) and four epilogue warps (each CTA drains its own 128 TMEM lanes).
// ============================================================================================
namespace pair {
constexpr uint32_t kBN = 256;                                   // tokens per pair tile
constexpr uint32_t kHalfTok = 128;                              // tokens staged per CTA
constexpr uint32_t kABytes = kBM * kBKBytes;                    // 16384
constexpr uint32_t kBBytes = kHalfTok * kBKBytes;               // 16384
constexpr uint32_t kSfaBytes = 2048;
constexpr uint32_t kSfbBytes = 4096;                            // both 128-token scale blocks
constexpr uint32_t kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;   // 38912
constexpr uint32_t kStages = 5;
constexpr uint32_t kSfCols = 16 + 32;
constexpr uint32_t kTmemCols = 512;                             // 256 accumulator + 5 x 48 scale columns
constexpr uint32_t kSmemBytes = 1024 + 1024 + kStages * kStageBytes;
constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((256u >> 4) << 24);
static_assert(256 + kStages * kSfCols <= kTmemCols, "TMEM budget");
}  // namespace pair

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t v;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(v));
  return v;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(v) : "r"(smem_addr), "r"(rank));
  return v;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Tiled TMA load whose completion is counted on a barrier that may live in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, uint32_t c0, uint32_t c1, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void mma_mxf4nvf4_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                  uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// Arrives (once the pair's earlier tcgen05 operations have completed) on the barrier at the same
// shared-memory offset in every CTA of `cta_mask`.
__device__ __forceinline__ void mma_commit_pair_fanout(uint64_t *bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(cta_mask) : "memory");
}
__device__ __forceinline__ void mma_commit_pair(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
nvfp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                       __nv_bfloat16 *__restrict__ c, uint32_t m, uint32_t n, uint32_t k, float alpha) {
  namespace P = pair;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);                   // [kStages]   used in the leader
  uint64_t *empty = full + 8;                                            // [kStages]   one per CTA
  uint64_t *sf_full = empty + 8;                                         // [kStages]   used in the leader
  uint64_t *sf_landed = sf_full + 8;                                     // [kStages]   used in the leader
  uint64_t *acc_full = sf_landed + 8;                                    // one per CTA
  uint64_t *acc_empty = acc_full + 2;                                    // used in the leader: 8 epilogue warps
  uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
  uint8_t *stages = smem + 1024;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t rank = cluster_rank() & 1u;
  const bool leader = rank == 0u;
  const uint32_t pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const uint32_t m_blocks = m / 256u, n_blocks = (n + P::kBN - 1) / P::kBN;
  const uint32_t tiles = m_blocks * n_blocks;
  const uint32_t k_blocks = k / 256u;
  const uint32_t sf_tiles_per_block = k / 64u;                           // 512-byte tiles per 128 rows

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < P::kStages; ++s) {
      mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&sf_full[s], 1); mbar_init(&sf_landed[s], 1);
    }
    mbar_init(&acc_full[0], 1);
    mbar_init(&acc_empty[0], 16);           // eight epilogue warps in each CTA of the pair
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(P::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                       // both CTAs' barriers exist before anything crosses over
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_base_slot;
  const uint32_t tmem_sf = tmem_base + 256u;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t g = 0;
      for (uint32_t tile = pair_id; tile < tiles; tile += n_pairs) {
        const uint32_t nb = tile % n_blocks, mb = tile / n_blocks;
        const uint32_t row_block = mb * 2u + rank;                       // this CTA's 128 weight rows
        bool dead = false;
        for (uint32_t kb = 0; kb < k_blocks; ++kb, ++g) {
          const uint32_t s = g % P::kStages, ph = (g / P::kStages) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u)) { dead = true; break; }
          if (leader) Q36_GTRACE(g, 0); else Q36_GTRACE1(g, 0);
          uint8_t *st = stages + s * P::kStageBytes;
          // the leader's barriers count both CTAs' bytes; the (small) scale tiles go first and on a barrier
          // of their own, so that the copier warp moves them into TMEM while the operand tiles still travel
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0u), bar_sf = map_to_cta(smem_u32(&sf_landed[s]), 0u);
          if (leader) {
            mbar_expect_tx(&sf_landed[s], 2u * (P::kSfaBytes + P::kSfbBytes));
            mbar_expect_tx(&full[s], 2u * (P::kABytes + P::kBBytes));
          }
          tma_load_2d_pair(st + P::kABytes + P::kBBytes, &map_sfa, 0u, row_block * sf_tiles_per_block + kb * 4u, bar_sf);
          // token blocks past the end of the activation tensor lie outside the map and arrive as zeros
#pragma unroll
          for (uint32_t t = 0; t < 2; ++t)
            tma_load_2d_pair(st + P::kABytes + P::kBBytes + P::kSfaBytes + t * 2048u, &map_sfb, 0u,
                             (nb * 2u + t) * sf_tiles_per_block + kb * 4u, bar_sf);
          tma_load_2d_pair(st, &map_a, kb * kBKBytes, row_block * kBM, bar);
          tma_load_2d_pair(st + P::kABytes, &map_b, kb * kBKBytes, nb * P::kBN + rank * P::kHalfTok, bar);
          if (leader) Q36_GTRACE(g, 1); else Q36_GTRACE1(g, 1);
        }
        if (dead) break;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader only)
    if (leader && lane == 0) {
      uint32_t g = 0, t_local = 0;
      bool dead = false;
      for (uint32_t tile = pair_id; tile < tiles && !dead; tile += n_pairs, ++t_local) {
        if (!mbar_wait(&acc_empty[0], (t_local & 1u) ^ 1u)) { dead = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (uint32_t kb = 0; kb < k_blocks; ++kb, ++g) {
          const uint32_t s = g % P::kStages, ph = (g / P::kStages) & 1u;
          if (!mbar_wait(&full[s], ph)) { dead = true; break; }
          Q36_GTRACE(g, 4);
          if (!mbar_wait(&sf_full[s], ph)) { dead = true; break; }     // scales of this stage are in both TMEMs
          Q36_GTRACE(g, 5);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t st = smem_u32(stages + s * P::kStageBytes);
          const uint32_t sfa_t = tmem_sf + s * P::kSfCols, sfb_t = sfa_t + 16u;
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk)
            mma_mxf4nvf4_pair(tmem_base, desc_sw128(st + kk * 32u), desc_sw128(st + P::kABytes + kk * 32u), P::kIdesc,
                              sfa_t + kk * 4u, sfb_t + kk * 8u, (kb | kk) != 0u);
          mma_commit_pair_fanout(&empty[s], 3);  // frees the stage in both CTAs once these MMAs have read it
          Q36_GTRACE(g, 6);
        }
        if (!dead) mma_commit_pair_fanout(&acc_full[0], 3);   // accumulator complete, in both CTAs
      }
    }
  } else if (warp == kWarpCopier) {
    // ---------------------------------------------------------------- scale copier (leader only)
    if (leader && lane == 0) {
      uint32_t g = 0;
      bool dead = false;
      for (uint32_t tile = pair_id; tile < tiles && !dead; tile += n_pairs) {
        for (uint32_t kb = 0; kb < k_blocks; ++kb, ++g) {
          const uint32_t s = g % P::kStages, ph = (g / P::kStages) & 1u;
          if (!mbar_wait(&sf_landed[s], ph)) { dead = true; break; }
          Q36_GTRACE(g, 2);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t st = smem_u32(stages + s * P::kStageBytes);
          const uint32_t sfa_t = tmem_sf + s * P::kSfCols, sfb_t = sfa_t + 16u;
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk) {
            tmem_cp_sf_pair(sfa_t + kk * 4u, desc_sf(st + P::kABytes + P::kBBytes + kk * 512u));
#pragma unroll
            for (uint32_t t = 0; t < 2; ++t)
              tmem_cp_sf_pair(sfb_t + (kk * 2u + t) * 4u,
                              desc_sf(st + P::kABytes + P::kBBytes + P::kSfaBytes + t * 2048u + kk * 512u));
          }
          mma_commit_pair(&sf_full[s]);
          Q36_GTRACE(g, 3);
        }
      }
    }
  } else if (warp >= kWarpEpilogue) {
    // ---------------------------------------------------------------- epilogue warps 4..11 (both CTAs)
    const uint32_t quarter = warp & 3u;           // TMEM lanes [32*quarter, +32) are this warp's
    const uint32_t col0 = ((warp - kWarpEpilogue) >> 2) * (P::kBN / 2u);   // this warp's half of the columns
    const uint32_t acc_empty_leader = map_to_cta(smem_u32(&acc_empty[0]), 0u);
    uint32_t t_local = 0;
    for (uint32_t tile = pair_id; tile < tiles; tile += n_pairs, ++t_local) {
      const uint32_t nb = tile % n_blocks, mb = tile / n_blocks;
      if (!mbar_wait(&acc_full[0], t_local & 1u)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t row = (mb * 2u + rank) * kBM + quarter * 32u + lane;     // feature index
      const uint32_t taddr = tmem_base + col0 + ((quarter * 32u) << 16);
      const uint32_t tok0 = nb * P::kBN + col0;
      uint32_t packed[P::kBN / 4];
#pragma unroll
      for (uint32_t c0 = 0; c0 < P::kBN / 2u; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (uint32_t j = 0; j < 32; j += 2) {
          const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha);
          packed[(c0 + j) / 2] = *reinterpret_cast<const uint32_t *>(&v);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
      const bool odd = (lane & 1u) != 0u;
      __nv_bfloat16 *crow = c + (row & ~1u);
#pragma unroll
      for (uint32_t j = 0; j < P::kBN / 4; ++j) {
        const uint32_t got = __shfl_xor_sync(0xffffffffu, packed[j], 1);
        const uint32_t v = odd ? __byte_perm(got, packed[j], 0x7632) : __byte_perm(packed[j], got, 0x5410);
        const uint32_t tok = tok0 + 2u * j + (odd ? 1u : 0u);
        if (tok < n) *reinterpret_cast<uint32_t *>(crow + static_cast<size_t>(tok) * m) = v;
      }
    }
  }

  // Common exit: the pair meets (nobody may still read the other's shared or tensor memory),
  // then both allocating warps release TMEM.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P::kTmemCols) : "memory");
  }
}

// ============================================================================================
// CTA-pair form with the scale tiles on a pipeline of their own.  The pair form above keeps five
// 38 KB stages (operands + scale tiles) in flight, which a 2.7-3 us load round trip turns into a
// stage every 0.56 us although the SM could take one in every 0.43 us.  Here the operand ring holds
// six 32 KB stages, and the scale tiles (6 KB per stage) travel separately: a second producer
// thread loads them into a five-slot shared-memory ring, the copier moves a slot into one of five
// TMEM buffers as soon as that buffer's previous user has been multiplied, and frees the slot at
// once.  So the scales run up to ten stages ahead of the MMAs without holding operand space,
// and while an accumulator drains the operand ring fills up, which lets the MMA warp make up part
// of the bubble at its own rate afterwards.
// ============================================================================================
namespace pair6 {
constexpr uint32_t kBN = 256, kHalfTok = 128;
constexpr uint32_t kABytes = kBM * kBKBytes, kBBytes = kHalfTok * kBKBytes;   // 16384 each
constexpr uint32_t kAbStage = kABytes + kBBytes;                              // 32768
constexpr uint32_t kAbStages = 6;
constexpr uint32_t kSfaBytes = 2048, kSfbBytes = 4096, kSfSlot = kSfaBytes + kSfbBytes;
constexpr uint32_t kSfSlots = 5, kSfBufs = 5, kSfCols = 16 + 32;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSmemBytes = 1024 + 1024 + kAbStages * kAbStage + kSfSlots * kSfSlot;
constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((256u >> 4) << 24);
static_assert(256 + kSfBufs * kSfCols <= kTmemCols, "TMEM budget");
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
// Stream-K form: a (tile, K-block) pair is a unit and every CTA pair takes an equal, contiguous run
// of units, so a launch whose tiles do not fill the last round (40 tiles on 74 pairs) still keeps
// every pair busy to the end.  A pair's run may begin and end inside a tile.  The pair that holds a
// tile's FIRST K-blocks owns its output; pairs that hold later K-blocks of it (always the first
// thing they do) leave their float32 accumulator in a slot of the caller's workspace, epilogue
// thread by epilogue thread, and raise a per-warp flag that carries the launch's tag; the owner
// (for which that tile is the last thing it does) adds the slots in K order.  Bits differ from the
// one-pass sum only by that regrouping of float32 additions; they do not depend on timing.
constexpr uint32_t kSlotFloats = 2u * 8u * 128u * 32u;           // pair x epilogue warps x columns x lanes = 256 KB
constexpr uint32_t kFlagsPerPair = 16u;
}  // namespace pair6

// The segments (tile, K-blocks [kb0, kb1)) of one CTA pair, in the order every role walks them.
template <bool SK>
struct PairWalk {
  uint32_t a, b, step, k_blocks;       // tiles form: next tile, tile count, stride.  Stream-K: next unit, end unit
  __device__ __forceinline__ PairWalk(uint32_t pair_id, uint32_t n_pairs, uint32_t tiles, uint32_t kb) : k_blocks(kb) {
    if (SK) {
      const uint64_t total = static_cast<uint64_t>(tiles) * kb;
      a = static_cast<uint32_t>(total * pair_id / n_pairs);
      b = static_cast<uint32_t>(total * (pair_id + 1u) / n_pairs);
      step = 0u;
    } else {
      a = pair_id; b = tiles; step = n_pairs;
    }
  }
  __device__ __forceinline__ bool next(uint32_t &tile, uint32_t &kb0, uint32_t &kb1) {
    if (a >= b) return false;
    if (SK) {
      tile = a / k_blocks;
      kb0 = a - tile * k_blocks;
      kb1 = min(k_blocks, kb0 + (b - a));
      a += kb1 - kb0;
    } else {
      tile = a; kb0 = 0u; kb1 = k_blocks; a += step;
    }
    return true;
  }
};


template <bool SK>
__global__ void __launch_bounds__(kThreads, 1)
nvfp4_gemm_pair6_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                        __nv_bfloat16 *__restrict__ c, uint32_t m, uint32_t n, uint32_t k, float alpha,
                        float *__restrict__ ws, uint32_t tag) {
  namespace P = pair6;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t *ab_full = reinterpret_cast<uint64_t *>(smem);                // [6]  used in the leader
  uint64_t *ab_empty = ab_full + 8;                                      // [6]  one per CTA
  uint64_t *sfs_full = ab_empty + 8;                                     // [5]  used in the leader
  uint64_t *sfs_empty = sfs_full + 8;                                    // [5]  one per CTA
  uint64_t *sft_ready = sfs_empty + 8;                                   // [5]  used in the leader
  uint64_t *sft_free = sft_ready + 8;                                    // [5]  used in the leader
  uint64_t *acc_full = sft_free + 8;                                     // one per CTA
  uint64_t *acc_empty = acc_full + 2;                                    // used in the leader: 8 epilogue warps x 2 CTAs
  uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
  uint8_t *ab = smem + 1024;
  uint8_t *sfs = ab + P::kAbStages * P::kAbStage;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  // the four descriptors start their way into the TMA unit's cache while the barriers are set up
  // (measured: the first MMA 0.35 us earlier)
  if (threadIdx.x == 64) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_sfa) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_sfb) : "memory");
  }
  const uint32_t rank = cluster_rank() & 1u;
  const bool leader = rank == 0u;
  const uint32_t pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const uint32_t m_blocks = m / 256u, n_blocks = (n + P::kBN - 1) / P::kBN;
  const uint32_t tiles = m_blocks * n_blocks;
  const uint32_t k_blocks = k / 256u;
  const uint32_t sf_tiles_per_block = k / 64u;                           // 512-byte tiles per 128 rows

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < P::kAbStages; ++s) { mbar_init(&ab_full[s], 1); mbar_init(&ab_empty[s], 1); }
    for (uint32_t s = 0; s < P::kSfSlots; ++s) { mbar_init(&sfs_full[s], 1); mbar_init(&sfs_empty[s], 1); }
    for (uint32_t s = 0; s < P::kSfBufs; ++s) { mbar_init(&sft_ready[s], 1); mbar_init(&sft_free[s], 1); }
    mbar_init(&acc_full[0], 1);
    mbar_init(&acc_empty[0], 16);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(P::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                       // both CTAs' barriers exist before anything crosses over
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_base_slot;
  const uint32_t tmem_sf = tmem_base + 256u;

  if (warp == 0) {
    // ---------------------------------------------------------------- operand producer (both CTAs)
    if (lane == 0) {
      uint32_t g = 0;
      bool dead = false;
      PairWalk<SK> walk(pair_id, n_pairs, tiles, k_blocks);
      uint32_t tile, kb0, kb1;
      while (!dead && walk.next(tile, kb0, kb1)) {
        const uint32_t nb = tile % n_blocks, mb = tile / n_blocks;
        const uint32_t row_block = mb * 2u + rank;                       // this CTA's 128 weight rows
        for (uint32_t kb = kb0; kb < kb1; ++kb, ++g) {
          const uint32_t s = g % P::kAbStages, ph = (g / P::kAbStages) & 1u;
          if (!mbar_wait(&ab_empty[s], ph ^ 1u)) { dead = true; break; }
          if (leader) Q36_GTRACE(g, 0);
          uint8_t *st = ab + s * P::kAbStage;
          const uint32_t bar = map_to_cta(smem_u32(&ab_full[s]), 0u);    // the leader's barrier counts both CTAs' bytes
          if (leader) mbar_expect_tx(&ab_full[s], 2u * P::kAbStage);
          tma_load_2d_pair(st, &map_a, kb * kBKBytes, row_block * kBM, bar);
          // token blocks past the end of the activation tensor lie outside the map and arrive as zeros
          tma_load_2d_pair(st + P::kABytes, &map_b, kb * kBKBytes, nb * P::kBN + rank * P::kHalfTok, bar);
          if (leader) Q36_GTRACE(g, 1);
        }
      }
    } else if (lane == 1) {
      // -------------------------------------------------------------- scale-tile producer (both CTAs): the other
      // side of the same branch, so that the two lanes run their loops side by side
      uint32_t g = 0;
      bool dead = false;
      PairWalk<SK> walk(pair_id, n_pairs, tiles, k_blocks);
      uint32_t tile, kb0, kb1;
      while (!dead && walk.next(tile, kb0, kb1)) {
        const uint32_t nb = tile % n_blocks, mb = tile / n_blocks;
        const uint32_t row_block = mb * 2u + rank;
        for (uint32_t kb = kb0; kb < kb1; ++kb, ++g) {
          const uint32_t s = g % P::kSfSlots, ph = (g / P::kSfSlots) & 1u;
          if (!mbar_wait(&sfs_empty[s], ph ^ 1u)) { dead = true; break; }
          uint8_t *st = sfs + s * P::kSfSlot;
          const uint32_t bar = map_to_cta(smem_u32(&sfs_full[s]), 0u);
          if (leader) mbar_expect_tx(&sfs_full[s], 2u * P::kSfSlot);
          tma_load_2d_pair(st, &map_sfa, 0u, row_block * sf_tiles_per_block + kb * 4u, bar);
#pragma unroll
          for (uint32_t t = 0; t < 2; ++t)
            tma_load_2d_pair(st + P::kSfaBytes + t * 2048u, &map_sfb, 0u, (nb * 2u + t) * sf_tiles_per_block + kb * 4u, bar);
        }
      }
    }
  } else if (warp == kWarpCopier || warp == 3u) {
    // ---------------------------------------------------------------- scale copiers (leader only)
    // Twelve tcgen05.cp per stage take one thread longer to issue than a stage may last, so two
    // threads (warps 2 and 3) take alternate stages.
    if (leader && lane == 0) {
      const uint32_t mine = warp == 3u ? 1u : 0u;
      uint32_t g = 0;
      bool dead = false;
      PairWalk<SK> walk(pair_id, n_pairs, tiles, k_blocks);
      uint32_t tile, kb0, kb1;
      while (!dead && walk.next(tile, kb0, kb1)) {
        for (uint32_t kb = kb0; kb < kb1; ++kb, ++g) {
          if ((g & 1u) != mine) continue;
          const uint32_t s = g % P::kSfSlots, phs = (g / P::kSfSlots) & 1u;
          const uint32_t b = g % P::kSfBufs, phb = (g / P::kSfBufs) & 1u;
          if (!mbar_wait(&sfs_full[s], phs)) { dead = true; break; }
          Q36_GTRACE(g, 2);
          // The TMEM buffer is free once the MMAs of stage g - 5 are done, which is what frees that
          // stage's operand slot too: the copier watches the same barrier as the operand producer
          // (the MMA thread issues one commit per stage, not two: it is the issue-bound one).  The
          // barrier cannot be more than that one phase ahead, since the MMAs of stage g + 1 need this copy.
          if (g >= P::kSfBufs) {
            const uint32_t gp = g - P::kSfBufs;
            if (!mbar_wait(&ab_empty[gp % P::kAbStages], (gp / P::kAbStages) & 1u)) { dead = true; break; }
          }
          (void)phb;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t st = smem_u32(sfs + s * P::kSfSlot);
          const uint32_t sfa_t = tmem_sf + b * P::kSfCols, sfb_t = sfa_t + 16u;
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk) {
            tmem_cp_sf_pair(sfa_t + kk * 4u, desc_sf(st + kk * 512u));
#pragma unroll
            for (uint32_t t = 0; t < 2; ++t)
              tmem_cp_sf_pair(sfb_t + (kk * 2u + t) * 4u, desc_sf(st + P::kSfaBytes + t * 2048u + kk * 512u));
          }
          mma_commit_pair(&sft_ready[b]);                    // scales of this stage are in both TMEMs
          mma_commit_pair_fanout(&sfs_empty[s], 3);          // and the slot is free again in both CTAs
          Q36_GTRACE(g, 3);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader only)
    if (leader && lane == 0) {
      uint32_t g = 0, t_local = 0;
      bool dead = false;
      PairWalk<SK> walk(pair_id, n_pairs, tiles, k_blocks);
      uint32_t tile, kb0, kb1;
      for (; !dead && walk.next(tile, kb0, kb1); ++t_local) {
        if (!mbar_wait(&acc_empty[0], (t_local & 1u) ^ 1u)) { dead = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (uint32_t kb = kb0; kb < kb1; ++kb, ++g) {
          const uint32_t s = g % P::kAbStages, ph = (g / P::kAbStages) & 1u;
          const uint32_t b = g % P::kSfBufs, phb = (g / P::kSfBufs) & 1u;
          if (!mbar_wait(&ab_full[s], ph)) { dead = true; break; }
          Q36_GTRACE(g, 4);
          if (!mbar_wait(&sft_ready[b], phb)) { dead = true; break; }
          Q36_GTRACE(g, 5);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t st = smem_u32(ab + s * P::kAbStage);
          const uint32_t sfa_t = tmem_sf + b * P::kSfCols, sfb_t = sfa_t + 16u;
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk)
            mma_mxf4nvf4_pair(tmem_base, desc_sw128(st + kk * 32u), desc_sw128(st + P::kABytes + kk * 32u), P::kIdesc,
                              sfa_t + kk * 4u, sfb_t + kk * 8u, kb != kb0 || kk != 0u);
          mma_commit_pair_fanout(&ab_empty[s], 3);           // frees the operand stage in both CTAs (and, for the copier, the scale buffer)
          Q36_GTRACE(g, 6);
        }
        if (!dead) mma_commit_pair_fanout(&acc_full[0], 3);  // accumulator complete, in both CTAs
      }
    }
  } else if (warp >= kWarpEpilogue) {
    // ---------------------------------------------------------------- epilogue warps 4..11 (both CTAs)
    const uint32_t quarter = warp & 3u;           // TMEM lanes [32*quarter, +32) are this warp's
    const uint32_t col0 = ((warp - kWarpEpilogue) >> 2) * (P::kBN / 2u);   // this warp's half of the columns
    const uint32_t acc_empty_leader = map_to_cta(smem_u32(&acc_empty[0]), 0u);
    uint32_t t_local = 0;
    PairWalk<SK> walk(pair_id, n_pairs, tiles, k_blocks);
    uint32_t tile, kb0, kb1;
    for (; walk.next(tile, kb0, kb1); ++t_local) {
      const uint32_t nb = tile % n_blocks, mb = tile / n_blocks;
      if (!mbar_wait(&acc_full[0], t_local & 1u)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t row = (mb * 2u + rank) * kBM + quarter * 32u + lane;     // feature index
      const uint32_t taddr = tmem_base + col0 + ((quarter * 32u) << 16);
      const uint32_t tok0 = nb * P::kBN + col0;
      if (SK && kb0 == 0u && kb1 != k_blocks) {
        // Owner of a tile that other pairs finish (always the last piece of this pair's run, so the
        // accumulator can stay in tensor memory meanwhile): 32 columns at a time, the partial sums of
        // kFly contributors in flight together, added in K order.
        constexpr uint32_t kFly = 3;
        const uint32_t ew = warp - kWarpEpilogue;
        const size_t mine = ((static_cast<size_t>(rank) * 8u + ew) * 32u) * 32u + lane;
        uint32_t *flags = reinterpret_cast<uint32_t *>(ws + static_cast<size_t>(n_pairs) * P::kSlotFloats);
        const uint64_t total = static_cast<uint64_t>(tiles) * k_blocks;
        const uint64_t tile_end = static_cast<uint64_t>(tile + 1u) * k_blocks;
        uint32_t q_end = pair_id + 1u;                          // contributors: pairs [pair_id + 1, q_end)
        while (q_end < n_pairs && total * q_end / n_pairs < tile_end) ++q_end;
        for (uint32_t q = pair_id + 1u; q < q_end; ++q) {
          const volatile uint32_t *flag = flags + q * P::kFlagsPerPair + rank * 8u + ew;
          bool there = false;
          for (uint32_t spin = 0; spin < (1u << 22); ++spin) {        // x 64 ns: a quarter of a second
            if (*flag == tag) { there = true; break; }
            __nanosleep(64);
          }
          if (!there) atomicExch(&g_gemm_error, 1u);
        }
        __threadfence();
        const bool odd = (lane & 1u) != 0u;
        __nv_bfloat16 *crow = c + (row & ~1u);
#pragma unroll 1
        for (uint32_t chunk = 0; chunk < 4; ++chunk) {
          uint32_t r[32];
          tmem_ld32(taddr + chunk * 32u, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          for (uint32_t q0 = pair_id + 1u; q0 < q_end; q0 += kFly) {
            float4 v[kFly][8];
#pragma unroll
            for (uint32_t f = 0; f < kFly; ++f) {
              const uint32_t q = q0 + f < q_end ? q0 + f : q0;    // a repeat of the first one where the group is short (not added)
              const float4 *slot = reinterpret_cast<const float4 *>(ws + static_cast<size_t>(q) * P::kSlotFloats) + mine;
#pragma unroll
              for (uint32_t g4 = 0; g4 < 8; ++g4) v[f][g4] = __ldcg(slot + (chunk * 8u + g4) * 32u);
            }
#pragma unroll
            for (uint32_t f = 0; f < kFly; ++f) {
              if (q0 + f < q_end) {
#pragma unroll
                for (uint32_t g4 = 0; g4 < 8; ++g4) {
                  r[4 * g4] = __float_as_uint(__uint_as_float(r[4 * g4]) + v[f][g4].x);
                  r[4 * g4 + 1] = __float_as_uint(__uint_as_float(r[4 * g4 + 1]) + v[f][g4].y);
                  r[4 * g4 + 2] = __float_as_uint(__uint_as_float(r[4 * g4 + 2]) + v[f][g4].z);
                  r[4 * g4 + 3] = __float_as_uint(__uint_as_float(r[4 * g4 + 3]) + v[f][g4].w);
                }
              }
            }
          }
#pragma unroll
          for (uint32_t j = 0; j < 32; j += 2) {
            const __nv_bfloat162 pv = __floats2bfloat162_rn(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha);
            const uint32_t mine_bits = *reinterpret_cast<const uint32_t *>(&pv);
            const uint32_t got = __shfl_xor_sync(0xffffffffu, mine_bits, 1);
            const uint32_t out = odd ? __byte_perm(got, mine_bits, 0x7632) : __byte_perm(mine_bits, got, 0x5410);
            const uint32_t tok = tok0 + chunk * 32u + j + (odd ? 1u : 0u);
            if (tok < n) *reinterpret_cast<uint32_t *>(crow + static_cast<size_t>(tok) * m) = out;
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_cluster(acc_empty_leader);
          // This warp is the flags' only reader: clear them, so that a replay of a captured launch (same
          // tag) does not find the flags of the replay before it.
          for (uint32_t q = pair_id + 1u; q < q_end; ++q)
            *reinterpret_cast<volatile uint32_t *>(flags + q * P::kFlagsPerPair + rank * 8u + ew) = 0u;
        }
        continue;
      }
      // All four loads of the warp's 128 columns go out before the one wait, and the accumulator is
      // handed back before anything is converted: the time the MMA warp stands still per tile is the
      // commit, one TMEM read and this arrival, nothing else.
      uint32_t r0[32], r1[32], r2[32], r3[32];
      tmem_ld32(taddr, r0);
      tmem_ld32(taddr + 32u, r1);
      tmem_ld32(taddr + 64u, r2);
      tmem_ld32(taddr + 96u, r3);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
      if (SK && kb0 != 0u) {
        // A partial tile whose first K-blocks belong to another pair: this thread's 128 sums, as 32 groups
        // of four columns, [pair][CTA][epilogue warp][group][lane] float4, so that a warp moves 512 contiguous
        // bytes per access; the owner of the tile adds them and writes the output.
        const uint32_t ew = warp - kWarpEpilogue;
        const size_t mine = ((static_cast<size_t>(rank) * 8u + ew) * 32u) * 32u + lane;
        uint32_t *flags = reinterpret_cast<uint32_t *>(ws + static_cast<size_t>(n_pairs) * P::kSlotFloats);
        float4 *slot = reinterpret_cast<float4 *>(ws + static_cast<size_t>(pair_id) * P::kSlotFloats) + mine;
#pragma unroll
        for (uint32_t g4 = 0; g4 < 8; ++g4) {
          slot[g4 * 32u] = make_float4(__uint_as_float(r0[4 * g4]), __uint_as_float(r0[4 * g4 + 1]),
                                       __uint_as_float(r0[4 * g4 + 2]), __uint_as_float(r0[4 * g4 + 3]));
          slot[(8u + g4) * 32u] = make_float4(__uint_as_float(r1[4 * g4]), __uint_as_float(r1[4 * g4 + 1]),
                                              __uint_as_float(r1[4 * g4 + 2]), __uint_as_float(r1[4 * g4 + 3]));
          slot[(16u + g4) * 32u] = make_float4(__uint_as_float(r2[4 * g4]), __uint_as_float(r2[4 * g4 + 1]),
                                               __uint_as_float(r2[4 * g4 + 2]), __uint_as_float(r2[4 * g4 + 3]));
          slot[(24u + g4) * 32u] = make_float4(__uint_as_float(r3[4 * g4]), __uint_as_float(r3[4 * g4 + 1]),
                                               __uint_as_float(r3[4 * g4 + 2]), __uint_as_float(r3[4 * g4 + 3]));
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) *reinterpret_cast<volatile uint32_t *>(flags + pair_id * P::kFlagsPerPair + rank * 8u + ew) = tag;
        continue;
      }
      uint32_t packed[P::kBN / 4];
#pragma unroll
      for (uint32_t j = 0; j < 32; j += 2) {
        const __nv_bfloat162 v0 = __floats2bfloat162_rn(__uint_as_float(r0[j]) * alpha, __uint_as_float(r0[j + 1]) * alpha);
        const __nv_bfloat162 v1 = __floats2bfloat162_rn(__uint_as_float(r1[j]) * alpha, __uint_as_float(r1[j + 1]) * alpha);
        const __nv_bfloat162 v2 = __floats2bfloat162_rn(__uint_as_float(r2[j]) * alpha, __uint_as_float(r2[j + 1]) * alpha);
        const __nv_bfloat162 v3 = __floats2bfloat162_rn(__uint_as_float(r3[j]) * alpha, __uint_as_float(r3[j + 1]) * alpha);
        packed[j / 2] = *reinterpret_cast<const uint32_t *>(&v0);
        packed[16 + j / 2] = *reinterpret_cast<const uint32_t *>(&v1);
        packed[32 + j / 2] = *reinterpret_cast<const uint32_t *>(&v2);
        packed[48 + j / 2] = *reinterpret_cast<const uint32_t *>(&v3);
      }
      const bool odd = (lane & 1u) != 0u;
      __nv_bfloat16 *crow = c + (row & ~1u);
#pragma unroll
      for (uint32_t j = 0; j < P::kBN / 4; ++j) {
        const uint32_t got = __shfl_xor_sync(0xffffffffu, packed[j], 1);
        const uint32_t v = odd ? __byte_perm(got, packed[j], 0x7632) : __byte_perm(packed[j], got, 0x5410);
        const uint32_t tok = tok0 + 2u * j + (odd ? 1u : 0u);
        if (tok < n) *reinterpret_cast<uint32_t *>(crow + static_cast<size_t>(tok) * m) = v;
      }
    }
  }

  // Common exit: the pair meets (nobody may still read the other's shared or tensor memory),
  // then both allocating warps release TMEM.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P::kTmemCols) : "memory");
  }
}

// ============================================================================================
// Split-K form for few tokens and few row blocks (decode: n <= 8, the k / v / o / down
// projections have only 8 or 40 row blocks, far fewer than SMs).  A cluster of S CTAs shares one
// 128-row x BN-token tile; CTA r streams K-blocks [r * kb / S, (r + 1) * kb / S) through the same
// TMA -> tcgen05 pipeline into its own TMEM accumulator.  The partial sums meet in the first
// CTA's shared memory (distributed shared memory stores, one cluster barrier), which adds them in
// rank order, applies alpha and writes bf16: no workspace, no atomics, deterministic.
// ============================================================================================
constexpr uint32_t kMaxSplit = 8;
// CTAs per row block that still leave room for the partial sums in the first CTA's shared memory
// ((S - 1) x 128 rows x BN floats beside the operand ring): 8 up to 16 tokens, 5 at 32, 2 at 64.
template <uint32_t BN> constexpr uint32_t max_split_for() { return BN <= 16 ? kMaxSplit : (BN <= 32 ? 5u : 2u); }

__device__ __forceinline__ void st_cluster_v4f(uint32_t addr, float a, float b, float c4, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c4), "f"(d) : "memory");
}

template <uint32_t BN>
__global__ void __launch_bounds__(kThreads, 1)
nvfp4_gemm_splitk_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const uint8_t *__restrict__ a_sf, const uint8_t *__restrict__ b_sf,
                         __nv_bfloat16 *__restrict__ c, uint32_t m, uint32_t n, uint32_t k, float alpha) {
  using C = Cfg<BN>;
  static_assert(BN <= 64, "split-K form is for small token counts");
  constexpr uint32_t kCols = C::kBRows;                                  // accumulator columns that hold data
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + 8;
  uint64_t *sf_full = empty + 8;
  uint64_t *acc_full = sf_full + 8;
  uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(acc_full + 2);
  uint8_t *stages = smem + 1024;
  float *partials = reinterpret_cast<float *>(stages + C::kStages * C::kStageBytes);   // [S-1][128 rows][kCols], first CTA only

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  uint32_t S, rank;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(S));
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const uint32_t mb = blockIdx.x / S;                                    // one tile per cluster, one token block
  const uint32_t k_blocks = k / 256u;
  const uint32_t kb_begin = rank * k_blocks / S, kb_end = (rank + 1u) * k_blocks / S;
  const uint32_t sf_tiles_per_block = k / 64u;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < C::kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&sf_full[s], 1); }
    mbar_init(&acc_full[0], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_base_slot;
  const uint32_t tmem_sf = tmem_base + C::kAccStages * C::kAccCols;

  float acc[kCols];                                                      // epilogue warps: this lane's row
#pragma unroll
  for (uint32_t j = 0; j < kCols; ++j) acc[j] = 0.f;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      for (uint32_t kb = kb_begin, g = 0; kb < kb_end; ++kb, ++g) {
        const uint32_t s = g % C::kStages, ph = (g / C::kStages) & 1u;
        if (!mbar_wait(&empty[s], ph ^ 1u)) break;
        uint8_t *st = stages + s * C::kStageBytes;
        mbar_expect_tx(&full[s], C::kABytes + C::kBRows * kBKBytes + C::kSfaBytes + 2048u);
        tma_load_2d(st, &map_a, kb * kBKBytes, mb * kBM, &full[s]);
        tma_load_2d(st + C::kABytes, &map_b, kb * kBKBytes, 0u, &full[s]);
        bulk_g2s(st + C::kABytes + C::kBBytes, a_sf + (static_cast<size_t>(mb) * sf_tiles_per_block + kb * 4u) * 512u,
                 2048u, &full[s]);
        bulk_g2s(st + C::kABytes + C::kBBytes + C::kSfaBytes, b_sf + static_cast<size_t>(kb * 4u) * 512u, 2048u, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool dead = false;
      for (uint32_t kb = kb_begin, g = 0; kb < kb_end; ++kb, ++g) {
        const uint32_t s = g % C::kStages, ph = (g / C::kStages) & 1u;
        if (!mbar_wait(&full[s], ph) || !mbar_wait(&sf_full[s], ph)) { dead = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t st = smem_u32(stages + s * C::kStageBytes);
        const uint32_t sfa_t = tmem_sf + s * C::kSfCols, sfb_t = sfa_t + 16u;
#pragma unroll
        for (uint32_t kk = 0; kk < 4; ++kk)
          mma_mxf4nvf4(tmem_base, desc_sw128(st + kk * 32u), desc_sw128(st + C::kABytes + kk * 32u), C::kIdesc,
                       sfa_t + kk * 4u, sfb_t + kk * 4u, (g | kk) != 0u);
        mma_commit(&empty[s]);
      }
      if (!dead) mma_commit(&acc_full[0]);
    }
  } else if (warp == kWarpCopier) {
    if (lane == 0) {
      for (uint32_t kb = kb_begin, g = 0; kb < kb_end; ++kb, ++g) {
        const uint32_t s = g % C::kStages, ph = (g / C::kStages) & 1u;
        if (!mbar_wait(&full[s], ph)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t st = smem_u32(stages + s * C::kStageBytes);
        const uint32_t sfa_t = tmem_sf + s * C::kSfCols, sfb_t = sfa_t + 16u;
#pragma unroll
        for (uint32_t kk = 0; kk < 4; ++kk) {
          tmem_cp_sf(sfa_t + kk * 4u, desc_sf(st + C::kABytes + C::kBBytes + kk * 512u));
          tmem_cp_sf(sfb_t + kk * 4u, desc_sf(st + C::kABytes + C::kBBytes + C::kSfaBytes + kk * 512u));
        }
        mma_commit(&sf_full[s]);
      }
    }
  } else if (warp >= kWarpEpilogue && warp < kWarpEpilogue + 4u) {
    // epilogue warps 4..7: drain this CTA's partial sums; ranks > 0 hand them to the first CTA
    const uint32_t quarter = warp & 3u;
    if (kb_end > kb_begin) {
      ok = mbar_wait(&acc_full[0], 0u);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (ok) {
        const uint32_t taddr = tmem_base + ((quarter * 32u) << 16);
#pragma unroll
        for (uint32_t c0 = 0; c0 < kCols; c0 += 8) {
          uint32_t r[8];
          tmem_ld8(taddr + c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j) acc[c0 + j] = __uint_as_float(r[j]);
        }
      }
    }
    if (rank != 0u) {
      const uint32_t row = quarter * 32u + lane;
      const uint32_t dst = map_to_cta(smem_u32(partials + (static_cast<size_t>(rank - 1u) * kBM + row) * kCols), 0u);
#pragma unroll
      for (uint32_t j = 0; j < kCols; j += 4) st_cluster_v4f(dst + j * 4u, acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    }
  }

  // The cluster meets: every partial sum has landed in the first CTA's shared memory.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();
  if (rank == 0u && warp >= kWarpEpilogue && warp < kWarpEpilogue + 4u && ok) {
    const uint32_t quarter = warp & 3u;
    const uint32_t row_in = quarter * 32u + lane, row = mb * kBM + row_in;
    for (uint32_t r = 1; r < S; ++r) {                                   // fixed order: rank 1, 2, ...
      const float4 *src = reinterpret_cast<const float4 *>(partials + (static_cast<size_t>(r - 1u) * kBM + row_in) * kCols);
#pragma unroll
      for (uint32_t j = 0; j < kCols; j += 4) {
        const float4 v = src[j / 4];
        acc[j] += v.x; acc[j + 1] += v.y; acc[j + 2] += v.z; acc[j + 3] += v.w;
      }
    }
#pragma unroll
    for (uint32_t j = 0; j < kCols; ++j)
      if (j < n) c[static_cast<size_t>(j) * m + row] = __float2bfloat16(acc[j] * alpha);
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::kTmemCols) : "memory");
  }
}

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

// Packed fp4 bytes [rows][k/2] -> 2-D map, box = 128 bytes x box_rows, 128-byte swizzle.
// A tensor map depends only on (pointer, extents, box): weights and activation buffers come back
// with the same few hundred combinations on every step, so the encoded maps are kept in a small
// direct-mapped cache instead of being rebuilt by the driver on every launch (a cost only eager
// callers see; a replayed graph holds the maps).
struct MapKey {
  uint64_t ptr = 0, rows = 0, k = 0;
  uint32_t box = 0, kind = 0;          // kind 1 = operand map, 2 = scale map
  bool operator==(const MapKey &o) const { return ptr == o.ptr && rows == o.rows && k == o.k && box == o.box && kind == o.kind; }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
};
constexpr size_t kMapSlots = 512;
std::mutex g_map_mu;
MapSlot g_map_slots[kMapSlots];

bool cached_map(const MapKey &key, CUtensorMap *out, bool (*build)(CUtensorMap *, const MapKey &)) {
  const uint64_t h = ((key.ptr >> 8) * 0x9E3779B97F4A7C15ull) ^ (key.rows * 31u + key.k * 7u + key.box + key.kind);
  MapSlot &slot = g_map_slots[(h >> 24) % kMapSlots];
  {
    std::lock_guard<std::mutex> lock(g_map_mu);
    if (slot.key == key) { *out = slot.map; return true; }
  }
  if (!build(out, key)) return false;
  std::lock_guard<std::mutex> lock(g_map_mu);
  slot.key = key;
  slot.map = *out;
  return true;
}

bool build_operand_map(CUtensorMap *map, const MapKey &key) {
  EncodeFn enc = encode_fn();
  if (enc == nullptr) return false;
  const uint64_t ptr = key.ptr, rows = key.rows, k = key.k;
  const uint32_t box_rows = key.box;
  const cuuint64_t dims[2] = {k / 2, rows};
  const cuuint64_t strides[1] = {k / 2};
  const cuuint32_t box[2] = {kBKBytes, box_rows};
  const cuuint32_t ones[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, reinterpret_cast<void *>(ptr), dims, strides, box, ones,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_operand_map(CUtensorMap *map, uint64_t ptr, uint64_t rows, uint64_t k, uint32_t box_rows) {
  MapKey key;
  key.ptr = ptr; key.rows = rows; key.k = k; key.box = box_rows; key.kind = 1;
  return cached_map(key, map, build_operand_map);
}

int sm_count() { return q36::sm_count_current_device(); }

template <uint32_t BN>
int launch(const qwen36_nvfp4_gemm_spec_t *s, float alpha) {
  using C = Cfg<BN>;
  CUtensorMap map_a, map_b;
  if (!make_operand_map(&map_a, s->a_fp4.ptr, s->m, s->k, kBM) ||
      !make_operand_map(&map_b, s->b_fp4.ptr, s->n, s->k, C::kBRows))
    return QWEN36_STATUS_NOT_IMPLEMENTED;
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(nvfp4_gemm_tc_kernel<BN>), static_cast<int>(C::kSmemBytes)) !=
      cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  const uint32_t tiles = static_cast<uint32_t>((s->m / kBM) * ((s->n + BN - 1) / BN));
  const uint32_t grid = tiles < static_cast<uint32_t>(sm_count()) ? tiles : static_cast<uint32_t>(sm_count());
  nvfp4_gemm_tc_kernel<BN><<<grid, kThreads, C::kSmemBytes, q36::stream()>>>(
      map_a, map_b, as_ptr<const uint8_t>(s->a_scale), as_ptr<const uint8_t>(s->b_scale),
      as_ptr<__nv_bfloat16>(s->c_bf16), static_cast<uint32_t>(s->m), static_cast<uint32_t>(s->n),
      static_cast<uint32_t>(s->k), alpha);
  return q36::launch_status();
}

// Tiled scale buffer as uint32 [tiles][128]: one 512-byte scale tile per row, box = four tiles (one 256-K stage).
bool build_scale_map(CUtensorMap *map, const MapKey &key) {
  EncodeFn enc = encode_fn();
  if (enc == nullptr) return false;
  const uint64_t ptr = key.ptr, tiles = key.rows;
  const cuuint64_t dims[2] = {128, tiles};
  const cuuint64_t strides[1] = {512};
  const cuuint32_t box[2] = {128, 4};
  const cuuint32_t ones[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, reinterpret_cast<void *>(ptr), dims, strides, box, ones,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_scale_map(CUtensorMap *map, uint64_t ptr, uint64_t tiles) {
  MapKey key;
  key.ptr = ptr; key.rows = tiles; key.kind = 2;
  return cached_map(key, map, build_scale_map);
}

// Pairs of CTAs of `kernel` that the current device can host at once (asked once per kernel and device).
int max_active_pairs(const void *kernel, const cudaLaunchConfig_t *cfg) {
  static std::mutex mu;
  static std::vector<std::tuple<const void *, int, int>> known;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const auto &e : known)
      if (std::get<0>(e) == kernel && std::get<1>(e) == dev) return std::get<2>(e);
  }
  int v = 0;
  if (cudaOccupancyMaxActiveClusters(&v, kernel, cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    v = 0;
  }
  std::lock_guard<std::mutex> lock(mu);
  known.emplace_back(kernel, dev, v);
  return v;
}

int launch_pair(const qwen36_nvfp4_gemm_spec_t *s, float alpha) {
  namespace P = pair;
  CUtensorMap map_a, map_b, map_sfa, map_sfb;
  const uint64_t sf_tiles = s->k / 64;
  if (!make_operand_map(&map_a, s->a_fp4.ptr, s->m, s->k, kBM) ||
      !make_operand_map(&map_b, s->b_fp4.ptr, s->n, s->k, P::kHalfTok) ||
      !make_scale_map(&map_sfa, s->a_scale.ptr, (s->m / 128) * sf_tiles) ||
      !make_scale_map(&map_sfb, s->b_scale.ptr, ((s->n + 127) / 128) * sf_tiles))
    return QWEN36_STATUS_NOT_IMPLEMENTED;
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(nvfp4_gemm_pair_kernel), static_cast<int>(P::kSmemBytes)) !=
      cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  const uint32_t tiles = static_cast<uint32_t>((s->m / 256) * ((s->n + P::kBN - 1) / P::kBN));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<uint32_t>(sm_count()) & ~1u);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = P::kSmemBytes;
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // The grid is persistent with a static tile stride, so it must never exceed the number of
  // pairs the device can host at the same time (some SMs may have no free partner).
  const int max_pairs = max_active_pairs(reinterpret_cast<const void *>(nvfp4_gemm_pair_kernel), &cfg);
  if (max_pairs <= 0) return QWEN36_STATUS_NOT_IMPLEMENTED;
  const uint32_t pairs = tiles < static_cast<uint32_t>(max_pairs) ? tiles : static_cast<uint32_t>(max_pairs);
  cfg.gridDim = dim3(pairs * 2u);
  return q36::cuda_status(cudaLaunchKernelEx(&cfg, nvfp4_gemm_pair_kernel, map_a, map_b, map_sfa, map_sfb,
                                             as_ptr<__nv_bfloat16>(s->c_bf16), static_cast<uint32_t>(s->m),
                                             static_cast<uint32_t>(s->n), static_cast<uint32_t>(s->k), alpha));
}

std::atomic<uint32_t> g_streamk_tag{0};
std::atomic<int> g_streamk_mode{0};       // test hook: 0 = by the fill of the last round, 1 = never, 2 = whenever the workspace allows

// Does cutting tiles along K pay for this launch?  Whole tiles cost ceil(tiles / pairs) rounds of k_blocks
// stages.  Stream-K costs tiles * k_blocks / pairs stages, each about a tenth slower (pairs that run side
// by side no longer share weight rows in L2), plus the fix-up and the extra segment turn-arounds (8 us,
// 17 stages).  Measured on down 5120 x 17408: 46 -> 43 / 82 -> 61 / 110 -> 93 us at 512 / 1024 / 2048
// tokens, and the other way round (170 -> 182 us) at 4096, where this rule declines.
bool stream_k_pays(uint32_t tiles, uint32_t pairs, uint32_t k_blocks) {
  const uint64_t whole = static_cast<uint64_t>((tiles + pairs - 1u) / pairs) * k_blocks;
  const uint64_t cut = (static_cast<uint64_t>(tiles) * k_blocks + pairs - 1u) / pairs;
  return cut * 11u + 170u < whole * 10u;
}

template <bool SK>
int launch_pair6_form(const qwen36_nvfp4_gemm_spec_t *s, float alpha, const CUtensorMap &map_a, const CUtensorMap &map_b,
                      const CUtensorMap &map_sfa, const CUtensorMap &map_sfb, cudaLaunchConfig_t &cfg, uint32_t pairs) {
  namespace P = pair6;
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(nvfp4_gemm_pair6_kernel<SK>), static_cast<int>(P::kSmemBytes)) !=
      cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  cfg.gridDim = dim3(pairs * 2u);
  uint32_t tag = 0;
  if (SK) {
    do { tag = g_streamk_tag.fetch_add(1u) + 1u; } while (tag == 0u);   // never 0: a cleared workspace must not look flagged
  }
  return q36::cuda_status(cudaLaunchKernelEx(&cfg, nvfp4_gemm_pair6_kernel<SK>, map_a, map_b, map_sfa, map_sfb,
                                             as_ptr<__nv_bfloat16>(s->c_bf16), static_cast<uint32_t>(s->m),
                                             static_cast<uint32_t>(s->n), static_cast<uint32_t>(s->k), alpha,
                                             as_ptr<float>(s->workspace), tag));
}

int launch_pair6(const qwen36_nvfp4_gemm_spec_t *s, float alpha) {
  namespace P = pair6;
  CUtensorMap map_a, map_b, map_sfa, map_sfb;
  const uint64_t sf_tiles = s->k / 64;
  if (!make_operand_map(&map_a, s->a_fp4.ptr, s->m, s->k, kBM) ||
      !make_operand_map(&map_b, s->b_fp4.ptr, s->n, s->k, P::kHalfTok) ||
      !make_scale_map(&map_sfa, s->a_scale.ptr, (s->m / 128) * sf_tiles) ||
      !make_scale_map(&map_sfb, s->b_scale.ptr, ((s->n + 127) / 128) * sf_tiles))
    return QWEN36_STATUS_NOT_IMPLEMENTED;
  const uint32_t tiles = static_cast<uint32_t>((s->m / 256) * ((s->n + P::kBN - 1) / P::kBN));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<uint32_t>(sm_count()) & ~1u);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = P::kSmemBytes;
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // The grid is persistent with a static walk over the work, so it must never exceed the number of
  // pairs the device can host at the same time (some SMs may have no free partner).
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(nvfp4_gemm_pair6_kernel<false>), static_cast<int>(P::kSmemBytes)) !=
      cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  const int max_pairs = max_active_pairs(reinterpret_cast<const void *>(nvfp4_gemm_pair6_kernel<false>), &cfg);
  if (max_pairs <= 0) return QWEN36_STATUS_NOT_IMPLEMENTED;
  const uint32_t all = static_cast<uint32_t>(max_pairs);
  const uint64_t units = static_cast<uint64_t>(tiles) * (s->k / 256);
  const size_t need = static_cast<size_t>(all) * (P::kSlotFloats * sizeof(float) + P::kFlagsPerPair * sizeof(uint32_t));
  const int mode = g_streamk_mode.load();
  const bool fits = s->workspace.ptr != 0 && (s->workspace.ptr & 15u) == 0 && s->workspace_bytes >= need && units >= all &&
                    units < (1ull << 32);
  if (fits && (mode == 2 || (mode == 0 && stream_k_pays(tiles, all, static_cast<uint32_t>(s->k / 256)))))
    return launch_pair6_form<true>(s, alpha, map_a, map_b, map_sfa, map_sfb, cfg, all);
  const uint32_t pairs = tiles < all ? tiles : all;
  return launch_pair6_form<false>(s, alpha, map_a, map_b, map_sfa, map_sfb, cfg, pairs);
}

// Split-K launch: `split` CTAs per 128-row block (cluster), one token block (n <= BN).
template <uint32_t BN>
int launch_splitk(const qwen36_nvfp4_gemm_spec_t *s, float alpha, uint32_t split) {
  using C = Cfg<BN>;
  CUtensorMap map_a, map_b;
  if (!make_operand_map(&map_a, s->a_fp4.ptr, s->m, s->k, kBM) ||
      !make_operand_map(&map_b, s->b_fp4.ptr, s->n, s->k, C::kBRows))
    return QWEN36_STATUS_NOT_IMPLEMENTED;
  constexpr uint32_t kSmem = C::kSmemBytes + (max_split_for<BN>() - 1) * kBM * C::kBRows * 4u;
  static_assert(kSmem <= 227u * 1024u, "split-K shared memory");
  if (split > max_split_for<BN>()) split = max_split_for<BN>();
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(nvfp4_gemm_splitk_kernel<BN>), static_cast<int>(kSmem)) !=
      cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<uint32_t>(s->m / kBM) * split);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return q36::cuda_status(cudaLaunchKernelEx(&cfg, nvfp4_gemm_splitk_kernel<BN>, map_a, map_b,
                                             as_ptr<const uint8_t>(s->a_scale), as_ptr<const uint8_t>(s->b_scale),
                                             as_ptr<__nv_bfloat16>(s->c_bf16), static_cast<uint32_t>(s->m),
                                             static_cast<uint32_t>(s->n), static_cast<uint32_t>(s->k), alpha));
}

// CTAs per row block for the split-K form, 1 when the plain persistent kernel should run: split
// only when the row blocks alone leave most SMs idle, as far as that fills the device, keeping at
// least two K-blocks per CTA.
uint32_t choose_split(const qwen36_nvfp4_gemm_spec_t *s) {
  const int forced = g_force_split.load();
  const uint32_t m_blocks = static_cast<uint32_t>(s->m / kBM), k_blocks = static_cast<uint32_t>(s->k / 256);
  uint32_t split = forced > 0 ? static_cast<uint32_t>(forced) : static_cast<uint32_t>(sm_count()) / m_blocks;
  if (split > kMaxSplit) split = kMaxSplit;
  if (split > k_blocks / 2u) split = k_blocks / 2u;
  return split < 2u ? 1u : split;
}

}  // namespace

bool nvfp4_gemm_tc_forced() { return g_force_bn.load() != 0 || g_force_split.load() != 0; }

int nvfp4_gemm_tc(const qwen36_nvfp4_gemm_spec_t *s, float alpha) {
  if (s->m % kBM != 0 || s->k % 256 != 0 || s->m > (1u << 30) || s->n > (1u << 30) || s->k > (1u << 30) ||
      ((s->a_fp4.ptr | s->b_fp4.ptr | s->a_scale.ptr | s->b_scale.ptr) & 15u) != 0 || (s->c_bf16.ptr & 3u) != 0)
    return QWEN36_STATUS_NOT_IMPLEMENTED;
  const int forced = g_force_bn.load();
  if (forced == 128 && s->n > 128) return launch<128>(s, alpha);
  // CTA pairs (256 x 256 tiles): measured ahead of single-CTA tiles only for long K with many
  // tokens (+5 % at k = 17408, n = 8192; level or slightly behind elsewhere).
  // CTA pairs with six operand stages and a separate scale pipeline: ahead of every other form from
  // 512 tokens up (gate_up 34816 x 5120: 56 / 178 / 673 us at 512 / 2048 / 8192 tokens against 58 / 187 / 724;
  // down 5120 x 17408: 44 / 114 / 336 against 48 / 128 / 373).
  if (s->n > 128 && s->m % 256 == 0 && (forced == 768 || (forced == 0 && s->n >= 512))) {
    const int rc = launch_pair6(s, alpha);
    if (rc != QWEN36_STATUS_NOT_IMPLEMENTED) return rc;      // pairs unavailable: the older forms below
  }
  if (s->n > 128 && s->m % 256 == 0 && (forced == 512 || (forced == 0 && s->k >= 8192 && s->n >= 4096))) {
    const int rc = launch_pair(s, alpha);
    if (rc != QWEN36_STATUS_NOT_IMPLEMENTED) return rc;      // pairs unavailable: single-CTA tiles below
  }
  if (s->n <= 64) {
    // few row blocks (k / v / o / down: 8 or 40 on 148 SMs): clusters share a tile along K.  Up to 16 tokens
    // as many CTAs per row block as fit the GPU; 32 and 64 tokens as many as the partial sums leave room for
    // (down 5120 x 17408 at 32 tokens: 29 -> 16 us).
    const uint32_t split = choose_split(s);
    if (split > 1u) {
      if (s->n <= 8) return launch_splitk<8>(s, alpha, split);
      if (s->n <= 16) return launch_splitk<16>(s, alpha, split);
      if (s->n <= 32) return launch_splitk<32>(s, alpha, split);
      // two CTAs per row block: pays for long K only (k = 17408: 30 -> 23 us; k = 6144: 13.7 -> 14.6 us)
      if (s->k >= 48u * 256u) return launch_splitk<64>(s, alpha, split);
    }
  }
  if (s->n <= 8) return launch<8>(s, alpha);
  if (s->n <= 16) return launch<16>(s, alpha);
  if (s->n <= 32) return launch<32>(s, alpha);
  if (s->n <= 64) return launch<64>(s, alpha);
  if (s->n <= 128) return launch<128>(s, alpha);
  return launch<256>(s, alpha);
}

// Tuning hook: 128 forces 128-token tiles (two accumulator stages) for large n, 256 single-CTA
// 256-token tiles, 512 CTA pairs with five combined stages, 768 CTA pairs with six operand stages
// and the separate scale pipeline (where the shape allows pairs); 0 = default.
extern "C" void qwen36_nvfp4_gemm_force_bn(int bn) { g_force_bn.store(bn); }
// Tuning / test hook for the stream-K form of the CTA-pair kernel: 0 = by the fill of the last round of
// tiles (default), 1 = never, 2 = whenever the workspace allows.
extern "C" void qwen36_nvfp4_gemm_stream_k(int mode) { g_streamk_mode.store(mode < 0 || mode > 2 ? 0 : mode); }
// Tuning hook: CTAs per row block of the split-K form for n <= 16 (1 = never split, 0 = heuristic).
extern "C" void qwen36_nvfp4_gemm_force_split(int split) { g_force_split.store(split); }

#ifdef Q36_GEMM_TRACE
extern "C" int qwen36_nvfp4_gemm_trace_read(void *dst) {
  return cudaMemcpyFromSymbol(dst, g_gemm_trace, sizeof(g_gemm_trace)) == cudaSuccess ? 0 : -1;
}
#endif

// 1 when a bounded wait inside the tensor-core GEMM ever gave up.  Synchronises.
extern "C" int qwen36_nvfp4_gemm_last_error(void) {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(v)) != cudaSuccess) return -1;
  return static_cast<int>(v);
}

}  // namespace q36
