// NVFP4 GEMV for decode (one token), HBM-bound weight streaming with the arithmetic on the
// tensor cores:
//   W4A16  y[row] = bf16( global * sum_g ue4m3(sf[g,row]) * sum_{i<16} x[16g+i] * e2m1(w[row,16g+i]) )
//          (semantics of kernels-cuda/ops.cu:547-639 in the reference; x is a bf16 vector)
//   W4A4   the same with x = e2m1(b) * ue4m3(sfb), exact in float16, and alpha in place of global
//          (kernels-cuda/decode_gemv/nvfp4_gemv_sm120.cu:203-331, n = 1)
//
// Why tensor cores for a matrix-vector product: at the HBM rate a SIMT inner loop (one
// conversion per two weights, one FMA per weight, scale handling) needs nearly every issue slot
// of the SM, so any stall of the weight stream is lost for good.  Here a warp turns a 16-row x
// 16-column weight block into ONE mma.sync.m16n8k16 (float16 operands, float32 accumulation):
// the only per-weight instruction left is the e2m1x2 -> f16x2 conversion, which leaves the SM
// about twice the HBM rate in hand to catch up after the serial part of a launch.
//
// Block scales without a per-weight multiply.  The B operand (activations, 16 x 8) is filled so
// that column n holds the activations of the four k-slots that lane-in-group n supplies and zeros
// elsewhere.  Four chained MMAs then leave in D[row][n] the exact partial dot product of ONE
// 16-column scale group per column n, and the block scale is applied to that sum with one
// float32 FMA per (row, group), which is the reference's own order of operations.
//
// Pipeline.  Persistent CTAs: one producer warp, eight consumer warps, one epilogue warp.  A work
// unit is 32 rows (rows r0+q+32j of a 128-row block, q < 8, j < 4); a stage is 1024 columns of it:
// ONE 5-D tiled TMA box of weights (128-byte swizzle, 16 KB) + ONE 3-D box of scale tiles (2 KB),
// four stages in flight per CTA.  Every consumer warp owns 128 of a stage's 1024 columns for all
// 32 rows, so all warps are busy on every stage whatever the matrix shape; their partial sums go
// through shared memory to the epilogue warp, which forms the rows while the consumers are already
// on the next item.  The activation slice of a warp is staged by that warp alone (no CTA barrier
// between the end of the producing kernel and the first MMA).  Up to four matrices that share the
// activation vector run as one launch.
//
// Work decomposition.  For K of more than kChunkStages stages a unit is cut along K into chunks, an
// item is one chunk of one unit, and every CTA takes a contiguous run of the chunk-major item list
// that holds 1 / grid of the launch's stages: matrices with few rows (o: 160 units, down: 160
// units of 17 stages) then fill all CTA slots evenly instead of leaving half of them idle, and a
// CTA stages only the part of x its chunks touch.  The chunks of a unit meet in global memory
// (see the epilogue warp).  The cut depends on K alone, so a row's sum is formed in the same order
// whatever the matrix height, the grouping or the GPU.  Units of shorter K stay whole and are
// dealt round-robin over a grid sized so that every CTA gets the same number of them.
//
// Weights and scales stream before griddepcontrol.wait: under programmatic dependent launch the
// ring fills while the kernel that produces x is still finishing.
//
// Tensor-parallel form (PEER = true; the output rows of a matrix are split over the GPUs of a node).
// The epilogue stores the rank's rows straight into EVERY rank's copy of the full output vector
// (stores over NVLink into an arena the peers have mapped).  The vector travels in flagged cells:
// 8 bytes = two bf16 values + the 32-bit number of the call that wrote them, two cells per 16-byte
// store.  An 8-byte aligned word arrives whole, so a consumer that reads a cell with the expected
// call number has its data: no fence, no flag, no ticket on the path between the producer's last
// FMA and the consumer's first MMA, which is what a chain of dependent few-microsecond launches
// needs (a system-scope fence alone costs about 4 us here).  The launch that consumes the vector
// polls (bounded) the cells of ITS columns while it stages them, with its weight ring already
// full.  Call numbers live in device memory and are advanced by the kernel, so a CUDA graph can
// hold the launches.  A wait that runs out poisons the rows (NaN) and records the call number.
#include "nvfp4_gemv_mma.cuh"

#include <atomic>
#include <mutex>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace {

using q36::as_ptr;

constexpr int kWarps = 8;                           // consumer warps
constexpr uint32_t kWarpProducer = kWarps, kWarpEpilogue = kWarps + 1;
constexpr int kBlock = (kWarps + 2) * 32;
constexpr uint32_t kRed = 3;                        // items' partial sums in flight to the epilogue warp
#ifndef Q36_GEMV_CHUNK
#define Q36_GEMV_CHUNK 6
#endif
constexpr uint32_t kChunkStages = Q36_GEMV_CHUNK;   // stages per K-chunk, at most
constexpr uint32_t kMaxChunks = 16;                 // K-chunks per unit (kMaxK / 1024 stages over kChunkStages)
constexpr uint32_t kMaxMats = 4;
#ifndef Q36_GEMV_STAGES
#define Q36_GEMV_STAGES 4
#endif
constexpr uint32_t kStages = Q36_GEMV_STAGES;
#ifndef Q36_GEMV_AHEAD
#define Q36_GEMV_AHEAD 4
#endif
constexpr uint32_t kAhead = Q36_GEMV_AHEAD;         // stages of L2 prefetch kept ahead of the ring
constexpr uint32_t kStageW = 16384;                 // 32 rows x 512 B
constexpr uint32_t kStageSf = 2048;                 // 16 scale tiles x 8 row-words x 16 B
constexpr uint32_t kStageBytes = kStageW + kStageSf;
constexpr uint32_t kRingBytes = kStages * kStageBytes;
constexpr uint32_t kHeaderBytes = 4096;             // barriers, slice scales, zero chunk, partial sums
constexpr uint32_t kSpinLimit = 1u << 24;
constexpr uint32_t kMaxK = 32768;
constexpr uint32_t kMaxPeers = 8;                   // tensor-parallel form: ranks of one node
constexpr uint32_t kNoSlot = 0xffffffffu;
constexpr uint32_t kPeerSpinLimit = 1u << 21;       // x (200 ns back-off + one read of the cells): 1-2 s
constexpr uint32_t kPeerEagerPolls = 2048;
constexpr uint32_t kParkSpinLimit = 1u << 20;       // x (100 ns back-off + one round trip to L2): about a second

__device__ unsigned int g_gemv_mma_error = 0;       // set when a bounded wait gives up
constexpr uint32_t kPoolSets = 16, kScratchCells = 1u << 19, kTicketWords = 1u << 15;
__device__ unsigned long long g_scratch[kPoolSets * kScratchCells];   // 64 MB, zero-initialised like every device global
__device__ uint32_t g_tickets[kPoolSets * kTicketWords];

// Per-CTA %globaltimer stamps for pipeline analysis; compiled in only with -DQ36_GEMV_TRACE.
#ifdef Q36_GEMV_TRACE
constexpr uint32_t kTraceLaunches = 64, kTraceCtas = 320, kTraceEvents = 8;
__device__ unsigned long long g_trace[kTraceLaunches][kTraceCtas][kTraceEvents];
#define Q36_TRACE(ev)                                                                       \
  do {                                                                                      \
    unsigned long long t_;                                                                  \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                  \
    if (blockIdx.x < kTraceCtas) g_trace[p.trace_id % kTraceLaunches][blockIdx.x][ev] = t_; \
  } while (0)
#else
#define Q36_TRACE(ev)
#endif

struct GemvParams {
  CUtensorMap map_w[kMaxMats];
  CUtensorMap map_sf[kMaxMats];
  const uint8_t *w[kMaxMats];
  const uint8_t *sf[kMaxMats];
  __nv_bfloat16 *y[kMaxMats];
  const float *tensor_scale[kMaxMats];   // W4A16: per-matrix global scale (may be null)
  uint32_t unit_end[kMaxMats];           // running total of 32-row units
  const void *x;                         // bf16 vector (W4A16) or packed E2M1 codes (W4A4)
  const uint8_t *x_sf;                   // W4A4: tiled UE4M3 scales of the activation row
  uint32_t K, iters, units, count;
  uint32_t chunk, cpu;                   // stages per K-chunk, chunks per unit
  uint32_t set;                          // which parking set of g_scratch / g_tickets this launch uses
  uint32_t tag;                          // nonzero, differs between launches that may meet in one scratch set
  float alpha;                           // W4A4
  // tensor-parallel form only
  uint8_t *const *peer_arena;            // device array [world]: base of every rank's arena (own one included)
  uint32_t *state;                       // local [slots][4]: calls completed, CTA ticket, first failed call, -
  uint32_t world, rank, out_slot, in_slot;
  uint32_t row_off[kMaxMats];            // first row of this rank's slice in the full vector
  uint64_t y_off[kMaxMats];              // byte offset of the full output vector (flagged cells) inside an arena
#ifdef Q36_GEMV_TRACE
  uint32_t trace_id;
#endif
};

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
  atomicExch(&g_gemv_mma_error, 1u);
  return false;
}
__device__ __forceinline__ void tma_load_5d(void *dst, const CUtensorMap *map, uint32_t c0, uint32_t c1, uint32_t c2,
                                            uint32_t c3, uint32_t c4, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
// L2 prefetch of the same boxes (no shared memory involved).
__device__ __forceinline__ void tma_prefetch_5d(const CUtensorMap *map, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                uint32_t c4) {
  asm volatile("cp.async.bulk.prefetch.tensor.5d.L2.global.tile [%0, {%1, %2, %3, %4, %5}];"
               ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap *map, uint32_t c0, uint32_t c1, uint32_t c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
               ::"l"(map), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint32_t c0, uint32_t c1, uint32_t c2,
                                            uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// Four bytes of packed E2M1 -> four f16x2 (low nibble in the low half).
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

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Two UE4M3 bytes -> two floats through the hardware E4M3 conversion (exact).  The bytes 0x7F and
// 0xFF convert to NaN here while the reference reads them as 448: the NaN reaches the row's sum,
// and a row whose sum is NaN is redone by exact_row() below with the reference's decoder.
__device__ __forceinline__ float2 ue4m3x2_to_f32(uint32_t two_bytes) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two_bytes), __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2 *>(&h));
}

__device__ __forceinline__ void st_cells(void *p, uint32_t d0, uint32_t d1, uint32_t call) {
  asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1, %2, %3, %2};" ::"l"(p), "r"(d0), "r"(call), "r"(d1) : "memory");
}
__device__ __forceinline__ uint4 ld_cells(const void *p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Position of 16-byte chunk `chunk` (0..15) inside a warp's 256-byte activation slot: the four
// chunks that the four reading lanes fetch together (64 bytes apart) land on different banks.
__device__ __forceinline__ uint32_t x_chunk_pos(uint32_t chunk) {
  const uint32_t kc = chunk >> 2, m = chunk & 3u;
  return kc * 4u + (m ^ (kc >> 1));
}

// One row with the reference's scalar arithmetic, from global memory (rare: see ue4m3x2_to_f32).
template <int XKIND>
__device__ __noinline__ float exact_row(const GemvParams &p, uint32_t mat, uint32_t row, float global) {
  const uint32_t K = p.K, groups = K / 16u;
  const size_t sf_inner = q36::round_up(groups, 4);
  const uint8_t *wrow = p.w[mat] + static_cast<size_t>(row) * (K / 2u);
  float sum = 0.f;
  for (uint32_t g = 0; g < groups; ++g) {
    float scale = q36::decode_e4m3(p.sf[mat][q36::sf_offset(g, row, sf_inner)]);
    float local = 0.f;
    for (uint32_t i = 0; i < 8u; ++i) {
      const uint32_t byte = wrow[g * 8u + i];
      float x0, x1;
      if (XKIND == 0) {
        const __nv_bfloat16 *x = static_cast<const __nv_bfloat16 *>(p.x);
        x0 = __bfloat162float(x[g * 16u + 2u * i]);
        x1 = __bfloat162float(x[g * 16u + 2u * i + 1u]);
      } else {
        const uint32_t xb = static_cast<const uint8_t *>(p.x)[g * 8u + i];
        x0 = q36::e2m1_value(xb);
        x1 = q36::e2m1_value(xb >> 4);
      }
      local = fmaf(x0, q36::e2m1_value(byte), local);
      local = fmaf(x1, q36::e2m1_value(byte >> 4), local);
    }
    if (XKIND == 0) scale = __fmul_rn(scale, global);
    else scale = __fmul_rn(scale, q36::decode_e4m3(p.x_sf[q36::sf_offset(g, 0, sf_inner)]));
    sum = fmaf(local, scale, sum);
  }
  return XKIND == 0 ? sum : sum * global;
}

// Work decomposition.  A unit (32 rows over all of K) is cut along K into `cpu` chunks of `chunk`
// stages (the last one may be shorter); the chunk boundaries depend on K alone.  An ITEM is one
// chunk of one unit; items are numbered chunk-major (all units' chunk 0, then chunk 1, ...) and
// every CTA takes a contiguous range of them holding 1/grid of the launch's stages.  So every CTA
// streams the same number of bytes whatever the matrix shape (two CTAs per SM: every SM too),
// and a CTA touches few distinct K-chunks, of which alone it stages the activations.
struct Item {
  uint32_t unit, kc, it0, nit;        // global unit, chunk index, first stage, stages
  uint32_t mat, lu, rb, r0;           // matrix, unit inside it, 128-row block, first q-row of the unit
};
__device__ __forceinline__ Item decode_item(const GemvParams &p, uint32_t j) {
  Item t;
  t.kc = j / p.units;
  t.unit = j - t.kc * p.units;
  t.it0 = t.kc * p.chunk;
  t.nit = min(p.chunk, p.iters - t.it0);
  uint32_t mat = 0, first = 0;
  while (mat + 1u < p.count && t.unit >= p.unit_end[mat]) { first = p.unit_end[mat]; ++mat; }
  t.mat = mat;
  t.lu = t.unit - first;
  t.rb = t.lu >> 2;
  t.r0 = (t.lu & 3u) * 8u;
  return t;
}
// Units that stay whole (cpu == 1) are dealt round-robin instead: item k of CTA b is unit b + k * grid,
// so that the CTAs running at the same time read neighbouring rows (measured faster than one
// contiguous band per CTA); the grid is then sized so that every CTA gets the same number of units.
// Items [begin, end) of CTA b otherwise: boundaries at b / grid of the launch's stages, rounded down
// to an item.
__device__ __forceinline__ uint32_t item_at(const GemvParams &p, uint32_t b, uint32_t grid) {
  if (b >= grid) return p.units * p.cpu;
  const uint32_t last = p.iters - (p.cpu - 1u) * p.chunk;
  const uint64_t total = static_cast<uint64_t>(p.units) * p.iters;
  const uint64_t full_part = static_cast<uint64_t>(p.cpu - 1u) * p.units * p.chunk;
  const uint64_t pos = total * b / grid;
  return pos < full_part ? static_cast<uint32_t>(pos / p.chunk)
                         : (p.cpu - 1u) * p.units + static_cast<uint32_t>((pos - full_part) / last);
}

__device__ __forceinline__ uint32_t atom_add_acq_rel_gpu(uint32_t *p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}

// XKIND 0: x is a bf16 vector.  XKIND 1: x is one NVFP4-quantised activation row.
template <int XKIND, bool PEER>
__global__ void __launch_bounds__(kBlock, 2)
nvfp4_gemv_mma_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  // the swizzled boxes need 1024-byte aligned stages
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);                 // [kStages]
  uint64_t *empty = full + kStages;                                    // [kStages]
  uint64_t *red_full = empty + kStages;                                // [kRed]
  uint64_t *red_empty = red_full + kRed;                               // [kRed]
  static_assert((2 * kStages + 2 * kRed) * sizeof(uint64_t) <= 128, "barriers overlap the header fields");
  uint4 *zero_chunk = reinterpret_cast<uint4 *>(smem + 128);           // 16 bytes of zeros
  uint32_t *peer_fail = reinterpret_cast<uint32_t *>(smem + 160);      // [kWarps] 1 = this warp's wait for a peer ran out
  float *slice_inv = reinterpret_cast<float *>(smem + 256);            // [kMaxChunks][kWarps] inverse scale of a warp's x slice
  static_assert(256 + kMaxChunks * kWarps * sizeof(float) <= 1024, "slice scales overlap the partial sums");
  float *red = reinterpret_cast<float *>(smem + 1024);                 // [kRed][kWarps][32] partial row sums
  static_assert(1024 + kRed * kWarps * 32 * sizeof(float) <= kHeaderBytes, "partial sums overlap the ring");
  uint8_t *ring = smem + kHeaderBytes;
  uint8_t *xs = ring + kRingBytes;                                     // [kWarps][iters][256 B] float16 activations

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t iters = p.iters;
  const bool strided = p.cpu == 1u;
  const uint32_t j_begin = strided ? blockIdx.x : item_at(p, blockIdx.x, gridDim.x);
  const uint32_t j_end = strided ? p.units : item_at(p, blockIdx.x + 1u, gridDim.x);
  const uint32_t j_step = strided ? gridDim.x : 1u;

  if (threadIdx.x == 0) Q36_TRACE(0);
  if (warp == kWarpProducer) {
    // ------------------------------------------------------------------ producer warp
    // It owns the barriers: initialises them, signals the others through a named barrier it does
    // not wait on, and starts streaming at once (weights do not depend on the kernel that
    // produced x).
    if (lane < kStages) { mbar_init(&full[lane], 1); mbar_init(&empty[lane], kWarps); }
    if (lane < kRed) { mbar_init(&red_full[lane], kWarps); mbar_init(&red_empty[lane], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("bar.arrive 2, %0;" ::"n"(kBlock) : "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (lane == 0 && j_begin < j_end) {
      // Run-ahead cursor: asks L2 for the boxes the ring will want `kAhead` stages later.  The ring
      // itself is full long before x is ready (that is the point of streaming early); without the
      // run-ahead HBM would idle from then until the first stage is released.  With it the next
      // stages are already in L2 when the consumers start, and they work them off faster than HBM
      // could deliver them.
      uint32_t pf_j = j_begin, pf_issued = 0;
      Item pf = decode_item(p, pf_j);
      uint32_t pf_it = pf.it0;
      auto prefetch_one = [&]() {
        if (pf_j >= j_end) return;
        tma_prefetch_5d(&p.map_w[pf.mat], 0u, pf.r0, 0u, pf_it * 4u, pf.rb);
        tma_prefetch_3d(&p.map_sf[pf.mat], pf.r0 * 4u, pf_it * 16u, pf.rb);
        ++pf_issued;
        if (++pf_it == pf.it0 + pf.nit && (pf_j += j_step) < j_end) { pf = decode_item(p, pf_j); pf_it = pf.it0; }
      };
      uint32_t g = 0;
      for (uint32_t j = j_begin; j < j_end; j += j_step) {
        const Item t = decode_item(p, j);
        for (uint32_t it = t.it0; it < t.it0 + t.nit; ++it, ++g) {
          const uint32_t stage = g % kStages, phase = (g / kStages) & 1u;
          if (kAhead != 0u && g >= kStages)                  // the ring is full: keep L2 `kAhead` stages ahead
            while (pf_issued < g + kAhead + 1u && pf_j < j_end) prefetch_one();
          if (!mbar_wait(&empty[stage], phase ^ 1u)) return;
          uint8_t *dst = ring + stage * kStageBytes;
          mbar_expect_tx(&full[stage], kStageBytes);        // whole boxes; columns past K arrive as zeros
          tma_load_5d(dst, &p.map_w[t.mat], 0u, t.r0, 0u, it * 4u, t.rb, &full[stage]);
          tma_load_3d(dst + kStageW, &p.map_sf[t.mat], t.r0 * 4u, it * 16u, t.rb, &full[stage]);
          if (kAhead != 0u && pf_issued <= g) prefetch_one();   // cursor never falls behind the loads (skips what they fetched)
          if (g == 0) Q36_TRACE(1);
        }
      }
      Q36_TRACE(2);
    }
    return;
  }

  if (warp == kWarpEpilogue) {
    // ------------------------------------------------------------------ epilogue warp
    // Takes the eight warps' partial row sums of an item out of shared memory, so that the
    // consumers go straight on to the next item.  Lane = row of the unit.  A unit that was cut
    // along K meets in global memory: every chunk's 32 sums are parked there, a ticket per unit
    // tells the last chunk to arrive, and that one adds them in chunk order (the order of
    // arrival plays no part in the result).
    asm volatile("griddepcontrol.wait;" ::: "memory");        // outputs and scratch may still be in use by the grid before
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("bar.sync 2, %0;" ::"n"(kBlock) : "memory");
    // tensor-parallel form: lane L stores cell pair L / 4 (four consecutive rows) to ranks L % 4 and L % 4 + 4
    uint8_t *peer_lo = nullptr, *peer_hi = nullptr;
    bool poisoned = false;
    uint32_t call = 0;
    if (PEER) {
      if ((lane & 3u) < p.world) peer_lo = p.peer_arena[lane & 3u];
      if ((lane & 3u) + 4u < p.world) peer_hi = p.peer_arena[(lane & 3u) + 4u];
      call = *reinterpret_cast<const volatile uint32_t *>(p.state + p.out_slot * 4u) + 1u;
#pragma unroll
      for (uint32_t w = 0; w < static_cast<uint32_t>(kWarps); ++w) poisoned |= peer_fail[w] != 0u;
    }
    // [units][cpu][32] parked partial sums of units cut along K, (float, launch tag) per cell; [units] tickets
    unsigned long long *const scratch = g_scratch + static_cast<size_t>(p.set) * kScratchCells;
    uint32_t *const tickets = g_tickets + static_cast<size_t>(p.set) * kTicketWords;
    float gscale[kMaxMats];
#pragma unroll
    for (uint32_t i = 0; i < kMaxMats; ++i)
      gscale[i] = XKIND == 0 ? ((i < p.count && p.tensor_scale[i] != nullptr) ? __ldg(p.tensor_scale[i]) : 1.0f) : p.alpha;
    bool dead = false;
    // Writes a unit's 32 rows: v = the row sums before the tensor scale.
    auto write_rows = [&](const Item &t, float v) {
      const uint32_t row = (t.lu >> 2) * 128u + (t.lu & 3u) * 8u + (lane & 7u) + 32u * (lane >> 3);
      float global = gscale[0];
#pragma unroll
      for (uint32_t i = 1; i < kMaxMats; ++i) global = t.mat == i ? gscale[i] : global;
      v *= global;
      if (v != v && !dead) v = exact_row<XKIND>(p, t.mat, row, global);
      if (!PEER) {
        p.y[t.mat][row] = __float2bfloat16(v);
      } else {
        if (poisoned || dead) v = __uint_as_float(0x7fc00000u);
        const uint32_t bits = __bfloat16_as_ushort(__float2bfloat16(v));
        const uint32_t pair = bits | (__shfl_down_sync(0xffffffffu, bits, 1) << 16);      // even lanes: rows 2i, 2i + 1
        const uint32_t d0 = __shfl_sync(0xffffffffu, pair, lane & 28u), d1 = __shfl_sync(0xffffffffu, pair, (lane & 28u) + 2u);
        // lanes 4c .. 4c + 3 hold four consecutive rows: (4c & 7) + 32 (4c >> 3) of the unit
        const uint32_t row4 = (t.lu >> 2) * 128u + (t.lu & 3u) * 8u + (lane & 4u) + 32u * (lane >> 3);
        const size_t at = p.y_off[t.mat] + (static_cast<size_t>(p.row_off[t.mat]) + row4) * 4u;
        if (peer_lo != nullptr) st_cells(peer_lo + at, d0, d1, call);
        if (peer_hi != nullptr) st_cells(peer_hi + at, d0, d1, call);
      }
    };
    // A unit cut along K: every chunk takes a ticket of the unit when its CTA turns to it, and the
    // chunk that took the last one adds the unit up, in chunk order, once its own sums are there.
    // The others park theirs in global memory as 8-byte cells (value, launch tag).  Nothing orders
    // a parked cell before anything else: the reader looks again until the tag is there (its owner
    // took its ticket earlier, so it is at most about one item behind), and then wipes the cell
    // for the next launch that gets this scratch set.  The ticket is taken one item ahead, so its
    // round trip to L2 runs under the wait for the item's sums.
    auto add_up = [&](const Item &t, float own) {
      unsigned long long *parked = scratch + static_cast<size_t>(t.unit) * p.cpu * 32u + lane;
      float v = 0.f;
      for (uint32_t k0 = 0; k0 < p.cpu; k0 += 4u) {
        unsigned long long cell[4] = {0ull, 0ull, 0ull, 0ull};
        for (uint32_t spin = 0;; ++spin) {
#pragma unroll
          for (uint32_t i = 0; i < 4u; ++i)             // all loads first: one round trip
            if (k0 + i < p.cpu && k0 + i != t.kc)
              asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(cell[i]) : "l"(parked + (k0 + i) * 32u) : "memory");
          bool ok = true;
#pragma unroll
          for (uint32_t i = 0; i < 4u; ++i)
            ok = ok && (k0 + i >= p.cpu || k0 + i == t.kc || static_cast<uint32_t>(cell[i] >> 32) == p.tag);
          if (__all_sync(0xffffffffu, ok)) break;
          if (spin >= kParkSpinLimit) { dead = true; atomicExch(&g_gemv_mma_error, 1u); break; }
          if (spin > 64u) __nanosleep(100);
        }
#pragma unroll
        for (uint32_t i = 0; i < 4u; ++i) {
          if (k0 + i >= p.cpu) continue;
          if (k0 + i == t.kc) { v += own; continue; }
          v += __uint_as_float(static_cast<uint32_t>(cell[i]));
          parked[(k0 + i) * 32u] = 0ull;
        }
      }
      if (lane == 0) tickets[t.unit] = 0;                   // ready for the next launch that gets this scratch
      write_rows(t, v);
    };
    uint32_t next_ticket = 0;
    if (p.cpu > 1u && j_begin < j_end && lane == 0) next_ticket = atomicAdd(tickets + j_begin % p.units, 1u);
    uint32_t n_local = 0;
    for (uint32_t j = j_begin; j < j_end; j += j_step, ++n_local) {
      const Item t = decode_item(p, j);
      const uint32_t ticket = next_ticket;
      const uint32_t slot = n_local % kRed, ph = (n_local / kRed) & 1u;
      if (!dead && !mbar_wait(&red_full[slot], ph)) dead = true;
      const float *buf = red + slot * (kWarps * 32u);
      const float *inv = slice_inv + t.kc * kWarps;
      float v = 0.f;
#pragma unroll
      for (uint32_t w = 0; w < static_cast<uint32_t>(kWarps); ++w) v = fmaf(buf[w * 32u + lane], inv[w], v);
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_empty[slot]);
      if (p.cpu == 1u) {
        write_rows(t, v);
        continue;
      }
      if (j + 1u < j_end && lane == 0) next_ticket = atomicAdd(tickets + (j + 1u) % p.units, 1u);
      if (__shfl_sync(0xffffffffu, ticket, 0) == p.cpu - 1u) {
        add_up(t, v);
      } else {
        const unsigned long long cell = (static_cast<unsigned long long>(p.tag) << 32) | __float_as_uint(v);
        asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(scratch + (static_cast<size_t>(t.unit) * p.cpu + t.kc) * 32u + lane), "l"(cell) : "memory");
      }
    }
    if (threadIdx.x == kWarpEpilogue * 32u) Q36_TRACE(7);
    if (PEER && lane == 0u) {
      // The last CTA of the launch advances the slot's call number.  Nothing here orders the stores
      // above: the cells order themselves.
      uint32_t *st = p.state + p.out_slot * 4u;
      if (poisoned || dead) atomicCAS(&st[2], 0u, call);
      if (atomicAdd(&st[1], 1u) == gridDim.x - 1u) {
        st[1] = 0;
        *reinterpret_cast<volatile uint32_t *>(&st[0]) = call;
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  if (threadIdx.x == 0) *zero_chunk = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) Q36_TRACE(3);
  bool dead = false;
  // Tensor-parallel form: x may be a flagged vector that the ranks are still delivering.  Its cells
  // must carry the number of the call that produced it; this rank's own producer ran earlier in
  // the stream, so its count of completed calls is that number.
  const bool flagged = PEER && p.in_slot != kNoSlot;
  uint32_t want = 0;
  if (flagged) want = *reinterpret_cast<const volatile uint32_t *>(p.state + p.in_slot * 4u);

  // Each warp stages the activations of ITS columns (128 of every 1024) as float16, alone, and only
  // for the K-chunks this CTA's items touch.
  uint8_t *xw = xs + warp * iters * 256u;
  const uint32_t kc_lo = j_begin < j_end ? j_begin / p.units : 1u, kc_hi = j_begin < j_end ? (j_end - 1u) / p.units : 0u;
  for (uint32_t kc = kc_lo; kc <= kc_hi; ++kc) {
    const uint32_t it0 = kc * p.chunk, it_end = min(it0 + p.chunk, iters);
    if (XKIND == 0) {
      // bf16 -> float16 times a power of two that brings the slice's max|x| into [2^14, 2^15):
      // products with e2m1 weights stay exact, values more than 2^-38 below the maximum flush (far
      // below the float32 accumulation error); the inverse scale is applied to the warp's partial sum.
      // A pass of the warp covers two stages (16 lanes x 8 values each).  Four passes' loads go out
      // together; the bf16 values are parked in the warp's own float16 slot (same size) until the
      // chunk's maximum is known, then every lane converts what it parked.
      constexpr uint32_t kBatch = 4;
      const uint8_t *xc = static_cast<const uint8_t *>(p.x);
      uint32_t m2 = 0;
      for (uint32_t base = it0; base < it_end; base += 2u * kBatch) {
        uint4 v[kBatch];
        uint32_t its[kBatch];
        bool real[kBatch];
#pragma unroll
        for (uint32_t ps = 0; ps < kBatch; ++ps) {
          its[ps] = base + 2u * ps + (lane >> 4);
          real[ps] = its[ps] < it_end && its[ps] * 1024u + warp * 128u + (lane & 15u) * 8u < p.K;
        }
        if (!flagged) {
          const uint4 *xg = static_cast<const uint4 *>(p.x);
#pragma unroll
          for (uint32_t ps = 0; ps < kBatch; ++ps)
            v[ps] = real[ps] ? __ldcg(xg + (its[ps] * 1024u + warp * 128u) / 8u + (lane & 15u)) : make_uint4(0u, 0u, 0u, 0u);   // L2: x may be fresh
        } else {
          // Flagged cells: 16 bytes carry four values, so a lane's eight values are two loads.  All of
          // the batch's loads are issued before the first comparison (one round trip where everything
          // has arrived); the set is read again while any cell still carries an older call number.
          for (uint32_t attempt = 0; !dead; ++attempt) {
            uint4 ca[kBatch], cb[kBatch];
#pragma unroll
            for (uint32_t ps = 0; ps < kBatch; ++ps) {
              ca[ps] = cb[ps] = make_uint4(0u, want, 0u, want);
              if (real[ps]) {
                const uint8_t *src = xc + (static_cast<size_t>(its[ps]) * 1024u + warp * 128u + (lane & 15u) * 8u) * 4u;
                ca[ps] = ld_cells(src);
                cb[ps] = ld_cells(src + 16u);
              }
            }
            bool ok = true;
#pragma unroll
            for (uint32_t ps = 0; ps < kBatch; ++ps) {
              ok = ok && ca[ps].y == want && ca[ps].w == want && cb[ps].y == want && cb[ps].w == want;
              v[ps] = make_uint4(ca[ps].x, ca[ps].z, cb[ps].x, cb[ps].z);
            }
            if (__all_sync(0xffffffffu, ok)) break;
            if (attempt >= kPeerSpinLimit) dead = true;
            else if (attempt > kPeerEagerPolls) __nanosleep(200);
          }
        }
#pragma unroll
        for (uint32_t ps = 0; ps < kBatch; ++ps) {
          if (dead) v[ps] = make_uint4(0u, 0u, 0u, 0u);
          m2 = max_u16x2(m2, max_u16x2(max_u16x2(v[ps].x & 0x7fff7fffu, v[ps].y & 0x7fff7fffu),
                                       max_u16x2(v[ps].z & 0x7fff7fffu, v[ps].w & 0x7fff7fffu)));
          if (its[ps] < it_end) *reinterpret_cast<uint4 *>(xw + its[ps] * 256u + x_chunk_pos(lane & 15u) * 16u) = v[ps];
        }
      }
      const uint32_t mx = __reduce_max_sync(0xffffffffu, max(m2 & 0xffffu, m2 >> 16));
      const uint32_t e = (mx >> 7) & 0xffu;
      const int shift = e == 255u ? 0 : (e < 15u ? 126 : 141 - static_cast<int>(e));
      const float up = __uint_as_float(static_cast<uint32_t>(127 + shift) << 23);
      if (lane == 0) slice_inv[kc * kWarps + warp] = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
      for (uint32_t it = it0 + (lane >> 4); it < it_end; it += 2u) {
        uint4 *slot = reinterpret_cast<uint4 *>(xw + it * 256u + x_chunk_pos(lane & 15u) * 16u);
        const uint4 raw = *slot;
        const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
        __half2 h[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
          h[q] = __floats2half2_rn(__uint_as_float(wv[q] << 16) * up, __uint_as_float(wv[q] & 0xffff0000u) * up);
        *slot = *reinterpret_cast<uint4 *>(h);
      }
    } else {
      // e2m1 * ue4m3 is exact in float16 (at most 7 significant bits, magnitudes 2^-10 .. 2688).
      const uint8_t *xb = static_cast<const uint8_t *>(p.x);
      const uint32_t sub = lane & 7u;                                     // one 16-value group per lane
      for (uint32_t it = it0 + (lane >> 3); it < it_end; it += 4u) {
        const uint32_t col = it * 1024u + warp * 128u + sub * 16u;
        uint2 codes = make_uint2(0u, 0u);
        uint32_t sbyte = 0;
        if (col < p.K) {
          codes = __ldcg(reinterpret_cast<const uint2 *>(xb + col / 2u));
          const uint32_t grp = col / 16u;
          sbyte = __ldcg(p.x_sf + static_cast<size_t>(grp >> 2) * 512u + (grp & 3u));
        }
        const __half_raw sraw = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(sbyte), __NV_E4M3);
        const __half2 s2 = __half2half2(*reinterpret_cast<const __half *>(&sraw));
        uint32_t lo[4], hi[4];
        e2m1x8_to_h2(codes.x, lo);
        e2m1x8_to_h2(codes.y, hi);
        __half2 h[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          h[q] = __hmul2(*reinterpret_cast<__half2 *>(&lo[q]), s2);
          h[4 + q] = __hmul2(*reinterpret_cast<__half2 *>(&hi[q]), s2);
        }
        uint4 *dst = reinterpret_cast<uint4 *>(xw + it * 256u);
        dst[x_chunk_pos(sub * 2u)] = *reinterpret_cast<uint4 *>(&h[0]);
        dst[x_chunk_pos(sub * 2u + 1u)] = *reinterpret_cast<uint4 *>(&h[4]);
      }
      if (lane == 0) slice_inv[kc * kWarps + warp] = 1.0f;
    }
  }
  if (PEER) {
    dead = __any_sync(0xffffffffu, dead);
    if (dead) atomicExch(&g_gemv_mma_error, 2u);
    if (lane == 0) peer_fail[warp] = dead ? 1u : 0u;
  }
  // Meets the producer's arrival (barriers initialised); also publishes the slice scales and the zero chunk.
  asm volatile("bar.sync 2, %0;" ::"n"(kBlock) : "memory");
  if (threadIdx.x == 0) Q36_TRACE(4);

  // Fragment geometry.  Lane (r = lane / 4, c = lane % 4) of the MMA holds weight rows r and r + 8 of a
  // 16-row tile.  Tile t of a unit is {rows q + 32 (2t), q + 32 (2t + 1)}, q < 8, and MMA row r maps
  // to q = (r >> 1) | ((r & 1) << 2): with the 128-byte swizzle of the TMA box (chunk ^= q) the eight
  // lanes of a quarter warp then read eight different 16-byte bank groups.
  const uint32_t r = lane >> 2, c = lane & 3u;
  const uint32_t q = (r >> 1) | ((r & 1u) << 2);
  const uint32_t kcol = warp >> 1, ch = (warp & 1u) * 4u + c;
  const uint32_t w_off = (kcol * 32u + q) * 128u + ((ch ^ q) << 4);      // + j * 1024
  const uint32_t tile = 2u * warp + (c & 1u);                            // scale tile of this lane's groups
  const uint32_t sf_off = kStageW + tile * 128u + ((q ^ (tile & 7u)) << 4);
  // B operand: only lanes with r == c carry activations (k-slots of lane c, column c); the rest read zeros.
  const bool x_active = r == c;
  const uint8_t *x_base = x_active ? xw : reinterpret_cast<const uint8_t *>(zero_chunk);
  const uint32_t x_stride = x_active ? 256u : 0u;
  uint32_t x_pos[4];
#pragma unroll
  for (uint32_t m = 0; m < 4u; ++m) x_pos[m] = x_active ? x_chunk_pos(c * 4u + m) * 16u : 0u;

  uint32_t g = 0, n_local = 0;
  bool stalled = false;
  for (uint32_t j = j_begin; j < j_end; j += j_step, ++n_local) {
    const uint32_t kc = j / p.units;
    const uint32_t it0 = kc * p.chunk, it_end = min(it0 + p.chunk, iters);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};                                 // rows q + 32 j, j = 0..3
    for (uint32_t it = it0; it < it_end; ++it, ++g) {
      const uint32_t stage = g % kStages, phase = (g / kStages) & 1u;
      // A wait that gives up (never seen in practice) only stops the arithmetic: the warp keeps
      // walking its stages and barriers so that nobody else is left waiting for it.
      if (!stalled && !mbar_wait(&full[stage], phase)) stalled = true;
      if (threadIdx.x == 0 && g == 0) Q36_TRACE(5);
      if (!stalled) {
        const uint8_t *st = ring + stage * kStageBytes;
        uint4 bx[4];
#pragma unroll
        for (uint32_t m = 0; m < 4u; ++m) bx[m] = *reinterpret_cast<const uint4 *>(x_base + it * x_stride + x_pos[m]);
        const uint4 sq = *reinterpret_cast<const uint4 *>(st + sf_off);
        const uint32_t sw[4] = {sq.x, sq.y, sq.z, sq.w};                 // scale bytes [j][group 0..3 of the tile]
#pragma unroll
        for (uint32_t t = 0; t < 2u; ++t) {
          const uint4 wa = *reinterpret_cast<const uint4 *>(st + w_off + (2u * t) * 1024u);
          const uint4 wb = *reinterpret_cast<const uint4 *>(st + w_off + (2u * t + 1u) * 1024u);
          const uint32_t wav[4] = {wa.x, wa.y, wa.z, wa.w}, wbv[4] = {wb.x, wb.y, wb.z, wb.w};
          float de[4] = {0.f, 0.f, 0.f, 0.f}, dod[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (uint32_t m = 0; m < 4u; ++m) {                             // 8 weights of each row per word
            uint32_t ha[4], hb[4];
            e2m1x8_to_h2(wav[m], ha);
            e2m1x8_to_h2(wbv[m], hb);
            if (m < 2u) {
              mma_f16(de, ha[0], hb[0], ha[1], hb[1], bx[m].x, bx[m].y);
              mma_f16(de, ha[2], hb[2], ha[3], hb[3], bx[m].z, bx[m].w);
            } else {
              mma_f16(dod, ha[0], hb[0], ha[1], hb[1], bx[m].x, bx[m].y);
              mma_f16(dod, ha[2], hb[2], ha[3], hb[3], bx[m].z, bx[m].w);
            }
          }
          // D columns 2c, 2c + 1 of lanes c < 2: groups 4c .. 4c + 3 of the warp's eight, i.e. scale tile
          // 2 warp + c, bytes [j][0..3].
          const float2 s01a = ue4m3x2_to_f32(sw[2u * t] & 0xffffu), s23a = ue4m3x2_to_f32(sw[2u * t] >> 16);
          const float2 s01b = ue4m3x2_to_f32(sw[2u * t + 1u] & 0xffffu), s23b = ue4m3x2_to_f32(sw[2u * t + 1u] >> 16);
          float a0 = acc[2u * t], a1 = acc[2u * t + 1u];
          a0 = fmaf(de[0], s01a.x, a0); a0 = fmaf(dod[0], s01a.y, a0);
          a0 = fmaf(de[1], s23a.x, a0); a0 = fmaf(dod[1], s23a.y, a0);
          a1 = fmaf(de[2], s01b.x, a1); a1 = fmaf(dod[2], s01b.y, a1);
          a1 = fmaf(de[3], s23b.x, a1); a1 = fmaf(dod[3], s23b.y, a1);
          acc[2u * t] = a0; acc[2u * t + 1u] = a1;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
    }
    if (threadIdx.x == 0) Q36_TRACE(6);
    // Hand the item's sums to the epilogue warp.  Lanes c = 0 and c = 1 hold the two scale tiles of the
    // warp's columns; lanes c >= 2 hold zeros.
    const uint32_t slot = n_local % kRed, ph = (n_local / kRed) & 1u;
    if (!stalled && !mbar_wait(&red_empty[slot], ph ^ 1u)) stalled = true;
    float *buf = red + slot * (kWarps * 32u);
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      acc[jj] += __shfl_xor_sync(0xffffffffu, acc[jj], 1);
      if (c == 0u) buf[warp * 32u + static_cast<uint32_t>(jj) * 8u + q] = acc[jj];
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&red_full[slot]);
  }
}

// Unpacks a flagged vector of this rank's arena into plain bf16 once all of its cells carry the
// call number of `slot` (bounded wait; NaN where it ran out): for a consumer that is not one of
// these kernels.  One thread per four values.
__global__ void __launch_bounds__(256)
nvfp4_gemv_peer_collect_kernel(const uint8_t *cells, uint32_t *state, uint32_t slot, uint32_t n, __nv_bfloat16 *out) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t want = *reinterpret_cast<const volatile uint32_t *>(state + slot * 4u);
  const uint32_t i = (blockIdx.x * blockDim.x + threadIdx.x) * 4u;
  if (i >= n) return;
  uint2 v = make_uint2(0x7fc07fc0u, 0x7fc07fc0u);
  bool ok = false;
  for (uint32_t spin = 0; spin < kPeerSpinLimit && !ok; ++spin) {
    const uint4 c = ld_cells(cells + static_cast<size_t>(i) * 4u);
    if (c.y == want && c.w == want) { v = make_uint2(c.x, c.z); ok = true; }
    else if (spin > kPeerEagerPolls) __nanosleep(200);
  }
  if (!ok) {
    atomicExch(&g_gemv_mma_error, 2u);
    atomicCAS(&state[slot * 4u + 2u], 0u, want);
  }
  *reinterpret_cast<uint2 *>(out + i) = v;
}

// ---- host side ---------------------------------------------------------------------------------

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

// Tensor maps depend only on (pointer, rows, K): a decode loop asks for the same few hundred pairs
// on every token, so they are kept in a small direct-mapped cache instead of being encoded per call.
struct MapEntry {
  const void *w = nullptr, *sf = nullptr;
  uint64_t n = 0, k = 0;
  CUtensorMap map_w, map_sf;
};
constexpr size_t kMapCacheSize = 1024;
std::mutex g_map_mu;
MapEntry g_map_cache[kMapCacheSize];

bool encode_maps(const void *w, const void *sf, uint64_t N, uint64_t K, CUtensorMap *map_w, CUtensorMap *map_sf) {
  EncodeFn enc = encode_fn();
  if (enc == nullptr) return false;
  const uint64_t row_bytes = K / 2, blocks = N / 128, tiles = K / 64;
  const cuuint32_t ones[5] = {1, 1, 1, 1, 1};
  {   // weights as uint32 [blocks][K/256 column chunks][4 j][32 q][32 words = 128 B]
    const cuuint64_t dims[5] = {32, 32, 4, K / 256, blocks};
    const cuuint64_t strides[4] = {row_bytes, 32 * row_bytes, 128, 128 * row_bytes};
    const cuuint32_t box[5] = {32, 8, 4, 4, 1};
    if (enc(map_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 5, const_cast<void *>(w), dims, strides, box, ones,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  {   // scales as uint32 [blocks][tiles][128 words = one 512-byte tile]
    const cuuint64_t dims[3] = {128, tiles, blocks};
    const cuuint64_t strides[2] = {512, tiles * 512};
    const cuuint32_t box[3] = {32, 16, 1};
    if (enc(map_sf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void *>(sf), dims, strides, box, ones,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  return true;
}

bool get_maps(const void *w, const void *sf, uint64_t N, uint64_t K, CUtensorMap *map_w, CUtensorMap *map_sf) {
  const uint64_t h = (reinterpret_cast<uintptr_t>(w) >> 8) * 0x9E3779B97F4A7C15ull ^ (N * 31u + K);
  MapEntry &e = g_map_cache[(h >> 20) % kMapCacheSize];
  {
    std::lock_guard<std::mutex> lock(g_map_mu);
    if (e.w == w && e.sf == sf && e.n == N && e.k == K) {
      *map_w = e.map_w;
      *map_sf = e.map_sf;
      return true;
    }
  }
  if (!encode_maps(w, sf, N, K, map_w, map_sf)) return false;
  std::lock_guard<std::mutex> lock(g_map_mu);
  e.w = w; e.sf = sf; e.n = N; e.k = K;
  e.map_w = *map_w;
  e.map_sf = *map_sf;
  return true;
}

#ifdef Q36_GEMV_TRACE
std::atomic<uint32_t> g_trace_id{0};
#endif

// Parking area for the partial sums of units cut along K, and the per-unit tickets.  A launch
// touches its set only after the grid before it on its stream has completed, so the launches of
// one stream can share a set; every stream that launches through this file gets a set of its own,
// up to kPoolSets streams per process (further streams share by hash: callers that drive more
// than kPoolSets streams at once through these entry points must serialise the surplus).
struct ScratchSet {
  uint32_t set, tag;
};
std::atomic<uint32_t> g_pool_seq{0};
std::mutex g_pool_mu;
cudaStream_t g_pool_streams[kPoolSets];
uint32_t g_pool_streams_used = 0;

// The kernel addresses the sets itself (they are device globals), so nothing here touches the device:
// safe inside a stream capture, also as the first call of a process.
void scratch_for_launch(ScratchSet *out) {
  const cudaStream_t stream = q36::stream();
  uint32_t set = kPoolSets;
  {
    std::lock_guard<std::mutex> lock(g_pool_mu);
    for (uint32_t i = 0; i < g_pool_streams_used; ++i)
      if (g_pool_streams[i] == stream) set = i;
    if (set == kPoolSets && g_pool_streams_used < kPoolSets) {
      set = g_pool_streams_used++;
      g_pool_streams[set] = stream;
    }
  }
  if (set == kPoolSets) set = static_cast<uint32_t>((reinterpret_cast<uintptr_t>(stream) >> 4) % kPoolSets);
  out->set = set;
  out->tag = g_pool_seq.fetch_add(1u) % 0xfffffffeu + 1u;
}

struct Mat {
  const uint8_t *w, *sf;
  __nv_bfloat16 *y;
  const float *tensor_scale;
  uint64_t n;
};

bool shape_ok(uint64_t n, uint64_t k) {
  return n != 0 && n % 128 == 0 && n < (1ull << 31) && k >= 256 && k % 256 == 0 && k <= kMaxK;
}

template <int XKIND, bool PEER = false>
int launch(const Mat *mats, uint32_t count, uint64_t K, const void *x, const uint8_t *x_sf, float alpha,
           const qwen36_nvfp4_matvec_peer_spec_t *peer = nullptr) {
  GemvParams p{};
  if (PEER) {
    p.peer_arena = as_ptr<uint8_t *const>(peer->peer_arena);
    p.state = as_ptr<uint32_t>(peer->state);
    p.world = static_cast<uint32_t>(peer->world);
    p.rank = static_cast<uint32_t>(peer->rank);
    p.out_slot = static_cast<uint32_t>(peer->out_slot);
    p.in_slot = peer->in_slot == QWEN36_PEER_INPUT_LOCAL ? kNoSlot : static_cast<uint32_t>(peer->in_slot);
    for (uint32_t i = 0; i < count; ++i) {
      p.row_off[i] = static_cast<uint32_t>(peer->row_offset[i]);
      p.y_off[i] = peer->output_offset_bytes[i];
    }
  }
  uint32_t units = 0;
  for (uint32_t i = 0; i < count; ++i) {
    if (!get_maps(mats[i].w, mats[i].sf, mats[i].n, K, &p.map_w[i], &p.map_sf[i])) return QWEN36_STATUS_NOT_IMPLEMENTED;
    p.w[i] = mats[i].w;
    p.sf[i] = mats[i].sf;
    p.y[i] = mats[i].y;
    p.tensor_scale[i] = mats[i].tensor_scale;
    units += static_cast<uint32_t>(mats[i].n / 32);
    p.unit_end[i] = units;
  }
  for (uint32_t i = count; i < kMaxMats; ++i) p.unit_end[i] = units;
  p.x = x;
  p.x_sf = x_sf;
  p.K = static_cast<uint32_t>(K);
  p.iters = static_cast<uint32_t>((K + 1023) / 1024);
  p.units = units;
  p.count = count;
  p.alpha = alpha;
#ifdef Q36_GEMV_TRACE
  p.trace_id = g_trace_id.fetch_add(1u);
#endif
  // K-chunks of at most kChunkStages stages, as even as the stage count allows; the cut depends on K alone,
  // so a row's sum is formed in the same order whatever the matrix height, grouping or GPU.
  p.cpu = (p.iters + kChunkStages - 1u) / kChunkStages;
  p.chunk = (p.iters + p.cpu - 1u) / p.cpu;
  p.cpu = (p.iters + p.chunk - 1u) / p.chunk;
  if (p.cpu > 1u) {
    ScratchSet set;
    if (static_cast<size_t>(units) * p.cpu * 32u > kScratchCells || units > kTicketWords) {
      p.cpu = 1u;                          // too tall for the parking area: whole units, one CTA each
      p.chunk = p.iters;
    } else {
      scratch_for_launch(&set);
      p.set = set.set;
      p.tag = set.tag;
    }
  }
  const size_t smem = 1024 + kHeaderBytes + kRingBytes + static_cast<size_t>(p.iters) * 2048;
  if (q36::ensure_dynamic_smem(reinterpret_cast<const void *>(nvfp4_gemv_mma_kernel<XKIND, PEER>), 227 * 1024) != cudaSuccess)
    return QWEN36_STATUS_CUDA_ERROR;
  // One CTA per resident slot (two per SM while the activation vector leaves room), each with the
  // same share of the launch's stages; never more CTAs than items.
  const uint32_t per_sm = smem * 2 + 2048 <= 228u * 1024u ? 2u : 1u;
  const uint32_t cap = static_cast<uint32_t>(q36::sm_count_current_device()) * per_sm;
  const uint32_t items = units * p.cpu;
  const uint32_t passes = (units + cap - 1) / cap;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.cpu == 1u ? (units + passes - 1) / passes : (items < cap ? items : cap));
  cfg.blockDim = dim3(kBlock);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return q36::cuda_status(cudaLaunchKernelEx(&cfg, nvfp4_gemv_mma_kernel<XKIND, PEER>, p));
}

}  // namespace

namespace q36 {

int nvfp4_gemv_mma_bf16(const qwen36_nvfp4_matvec_spec_t *specs, size_t count) {
  if (count == 0 || count > kMaxMats) return QWEN36_STATUS_NOT_IMPLEMENTED;
  Mat mats[kMaxMats];
  const uint64_t K = specs[0].in_features;
  for (size_t i = 0; i < count; ++i) {
    const qwen36_nvfp4_matvec_spec_t &s = specs[i];
    if (s.in_features != K || s.input_bf16.ptr != specs[0].input_bf16.ptr || !shape_ok(s.out_features, K) ||
        ((s.input_bf16.ptr | s.weight_u8.ptr | s.block_scale_e4m3.ptr) & 15u) != 0)
      return QWEN36_STATUS_NOT_IMPLEMENTED;
    mats[i] = Mat{as_ptr<const uint8_t>(s.weight_u8), as_ptr<const uint8_t>(s.block_scale_e4m3),
                  as_ptr<__nv_bfloat16>(s.output_bf16), as_ptr<const float>(s.tensor_scale_f32), s.out_features};
  }
  return launch<0>(mats, static_cast<uint32_t>(count), K, as_ptr<const void>(specs[0].input_bf16), nullptr, 1.0f);
}

int nvfp4_gemv_mma_bf16_peer(const qwen36_nvfp4_matvec_spec_t *specs, size_t count,
                             const qwen36_nvfp4_matvec_peer_spec_t *peer) {
  if (count == 0 || count > kMaxMats) return QWEN36_STATUS_NOT_IMPLEMENTED;
  Mat mats[kMaxMats];
  const uint64_t K = specs[0].in_features;
  for (size_t i = 0; i < count; ++i) {
    const qwen36_nvfp4_matvec_spec_t &s = specs[i];
    if (s.in_features != K || s.input_bf16.ptr != specs[0].input_bf16.ptr || !shape_ok(s.out_features, K) ||
        ((s.input_bf16.ptr | s.weight_u8.ptr | s.block_scale_e4m3.ptr) & 15u) != 0)
      return QWEN36_STATUS_NOT_IMPLEMENTED;
    mats[i] = Mat{as_ptr<const uint8_t>(s.weight_u8), as_ptr<const uint8_t>(s.block_scale_e4m3), nullptr,
                  as_ptr<const float>(s.tensor_scale_f32), s.out_features};
  }
  return launch<0, true>(mats, static_cast<uint32_t>(count), K, as_ptr<const void>(specs[0].input_bf16), nullptr, 1.0f, peer);
}

int nvfp4_gemv_peer_collect(const qwen36_nvfp4_matvec_peer_spec_t *peer, size_t slot, size_t vector_offset_bytes,
                            size_t n, qwen36_device_ptr_t arena, qwen36_device_ptr_t out_bf16) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>((n / 4 + 255) / 256));
  cfg.blockDim = dim3(256);
  cfg.stream = q36::stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return q36::cuda_status(cudaLaunchKernelEx(&cfg, nvfp4_gemv_peer_collect_kernel,
                                             as_ptr<const uint8_t>(arena) + vector_offset_bytes, as_ptr<uint32_t>(peer->state),
                                             static_cast<uint32_t>(slot), static_cast<uint32_t>(n),
                                             as_ptr<__nv_bfloat16>(out_bf16)));
}

int nvfp4_gemv_mma_fp4(const qwen36_nvfp4_gemm_spec_t *s, float alpha) {
  if (s->n != 1 || !shape_ok(s->m, s->k) || ((s->a_fp4.ptr | s->a_scale.ptr) & 15u) != 0 || (s->b_fp4.ptr & 7u) != 0)
    return QWEN36_STATUS_NOT_IMPLEMENTED;
  const Mat mat{as_ptr<const uint8_t>(s->a_fp4), as_ptr<const uint8_t>(s->a_scale), as_ptr<__nv_bfloat16>(s->c_bf16),
                nullptr, s->m};
  return launch<1>(&mat, 1u, s->k, as_ptr<const void>(s->b_fp4), as_ptr<const uint8_t>(s->b_scale), alpha);
}

}  // namespace q36

#ifdef Q36_GEMV_TRACE
// Copies the timestamp table [64 launches][320 CTAs][8 events] (u64 ns) to `dst` and rewinds the
// launch counter.  Synchronises.
extern "C" int qwen36_nvfp4_gemv_trace_read(void *dst) {
  g_trace_id.store(0);
  return cudaMemcpyFromSymbol(dst, g_trace, sizeof(g_trace)) == cudaSuccess ? 0 : -1;
}
#endif

// 1 when a bounded wait inside the tensor-core GEMV pipeline ever gave up (a stage never arrived;
// the kernel then returns without finishing its rows), 2 when a wait for a peer's flag ran out in
// the tensor-parallel form (rows poisoned).  Sticky until reset.  Reads device memory: synchronises.
extern "C" int qwen36_nvfp4_gemv_mma_last_error(void) {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemv_mma_error, sizeof(v)) != cudaSuccess) return -1;
  return static_cast<int>(v);
}

extern "C" int qwen36_nvfp4_gemv_mma_reset_error(void) {
  const unsigned int v = 0;
  return cudaMemcpyToSymbol(g_gemv_mma_error, &v, sizeof(v)) == cudaSuccess ? 0 : -1;
}
