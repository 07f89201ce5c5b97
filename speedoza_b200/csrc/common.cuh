// Shared helpers of the sm_100a kernel library: status codes, pointer casts,
// the ambient stream, and the NVFP4 / UE4M3 codecs whose rounding rules the
// whole path depends on.  Citations name files of the reference project.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
#include <mutex>
#include <utility>
#include <vector>
#endif

#include "../../include/qwen36_fp4_b200.h"

namespace q36 {

template <typename T>
static inline T *as_ptr(qwen36_device_ptr_t p) {
  return reinterpret_cast<T *>(static_cast<uintptr_t>(p.ptr));
}

static inline int cuda_status(cudaError_t e) {
  return e == cudaSuccess ? QWEN36_STATUS_SUCCESS : QWEN36_STATUS_CUDA_ERROR;
}

// Status of the launch just issued (no synchronisation), as the reference's
// entry points report it (e.g. kernels-cuda/ops.cu:1178-1179).
static inline int launch_status() { return cuda_status(cudaGetLastError()); }

// The stream every launch goes to (runtime.cu).
static inline cudaStream_t stream() {
  return reinterpret_cast<cudaStream_t>(qwen36_internal_active_stream());
}

// Opts a kernel in to `bytes` of dynamic shared memory (more than the 48 KB default).  The
// attribute belongs to the (kernel, device) pair, so it is set once per pair: a process that drives
// several GPUs gets it on each of them.
inline cudaError_t ensure_dynamic_smem(const void *kernel, int bytes) {
  static std::mutex mu;
  static std::vector<std::pair<const void *, int>> done;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  std::lock_guard<std::mutex> lock(mu);
  for (const auto &e : done)
    if (e.first == kernel && e.second == dev) return cudaSuccess;
  err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (err == cudaSuccess) done.emplace_back(kernel, dev);
  return err;
}

// Multiprocessor count of the current device (cached per device ordinal).
inline int sm_count_current_device() {
  static std::mutex mu;
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev >= 0 && dev < 64) {
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] > 0) return cached[dev];
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
  if (dev >= 0 && dev < 64) {
    std::lock_guard<std::mutex> lock(mu);
    cached[dev] = n;
  }
  return n;
}

__host__ __device__ static inline size_t div_ceil(size_t a, size_t b) { return (a + b - 1) / b; }
__host__ __device__ static inline size_t round_up(size_t a, size_t b) { return div_ceil(a, b) * b; }

// Tiled block-scale layout (kernels-cuda/ops.cu:64-79): 128 outer rows x 4
// inner groups form one 512-byte tile; inside it row r sits at
// (r % 32) * 16 + (r / 32) * 4 and the 4 groups are adjacent bytes.  Tiles of
// one 128-row block are contiguous along the inner (K) direction.  This is
// also the shared-memory image that a tcgen05.cp 32x128b.warpx4 copy turns
// into the TMEM scale-factor operand of a block-scaled MMA.
__host__ __device__ static inline size_t sf_offset(size_t inner, size_t outer, size_t sf_inner_dim) {
  const size_t tile = (inner / 4) + (outer / 128) * (sf_inner_dim / 4);
  const size_t r = outer % 128;
  return tile * 512 + (r % 32) * 16 + (r / 32) * 4 + (inner % 4);
}
__host__ __device__ static inline size_t sf_bytes(size_t inner_groups, size_t outer) {
  return div_ceil(outer, 128) * (round_up(inner_groups, 4) / 4) * 512;
}

// UE4M3 / E4M3 byte -> float, all 256 codes as the reference reads them
// (kernels-cuda/ops.cu:39-54): sign honoured, 0x7F and 0xFF are 448.
__host__ __device__ static inline float decode_e4m3(uint32_t code) {
  const uint32_t e = (code >> 3) & 15u, m = code & 7u;
  if ((code & 0x7fu) == 0u) return 0.0f;   // 0x80 reads as +0, as in the reference
  float v;
  if (e == 0) {
    v = static_cast<float>(m) * 0x1p-9f;
  } else if (e == 15u && m == 7u) {
    v = 448.0f;
  } else {
#ifdef __CUDA_ARCH__
    v = __uint_as_float(((e + 120u) << 23) | (m << 20));
#else
    union { uint32_t u; float f; } cvt;
    cvt.u = ((e + 120u) << 23) | (m << 20);
    v = cvt.f;
#endif
  }
  return (code & 0x80u) ? -v : v;
}

#ifdef __CUDACC__
// Positive float -> UE4M3 byte (kernels-cuda/ops.cu:81-117): ties on the
// normal grid round DOWN (+0x7FFFF before the shift), the subnormal grid uses
// floorf(v / 2^-9 + 0.49999994f) in float32, 448 and above clamp to 0x7E.
__device__ static inline uint32_t encode_ue4m3(float v) {
  if (!(v > 0.0f)) return 0u;
  if (v >= 448.0f) return 0x7eu;
  if (v < 0x1p-6f) {
    if (v >= (7.0f * 0x1p-9f + 0x1p-6f) * 0.5f) return 0x08u;
    const int m = static_cast<int>(floorf(__fadd_rn(__fmul_rn(v, 512.0f), 0.49999994f)));
    return m <= 0 ? 0u : static_cast<uint32_t>(m);
  }
  const uint32_t bits = __float_as_uint(v);
  uint32_t e = ((bits >> 23) & 0xffu) - 120u;
  uint32_t m = ((bits & 0x007fffffu) + 0x0007ffffu) >> 20;
  if (m >= 8u) { m = 0u; ++e; }
  if (e >= 15u) { e = 15u; if (m > 6u) m = 6u; }
  return (e << 3) | m;
}

// float -> E2M1 nibble (kernels-cuda/ops.cu:119-139): `<=` thresholds, so
// exact ties go toward zero; NaN lands on magnitude 7; -0.0 keeps sign clear.
__device__ static inline uint32_t encode_e2m1(float v) {
  const float a = fminf(fabsf(v), 6.0f);
  uint32_t idx = 7u;
  if (a <= 0.25f) idx = 0u;
  else if (a <= 0.75f) idx = 1u;
  else if (a <= 1.25f) idx = 2u;
  else if (a <= 1.75f) idx = 3u;
  else if (a <= 2.5f) idx = 4u;
  else if (a <= 3.5f) idx = 5u;
  else if (a <= 5.0f) idx = 6u;
  return (v < 0.0f ? 8u : 0u) | idx;
}

// Two floats -> one packed byte (lo in the low nibble), same result as two encode_e2m1 calls,
// built on the hardware conversion cvt.rn.satfinite.e2m1x2.f32.  The hardware rounds to nearest
// with ties to even and saturates at 6; the reference rule sends ties toward zero, which differs
// only at the exact magnitudes 0.75, 1.75 and 3.5 (even would go up), and reports -0.0 as code 0
// where the hardware keeps the sign.  NaN gives +6 (code 7) on both.
__device__ static inline uint32_t encode_e2m1x2(float lo, float hi) {
  uint32_t packed;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}"
      : "=r"(packed) : "f"(hi), "f"(lo));
  const uint32_t bl = __float_as_uint(lo) & 0x7fffffffu, bh = __float_as_uint(hi) & 0x7fffffffu;
  // ties that round-to-even takes up: step the magnitude back down
  if (bl == 0x3f400000u || bl == 0x3fe00000u || bl == 0x40600000u) packed -= 1u;
  if (bh == 0x3f400000u || bh == 0x3fe00000u || bh == 0x40600000u) packed -= 16u;
  if (bl == 0u) packed &= 0xf0u;     // +-0 -> code 0
  if (bh == 0u) packed &= 0x0fu;
  return packed;
}

// E2M1 nibble -> float (kernels-cuda/ops.cu:520-523) without a table:
// magnitude code c = (e << 1) | m is 0.5 * m for e == 0, else 2^(e-1)*(1+m/2).
__device__ static inline float e2m1_value(uint32_t code) {
  const uint32_t c = code & 7u;
  const uint32_t e = c >> 1, m = c & 1u;
  const float mag = e == 0u ? 0.5f * static_cast<float>(m)
                            : __uint_as_float(((e + 126u) << 23) | (m << 22));
  return (code & 8u) ? -mag : mag;
}

__device__ static inline float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }
#endif  // __CUDACC__

}  // namespace q36
