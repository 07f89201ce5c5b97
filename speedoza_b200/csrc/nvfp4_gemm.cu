// W4A4 NVFP4 product behind qwen36_nvfp4_gemm / qwen36_decode_nvfp4_gemv:
//   c[token][row] = bf16( alpha * sum_k e2m1(a[row,k]) * ue4m3(sfa) * e2m1(b[token,k]) * ue4m3(sfb) )
// Entry points, shape routing, and the generic SIMT kernel that takes every
// shape the tensor-core kernels (nvfp4_gemm_tc.cu) decline.
#include "common.cuh"
#include "nvfp4_gemm_tc.cuh"
#include "nvfp4_gemv_mma.cuh"

namespace {

using q36::as_ptr;

constexpr int kWarps = 8;
constexpr int kTok = 8;   // tokens per warp pass

// One warp per weight row and up to kTok tokens; lanes stride over 16-groups.
// Inside a group the 16 products are small dyadic rationals, so their float32
// sum is exact; rounding happens only in the scaled accumulation.
__global__ void __launch_bounds__(kWarps * 32)
nvfp4_gemm_generic_kernel(const uint8_t *__restrict__ a, const uint8_t *__restrict__ a_sf,
                          const uint8_t *__restrict__ b, const uint8_t *__restrict__ b_sf, float alpha,
                          __nv_bfloat16 *__restrict__ c, size_t m, size_t n, size_t k) {
  const size_t row = static_cast<size_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  const size_t tok0 = static_cast<size_t>(blockIdx.y) * kTok;
  const unsigned lane = threadIdx.x & 31u;
  if (row >= m) return;
  const size_t groups = k / 16, sf_inner = q36::round_up(groups, 4), packed = k / 2;
  float acc[kTok];
#pragma unroll
  for (int t = 0; t < kTok; ++t) acc[t] = 0.f;
  for (size_t g = lane; g < groups; g += 32) {
    const uint8_t *wa = a + row * packed + g * 8;
    float av[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t byte = __ldg(wa + i);
      av[2 * i] = q36::e2m1_value(byte);
      av[2 * i + 1] = q36::e2m1_value(byte >> 4);
    }
    const float sa = q36::decode_e4m3(__ldg(a_sf + q36::sf_offset(g, row, sf_inner)));
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
      const size_t tok = tok0 + t;
      if (tok >= n) break;
      const uint8_t *wb = b + tok * packed + g * 8;
      float local = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t byte = __ldg(wb + i);
        local = fmaf(av[2 * i], q36::e2m1_value(byte), local);
        local = fmaf(av[2 * i + 1], q36::e2m1_value(byte >> 4), local);
      }
      const float sb = q36::decode_e4m3(__ldg(b_sf + q36::sf_offset(g, tok, sf_inner)));
      acc[t] = fmaf(local, sa * sb, acc[t]);
    }
  }
#pragma unroll
  for (int t = 0; t < kTok; ++t) {
    float v = acc[t];
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == 0 && tok0 + t < n) c[(tok0 + t) * m + row] = __float2bfloat16(v * alpha);
  }
}

int check(const qwen36_nvfp4_gemm_spec_t *s) {
  if (s == nullptr) return QWEN36_STATUS_NULL_POINTER;
  if (s->m == 0 || s->n == 0 || s->k == 0 || s->a_fp4.ptr == 0 || s->b_fp4.ptr == 0 || s->c_bf16.ptr == 0 ||
      s->a_scale.ptr == 0 || s->b_scale.ptr == 0)
    return QWEN36_STATUS_INVALID_ARGUMENT;
  return QWEN36_STATUS_SUCCESS;
}

int launch_generic(const qwen36_nvfp4_gemm_spec_t *s, float alpha) {
  if (s->k % 16 != 0) return QWEN36_STATUS_INVALID_ARGUMENT;
  const dim3 grid(static_cast<unsigned>(q36::div_ceil(s->m, kWarps)),
                  static_cast<unsigned>(q36::div_ceil(s->n, kTok)));
  if (grid.y > 65535u) return QWEN36_STATUS_INVALID_ARGUMENT;
  nvfp4_gemm_generic_kernel<<<grid, kWarps * 32, 0, q36::stream()>>>(
      as_ptr<const uint8_t>(s->a_fp4), as_ptr<const uint8_t>(s->a_scale), as_ptr<const uint8_t>(s->b_fp4),
      as_ptr<const uint8_t>(s->b_scale), alpha, as_ptr<__nv_bfloat16>(s->c_bf16), s->m, s->n, s->k);
  return q36::launch_status();
}

}  // namespace

extern "C" int qwen36_nvfp4_gemm(const qwen36_nvfp4_gemm_spec_t *spec) {
  const int rc = check(spec);
  if (rc != QWEN36_STATUS_SUCCESS) return rc;
  const float alpha = spec->alpha == 0.0f ? 1.0f : spec->alpha;   // kernels-cuda/nvfp4_gemm.cu:380
  if (spec->n == 1 && !q36::nvfp4_gemm_tc_forced()) {              // one token: the HBM-bound GEMV
    const int gv = q36::nvfp4_gemv_mma_fp4(spec, alpha);
    if (gv != QWEN36_STATUS_NOT_IMPLEMENTED) return gv;
  }
  const int tc = q36::nvfp4_gemm_tc(spec, alpha);
  if (tc != QWEN36_STATUS_NOT_IMPLEMENTED) return tc;
  return launch_generic(spec, alpha);
}

extern "C" int qwen36_decode_nvfp4_gemv(const qwen36_nvfp4_gemm_spec_t *spec) {
  const int rc = check(spec);
  if (rc != QWEN36_STATUS_SUCCESS) return rc;
  if (spec->n > 8) return QWEN36_STATUS_NOT_IMPLEMENTED;
  if (spec->n == 1 && !q36::nvfp4_gemm_tc_forced()) {
    const int gv = q36::nvfp4_gemv_mma_fp4(spec, spec->alpha);
    if (gv != QWEN36_STATUS_NOT_IMPLEMENTED) return gv;
  }
  return q36::nvfp4_gemm_tc(spec, spec->alpha);   // NOT_IMPLEMENTED for shapes it declines
}

extern "C" void qwen36_nvfp4_chunk_gemv_set_mtile(int mtile) { (void)mtile; }
