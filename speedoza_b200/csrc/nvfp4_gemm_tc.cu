#include "nvfp4_gemm_tc.cuh"
namespace q36 {
int nvfp4_gemm_tc(const qwen36_nvfp4_gemm_spec_t *spec, float alpha) {
  (void)spec; (void)alpha;
  return QWEN36_STATUS_NOT_IMPLEMENTED;
}
}  // namespace q36
