// Tensor-core NVFP4 GEMV (nvfp4_gemv_mma.cu): entry points for the C-ABI wrappers.
#pragma once

#include "common.cuh"

namespace q36 {

// W4A16: up to four matrices that share one bf16 activation vector, one launch.  Returns
// QWEN36_STATUS_NOT_IMPLEMENTED when a shape or pointer is outside what the kernel takes
// (out_features % 128, in_features % 256, in_features <= 32768, 16-byte aligned pointers).
int nvfp4_gemv_mma_bf16(const qwen36_nvfp4_matvec_spec_t *specs, size_t count);

// W4A4, one token: activation given as packed E2M1 codes + tiled UE4M3 scales.  Same return rule.
int nvfp4_gemv_mma_fp4(const qwen36_nvfp4_gemm_spec_t *spec, float alpha);

}  // namespace q36
