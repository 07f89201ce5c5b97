// Tensor-core NVFP4 GEMV (nvfp4_gemv_mma.cu): entry points for the C-ABI wrappers.
#pragma once

#include "common.cuh"

namespace q36 {

// W4A16: up to four matrices that share one bf16 activation vector, one launch.  Returns
// QWEN36_STATUS_NOT_IMPLEMENTED when a shape or pointer is outside what the kernel takes
// (out_features % 128, in_features % 256, in_features <= 32768, 16-byte aligned pointers).
int nvfp4_gemv_mma_bf16(const qwen36_nvfp4_matvec_spec_t *specs, size_t count);

// W4A16, tensor-parallel form: the rows of the specs are this rank's slices; the results go into every
// rank's arena over NVLink (qwen36_nvfp4_matvec_peer).  Same return rule.
int nvfp4_gemv_mma_bf16_peer(const qwen36_nvfp4_matvec_spec_t *specs, size_t count,
                             const qwen36_nvfp4_matvec_peer_spec_t *peer);
// Unpacks n values of a flagged vector at arena + offset into plain bf16 once they have arrived.
int nvfp4_gemv_peer_collect(const qwen36_nvfp4_matvec_peer_spec_t *peer, size_t slot, size_t vector_offset_bytes,
                            size_t n, qwen36_device_ptr_t arena, qwen36_device_ptr_t out_bf16);

// W4A4, one token: activation given as packed E2M1 codes + tiled UE4M3 scales.  Same return rule.
int nvfp4_gemv_mma_fp4(const qwen36_nvfp4_gemm_spec_t *spec, float alpha);

}  // namespace q36
