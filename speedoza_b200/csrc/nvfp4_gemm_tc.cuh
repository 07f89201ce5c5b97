// Interface between the GEMM entry points and the tcgen05 kernels.
#pragma once
#include "common.cuh"

namespace q36 {
// Runs the product on tcgen05 block-scaled MMA when the shape allows it;
// returns QWEN36_STATUS_NOT_IMPLEMENTED (nothing launched) when it does not.
int nvfp4_gemm_tc(const qwen36_nvfp4_gemm_spec_t *spec, float alpha);
}  // namespace q36
