// Interface between the GEMM entry points and the tcgen05 kernels.
#pragma once
#include "common.cuh"

namespace q36 {
// Runs the product on tcgen05 block-scaled MMA when the shape allows it;
// returns QWEN36_STATUS_NOT_IMPLEMENTED (nothing launched) when it does not.
int nvfp4_gemm_tc(const qwen36_nvfp4_gemm_spec_t *spec, float alpha);
// True while a test hook pins the tile form or the split factor of these kernels: one-token calls
// then stay on this path instead of the GEMV.
bool nvfp4_gemm_tc_forced();
}  // namespace q36
