// Internal: launch of the cross-rank attention merge, shared by the two entry points that end in it.
#pragma once
#include "common.cuh"

namespace q36 {

// part_* : [q_heads, n_parts(, head_dim)] split partials of this rank (n_parts = 1: finished partials).
int launch_attention_peer_merge(const float *part_o, const float *part_m, const float *part_l, uint32_t n_parts,
                                qwen36_device_ptr_t peer_inbox, qwen36_device_ptr_t peer_flags,
                                qwen36_device_ptr_t state, qwen36_device_ptr_t output_bf16, size_t world, size_t rank,
                                size_t q_heads, size_t head_dim);

}  // namespace q36
