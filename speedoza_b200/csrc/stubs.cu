// Operators of the reference ABI that lie outside the quantized-matmul path.
// They are exported so that crates/kernels (backend.rs:1724-1770) links
// against this library, and report NOT_IMPLEMENTED without touching their
// argument.  The three mode hooks are accepted and ignored.
#include "common.cuh"

#define Q36_STUB(name) \
  extern "C" int name(const void *spec) { (void)spec; return QWEN36_STATUS_NOT_IMPLEMENTED; }

Q36_STUB(qwen36_bf16_gemm)
Q36_STUB(qwen36_bf16_matvec)
Q36_STUB(qwen36_attention_prefill)
Q36_STUB(qwen36_attention_flash_prefill)
Q36_STUB(qwen36_attention_sage_prefill)
Q36_STUB(qwen36_deltanet_decode)
Q36_STUB(qwen36_deltanet_prefill)
Q36_STUB(qwen36_interpreter_decode_sm120)
Q36_STUB(qwen36_drafter_attention_block_bf16)
Q36_STUB(qwen36_drafter_attention_block_flash_bf16)
Q36_STUB(qwen36_rmsnorm)
Q36_STUB(qwen36_partial_rope)
Q36_STUB(qwen36_swiglu)
Q36_STUB(qwen36_topk_argmax)
Q36_STUB(qwen36_embedding_lookup)
Q36_STUB(qwen36_conv1d_update)
Q36_STUB(qwen36_conv1d_prefill)
Q36_STUB(qwen36_gdn_gate)
Q36_STUB(qwen36_conv1d_gdn_gate_fused)
Q36_STUB(qwen36_sigmoid_gate)
Q36_STUB(qwen36_sigmoid_gate_strided)
Q36_STUB(qwen36_q_proj_deinterleave)
Q36_STUB(qwen36_q_proj_sigmoid_gate)
Q36_STUB(qwen36_copy_strided_rows)

extern "C" void qwen36_deltanet_set_resident(int mode) { (void)mode; }
extern "C" void qwen36_deltanet_prefill_set_tiny(int mode) { (void)mode; }
