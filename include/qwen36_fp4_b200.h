/*
 * C ABI of libqwen36_fp4_kernels.so, the sm_100a (B200) build of the
 * quantized-matmul hot path.
 *
 * Every "replaces" note names the interface of the reference project that the
 * entry point is binary-compatible with (paths relative to the reference
 * root; the reference header is kernels-cuda/include/qwen36_fp4.h).  Struct
 * field order and types are ABI: the Rust side binds them as #[repr(C)]
 * mirrors (crates/kernels/src/backend.rs:600-1771).  New fields and new entry
 * points are only ever appended.
 *
 * Conventions (same as the reference): every entry point returns an int
 * status, validates its arguments on the host, launches on the process-wide
 * ambient stream (qwen36_set_active_stream) and returns without
 * synchronising.  Device pointers travel as 64-bit integers.  Nothing here
 * allocates device memory except qwen36_cuda_malloc.
 *
 * Dimension names: the GEMM spec uses m = output features (weight rows),
 * n = tokens, k = input features.  The output c_bf16 is column-major [m, n]
 * with ld = m, i.e. row-major [tokens, features].
 */
#ifndef QWEN36_FP4_B200_H_
#define QWEN36_FP4_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- handles and status -------------------------------------------------- */

typedef struct { uint64_t ptr; } qwen36_device_ptr_t;            /* qwen36_fp4.h:10-12 */
typedef struct { qwen36_device_ptr_t ptr; size_t bytes; } qwen36_device_allocation_t; /* :14-17 */

enum {                                   /* qwen36_fp4.h:54-65 */
  QWEN36_STATUS_SUCCESS = 0,
  QWEN36_STATUS_NULL_POINTER = 1,
  QWEN36_STATUS_INVALID_ARGUMENT = 2,
  QWEN36_STATUS_CUDA_ERROR = 3,
  QWEN36_STATUS_CUBLAS_ERROR = 4,        /* never produced by this build */
  QWEN36_STATUS_NOT_IMPLEMENTED = 5      /* soft "use another path" signal */
};

typedef struct CUstream_st *qwen36_cuda_stream_t;
typedef struct CUevent_st *qwen36_cuda_event_t;
typedef struct CUgraph_st *qwen36_cuda_graph_t;
typedef struct CUgraphExec_st *qwen36_cuda_graph_exec_t;

typedef struct {                         /* qwen36_fp4.h:19-34 */
  int driver_version, runtime_version, device_count, active_device;
  int sm_major, sm_minor, multiprocessor_count;
  size_t total_global_mem;
  char device_name[128];
  char libcuda_path[512];
  char cudart_path[512];
  int last_cuda_error;
  char last_cuda_error_name[64];
  char last_cuda_error_string[256];
} qwen36_cuda_diagnostics_t;

typedef struct {                         /* qwen36_fp4.h:36-52 */
  uint64_t malloc_calls, free_calls, h2d_calls, h2d_bytes, d2h_calls, d2h_bytes;
  uint64_t d2d_calls, d2d_bytes, d2d_async_calls, d2d_async_bytes;
  uint64_t memset_calls, memset_bytes, synchronize_calls, stream_synchronize_calls;
  uint64_t graph_launch_calls;
} qwen36_cuda_counters_t;

/* ---- NVFP4 linear layers -------------------------------------------------- */

/* qwen36_fp4.h:67-81.  A = weights [m, k/2] packed E2M1 (low nibble = even
 * column) with UE4M3 block scales in the 128x4 tiled layout (outer = feature);
 * B = activations [n, k/2] with tiled scales (outer = token).  alpha carries
 * both per-tensor scales; a_scale_2 / b_scale_2 are accepted and ignored.
 * workspace (the buffer the reference hands to cuBLASLt) is optional: when it is
 * 16-byte aligned and holds 256 KB + 64 B per pair of SMs (19.4 MB on a B200),
 * prefill shapes whose tiles fill the SMs badly (e.g. 5120 x 17408 at 512-2048
 * tokens) are cut along K and their partial tiles meet in it; its contents need no
 * initialisation and mean nothing afterwards.  Calls that share a workspace must
 * not overlap (same rule as for cuBLASLt).  Without it every tile is summed by
 * one CTA pair, and the two routes differ only in the grouping of float32
 * additions. */
typedef struct {
  size_t m, n, k;
  qwen36_device_ptr_t a_fp4, a_scale, a_scale_2;
  qwen36_device_ptr_t b_fp4, b_scale, b_scale_2;
  qwen36_device_ptr_t c_bf16;
  qwen36_device_ptr_t workspace;
  size_t workspace_bytes;
  float alpha;
} qwen36_nvfp4_gemm_spec_t;

/* qwen36_fp4.h:463-471.  W4A16: bf16 activation [in_features]. */
typedef struct {
  size_t out_features, in_features;
  qwen36_device_ptr_t input_bf16, weight_u8, block_scale_e4m3, tensor_scale_f32, output_bf16;
} qwen36_nvfp4_matvec_spec_t;

/* qwen36_fp4.h:473-480 */
typedef struct {
  size_t values;
  qwen36_device_ptr_t input_bf16, output_fp4, output_scale_e4m3, output_tensor_scale_f32;
  float input_tensor_scale_f32;
} qwen36_nvfp4_quantize_spec_t;

/* qwen36_fp4.h:482-490 */
typedef struct {
  size_t rows, values;
  qwen36_device_ptr_t input_bf16, output_fp4, output_scale_e4m3, output_tensor_scale_f32;
  float input_tensor_scale_f32;
} qwen36_nvfp4_quantize_rows_spec_t;

/* qwen36_fp4.h:492-497 */
typedef struct {
  size_t rows, inner_groups;
  qwen36_device_ptr_t input_row_major_u8, output_tiled_u8;
} qwen36_nvfp4_retile_scales_spec_t;

/* ---- exact-argmax guards of the FP8 lm_head -------------------------------- */

#define QWEN36_LM_HEAD_TOP2_BLOCKS 240     /* qwen36_fp4.h:414: blocks of the vocabulary scan */

/* qwen36_fp4.h:384-400.  Full bf16 lm_head + argmax for rows whose
 * skip_flags_u32 entry is zero (NULL: every row); flagged rows keep their
 * token.  workspace: rows * 8 bytes. */
typedef struct {
  size_t rows;
  size_t out_features;
  size_t in_features;
  qwen36_device_ptr_t input_bf16;
  qwen36_device_ptr_t weight_bf16;
  qwen36_device_ptr_t output_token_u32;
  qwen36_device_ptr_t mirror_last_output_token_u32;
  qwen36_device_ptr_t workspace;
  size_t workspace_bytes;
  qwen36_device_ptr_t skip_flags_u32;
} qwen36_bf16_matvec_argmax_rows_spec_t;

/* qwen36_fp4.h:416-427.  tokens = argmax of the bf16 logits (lowest index on
 * ties), flags = 1 when top1 - top2 >= eps.  workspace: rows * 240 * 16 bytes. */
typedef struct {
  size_t rows;
  size_t vocab;
  float eps;
  qwen36_device_ptr_t logits_bf16;
  qwen36_device_ptr_t tokens_u32;
  qwen36_device_ptr_t flags_u32;
  qwen36_device_ptr_t mirror_last_token_u32;
  qwen36_device_ptr_t fallback_count_u32;
  qwen36_device_ptr_t workspace;
  size_t workspace_bytes;
} qwen36_lm_head_top2_margin_spec_t;

/* qwen36_fp4.h:447-461.  Top-8 block winners rescored against the bf16 weight. */
typedef struct {
  size_t rows;
  size_t vocab;
  size_t cols;
  float eps;
  qwen36_device_ptr_t logits_bf16;
  qwen36_device_ptr_t weight_bf16;
  qwen36_device_ptr_t input_bf16;
  qwen36_device_ptr_t tokens_u32;
  qwen36_device_ptr_t flags_u32;
  qwen36_device_ptr_t mirror_last_token_u32;
  qwen36_device_ptr_t fallback_count_u32;
  qwen36_device_ptr_t workspace;
  size_t workspace_bytes;
} qwen36_lm_head_top8_rescore_spec_t;

/* Replace kernels-cuda/lm_head_fp8.cu:528-590 and kernels-cuda/ops.cu:1104-1153.
 * Same tokens and flags as the reference for every input (same vocabulary
 * partition, same float64 / float32 summation orders, same tie rules); the
 * bf16 lm_head reads the weight once for up to eight rows instead of once per
 * row. */
int qwen36_lm_head_top2_margin(const qwen36_lm_head_top2_margin_spec_t *spec);
int qwen36_lm_head_top8_rescore(const qwen36_lm_head_top8_rescore_spec_t *spec);
int qwen36_bf16_matvec_argmax_rows(const qwen36_bf16_matvec_argmax_rows_spec_t *spec);

/* ---- fused producers of NVFP4 activations (decode path) -------------------- */

/* qwen36_fp4.h:264-276.  out = (input [+ residual]) * rsqrt(mean(sq) + eps) *
 * (1 + weight), written as bf16 (optional), as NVFP4 codes and as tiled block
 * scales (outer row 0); residual_out (optional) receives input + residual. */
typedef struct {
  size_t hidden;
  float eps;
  qwen36_device_ptr_t input_bf16;
  qwen36_device_ptr_t weight_bf16;
  qwen36_device_ptr_t residual_bf16;
  qwen36_device_ptr_t residual_out_bf16;
  qwen36_device_ptr_t output_bf16;
  qwen36_device_ptr_t output_fp4;
  qwen36_device_ptr_t output_scale_e4m3;
  qwen36_device_ptr_t output_tensor_scale_f32;
  float input_tensor_scale_f32;
} qwen36_rmsnorm_nvfp4_quantize_spec_t;

/* qwen36_fp4.h:304-312.  y = silu(gate) * up in float32, quantised like
 * qwen36_nvfp4_quantize_bf16 without the bf16 round trip. */
typedef struct {
  size_t intermediate;
  qwen36_device_ptr_t gate_bf16;
  qwen36_device_ptr_t up_bf16;
  qwen36_device_ptr_t output_fp4;
  qwen36_device_ptr_t output_scale_e4m3;
  qwen36_device_ptr_t output_tensor_scale_f32;
  float input_tensor_scale_f32;
} qwen36_swiglu_nvfp4_quantize_spec_t;

/* Replaces qwen36_rmsnorm_nvfp4_quantize (kernels-cuda/ops.cu:1007-1031, body
 * interpreter/opcodes/rmsnorm_nvfp4_quant.cuh:113-281): one launch, same
 * arithmetic order (256 strided partial sums + halving tree, rsqrtf), eps == 0
 * is read as 1e-6. */
int qwen36_rmsnorm_nvfp4_quantize(const qwen36_rmsnorm_nvfp4_quantize_spec_t *spec);

/* Replaces qwen36_swiglu_nvfp4_quantize (kernels-cuda/ops.cu:1500-1521, body
 * interpreter/opcodes/swiglu_nvfp4_quant.cuh:13-75). */
int qwen36_swiglu_nvfp4_quantize(const qwen36_swiglu_nvfp4_quantize_spec_t *spec);

/* Additive (no counterpart in qwen36_fp4.h): the prefill form of
 * qwen36_swiglu_nvfp4_quantize.  y[r] = silu(gate[r]) * up[r] for `rows` rows of
 * `intermediate` values (a multiple of 16), quantised row by row exactly as the
 * single-vector entry does it (float32, no bf16 round trip): output_fp4 is
 * [rows, intermediate / 2], output_scale_e4m3 the tiled 128 x 4 layout of
 * [rows, intermediate / 16], i.e. the activation operand of qwen36_nvfp4_gemm for the
 * down projection.  It replaces the reference's prefill chain "SwiGLU kernel ->
 * bf16 [rows, intermediate] -> qwen36_nvfp4_quantize_rows"
 * (crates/runtime/src/engine.rs:7395-7413) without the intermediate.  gate and up
 * are rows of `input_row_stride` elements (>= intermediate, a multiple of 8; both
 * halves of one [rows, 2 * intermediate] GEMM output qualify), 16-byte aligned. */
typedef struct {
  size_t rows;
  size_t intermediate;
  size_t input_row_stride;
  qwen36_device_ptr_t gate_bf16;
  qwen36_device_ptr_t up_bf16;
  qwen36_device_ptr_t output_fp4;
  qwen36_device_ptr_t output_scale_e4m3;
  qwen36_device_ptr_t output_tensor_scale_f32;
  float input_tensor_scale_f32;
} qwen36_swiglu_nvfp4_quantize_rows_spec_t;
int qwen36_swiglu_nvfp4_quantize_rows(const qwen36_swiglu_nvfp4_quantize_rows_spec_t *spec);

/* Replaces qwen36_nvfp4_gemm (kernels-cuda/nvfp4_gemm.cu:341-409, a cuBLASLt
 * call).  Any m, n, k with k % 16 == 0.  alpha == 0 is read as 1.  Shapes with
 * m % 128 == 0 and k % 256 == 0 run on tcgen05 block-scaled MMA: persistent
 * 128-row x {8..256}-token tiles; for n <= 16 with fewer row blocks than SMs,
 * clusters of CTAs split K and add their partial sums through distributed
 * shared memory; for long K and thousands of tokens, CTA pairs (cta_group::2)
 * share 256 x 256 tiles.  Anything else takes a generic SIMT kernel. */
int qwen36_nvfp4_gemm(const qwen36_nvfp4_gemm_spec_t *spec);

/* Replaces qwen36_decode_nvfp4_gemv
 * (kernels-cuda/decode_gemv/nvfp4_gemv_sm120.cu:203-331).  n in [1, 8],
 * m % 128 == 0, k % 256 == 0; other shapes return NOT_IMPLEMENTED, which the
 * Rust dispatcher turns into a qwen36_nvfp4_gemm call
 * (crates/kernels/src/backend.rs:225-229).  alpha is used as given. */
int qwen36_decode_nvfp4_gemv(const qwen36_nvfp4_gemm_spec_t *spec);

/* Replaces the test hook of the same name (nvfp4_gemv_sm120.cu:173-175);
 * kept for linkage, has no effect. */
void qwen36_nvfp4_chunk_gemv_set_mtile(int mtile);

/* Replaces qwen36_nvfp4_matvec (kernels-cuda/ops.cu:547-639,1155-1180). */
int qwen36_nvfp4_matvec(const qwen36_nvfp4_matvec_spec_t *spec);

/* Additive: `count` (1..4) GEMVs that share input_bf16 and in_features, as ONE launch whose work
 * list spans all of the matrices (q / k / v projections of a decode layer).  Same results as
 * `count` qwen36_nvfp4_matvec calls.  The reference reaches the same effect by concatenating such
 * weights along N at load time (crates/runtime/src/gpu.rs:181-225,410-467); this entry needs no
 * re-layout of the checkpoint.  INVALID_ARGUMENT when the specs do not share their input. */
int qwen36_nvfp4_matvec_group(const qwen36_nvfp4_matvec_spec_t *specs, size_t count);

/* Replace qwen36_nvfp4_quantize_bf16 / _rows
 * (kernels-cuda/ops.cu:641-761,1182-1227).  Codes, packing and scale bytes
 * follow the reference bit for bit (E2M1 ties toward zero, UE4M3 ties down).
 * Only scale bytes of real (row, group) pairs are written. */
int qwen36_nvfp4_quantize_bf16(const qwen36_nvfp4_quantize_spec_t *spec);
int qwen36_nvfp4_quantize_rows(const qwen36_nvfp4_quantize_rows_spec_t *spec);

/* Replaces qwen36_nvfp4_retile_scales (kernels-cuda/ops.cu:763-774,1229-1255).
 * Padding bytes are zeroed by the same kernel on the ambient stream (the
 * reference issues a synchronous cudaMemset first). */
int qwen36_nvfp4_retile_scales(const qwen36_nvfp4_retile_scales_spec_t *spec);

/* ---- lm_head: FP8 weight, greedy argmax ----------------------------------- */

#define QWEN36_LM_HEAD_FP8_MAX_N 16      /* qwen36_fp4.h:364 */

typedef struct {                         /* qwen36_fp4.h:366-372 */
  size_t rows, cols;
  qwen36_device_ptr_t weight_bf16, weight_e4m3, row_scales_f32;
} qwen36_lm_head_fp8_quantize_spec_t;

typedef struct {                         /* qwen36_fp4.h:374-382 */
  size_t rows, cols, n;
  qwen36_device_ptr_t weight_e4m3, row_scales_f32, input_bf16, output_bf16;
} qwen36_lm_head_fp8_gemv_spec_t;

typedef struct {                         /* qwen36_fp4.h:314-323 */
  size_t vocab_size;
  qwen36_device_ptr_t logits_bf16, output_token_u32;
  float temperature;
  size_t top_k;
  float top_p, repetition_penalty;
  qwen36_device_ptr_t mirror_output_token_u32;
} qwen36_sampling_spec_t;

typedef struct {                         /* qwen36_fp4.h:334-341 */
  size_t rows, vocab_size;
  qwen36_device_ptr_t logits_bf16, output_token_u32, mirror_last_output_token_u32;
  float temperature;
} qwen36_sampling_rows_spec_t;

/* Replace kernels-cuda/lm_head_fp8.cu:511-526 and :592-620.  The GEMV keeps
 * the reference's float32 summation order, so its bf16 logits are identical. */
int qwen36_lm_head_fp8_quantize(const qwen36_lm_head_fp8_quantize_spec_t *spec);
int qwen36_lm_head_fp8_gemv(const qwen36_lm_head_fp8_gemv_spec_t *spec);

/* Replace qwen36_sample / qwen36_sample_rows (kernels-cuda/ops.cu:299-427,
 * 1523-1560): greedy argmax over bf16 logits, ties to the lowest index. */
int qwen36_sample(const qwen36_sampling_spec_t *spec);
int qwen36_sample_rows(const qwen36_sampling_rows_spec_t *spec);

/* ---- int8 per-vector KV cache + decode attention --------------------------- */

typedef struct { size_t q_heads, kv_heads, head_dim, rope_dims; } qwen36_attention_shape_t; /* :94-99 */

typedef struct {                         /* qwen36_fp4.h:185-194 */
  size_t layer_index, position;
  qwen36_device_ptr_t k_bf16, v_bf16, k_quantized_i8, v_quantized_i8, metadata_f32;
  qwen36_attention_shape_t shape;
} qwen36_turboquant_encode_spec_t;

typedef struct {                         /* qwen36_fp4.h:196-208 */
  size_t layer_index, position;
  qwen36_device_ptr_t q_bf16, k_quantized_i8, v_quantized_i8, metadata_f32, output_bf16;
  qwen36_device_ptr_t workspace;
  size_t workspace_bytes;
  qwen36_attention_shape_t shape;
  int mode;
} qwen36_turboquant_attention_spec_t;

/* Replaces qwen36_turboquant_encode_kv (kernels-cuda/turboquant.cu:23-67,
 * 139-159): one position, K and V of every kv head. */
int qwen36_turboquant_encode_kv(const qwen36_turboquant_encode_spec_t *spec);

/* Replaces qwen36_turboquant_attention (kernels-cuda/turboquant.cu:69-135,
 * 161-183).  Split-KV: needs qwen36_turboquant_attention_workspace_bytes()
 * of caller scratch in `workspace` (the reference ignores the field); returns
 * INVALID_ARGUMENT when it is missing or too small.  `mode` is ignored. */
int qwen36_turboquant_attention(const qwen36_turboquant_attention_spec_t *spec);

/* ---- decode attention over a BF16 / FP8 (E4M3) KV cache --------------------- */

typedef struct {                         /* qwen36_fp4.h:151-183 */
  size_t layer_index, position;
  qwen36_device_ptr_t q_bf16, k_bf16, v_bf16, kv_cache_k, kv_cache_v, kv_cache_metadata, output_bf16;
  qwen36_attention_shape_t shape;
  int kv_cache_dtype;                    /* 0 = BF16, 1 = FP8 E4M3, 2 / 3 = TurboQuant3 / 3.5 */
  qwen36_device_ptr_t position_device_i32;
  qwen36_device_ptr_t partial_acc_f32, partial_max_f32, partial_denom_f32;
  size_t decode_n_splits, split_timesteps_per_block;
} qwen36_attention_decode_spec_t;

/* Replaces qwen36_attention_decode (kernels-cuda/attention.cu:2716-2876 and the
 * kernels it launches: attention.cu:842-1000, 1036-1223, 1225-1471, 1473-1554,
 * attention_decode_tiled.cu:159-357) for kv_cache_dtype 0 and 1: one query token
 * attends to cache rows [0, position) plus the new k_bf16 / v_bf16 row, and that
 * row is appended to the cache at `position` (copied for BF16; for FP8 encoded
 * with the reference's round-half-up E4M3 encoder, attention.cu:118-160).  The
 * position comes from position_device_i32 when that is non-zero.  With the three
 * partial buffers and decode_n_splits >= 2 the cached rows are split across up
 * to decode_n_splits CTAs per head (the buffers are laid out as the reference
 * says: [q_heads, decode_n_splits, head_dim] and 2 x [q_heads, decode_n_splits]);
 * how many of them are used and which rows each one takes is this library's
 * choice, so split_timesteps_per_block is only validated (>= 64 or 0).  Without
 * the buffers one CTA per q head walks the whole context.  TurboQuant3 / 3.5
 * caches (dtype 2 / 3) return QWEN36_STATUS_NOT_IMPLEMENTED. */
int qwen36_attention_decode(const qwen36_attention_decode_spec_t *spec);

/* Replaces qwen36_attention_decode_split_tiled (kernels-cuda/attention_decode_tiled.cu:159-357,
 * 370-403; not in the reference's public header, declared in attention.cu:2408-2418): the split-KV
 * half of a decode step on its own.  Split s covers timesteps [s * split_timesteps_per_block,
 * (s + 1) * split_timesteps_per_block) cut at position + 1, the timestep at `position` being the new
 * k_bf16 / v_bf16 row; it writes only the partials ([q_heads, n_splits(, head_dim)], an empty split
 * as (-inf, 0, 0)) and the split that owns `position` appends the row to the cache.  A merge
 * (qwen36_attention_merge_partials) turns the partials into the output.  head_dim 256, 2..8 q heads
 * per kv head, BF16 / FP8 cache, block a multiple of 8: other shapes return NOT_IMPLEMENTED, as the
 * reference's entry does. */
int qwen36_attention_decode_split_tiled(const qwen36_attention_decode_spec_t *spec, int n_splits,
                                        int split_timesteps_per_block);

/* ---- speculative-verify attention: a short query chunk over a long cache ---- */

typedef struct {                         /* qwen36_fp4.h:108-147 */
  size_t layer_index, start_position, tokens;
  qwen36_device_ptr_t q_bf16, k_bf16, v_bf16, kv_cache_k, kv_cache_v, kv_cache_metadata, output_bf16;
  qwen36_attention_shape_t shape;
  int kv_cache_dtype;                    /* 0 = BF16, 1 = FP8 E4M3 */
  qwen36_device_ptr_t start_position_device_i32;
  qwen36_device_ptr_t partial_acc_f32, partial_max_f32, partial_denom_f32;
  size_t prefill_n_splits, split_timesteps_per_block;
  qwen36_device_ptr_t tree_ancestor_bitmap_u64;
  size_t verify_chunk_rows;
} qwen36_attention_prefill_spec_t;

/* Replaces qwen36_attention_flash_splitk_prefill_bf16 (kernels-cuda/attention_flash_splitk.cu:96-420,
 * 504-600; declared in attention.cu:2408): `tokens` <= 32 query rows x q_heads, already appended to
 * the cache, attend to cache rows [0, start_position + tokens) under the causal mask of the chunk
 * (row i sees rows <= start_position + i); head_dim 256, BF16 or FP8 cache.  The 64-row K iterations
 * are dealt evenly to `n_splits` splits; partials are token-major
 * ([tokens, q_heads, n_splits(, head_dim)]) in the spec's three partial buffers, or, when the spec
 * has none, in a scratch the library grows on demand (growing allocates: during a stream capture the
 * call returns NOT_IMPLEMENTED instead, which the reference's dispatcher treats as "use another
 * path", attention.cu:2666-2671).  k_bf16 / v_bf16, the split fields and the tree bitmap of the spec
 * are not read by this entry (nor by the reference's). */
int qwen36_attention_flash_splitk_prefill_bf16(const qwen36_attention_prefill_spec_t *spec, int n_splits);
/* Test hooks: mode 0 = general kernel only, 1 = tensor-core kernels where they
 * apply (default); n > 0 overrides the number of splits used. */
void qwen36_attention_decode_set_mode(int mode);
void qwen36_attention_decode_force_splits(int n);

/* ---- additions of this build (no ABI change to anything above) ------------ */

/* Scratch needed by qwen36_turboquant_attention / _partial for a shape. */
size_t qwen36_turboquant_attention_workspace_bytes(size_t q_heads, size_t head_dim);

/* Batched form of qwen36_turboquant_encode_kv: k, v bf16
 * [tokens, kv_heads, head_dim] are written to cache rows
 * [position, position + tokens).  Same arithmetic per (token, head). */
typedef struct {
  size_t position, tokens;
  qwen36_device_ptr_t k_bf16, v_bf16, k_quantized_i8, v_quantized_i8, metadata_f32;
  qwen36_attention_shape_t shape;
} qwen36_turboquant_encode_rows_spec_t;
int qwen36_turboquant_encode_kv_rows(const qwen36_turboquant_encode_rows_spec_t *spec);

/* Attention over cache rows [t_begin, t_end) only, leaving one un-normalised
 * partial per q head in the (m, l, o) form of the reference's split paths
 * (kernels-cuda/attention.cu:1083-1094,1473-1554): partial_max_f32 [q_heads],
 * partial_denom_f32 [q_heads], partial_acc_f32 [q_heads, head_dim].  An empty
 * range yields (-inf, 0, 0).  Used to shard a long context across GPUs. */
typedef struct {
  size_t t_begin, t_end;
  qwen36_device_ptr_t q_bf16, k_quantized_i8, v_quantized_i8, metadata_f32;
  qwen36_device_ptr_t partial_acc_f32, partial_max_f32, partial_denom_f32;
  qwen36_device_ptr_t workspace;
  size_t workspace_bytes;
  qwen36_attention_shape_t shape;
} qwen36_turboquant_attention_partial_spec_t;
int qwen36_turboquant_attention_partial(const qwen36_turboquant_attention_partial_spec_t *spec);

/* No counterpart in the reference.  Same computation and same spec as
 * qwen36_turboquant_attention, for callers that cannot hand over scratch
 * memory: code running where cudaMalloc is off limits (inside a stream capture,
 * under a memory budget that is already fully committed, in a plug-in whose host
 * forbids allocation after start-up).  The split-KV partials go to a fixed
 * 4 MiB buffer inside the library image instead of `workspace` /
 * `workspace_bytes`, which are ignored.  The entry point allocates nothing.
 * Limits and rules:
 *  - q_heads * (head_dim + 2) must not exceed
 *    qwen36_turboquant_attention_static_max_head_floats() (8256: e.g. 32 heads of
 *    256 dims); larger shapes return QWEN36_STATUS_INVALID_ARGUMENT.
 *  - The first call on each device looks up the buffer's device address; make that
 *    call once, with the device current, before any stream capture.
 *  - All calls on a device share the one buffer: two calls whose kernels overlap
 *    on the GPU (different streams, or graphs launched side by side) race.  Calls
 *    ordered on one stream are fine; nothing in the buffer has to be cleared
 *    between them, every partial is written before it is read.
 *  - Every GPU that loads the library carries the 4 MiB until the process exits. */
int qwen36_turboquant_attention_static(const qwen36_turboquant_attention_spec_t *spec);
size_t qwen36_turboquant_attention_static_max_head_floats(void);

/* Log-sum-exp merge of n_parts partials laid out [q_heads, n_parts(, head_dim)]
 * into bf16 [q_heads, head_dim]; the arithmetic of
 * kernels-cuda/attention.cu:1473-1554 with the zero-denominator guard of
 * kernels-cuda/attention_flash_splitk.cu:419. */
typedef struct {
  size_t q_heads, head_dim, n_parts;
  qwen36_device_ptr_t partial_acc_f32, partial_max_f32, partial_denom_f32, output_bf16;
} qwen36_attention_merge_spec_t;
int qwen36_attention_merge_partials(const qwen36_attention_merge_spec_t *spec);

/* ---- Multi-GPU combine over NVLink peer memory (no reference counterpart: the
 * reference is single-GPU).  One process per GPU on one node.  Every rank
 * allocates an inbox and a flag array with qwen36_cuda_malloc plus a local
 * 4-word state, all zero-filled once; exports inbox and flags with
 * qwen36_ipc_get_handle, opens the peers' handles with qwen36_ipc_open_handle,
 * and keeps two device arrays of `world` pointers in rank order (its own
 * entries are the local pointers).  A combine kernel pushes this rank's piece
 * into every peer's inbox with plain peer stores, raises a flag there, waits
 * on its own flags and combines out of its own memory.  Every wait is bounded
 * (a few seconds at most).  A wait that runs out is visible without a
 * synchronising query: the call's output is poisoned (NaN rows of the merge,
 * token 0xFFFFFFFF of the argmax), state[2] receives the number of the first
 * failed call, and qwen36_peer_last_error() returns 1 from then on.  After any
 * reported failure the exchange is out of step: state, flags and inbox must be
 * re-zeroed on ALL ranks under a host barrier before it is used again.  The call number is kept in `state` and
 * advanced by the kernel, so a captured launch can be replayed; all ranks must
 * make the same sequence of calls on one set of buffers. */
int qwen36_ipc_get_handle(qwen36_device_ptr_t ptr, void *handle_out_64_bytes);
int qwen36_ipc_open_handle(const void *handle_64_bytes, qwen36_device_ptr_t *out);
int qwen36_ipc_close_handle(qwen36_device_ptr_t ptr);
int qwen36_peer_last_error(void);   /* sticky */
int qwen36_peer_reset_error(void);

/* Tensor-parallel W4A16 GEMV: the output rows of every matrix are split over
 * the ranks in whole 128-row blocks (the blocking of the scale tiles,
 * crates/runtime/src/gpu.rs:329-339 in the reference).  Each rank holds an
 * ARENA (an inbox of the exchange above; the flag array is not used) with one
 * full-length copy of every activation vector of the chain, kept as FLAGGED
 * CELLS: 8 bytes per two values = {bf16 pair, uint32 number of the call that
 * wrote them}, so a vector of n values takes 4 n bytes.
 * qwen36_nvfp4_matvec_peer computes this rank's rows of 1..4 matrices that
 * share their input (as qwen36_nvfp4_matvec_group does; output_bf16 of the
 * specs is not used) and its epilogue stores them, as cells, at
 * output_offset_bytes[i] + 4 * row_offset[i] of EVERY rank's arena.  A call
 * whose input is such a vector passes the address of the cells as input_bf16
 * and names the producing call's slot as `in_slot`: it then reads a cell only
 * once the cell carries that call's number (bounded wait), while its weights
 * stream.  QWEN36_PEER_INPUT_LOCAL = input_bf16 is a plain local bf16 vector.
 * state: slots x 4 uint32, local, zero-filled once ({calls completed, CTA
 * ticket, number of the first failed call, unused} per slot); the arenas
 * start zero-filled too.  All ranks make the same sequence of calls.  A
 * vector may be overwritten by a later call once it has been consumed on
 * every rank, which a dependent chain (each call consuming the previous
 * call's vector) guarantees.  A wait that runs out gives NaN rows that
 * propagate down the chain, the call number in state[4 * slot + 2] and
 * qwen36_nvfp4_gemv_mma_last_error() == 2.  NOT_IMPLEMENTED unless
 * out_features % 128 == 0 and in_features % 256 == 0, in_features <= 32768.
 * qwen36_nvfp4_matvec_peer_collect unpacks n values (a multiple of 4) of a
 * flagged vector of this rank's arena into plain bf16, waiting the same way:
 * for a consumer that is not one of these calls. */
#define QWEN36_PEER_INPUT_LOCAL ((size_t)-1)
typedef struct {
  size_t world, rank;                 /* world <= 8 */
  qwen36_device_ptr_t peer_arena;     /* device array: world x (uint8_t *)  */
  qwen36_device_ptr_t state;          /* local, slots x 4 uint32            */
  size_t slots, out_slot, in_slot;
  size_t output_offset_bytes[4];      /* multiples of 16                    */
  size_t row_offset[4];               /* multiples of 8                     */
} qwen36_nvfp4_matvec_peer_spec_t;
int qwen36_nvfp4_matvec_peer(const qwen36_nvfp4_matvec_spec_t *specs, size_t count,
                             const qwen36_nvfp4_matvec_peer_spec_t *peer);
int qwen36_nvfp4_matvec_peer_collect(const qwen36_nvfp4_matvec_peer_spec_t *peer, size_t slot,
                                     qwen36_device_ptr_t cells, size_t n, qwen36_device_ptr_t output_bf16);
/* 0 = no bounded wait of the tensor-core GEMV ever ran out in this process; 1 = a pipeline stage
 * never arrived; 2 = a peer's cells never arrived.  Sticky; both calls synchronise. */
int qwen36_nvfp4_gemv_mma_last_error(void);
int qwen36_nvfp4_gemv_mma_reset_error(void);

/* Cross-rank log-sum-exp merge of one (m, l, o) partial per q head and rank
 * (the arithmetic of qwen36_attention_merge_partials with n_parts = world, in
 * rank order, so every rank gets the same bits).  The three inputs are the
 * outputs of qwen36_turboquant_attention_partial.  Inbox:
 * qwen36_attention_peer_inbox_bytes(world, q_heads, head_dim); flag array:
 * world * q_heads uint32; state: 2 uint32. */
typedef struct {
  size_t world, rank, q_heads, head_dim;
  qwen36_device_ptr_t partial_acc_f32, partial_max_f32, partial_denom_f32;
  qwen36_device_ptr_t peer_inbox;     /* device array: world x (float *)    */
  qwen36_device_ptr_t peer_flags;     /* device array: world x (uint32_t *) */
  qwen36_device_ptr_t state;          /* local, 2 x uint32                  */
  qwen36_device_ptr_t output_bf16;    /* [q_heads, head_dim]                */
} qwen36_attention_peer_merge_spec_t;
size_t qwen36_attention_peer_inbox_bytes(size_t world, size_t q_heads, size_t head_dim);
int qwen36_attention_peer_merge(const qwen36_attention_peer_merge_spec_t *spec);

/* qwen36_turboquant_attention_partial over this rank's rows [t_begin, t_end) of
 * its local cache and the cross-rank merge in two launches (the split kernel,
 * then one kernel that merges the splits, pushes and merges the peers'
 * results); same bits as _partial + qwen36_attention_peer_merge. */
typedef struct {
  size_t t_begin, t_end;
  qwen36_device_ptr_t q_bf16, k_quantized_i8, v_quantized_i8, metadata_f32;
  qwen36_device_ptr_t workspace;
  size_t workspace_bytes;
  qwen36_attention_shape_t shape;
  size_t world, rank;
  qwen36_device_ptr_t peer_inbox, peer_flags, state, output_bf16;
} qwen36_turboquant_attention_peer_spec_t;
int qwen36_turboquant_attention_peer(const qwen36_turboquant_attention_peer_spec_t *spec);

/* Cross-rank greedy argmax of one (value, index) pair per token and rank, the
 * rule of kernels-cuda/ops.cu:19-23 (strictly greater wins, equal values keep
 * the lower index).  The two inputs are best_value_f32 / output_token_u32 of
 * qwen36_lm_head_fp8_gemv_argmax.  Inbox:
 * qwen36_argmax_peer_inbox_bytes(world, tokens); flag array: world uint32;
 * state: 2 uint32. */
typedef struct {
  size_t world, rank, tokens;
  qwen36_device_ptr_t best_value_f32, best_index_u32;
  qwen36_device_ptr_t peer_inbox;     /* device array: world x (uint32_t *) */
  qwen36_device_ptr_t peer_flags;     /* device array: world x (uint32_t *) */
  qwen36_device_ptr_t state;          /* local, 2 x uint32                  */
  qwen36_device_ptr_t output_token_u32;
} qwen36_argmax_peer_combine_spec_t;
size_t qwen36_argmax_peer_inbox_bytes(size_t world, size_t tokens);
int qwen36_argmax_peer_combine(const qwen36_argmax_peer_combine_spec_t *spec);

/* lm_head GEMV fused with the greedy argmax: no logits are written.  Each
 * logit is rounded to bf16 exactly as qwen36_lm_head_fp8_gemv would store it
 * before it is compared, so the winner equals qwen36_sample_rows over that
 * GEMV's output.  row_offset is added to every index (vocab shards);
 * best_value_f32 (optional) receives the winning bf16 logit as float per
 * token, for the cross-shard combine.  workspace: at least
 * qwen36_lm_head_fp8_argmax_workspace_bytes(rows, n) bytes, zero-filled once
 * before first use (the kernel leaves it zeroed). */
typedef struct {
  size_t rows, cols, n;
  qwen36_device_ptr_t weight_e4m3, row_scales_f32, input_bf16;
  qwen36_device_ptr_t output_token_u32, best_value_f32;
  qwen36_device_ptr_t workspace;
  size_t workspace_bytes;
  uint32_t row_offset;
} qwen36_lm_head_fp8_argmax_spec_t;
size_t qwen36_lm_head_fp8_argmax_workspace_bytes(size_t rows, size_t n);
int qwen36_lm_head_fp8_gemv_argmax(const qwen36_lm_head_fp8_argmax_spec_t *spec);

/* Dequantised NVFP4 weight as float32 [out_features, in_features]:
 * lut(code) * (decode(scale) * tensor_scale), the value the reference matvec
 * multiplies by (kernels-cuda/ops.cu:574-575,622-631).  For parity checks. */
typedef struct {
  size_t out_features, in_features;
  qwen36_device_ptr_t weight_u8, block_scale_e4m3, tensor_scale_f32, output_f32;
} qwen36_nvfp4_dequantize_spec_t;
int qwen36_nvfp4_dequantize(const qwen36_nvfp4_dequantize_spec_t *spec);

/* Host-side producer of the tiled scale layout, for loaders that want to
 * upload block scales already tiled instead of staging them row-major and
 * calling qwen36_nvfp4_retile_scales (crates/runtime/src/gpu.rs:1199-1239).
 * `tiled` must hold qwen36_nvfp4_tiled_scale_bytes(rows, inner_groups) bytes;
 * padding is zero-filled.  Pure CPU code, no CUDA call. */
size_t qwen36_nvfp4_tiled_scale_bytes(size_t rows, size_t inner_groups);
int qwen36_nvfp4_tile_scales_host(const uint8_t *row_major, uint8_t *tiled, size_t rows,
                                  size_t inner_groups);

/* ---- runtime plumbing (replaces kernels-cuda/runtime.cu) ------------------- */

int qwen36_cuda_malloc(qwen36_device_allocation_t *out, size_t bytes);
int qwen36_cuda_free(qwen36_device_ptr_t ptr);
int qwen36_cuda_memcpy_h2d(qwen36_device_ptr_t dst, const void *src, size_t bytes);
int qwen36_cuda_memcpy_d2h(void *dst, qwen36_device_ptr_t src, size_t bytes);
int qwen36_cuda_memcpy_d2d(qwen36_device_ptr_t dst, qwen36_device_ptr_t src, size_t bytes);
int qwen36_cuda_memcpy_d2d_async(qwen36_device_ptr_t dst, qwen36_device_ptr_t src, size_t bytes);
int qwen36_cuda_memset(qwen36_device_ptr_t dst, int value, size_t bytes);
int qwen36_cuda_memset_async(qwen36_device_ptr_t dst, int value, size_t bytes);
int qwen36_cuda_synchronize(void);
int qwen36_cuda_get_diagnostics(qwen36_cuda_diagnostics_t *out);
int qwen36_cuda_counters_reset(void);
int qwen36_cuda_counters_read(qwen36_cuda_counters_t *out);
int qwen36_cuda_set_l2_access_window(qwen36_device_ptr_t base, size_t bytes, float hit_ratio);
int qwen36_cuda_clear_l2_access_window(void);
int qwen36_l2_prefetch(qwen36_device_ptr_t base, size_t bytes, int target_cta_count);
qwen36_cuda_stream_t qwen36_get_active_stream(void);
void qwen36_set_active_stream(qwen36_cuda_stream_t stream);
qwen36_cuda_stream_t qwen36_get_prefetch_stream(void);
void qwen36_set_prefetch_stream(qwen36_cuda_stream_t stream);
qwen36_cuda_stream_t qwen36_internal_active_stream(void);
qwen36_cuda_stream_t qwen36_internal_prefetch_stream(void);
int qwen36_cuda_stream_create(qwen36_cuda_stream_t *out);
int qwen36_cuda_stream_destroy(qwen36_cuda_stream_t stream);
int qwen36_cuda_stream_synchronize(qwen36_cuda_stream_t stream);
int qwen36_cuda_event_create(qwen36_cuda_event_t *out);
int qwen36_cuda_event_destroy(qwen36_cuda_event_t event);
int qwen36_cuda_event_record(qwen36_cuda_event_t event, qwen36_cuda_stream_t stream);
int qwen36_cuda_stream_wait_event(qwen36_cuda_stream_t stream, qwen36_cuda_event_t event);
int qwen36_cuda_stream_begin_capture(qwen36_cuda_stream_t stream);
int qwen36_cuda_stream_end_capture(qwen36_cuda_stream_t stream, qwen36_cuda_graph_t *out);
int qwen36_cuda_graph_instantiate(qwen36_cuda_graph_t graph, qwen36_cuda_graph_exec_t *out);
int qwen36_cuda_graph_destroy(qwen36_cuda_graph_t graph);
int qwen36_cuda_graph_exec_destroy(qwen36_cuda_graph_exec_t exec);
int qwen36_cuda_graph_launch(qwen36_cuda_graph_exec_t exec, qwen36_cuda_stream_t stream);
int qwen36_increment_i32(qwen36_device_ptr_t target_i32);
int qwen36_mtp_assume_accept_chain_advance(qwen36_device_ptr_t position_i32, size_t draft_count,
                                           size_t position_count, int32_t position_delta);

/* ---- exported so crates/kernels links; not part of this path --------------- */
/* Each returns QWEN36_STATUS_NOT_IMPLEMENTED.  The argument is the reference's
 * spec struct for that operator (qwen36_fp4.h), which this build never reads. */
int qwen36_bf16_gemm(const void *spec);
int qwen36_bf16_matvec(const void *spec);
int qwen36_attention_prefill(const void *spec);
int qwen36_attention_flash_prefill(const void *spec);
int qwen36_attention_sage_prefill(const void *spec);
int qwen36_deltanet_decode(const void *spec);
int qwen36_deltanet_prefill(const void *spec);
void qwen36_deltanet_set_resident(int mode);
void qwen36_deltanet_prefill_set_tiny(int mode);
int qwen36_interpreter_decode_sm120(const void *program);
int qwen36_drafter_attention_block_bf16(const void *spec);
int qwen36_drafter_attention_block_flash_bf16(const void *spec);
int qwen36_rmsnorm(const void *spec);
int qwen36_partial_rope(const void *spec);
int qwen36_swiglu(const void *spec);
int qwen36_topk_argmax(const void *spec);
int qwen36_embedding_lookup(const void *spec);
int qwen36_conv1d_update(const void *spec);
int qwen36_conv1d_prefill(const void *spec);
int qwen36_gdn_gate(const void *spec);
int qwen36_conv1d_gdn_gate_fused(const void *spec);
int qwen36_sigmoid_gate(const void *spec);
int qwen36_sigmoid_gate_strided(const void *spec);
int qwen36_q_proj_deinterleave(const void *spec);
int qwen36_q_proj_sigmoid_gate(const void *spec);
int qwen36_copy_strided_rows(const void *spec);

#ifdef __cplusplus
}
#endif
#endif /* QWEN36_FP4_B200_H_ */
