"""ctypes view of the C ABI declared in include/qwen36_fp4_b200.h.

The library is the product; this module only loads it and mirrors its structs.
There is no fallback: if libqwen36_fp4_kernels.so is missing or a symbol does
not resolve, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libqwen36_fp4_kernels.so")

SUCCESS, NULL_POINTER, INVALID_ARGUMENT, CUDA_ERROR, CUBLAS_ERROR, NOT_IMPLEMENTED = range(6)
STATUS_NAMES = ["SUCCESS", "NULL_POINTER", "INVALID_ARGUMENT", "CUDA_ERROR", "CUBLAS_ERROR",
                "NOT_IMPLEMENTED"]

size_t = C.c_size_t


class DevicePtr(C.Structure):
    _fields_ = [("ptr", C.c_uint64)]


class DeviceAllocation(C.Structure):
    _fields_ = [("ptr", DevicePtr), ("bytes", size_t)]


class AttentionShape(C.Structure):
    _fields_ = [("q_heads", size_t), ("kv_heads", size_t), ("head_dim", size_t), ("rope_dims", size_t)]


class Nvfp4GemmSpec(C.Structure):
    _fields_ = [("m", size_t), ("n", size_t), ("k", size_t),
                ("a_fp4", DevicePtr), ("a_scale", DevicePtr), ("a_scale_2", DevicePtr),
                ("b_fp4", DevicePtr), ("b_scale", DevicePtr), ("b_scale_2", DevicePtr),
                ("c_bf16", DevicePtr), ("workspace", DevicePtr), ("workspace_bytes", size_t),
                ("alpha", C.c_float)]


class Nvfp4MatvecSpec(C.Structure):
    _fields_ = [("out_features", size_t), ("in_features", size_t), ("input_bf16", DevicePtr),
                ("weight_u8", DevicePtr), ("block_scale_e4m3", DevicePtr),
                ("tensor_scale_f32", DevicePtr), ("output_bf16", DevicePtr)]


PEER_INPUT_LOCAL = (1 << (8 * C.sizeof(size_t))) - 1


class Nvfp4MatvecPeerSpec(C.Structure):
    _fields_ = [("world", size_t), ("rank", size_t), ("peer_arena", DevicePtr), ("state", DevicePtr), ("slots", size_t), ("out_slot", size_t), ("in_slot", size_t),
                ("output_offset_bytes", size_t * 4), ("row_offset", size_t * 4)]


class Nvfp4QuantizeSpec(C.Structure):
    _fields_ = [("values", size_t), ("input_bf16", DevicePtr), ("output_fp4", DevicePtr),
                ("output_scale_e4m3", DevicePtr), ("output_tensor_scale_f32", DevicePtr),
                ("input_tensor_scale_f32", C.c_float)]


class Nvfp4QuantizeRowsSpec(C.Structure):
    _fields_ = [("rows", size_t), ("values", size_t), ("input_bf16", DevicePtr),
                ("output_fp4", DevicePtr), ("output_scale_e4m3", DevicePtr),
                ("output_tensor_scale_f32", DevicePtr), ("input_tensor_scale_f32", C.c_float)]


class RmsnormNvfp4QuantizeSpec(C.Structure):
    _fields_ = [("hidden", size_t), ("eps", C.c_float), ("input_bf16", DevicePtr), ("weight_bf16", DevicePtr),
                ("residual_bf16", DevicePtr), ("residual_out_bf16", DevicePtr), ("output_bf16", DevicePtr),
                ("output_fp4", DevicePtr), ("output_scale_e4m3", DevicePtr),
                ("output_tensor_scale_f32", DevicePtr), ("input_tensor_scale_f32", C.c_float)]


class SwigluNvfp4QuantizeSpec(C.Structure):
    _fields_ = [("intermediate", size_t), ("gate_bf16", DevicePtr), ("up_bf16", DevicePtr),
                ("output_fp4", DevicePtr), ("output_scale_e4m3", DevicePtr),
                ("output_tensor_scale_f32", DevicePtr), ("input_tensor_scale_f32", C.c_float)]


class SwigluNvfp4QuantizeRowsSpec(C.Structure):
    _fields_ = [("rows", size_t), ("intermediate", size_t), ("input_row_stride", size_t), ("gate_bf16", DevicePtr),
                ("up_bf16", DevicePtr), ("output_fp4", DevicePtr), ("output_scale_e4m3", DevicePtr),
                ("output_tensor_scale_f32", DevicePtr), ("input_tensor_scale_f32", C.c_float)]


class Bf16MatvecArgmaxRowsSpec(C.Structure):
    _fields_ = [("rows", size_t), ("out_features", size_t), ("in_features", size_t), ("input_bf16", DevicePtr),
                ("weight_bf16", DevicePtr), ("output_token_u32", DevicePtr),
                ("mirror_last_output_token_u32", DevicePtr), ("workspace", DevicePtr), ("workspace_bytes", size_t),
                ("skip_flags_u32", DevicePtr)]


class LmHeadTop2MarginSpec(C.Structure):
    _fields_ = [("rows", size_t), ("vocab", size_t), ("eps", C.c_float), ("logits_bf16", DevicePtr),
                ("tokens_u32", DevicePtr), ("flags_u32", DevicePtr), ("mirror_last_token_u32", DevicePtr),
                ("fallback_count_u32", DevicePtr), ("workspace", DevicePtr), ("workspace_bytes", size_t)]


class LmHeadTop8RescoreSpec(C.Structure):
    _fields_ = [("rows", size_t), ("vocab", size_t), ("cols", size_t), ("eps", C.c_float), ("logits_bf16", DevicePtr),
                ("weight_bf16", DevicePtr), ("input_bf16", DevicePtr), ("tokens_u32", DevicePtr),
                ("flags_u32", DevicePtr), ("mirror_last_token_u32", DevicePtr), ("fallback_count_u32", DevicePtr),
                ("workspace", DevicePtr), ("workspace_bytes", size_t)]


class Nvfp4RetileScalesSpec(C.Structure):
    _fields_ = [("rows", size_t), ("inner_groups", size_t), ("input_row_major_u8", DevicePtr),
                ("output_tiled_u8", DevicePtr)]


class Nvfp4DequantizeSpec(C.Structure):
    _fields_ = [("out_features", size_t), ("in_features", size_t), ("weight_u8", DevicePtr),
                ("block_scale_e4m3", DevicePtr), ("tensor_scale_f32", DevicePtr),
                ("output_f32", DevicePtr)]


class LmHeadFp8QuantizeSpec(C.Structure):
    _fields_ = [("rows", size_t), ("cols", size_t), ("weight_bf16", DevicePtr),
                ("weight_e4m3", DevicePtr), ("row_scales_f32", DevicePtr)]


class LmHeadFp8GemvSpec(C.Structure):
    _fields_ = [("rows", size_t), ("cols", size_t), ("n", size_t), ("weight_e4m3", DevicePtr),
                ("row_scales_f32", DevicePtr), ("input_bf16", DevicePtr), ("output_bf16", DevicePtr)]


class LmHeadFp8ArgmaxSpec(C.Structure):
    _fields_ = [("rows", size_t), ("cols", size_t), ("n", size_t), ("weight_e4m3", DevicePtr),
                ("row_scales_f32", DevicePtr), ("input_bf16", DevicePtr),
                ("output_token_u32", DevicePtr), ("best_value_f32", DevicePtr),
                ("workspace", DevicePtr), ("workspace_bytes", size_t), ("row_offset", C.c_uint32)]


class SamplingSpec(C.Structure):
    _fields_ = [("vocab_size", size_t), ("logits_bf16", DevicePtr), ("output_token_u32", DevicePtr),
                ("temperature", C.c_float), ("top_k", size_t), ("top_p", C.c_float),
                ("repetition_penalty", C.c_float), ("mirror_output_token_u32", DevicePtr)]


class SamplingRowsSpec(C.Structure):
    _fields_ = [("rows", size_t), ("vocab_size", size_t), ("logits_bf16", DevicePtr),
                ("output_token_u32", DevicePtr), ("mirror_last_output_token_u32", DevicePtr),
                ("temperature", C.c_float)]


class TurboquantEncodeSpec(C.Structure):
    _fields_ = [("layer_index", size_t), ("position", size_t), ("k_bf16", DevicePtr),
                ("v_bf16", DevicePtr), ("k_quantized_i8", DevicePtr), ("v_quantized_i8", DevicePtr),
                ("metadata_f32", DevicePtr), ("shape", AttentionShape)]


class TurboquantEncodeRowsSpec(C.Structure):
    _fields_ = [("position", size_t), ("tokens", size_t), ("k_bf16", DevicePtr), ("v_bf16", DevicePtr),
                ("k_quantized_i8", DevicePtr), ("v_quantized_i8", DevicePtr),
                ("metadata_f32", DevicePtr), ("shape", AttentionShape)]


class TurboquantAttentionSpec(C.Structure):
    _fields_ = [("layer_index", size_t), ("position", size_t), ("q_bf16", DevicePtr),
                ("k_quantized_i8", DevicePtr), ("v_quantized_i8", DevicePtr),
                ("metadata_f32", DevicePtr), ("output_bf16", DevicePtr), ("workspace", DevicePtr),
                ("workspace_bytes", size_t), ("shape", AttentionShape), ("mode", C.c_int)]


class AttentionDecodeSpec(C.Structure):
    _fields_ = [("layer_index", size_t), ("position", size_t), ("q_bf16", DevicePtr), ("k_bf16", DevicePtr),
                ("v_bf16", DevicePtr), ("kv_cache_k", DevicePtr), ("kv_cache_v", DevicePtr),
                ("kv_cache_metadata", DevicePtr), ("output_bf16", DevicePtr), ("shape", AttentionShape),
                ("kv_cache_dtype", C.c_int), ("position_device_i32", DevicePtr),
                ("partial_acc_f32", DevicePtr), ("partial_max_f32", DevicePtr), ("partial_denom_f32", DevicePtr),
                ("decode_n_splits", size_t), ("split_timesteps_per_block", size_t)]


class AttentionPrefillSpec(C.Structure):
    _fields_ = [("layer_index", size_t), ("start_position", size_t), ("tokens", size_t), ("q_bf16", DevicePtr),
                ("k_bf16", DevicePtr), ("v_bf16", DevicePtr), ("kv_cache_k", DevicePtr), ("kv_cache_v", DevicePtr),
                ("kv_cache_metadata", DevicePtr), ("output_bf16", DevicePtr), ("shape", AttentionShape),
                ("kv_cache_dtype", C.c_int), ("start_position_device_i32", DevicePtr),
                ("partial_acc_f32", DevicePtr), ("partial_max_f32", DevicePtr), ("partial_denom_f32", DevicePtr),
                ("prefill_n_splits", size_t), ("split_timesteps_per_block", size_t),
                ("tree_ancestor_bitmap_u64", DevicePtr), ("verify_chunk_rows", size_t)]


class TurboquantAttentionPartialSpec(C.Structure):
    _fields_ = [("t_begin", size_t), ("t_end", size_t), ("q_bf16", DevicePtr),
                ("k_quantized_i8", DevicePtr), ("v_quantized_i8", DevicePtr),
                ("metadata_f32", DevicePtr), ("partial_acc_f32", DevicePtr),
                ("partial_max_f32", DevicePtr), ("partial_denom_f32", DevicePtr),
                ("workspace", DevicePtr), ("workspace_bytes", size_t), ("shape", AttentionShape)]


class AttentionMergeSpec(C.Structure):
    _fields_ = [("q_heads", size_t), ("head_dim", size_t), ("n_parts", size_t),
                ("partial_acc_f32", DevicePtr), ("partial_max_f32", DevicePtr),
                ("partial_denom_f32", DevicePtr), ("output_bf16", DevicePtr)]


class AttentionPeerMergeSpec(C.Structure):
    _fields_ = [("world", size_t), ("rank", size_t), ("q_heads", size_t), ("head_dim", size_t),
                ("partial_acc_f32", DevicePtr), ("partial_max_f32", DevicePtr), ("partial_denom_f32", DevicePtr),
                ("peer_inbox", DevicePtr), ("peer_flags", DevicePtr), ("state", DevicePtr),
                ("output_bf16", DevicePtr)]


class TurboquantAttentionPeerSpec(C.Structure):
    _fields_ = [("t_begin", size_t), ("t_end", size_t), ("q_bf16", DevicePtr),
                ("k_quantized_i8", DevicePtr), ("v_quantized_i8", DevicePtr), ("metadata_f32", DevicePtr),
                ("workspace", DevicePtr), ("workspace_bytes", size_t), ("shape", AttentionShape),
                ("world", size_t), ("rank", size_t), ("peer_inbox", DevicePtr), ("peer_flags", DevicePtr),
                ("state", DevicePtr), ("output_bf16", DevicePtr)]


class ArgmaxPeerCombineSpec(C.Structure):
    _fields_ = [("world", size_t), ("rank", size_t), ("tokens", size_t),
                ("best_value_f32", DevicePtr), ("best_index_u32", DevicePtr),
                ("peer_inbox", DevicePtr), ("peer_flags", DevicePtr), ("state", DevicePtr),
                ("output_token_u32", DevicePtr)]


class CudaCounters(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "malloc_calls", "free_calls", "h2d_calls", "h2d_bytes", "d2h_calls", "d2h_bytes", "d2d_calls",
        "d2d_bytes", "d2d_async_calls", "d2d_async_bytes", "memset_calls", "memset_bytes",
        "synchronize_calls", "stream_synchronize_calls", "graph_launch_calls")]


class CudaDiagnostics(C.Structure):
    _fields_ = [("driver_version", C.c_int), ("runtime_version", C.c_int), ("device_count", C.c_int),
                ("active_device", C.c_int), ("sm_major", C.c_int), ("sm_minor", C.c_int),
                ("multiprocessor_count", C.c_int), ("total_global_mem", size_t),
                ("device_name", C.c_char * 128), ("libcuda_path", C.c_char * 512),
                ("cudart_path", C.c_char * 512), ("last_cuda_error", C.c_int),
                ("last_cuda_error_name", C.c_char * 64), ("last_cuda_error_string", C.c_char * 256)]


class KernelError(RuntimeError):
    """A non-zero status from the library (the Rust side's CoreError::KernelLaunch)."""

    def __init__(self, kernel: str, code: int):
        name = STATUS_NAMES[code] if 0 <= code < len(STATUS_NAMES) else str(code)
        super().__init__(f"{kernel} returned {code} ({name})")
        self.kernel = kernel
        self.code = code


_lib = None


def load() -> C.CDLL:
    """Loads the kernel library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m speedoza_b200.build` "
            "(there is no CPU or PyTorch fallback for these kernels)")
    lib = C.CDLL(LIB_PATH)
    lib.qwen36_get_active_stream.restype = C.c_void_p
    lib.qwen36_internal_active_stream.restype = C.c_void_p
    lib.qwen36_get_prefetch_stream.restype = C.c_void_p
    lib.qwen36_set_active_stream.argtypes = [C.c_void_p]
    lib.qwen36_set_active_stream.restype = None
    lib.qwen36_set_prefetch_stream.argtypes = [C.c_void_p]
    lib.qwen36_set_prefetch_stream.restype = None
    lib.qwen36_turboquant_attention_workspace_bytes.restype = size_t
    lib.qwen36_turboquant_attention_workspace_bytes.argtypes = [size_t, size_t]
    lib.qwen36_lm_head_fp8_argmax_workspace_bytes.restype = size_t
    lib.qwen36_lm_head_fp8_argmax_workspace_bytes.argtypes = [size_t, size_t]
    lib.qwen36_nvfp4_tiled_scale_bytes.restype = size_t
    lib.qwen36_nvfp4_tiled_scale_bytes.argtypes = [size_t, size_t]
    lib.qwen36_nvfp4_tile_scales_host.argtypes = [C.c_void_p, C.c_void_p, size_t, size_t]
    lib.qwen36_cuda_malloc.argtypes = [C.POINTER(DeviceAllocation), size_t]
    lib.qwen36_cuda_free.argtypes = [DevicePtr]
    lib.qwen36_cuda_memcpy_h2d.argtypes = [DevicePtr, C.c_void_p, size_t]
    lib.qwen36_cuda_memcpy_d2h.argtypes = [C.c_void_p, DevicePtr, size_t]
    lib.qwen36_cuda_memcpy_d2d.argtypes = [DevicePtr, DevicePtr, size_t]
    lib.qwen36_cuda_memcpy_d2d_async.argtypes = [DevicePtr, DevicePtr, size_t]
    lib.qwen36_cuda_memset.argtypes = [DevicePtr, C.c_int, size_t]
    lib.qwen36_cuda_memset_async.argtypes = [DevicePtr, C.c_int, size_t]
    lib.qwen36_cuda_stream_create.argtypes = [C.POINTER(C.c_void_p)]
    lib.qwen36_cuda_stream_destroy.argtypes = [C.c_void_p]
    lib.qwen36_cuda_stream_synchronize.argtypes = [C.c_void_p]
    lib.qwen36_cuda_stream_begin_capture.argtypes = [C.c_void_p]
    lib.qwen36_cuda_stream_end_capture.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    lib.qwen36_cuda_graph_instantiate.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    lib.qwen36_cuda_graph_destroy.argtypes = [C.c_void_p]
    lib.qwen36_cuda_graph_exec_destroy.argtypes = [C.c_void_p]
    lib.qwen36_cuda_graph_launch.argtypes = [C.c_void_p, C.c_void_p]
    lib.qwen36_cuda_event_create.argtypes = [C.POINTER(C.c_void_p)]
    lib.qwen36_cuda_event_destroy.argtypes = [C.c_void_p]
    lib.qwen36_cuda_event_record.argtypes = [C.c_void_p, C.c_void_p]
    lib.qwen36_cuda_stream_wait_event.argtypes = [C.c_void_p, C.c_void_p]
    lib.qwen36_increment_i32.argtypes = [DevicePtr]
    lib.qwen36_mtp_assume_accept_chain_advance.argtypes = [DevicePtr, size_t, size_t, C.c_int32]
    lib.qwen36_l2_prefetch.argtypes = [DevicePtr, size_t, C.c_int]
    lib.qwen36_cuda_set_l2_access_window.argtypes = [DevicePtr, size_t, C.c_float]
    lib.qwen36_ipc_get_handle.argtypes = [DevicePtr, C.c_void_p]
    lib.qwen36_ipc_open_handle.argtypes = [C.c_void_p, C.POINTER(DevicePtr)]
    lib.qwen36_ipc_close_handle.argtypes = [DevicePtr]
    lib.qwen36_attention_peer_inbox_bytes.restype = size_t
    lib.qwen36_attention_peer_inbox_bytes.argtypes = [size_t, size_t, size_t]
    lib.qwen36_argmax_peer_inbox_bytes.restype = size_t
    lib.qwen36_argmax_peer_inbox_bytes.argtypes = [size_t, size_t]
    lib.qwen36_attention_decode_set_mode.restype = None
    lib.qwen36_attention_decode_set_mode.argtypes = [C.c_int]
    lib.qwen36_attention_decode_force_splits.restype = None
    lib.qwen36_attention_decode_force_splits.argtypes = [C.c_int]
    lib.qwen36_nvfp4_chunk_gemv_set_mtile.restype = None
    lib.qwen36_nvfp4_matvec_force_quads.restype = None
    lib.qwen36_nvfp4_gemm_force_bn.restype = None
    lib.qwen36_nvfp4_gemm_force_bn.argtypes = [C.c_int]
    lib.qwen36_nvfp4_gemm_stream_k.restype = None
    lib.qwen36_nvfp4_gemm_stream_k.argtypes = [C.c_int]
    lib.qwen36_nvfp4_gemm_force_split.restype = None
    lib.qwen36_nvfp4_gemm_force_split.argtypes = [C.c_int]
    lib.qwen36_nvfp4_matvec_group.argtypes = [C.POINTER(Nvfp4MatvecSpec), size_t]
    lib.qwen36_nvfp4_matvec_peer.argtypes = [C.POINTER(Nvfp4MatvecSpec), size_t, C.POINTER(Nvfp4MatvecPeerSpec)]
    lib.qwen36_nvfp4_matvec_peer_collect.argtypes = [C.POINTER(Nvfp4MatvecPeerSpec), size_t, DevicePtr, size_t, DevicePtr]
    lib.qwen36_nvfp4_matvec_force_quads.argtypes = [C.c_int]
    lib.qwen36_attention_flash_splitk_prefill_bf16.argtypes = [C.POINTER(AttentionPrefillSpec), C.c_int]
    lib.qwen36_attention_decode_split_tiled.argtypes = [C.POINTER(AttentionDecodeSpec), C.c_int, C.c_int]
    lib.qwen36_lm_head_fp8_gemv_set_route.restype = None
    lib.qwen36_lm_head_fp8_gemv_set_route.argtypes = [C.c_int]
    lib.qwen36_nvfp4_quantize_set_path.restype = None
    lib.qwen36_nvfp4_quantize_set_path.argtypes = [C.c_int]
    _lib = lib
    return lib
