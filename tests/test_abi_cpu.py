"""CPU-only checks of the boundary: the library loads without a GPU, exports every
symbol the header declares, its struct layouts equal the reference header's, the
host-side scale tiling matches the oracle, and entry points reject bad arguments
before touching CUDA."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from oracle import oracle as orc
from speedoza_b200 import abi
from speedoza_b200.build import build_library

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "qwen36_fp4_b200.h")
REF_HEADER = os.path.join(orc.reference_dir(), "kernels-cuda", "include", "qwen36_fp4.h")


@pytest.fixture(scope="module")
def lib():
    build_library()
    return abi.load()


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qwen36_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) > 90
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_reference_abi_symbols_all_present(lib):
    """Every function the reference header declares (what crates/kernels links) resolves."""
    if not os.path.exists(REF_HEADER):
        pytest.skip("reference checkout not present")
    text = re.sub(r"/\*.*?\*/|//[^\n]*", "", open(REF_HEADER).read(), flags=re.S)
    names = sorted(set(re.findall(r"\b(qwen36_[a-z0-9_]+)\s*\(", text)))
    names += ["qwen36_cuda_memset_async", "qwen36_internal_active_stream", "qwen36_internal_prefetch_stream",
              "qwen36_attention_flash_splitk_prefill_bf16", "qwen36_attention_decode_split_tiled",
              "qwen36_drafter_attention_block_flash_bf16"]
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_struct_layouts_equal_reference_header(tmp_path):
    """sizeof/offsetof of every hot-path spec, reference header vs this header, via a C++ TU."""
    if not os.path.exists(REF_HEADER):
        pytest.skip("reference checkout not present")
    structs = {
        "qwen36_nvfp4_gemm_spec_t": ["m", "n", "k", "a_fp4", "a_scale", "a_scale_2", "b_fp4", "b_scale",
                                     "b_scale_2", "c_bf16", "workspace", "workspace_bytes", "alpha"],
        "qwen36_nvfp4_matvec_spec_t": ["out_features", "in_features", "input_bf16", "weight_u8",
                                       "block_scale_e4m3", "tensor_scale_f32", "output_bf16"],
        "qwen36_nvfp4_quantize_spec_t": ["values", "input_bf16", "output_fp4", "output_scale_e4m3",
                                         "output_tensor_scale_f32", "input_tensor_scale_f32"],
        "qwen36_nvfp4_quantize_rows_spec_t": ["rows", "values", "input_bf16", "output_fp4", "output_scale_e4m3",
                                              "output_tensor_scale_f32", "input_tensor_scale_f32"],
        "qwen36_nvfp4_retile_scales_spec_t": ["rows", "inner_groups", "input_row_major_u8", "output_tiled_u8"],
        "qwen36_rmsnorm_nvfp4_quantize_spec_t": ["hidden", "eps", "input_bf16", "weight_bf16", "residual_bf16",
                                                 "residual_out_bf16", "output_bf16", "output_fp4",
                                                 "output_scale_e4m3", "output_tensor_scale_f32",
                                                 "input_tensor_scale_f32"],
        "qwen36_swiglu_nvfp4_quantize_spec_t": ["intermediate", "gate_bf16", "up_bf16", "output_fp4",
                                                "output_scale_e4m3", "output_tensor_scale_f32",
                                                "input_tensor_scale_f32"],
        "qwen36_bf16_matvec_argmax_rows_spec_t": ["rows", "out_features", "in_features", "input_bf16", "weight_bf16",
                                                  "output_token_u32", "mirror_last_output_token_u32", "workspace",
                                                  "workspace_bytes", "skip_flags_u32"],
        "qwen36_lm_head_top2_margin_spec_t": ["rows", "vocab", "eps", "logits_bf16", "tokens_u32", "flags_u32",
                                              "mirror_last_token_u32", "fallback_count_u32", "workspace",
                                              "workspace_bytes"],
        "qwen36_lm_head_top8_rescore_spec_t": ["rows", "vocab", "cols", "eps", "logits_bf16", "weight_bf16",
                                               "input_bf16", "tokens_u32", "flags_u32", "mirror_last_token_u32",
                                               "fallback_count_u32", "workspace", "workspace_bytes"],
        "qwen36_lm_head_fp8_quantize_spec_t": ["rows", "cols", "weight_bf16", "weight_e4m3", "row_scales_f32"],
        "qwen36_lm_head_fp8_gemv_spec_t": ["rows", "cols", "n", "weight_e4m3", "row_scales_f32", "input_bf16",
                                           "output_bf16"],
        "qwen36_sampling_spec_t": ["vocab_size", "logits_bf16", "output_token_u32", "temperature", "top_k",
                                   "top_p", "repetition_penalty", "mirror_output_token_u32"],
        "qwen36_sampling_rows_spec_t": ["rows", "vocab_size", "logits_bf16", "output_token_u32",
                                        "mirror_last_output_token_u32", "temperature"],
        "qwen36_turboquant_encode_spec_t": ["layer_index", "position", "k_bf16", "v_bf16", "k_quantized_i8",
                                            "v_quantized_i8", "metadata_f32", "shape"],
        "qwen36_turboquant_attention_spec_t": ["layer_index", "position", "q_bf16", "k_quantized_i8",
                                               "v_quantized_i8", "metadata_f32", "output_bf16", "workspace",
                                               "workspace_bytes", "shape", "mode"],
        "qwen36_attention_decode_spec_t": ["layer_index", "position", "q_bf16", "k_bf16", "v_bf16", "kv_cache_k",
                                           "kv_cache_v", "kv_cache_metadata", "output_bf16", "shape",
                                           "kv_cache_dtype", "position_device_i32", "partial_acc_f32",
                                           "partial_max_f32", "partial_denom_f32", "decode_n_splits",
                                           "split_timesteps_per_block"],
        "qwen36_attention_prefill_spec_t": ["layer_index", "start_position", "tokens", "q_bf16", "k_bf16", "v_bf16",
                                            "kv_cache_k", "kv_cache_v", "kv_cache_metadata", "output_bf16", "shape",
                                            "kv_cache_dtype", "start_position_device_i32", "partial_acc_f32",
                                            "partial_max_f32", "partial_denom_f32", "prefill_n_splits",
                                            "split_timesteps_per_block", "tree_ancestor_bitmap_u64",
                                            "verify_chunk_rows"],
        "qwen36_attention_shape_t": ["q_heads", "kv_heads", "head_dim", "rope_dims"],
        "qwen36_cuda_counters_t": ["malloc_calls", "graph_launch_calls"],
        "qwen36_cuda_diagnostics_t": ["driver_version", "total_global_mem", "device_name", "last_cuda_error_string"],
        "qwen36_device_allocation_t": ["ptr", "bytes"],
    }
    lines = ["#include <stddef.h>", "#include <stdint.h>", "#include <cstddef>", "#include <cstdio>",
             "namespace ref {", f'#include "{REF_HEADER}"', "}",
             "namespace mine {", f'#include "{HEADER}"', "}", "int main() { int bad = 0;"]
    for s, fields in structs.items():
        lines.append(f'  if (sizeof(ref::{s}) != sizeof(mine::{s})) {{ printf("sizeof {s}\\n"); bad++; }}')
        for f in fields:
            lines.append(f'  if (offsetof(ref::{s}, {f}) != offsetof(mine::{s}, {f})) '
                         f'{{ printf("offsetof {s}.{f}\\n"); bad++; }}')
    lines += ['  static_assert(int(ref::QWEN36_STATUS_NOT_IMPLEMENTED) == int(mine::QWEN36_STATUS_NOT_IMPLEMENTED), "");',
              '  static_assert(int(ref::QWEN36_STATUS_CUDA_ERROR) == int(mine::QWEN36_STATUS_CUDA_ERROR), "");',
              "  return bad; }"]
    src = tmp_path / "layout.cpp"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["/usr/bin/g++", "-std=c++17", "-Wno-invalid-offsetof", str(src), "-o", str(exe)], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout


def test_ctypes_mirrors_match_header_sizes(tmp_path):
    names = {"qwen36_nvfp4_gemm_spec_t": abi.Nvfp4GemmSpec, "qwen36_nvfp4_matvec_spec_t": abi.Nvfp4MatvecSpec,
             "qwen36_nvfp4_quantize_rows_spec_t": abi.Nvfp4QuantizeRowsSpec,
             "qwen36_rmsnorm_nvfp4_quantize_spec_t": abi.RmsnormNvfp4QuantizeSpec,
             "qwen36_bf16_matvec_argmax_rows_spec_t": abi.Bf16MatvecArgmaxRowsSpec,
             "qwen36_lm_head_top2_margin_spec_t": abi.LmHeadTop2MarginSpec,
             "qwen36_lm_head_top8_rescore_spec_t": abi.LmHeadTop8RescoreSpec,
             "qwen36_swiglu_nvfp4_quantize_spec_t": abi.SwigluNvfp4QuantizeSpec,
             "qwen36_swiglu_nvfp4_quantize_rows_spec_t": abi.SwigluNvfp4QuantizeRowsSpec,
             "qwen36_lm_head_fp8_argmax_spec_t": abi.LmHeadFp8ArgmaxSpec,
             "qwen36_lm_head_fp8_gemv_spec_t": abi.LmHeadFp8GemvSpec,
             "qwen36_sampling_spec_t": abi.SamplingSpec, "qwen36_sampling_rows_spec_t": abi.SamplingRowsSpec,
             "qwen36_turboquant_encode_spec_t": abi.TurboquantEncodeSpec,
             "qwen36_turboquant_encode_rows_spec_t": abi.TurboquantEncodeRowsSpec,
             "qwen36_turboquant_attention_spec_t": abi.TurboquantAttentionSpec,
             "qwen36_attention_decode_spec_t": abi.AttentionDecodeSpec,
             "qwen36_attention_prefill_spec_t": abi.AttentionPrefillSpec,
             "qwen36_turboquant_attention_partial_spec_t": abi.TurboquantAttentionPartialSpec,
             "qwen36_attention_merge_spec_t": abi.AttentionMergeSpec,
             "qwen36_attention_peer_merge_spec_t": abi.AttentionPeerMergeSpec,
             "qwen36_argmax_peer_combine_spec_t": abi.ArgmaxPeerCombineSpec,
             "qwen36_turboquant_attention_peer_spec_t": abi.TurboquantAttentionPeerSpec,
             "qwen36_nvfp4_dequantize_spec_t": abi.Nvfp4DequantizeSpec,
             "qwen36_cuda_diagnostics_t": abi.CudaDiagnostics, "qwen36_cuda_counters_t": abi.CudaCounters}
    body = "\n".join(f'  printf("{n} %zu\\n", sizeof({n}));' for n in names)
    src = tmp_path / "sizes.c"
    src.write_text(f'#include <stdio.h>\n#include "{HEADER}"\nint main(void) {{\n{body}\n  return 0; }}\n')
    exe = tmp_path / "sizes"
    subprocess.run(["/usr/bin/gcc", str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout
    for line in out.strip().splitlines():
        n, sz = line.split()
        assert C.sizeof(names[n]) == int(sz), n


def test_host_scale_tiling_matches_oracle(lib):
    rng = np.random.default_rng(5)
    for rows, groups in ((1, 1), (130, 12), (257, 7), (128, 320)):
        sf = rng.integers(0, 256, size=(rows, groups), dtype=np.uint8)
        want = orc.retile_scales(sf)
        assert lib.qwen36_nvfp4_tiled_scale_bytes(rows, groups) == want.size
        got = np.full(want.size, 0xAA, dtype=np.uint8)
        rc = lib.qwen36_nvfp4_tile_scales_host(sf.ctypes.data, got.ctypes.data, rows, groups)
        assert rc == abi.SUCCESS and np.array_equal(got, want)
    assert lib.qwen36_nvfp4_tile_scales_host(None, None, 1, 1) == abi.NULL_POINTER


def test_argument_validation_needs_no_gpu(lib):
    assert lib.qwen36_nvfp4_gemm(None) == abi.NULL_POINTER
    assert lib.qwen36_nvfp4_matvec(None) == abi.NULL_POINTER
    assert lib.qwen36_nvfp4_gemm(C.byref(abi.Nvfp4GemmSpec())) == abi.INVALID_ARGUMENT
    assert lib.qwen36_decode_nvfp4_gemv(C.byref(abi.Nvfp4GemmSpec())) == abi.INVALID_ARGUMENT
    assert lib.qwen36_nvfp4_matvec(C.byref(abi.Nvfp4MatvecSpec())) == abi.INVALID_ARGUMENT
    assert lib.qwen36_nvfp4_quantize_rows(C.byref(abi.Nvfp4QuantizeRowsSpec())) == abi.INVALID_ARGUMENT
    assert lib.qwen36_lm_head_fp8_gemv(C.byref(abi.LmHeadFp8GemvSpec())) == abi.INVALID_ARGUMENT
    assert lib.qwen36_turboquant_attention(C.byref(abi.TurboquantAttentionSpec())) == abi.INVALID_ARGUMENT
    assert lib.qwen36_sample_rows(C.byref(abi.SamplingRowsSpec())) == abi.INVALID_ARGUMENT
    assert lib.qwen36_attention_peer_merge(None) == abi.NULL_POINTER
    assert lib.qwen36_attention_peer_merge(C.byref(abi.AttentionPeerMergeSpec())) == abi.INVALID_ARGUMENT
    assert lib.qwen36_argmax_peer_combine(C.byref(abi.ArgmaxPeerCombineSpec())) == abi.INVALID_ARGUMENT
    assert lib.qwen36_ipc_get_handle(abi.DevicePtr(0), None) == abi.NULL_POINTER
    assert lib.qwen36_swiglu_nvfp4_quantize_rows(None) == abi.NULL_POINTER
    assert lib.qwen36_swiglu_nvfp4_quantize_rows(C.byref(abi.SwigluNvfp4QuantizeRowsSpec())) == abi.INVALID_ARGUMENT
    ragged = abi.SwigluNvfp4QuantizeRowsSpec(rows=4, intermediate=40, input_row_stride=40, gate_bf16=abi.DevicePtr(16),
                                             up_bf16=abi.DevicePtr(16), output_fp4=abi.DevicePtr(16),
                                             output_scale_e4m3=abi.DevicePtr(16))
    assert lib.qwen36_swiglu_nvfp4_quantize_rows(C.byref(ragged)) == abi.INVALID_ARGUMENT      # whole 16-groups only
    # out-of-scope operators link and decline
    assert lib.qwen36_rmsnorm(None) == abi.NOT_IMPLEMENTED
    assert lib.qwen36_attention_flash_splitk_prefill_bf16(None, 4) == abi.NULL_POINTER
    assert lib.qwen36_attention_flash_splitk_prefill_bf16(C.byref(abi.AttentionPrefillSpec()), 4) == abi.INVALID_ARGUMENT
    assert lib.qwen36_attention_decode_split_tiled(None, 4, 64) == abi.NULL_POINTER
    assert lib.qwen36_attention_decode_split_tiled(C.byref(abi.AttentionDecodeSpec()), 4, 64) == abi.NOT_IMPLEMENTED
    # n > 8 on the decode GEMV entry is the soft "use the GEMM" code
    spec = abi.Nvfp4GemmSpec(m=128, n=9, k=256, a_fp4=abi.DevicePtr(16), a_scale=abi.DevicePtr(16),
                             b_fp4=abi.DevicePtr(16), b_scale=abi.DevicePtr(16), c_bf16=abi.DevicePtr(16))
    assert lib.qwen36_decode_nvfp4_gemv(C.byref(spec)) == abi.NOT_IMPLEMENTED


def test_runtime_entry_points_keep_the_reference_status_codes(lib):
    """kernels-cuda/runtime.cu:247-287 and decode_gemv/l2_prefetch.cu:41-53: a null target is
    INVALID_ARGUMENT (not NULL_POINTER), the MTP position advance refuses 0 or more than 4 drafts, an
    empty position list and a non-positive delta, a zero-byte prefetch is refused, and a failed
    malloc leaves an empty allocation behind.  All of it is decided before any CUDA call."""
    null, some = abi.DevicePtr(0), abi.DevicePtr(256)
    lib.qwen36_mtp_assume_accept_chain_advance.argtypes = [abi.DevicePtr, C.c_size_t, C.c_size_t, C.c_int32]
    lib.qwen36_l2_prefetch.argtypes = [abi.DevicePtr, C.c_size_t, C.c_int]
    lib.qwen36_increment_i32.argtypes = [abi.DevicePtr]
    assert lib.qwen36_increment_i32(null) == abi.INVALID_ARGUMENT
    adv = lib.qwen36_mtp_assume_accept_chain_advance
    assert adv(null, 1, 1, 1) == abi.INVALID_ARGUMENT
    for drafts, count, delta in ((0, 1, 1), (5, 1, 1), (2, 0, 1), (2, 3, 0), (2, 3, -1)):
        assert adv(some, drafts, count, delta) == abi.INVALID_ARGUMENT
    assert lib.qwen36_l2_prefetch(null, 64, 0) == abi.INVALID_ARGUMENT
    assert lib.qwen36_l2_prefetch(some, 0, 0) == abi.INVALID_ARGUMENT
    alloc = abi.DeviceAllocation(abi.DevicePtr(0xdead), 77)
    assert lib.qwen36_cuda_malloc(C.byref(alloc), 0) == abi.INVALID_ARGUMENT
    assert alloc.ptr.ptr == 0 and alloc.bytes == 0
    assert lib.qwen36_cuda_malloc(None, 16) == abi.NULL_POINTER


def test_product_code_never_touches_the_oracle():
    """Nothing under the package may import, load or mention the oracle."""
    pkg = os.path.join(ROOT, "speedoza_b200")
    for dirpath, _, files in os.walk(pkg):
        if "lib" in dirpath.split(os.sep):
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp", ".hpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "liboracle" not in text and "import oracle" not in text and "from oracle" not in text, f


def test_verify_attention_split_count_fills_the_sms_once():
    from speedoza_b200.backend import CudaBackend
    f = CudaBackend.attention_verify_splits
    assert f(4, 24, 4) == 37            # 24 rows per kv head: one CTA per (kv head, split) on 148 SMs
    assert f(16, 24, 4) == 18           # 96 rows: two row chunks per split
    assert f(32, 24, 4) == 12           # 192 rows: three
    assert f(1, 24, 4, sms=4) == 1 and f(32, 64, 1, sms=2) == 1      # never below one split
