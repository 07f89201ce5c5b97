"""Host-side mirror of the reference's ``KernelBackend`` for the hot path.

Method names, argument meaning and error behaviour follow
crates/kernels/src/backend.rs:38-275 of the reference: each method fills the
C spec struct and calls the matching ``qwen36_*`` entry point of
libqwen36_fp4_kernels.so; a non-zero status raises ``KernelError`` (the Rust
side's ``CoreError::KernelLaunch``), and ``nvfp4_gemm`` keeps the reference's
routing (decode GEMV first for n == 1, GEMM entry on NOT_IMPLEMENTED).

Tensors are torch CUDA tensors used purely as device buffers; all arithmetic
happens inside the library.  bf16 tensors are ``torch.bfloat16``; packed FP4,
scale bytes and FP8 weights are ``torch.uint8``; int8 caches ``torch.int8``.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import abi
from .abi import DevicePtr, KernelError


def _dp(t) -> DevicePtr:
    return DevicePtr(0 if t is None else t.data_ptr())


def _check(name: str, code: int) -> None:
    if code != abi.SUCCESS:
        raise KernelError(name, code)


def tiled_scale_bytes(rows: int, inner_groups: int) -> int:
    return int(abi.load().qwen36_nvfp4_tiled_scale_bytes(rows, inner_groups))


class CudaBackend:
    """One instance per process/device.  Launches go to torch's current stream:
    ``sync_stream()`` points the library's ambient stream at it."""

    name = "cuda-sm100a"

    def __init__(self) -> None:
        self.lib = abi.load()
        if not torch.cuda.is_available():
            raise RuntimeError("CudaBackend needs a CUDA device; there is no CPU fallback")
        self.sync_stream()

    # -- plumbing ---------------------------------------------------------
    def sync_stream(self) -> None:
        self.lib.qwen36_set_active_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))

    # -- NVFP4 ------------------------------------------------------------
    def nvfp4_retile_scales(self, sf_row_major: torch.Tensor) -> torch.Tensor:
        rows, groups = sf_row_major.shape
        out = torch.empty(tiled_scale_bytes(rows, groups), dtype=torch.uint8, device=sf_row_major.device)
        spec = abi.Nvfp4RetileScalesSpec(rows, groups, _dp(sf_row_major), _dp(out))
        _check("nvfp4_retile_scales", self.lib.qwen36_nvfp4_retile_scales(C.byref(spec)))
        return out

    def nvfp4_quantize_rows(self, x_bf16: torch.Tensor, input_tensor_scale: float = 0.0,
                            out_fp4=None, out_sf=None, out_ts=None):
        """x [rows, values] -> (fp4 [rows, values/2], tiled scales, tensor scale [1] f32)."""
        rows, values = x_bf16.shape
        dev = x_bf16.device
        if out_fp4 is None:
            out_fp4 = torch.empty((rows, (values + 1) // 2), dtype=torch.uint8, device=dev)
        if out_sf is None:
            out_sf = torch.zeros(tiled_scale_bytes(rows, (values + 15) // 16), dtype=torch.uint8, device=dev)
        if out_ts is None:
            out_ts = torch.empty(1, dtype=torch.float32, device=dev)
        spec = abi.Nvfp4QuantizeRowsSpec(rows, values, _dp(x_bf16), _dp(out_fp4), _dp(out_sf), _dp(out_ts),
                                         input_tensor_scale)
        _check("nvfp4_quantize_rows", self.lib.qwen36_nvfp4_quantize_rows(C.byref(spec)))
        return out_fp4, out_sf, out_ts

    def nvfp4_quantize_bf16(self, x_bf16: torch.Tensor, input_tensor_scale: float = 0.0):
        values = x_bf16.numel()
        dev = x_bf16.device
        out_fp4 = torch.empty((values + 1) // 2, dtype=torch.uint8, device=dev)
        out_sf = torch.zeros(tiled_scale_bytes(1, (values + 15) // 16), dtype=torch.uint8, device=dev)
        out_ts = torch.empty(1, dtype=torch.float32, device=dev)
        spec = abi.Nvfp4QuantizeSpec(values, _dp(x_bf16), _dp(out_fp4), _dp(out_sf), _dp(out_ts),
                                     input_tensor_scale)
        _check("nvfp4_quantize_bf16", self.lib.qwen36_nvfp4_quantize_bf16(C.byref(spec)))
        return out_fp4, out_sf, out_ts

    def rmsnorm_nvfp4_quantize(self, x_bf16, weight_bf16, residual_bf16=None, eps: float = 1e-6,
                               input_tensor_scale: float = 0.0, want_bf16: bool = True, want_residual_out: bool = False,
                               buffers=None):
        """One vector (crates/kernels/src/backend.rs `rmsnorm_nvfp4_quantize`).
        -> (out_bf16 | None, residual_out | None, fp4, tiled scales, tensor scale [1]);
        `buffers` = a previous result to write into instead of allocating."""
        hidden = x_bf16.numel()
        dev = x_bf16.device
        if buffers is not None:
            out, res_out, fp4, sf, ts = buffers
        else:
            out = torch.empty(hidden, dtype=torch.bfloat16, device=dev) if want_bf16 else None
            res_out = torch.empty(hidden, dtype=torch.bfloat16, device=dev) if want_residual_out else None
            fp4 = torch.empty((hidden + 1) // 2, dtype=torch.uint8, device=dev)
            sf = torch.zeros(tiled_scale_bytes(1, (hidden + 15) // 16), dtype=torch.uint8, device=dev)
            ts = torch.empty(1, dtype=torch.float32, device=dev)
        spec = abi.RmsnormNvfp4QuantizeSpec(hidden, eps, _dp(x_bf16), _dp(weight_bf16), _dp(residual_bf16),
                                            _dp(res_out), _dp(out), _dp(fp4), _dp(sf), _dp(ts), input_tensor_scale)
        _check("rmsnorm_nvfp4_quantize", self.lib.qwen36_rmsnorm_nvfp4_quantize(C.byref(spec)))
        return out, res_out, fp4, sf, ts

    def swiglu_nvfp4_quantize(self, gate_bf16, up_bf16, input_tensor_scale: float = 0.0, fp4=None, sf=None, ts=None):
        """One vector: silu(gate) * up -> (fp4, tiled scales, tensor scale [1])."""
        n = gate_bf16.numel()
        dev = gate_bf16.device
        if fp4 is None:
            fp4 = torch.empty((n + 1) // 2, dtype=torch.uint8, device=dev)
        if sf is None:
            sf = torch.zeros(tiled_scale_bytes(1, (n + 15) // 16), dtype=torch.uint8, device=dev)
        if ts is None:
            ts = torch.empty(1, dtype=torch.float32, device=dev)
        spec = abi.SwigluNvfp4QuantizeSpec(n, _dp(gate_bf16), _dp(up_bf16), _dp(fp4), _dp(sf), _dp(ts),
                                           input_tensor_scale)
        _check("swiglu_nvfp4_quantize", self.lib.qwen36_swiglu_nvfp4_quantize(C.byref(spec)))
        return fp4, sf, ts

    def swiglu_nvfp4_quantize_rows(self, gate_bf16, up_bf16, input_tensor_scale: float = 0.0, fp4=None, sf=None,
                                   ts=None):
        """[rows, n] blocks (views into one [rows, 2n] buffer are fine): silu(gate) * up, row by row as
        swiglu_nvfp4_quantize -> (fp4 [rows, n / 2], tiled scales of [rows, n / 16], tensor scale [1])."""
        rows, n = gate_bf16.shape
        dev = gate_bf16.device
        assert gate_bf16.stride(1) == 1 and up_bf16.stride(1) == 1 and gate_bf16.stride(0) == up_bf16.stride(0)
        if fp4 is None:
            fp4 = torch.empty((rows, n // 2), dtype=torch.uint8, device=dev)
        if sf is None:
            sf = torch.zeros(tiled_scale_bytes(rows, n // 16), dtype=torch.uint8, device=dev)
        if ts is None:
            ts = torch.empty(1, dtype=torch.float32, device=dev)
        spec = abi.SwigluNvfp4QuantizeRowsSpec(rows, n, gate_bf16.stride(0), _dp(gate_bf16), _dp(up_bf16), _dp(fp4),
                                               _dp(sf), _dp(ts), input_tensor_scale)
        _check("swiglu_nvfp4_quantize_rows", self.lib.qwen36_swiglu_nvfp4_quantize_rows(C.byref(spec)))
        return fp4, sf, ts

    def nvfp4_matvec(self, x_bf16, weight_u8, sf_tiled, tensor_scale, out=None) -> torch.Tensor:
        n_out, packed = weight_u8.shape
        k = x_bf16.numel()
        if out is None:
            out = torch.empty(n_out, dtype=torch.bfloat16, device=x_bf16.device)
        spec = abi.Nvfp4MatvecSpec(n_out, k, _dp(x_bf16), _dp(weight_u8), _dp(sf_tiled), _dp(tensor_scale),
                                   _dp(out))
        _check("nvfp4_matvec", self.lib.qwen36_nvfp4_matvec(C.byref(spec)))
        return out

    def nvfp4_matvec_group(self, x_bf16, mats) -> None:
        """`mats`: up to four (weight_u8, sf_tiled, tensor_scale, out) tuples that share `x_bf16`;
        one launch computes all of them (qwen36_nvfp4_matvec_group)."""
        specs = (abi.Nvfp4MatvecSpec * len(mats))()
        for i, (weight_u8, sf_tiled, tensor_scale, out) in enumerate(mats):
            n, kh = weight_u8.shape
            specs[i] = abi.Nvfp4MatvecSpec(n, x_bf16.numel(), _dp(x_bf16), _dp(weight_u8), _dp(sf_tiled),
                                           _dp(tensor_scale), _dp(out))
        _check("nvfp4_matvec_group", self.lib.qwen36_nvfp4_matvec_group(specs, len(mats)))

    def nvfp4_dequantize(self, weight_u8, sf_tiled, tensor_scale, in_features: int) -> torch.Tensor:
        n_out = weight_u8.shape[0]
        out = torch.empty((n_out, in_features), dtype=torch.float32, device=weight_u8.device)
        spec = abi.Nvfp4DequantizeSpec(n_out, in_features, _dp(weight_u8), _dp(sf_tiled), _dp(tensor_scale),
                                       _dp(out))
        _check("nvfp4_dequantize", self.lib.qwen36_nvfp4_dequantize(C.byref(spec)))
        return out

    GEMM_WORKSPACE_BYTES = 32 << 20

    def gemm_workspace(self, device):
        """The workspace the reference's callers hand to qwen36_nvfp4_gemm (there for cuBLASLt; here the
        stream-K form of the prefill GEMM parks partial tiles in it: 256 KB + 64 B per CTA pair).  One
        buffer per device, kept for the life of the backend; calls that share it must share a stream."""
        if not hasattr(self, "_gemm_ws"):
            self._gemm_ws = {}
        key = str(device)
        if key not in self._gemm_ws:
            self._gemm_ws[key] = torch.empty(self.GEMM_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        return self._gemm_ws[key]

    def _gemm_spec(self, a_fp4, a_sf, b_fp4, b_sf, alpha, m, n, k, out):
        ws = self.gemm_workspace(a_fp4.device) if n >= 512 else None
        return abi.Nvfp4GemmSpec(m, n, k, _dp(a_fp4), _dp(a_sf), DevicePtr(0), _dp(b_fp4), _dp(b_sf),
                                 DevicePtr(0), _dp(out), _dp(ws), 0 if ws is None else ws.numel(), alpha)

    def nvfp4_gemm(self, a_fp4, a_sf, b_fp4, b_sf, alpha: float, m: int, n: int, k: int,
                   out=None) -> torch.Tensor:
        """Reference routing (crates/kernels/src/backend.rs:213-233): n == 1 tries the decode
        GEMV unless the shape is the one the reference pins to its GEMM (m=5120, k=17408);
        NOT_IMPLEMENTED (5) falls through to qwen36_nvfp4_gemm.  Output [n, m] bf16."""
        if out is None:
            out = torch.empty((n, m), dtype=torch.bfloat16, device=a_fp4.device)
        spec = self._gemm_spec(a_fp4, a_sf, b_fp4, b_sf, alpha, m, n, k, out)
        if n == 1 and not (m == 5120 and k == 17408):
            code = self.lib.qwen36_decode_nvfp4_gemv(C.byref(spec))
            if code != abi.NOT_IMPLEMENTED:
                _check("decode_nvfp4_gemv", code)
                return out
        _check("nvfp4_gemm", self.lib.qwen36_nvfp4_gemm(C.byref(spec)))
        return out

    def decode_nvfp4_gemv_raw(self, a_fp4, a_sf, b_fp4, b_sf, alpha, m, n, k, out) -> int:
        spec = self._gemm_spec(a_fp4, a_sf, b_fp4, b_sf, alpha, m, n, k, out)
        return int(self.lib.qwen36_decode_nvfp4_gemv(C.byref(spec)))

    def nvfp4_gemm_raw(self, a_fp4, a_sf, b_fp4, b_sf, alpha, m, n, k, out) -> int:
        spec = self._gemm_spec(a_fp4, a_sf, b_fp4, b_sf, alpha, m, n, k, out)
        return int(self.lib.qwen36_nvfp4_gemm(C.byref(spec)))

    # -- lm_head ----------------------------------------------------------
    def lm_head_fp8_quantize(self, w_bf16: torch.Tensor):
        rows, cols = w_bf16.shape
        q = torch.empty((rows, cols), dtype=torch.uint8, device=w_bf16.device)
        s = torch.empty(rows, dtype=torch.float32, device=w_bf16.device)
        spec = abi.LmHeadFp8QuantizeSpec(rows, cols, _dp(w_bf16), _dp(q), _dp(s))
        _check("lm_head_fp8_quantize", self.lib.qwen36_lm_head_fp8_quantize(C.byref(spec)))
        return q, s

    # -- exact-argmax guards (crates/runtime/src/engine.rs:10705-10845) ------
    TOP2_BLOCKS = 240

    def lm_head_top2_margin(self, logits_bf16, eps: float, fallback_count=None, mirror=None):
        """[rows, vocab] bf16 logits -> (tokens u32 (as int32 tensor), flags)."""
        rows, vocab = logits_bf16.shape
        dev = logits_bf16.device
        tokens = torch.zeros(rows, dtype=torch.int32, device=dev)
        flags = torch.zeros(rows, dtype=torch.int32, device=dev)
        ws = torch.empty(rows * self.TOP2_BLOCKS * 16, dtype=torch.uint8, device=dev)
        spec = abi.LmHeadTop2MarginSpec(rows, vocab, eps, _dp(logits_bf16), _dp(tokens), _dp(flags), _dp(mirror),
                                        _dp(fallback_count), _dp(ws), ws.numel())
        _check("lm_head_top2_margin", self.lib.qwen36_lm_head_top2_margin(C.byref(spec)))
        return tokens, flags

    def lm_head_top8_rescore(self, logits_bf16, weight_bf16, input_bf16, eps: float, fallback_count=None, mirror=None):
        rows, vocab = logits_bf16.shape
        cols = weight_bf16.shape[1]
        dev = logits_bf16.device
        tokens = torch.zeros(rows, dtype=torch.int32, device=dev)
        flags = torch.zeros(rows, dtype=torch.int32, device=dev)
        ws = torch.empty(rows * self.TOP2_BLOCKS * 16, dtype=torch.uint8, device=dev)
        spec = abi.LmHeadTop8RescoreSpec(rows, vocab, cols, eps, _dp(logits_bf16), _dp(weight_bf16), _dp(input_bf16),
                                         _dp(tokens), _dp(flags), _dp(mirror), _dp(fallback_count), _dp(ws), ws.numel())
        _check("lm_head_top8_rescore", self.lib.qwen36_lm_head_top8_rescore(C.byref(spec)))
        return tokens, flags

    def bf16_matvec_argmax_rows(self, input_bf16, weight_bf16, tokens=None, skip_flags=None, mirror=None):
        """Rows whose skip flag is zero get argmax_v <x_row, W[v]>; the others keep `tokens`."""
        rows, in_features = input_bf16.shape
        out_features = weight_bf16.shape[0]
        dev = input_bf16.device
        if tokens is None:
            tokens = torch.zeros(rows, dtype=torch.int32, device=dev)
        ws = torch.empty(rows * 8, dtype=torch.uint8, device=dev)
        spec = abi.Bf16MatvecArgmaxRowsSpec(rows, out_features, in_features, _dp(input_bf16), _dp(weight_bf16),
                                            _dp(tokens), _dp(mirror), _dp(ws), ws.numel(), _dp(skip_flags))
        _check("bf16_matvec_argmax_rows", self.lib.qwen36_bf16_matvec_argmax_rows(C.byref(spec)))
        return tokens

    def lm_head_fp8_gemv(self, w_e4m3, row_scales, x_bf16, out=None) -> torch.Tensor:
        rows, cols = w_e4m3.shape
        n = x_bf16.shape[0]
        if out is None:
            out = torch.empty((n, rows), dtype=torch.bfloat16, device=x_bf16.device)
        spec = abi.LmHeadFp8GemvSpec(rows, cols, n, _dp(w_e4m3), _dp(row_scales), _dp(x_bf16), _dp(out))
        _check("lm_head_fp8_gemv", self.lib.qwen36_lm_head_fp8_gemv(C.byref(spec)))
        return out

    def lm_head_argmax_workspace(self, rows: int, n: int, device) -> torch.Tensor:
        nbytes = int(self.lib.qwen36_lm_head_fp8_argmax_workspace_bytes(rows, n))
        return torch.zeros(nbytes, dtype=torch.uint8, device=device)

    def lm_head_fp8_gemv_argmax(self, w_e4m3, row_scales, x_bf16, workspace, row_offset: int = 0,
                                out_tokens=None, out_best=None):
        rows, cols = w_e4m3.shape
        n = x_bf16.shape[0]
        dev = x_bf16.device
        if out_tokens is None:
            out_tokens = torch.empty(n, dtype=torch.int32, device=dev)
        if out_best is None:
            out_best = torch.empty(n, dtype=torch.float32, device=dev)
        spec = abi.LmHeadFp8ArgmaxSpec(rows, cols, n, _dp(w_e4m3), _dp(row_scales), _dp(x_bf16),
                                       _dp(out_tokens), _dp(out_best), _dp(workspace), workspace.numel(),
                                       row_offset)
        _check("lm_head_fp8_gemv_argmax", self.lib.qwen36_lm_head_fp8_gemv_argmax(C.byref(spec)))
        return out_tokens, out_best

    def sample(self, logits_bf16: torch.Tensor, temperature: float = 1.0, mirror=None) -> torch.Tensor:
        out = torch.empty(1, dtype=torch.int32, device=logits_bf16.device)
        spec = abi.SamplingSpec(logits_bf16.numel(), _dp(logits_bf16), _dp(out), temperature, 0, 1.0, 1.0,
                                _dp(mirror))
        _check("sample", self.lib.qwen36_sample(C.byref(spec)))
        return out

    def sample_rows(self, logits_bf16: torch.Tensor, temperature: float = 1.0, mirror=None) -> torch.Tensor:
        rows, vocab = logits_bf16.shape
        out = torch.empty(rows, dtype=torch.int32, device=logits_bf16.device)
        spec = abi.SamplingRowsSpec(rows, vocab, _dp(logits_bf16), _dp(out), _dp(mirror), temperature)
        _check("sample_rows", self.lib.qwen36_sample_rows(C.byref(spec)))
        return out

    # -- int8 KV ----------------------------------------------------------
    def attention_workspace(self, q_heads: int, head_dim: int, device) -> torch.Tensor:
        nbytes = int(self.lib.qwen36_turboquant_attention_workspace_bytes(q_heads, head_dim))
        return torch.empty(nbytes, dtype=torch.uint8, device=device)

    def turboquant_encode_kv(self, k_bf16, v_bf16, kq, vq, meta, position: int, q_heads: int = 0) -> None:
        kv_heads, head_dim = k_bf16.shape[-2], k_bf16.shape[-1]
        shape = abi.AttentionShape(q_heads, kv_heads, head_dim, 0)
        spec = abi.TurboquantEncodeSpec(0, position, _dp(k_bf16), _dp(v_bf16), _dp(kq), _dp(vq), _dp(meta), shape)
        _check("turboquant_encode_kv", self.lib.qwen36_turboquant_encode_kv(C.byref(spec)))

    def turboquant_encode_kv_rows(self, k_bf16, v_bf16, kq, vq, meta, position: int) -> None:
        tokens, kv_heads, head_dim = k_bf16.shape
        shape = abi.AttentionShape(0, kv_heads, head_dim, 0)
        spec = abi.TurboquantEncodeRowsSpec(position, tokens, _dp(k_bf16), _dp(v_bf16), _dp(kq), _dp(vq),
                                            _dp(meta), shape)
        _check("turboquant_encode_kv_rows", self.lib.qwen36_turboquant_encode_kv_rows(C.byref(spec)))

    def turboquant_attention(self, q_bf16, kq, vq, meta, position: int, workspace, out=None) -> torch.Tensor:
        q_heads, head_dim = q_bf16.shape
        kv_heads = kq.shape[1]
        if out is None:
            out = torch.empty((q_heads, head_dim), dtype=torch.bfloat16, device=q_bf16.device)
        shape = abi.AttentionShape(q_heads, kv_heads, head_dim, 0)
        spec = abi.TurboquantAttentionSpec(0, position, _dp(q_bf16), _dp(kq), _dp(vq), _dp(meta), _dp(out),
                                           _dp(workspace), 0 if workspace is None else workspace.numel(),
                                           shape, 0)
        _check("turboquant_attention", self.lib.qwen36_turboquant_attention(C.byref(spec)))
        return out

    def attention_decode(self, q_bf16, k_new, v_new, cache_k, cache_v, position: int, kv_cache_dtype: int,
                         partials=None, decode_n_splits: int = 0, position_device=None, out=None,
                         split_timesteps_per_block: int = 0) -> torch.Tensor:
        """Decode attention over a BF16 (dtype 0) or FP8 E4M3 (dtype 1) cache, with the reference's
        side effect: k_new / v_new are appended to cache row `position`.  `partials` is the
        (acc [q_heads, n, head_dim], max [q_heads, n], denom [q_heads, n]) float32 triple of the
        reference's split path, n = decode_n_splits."""
        q_heads, head_dim = q_bf16.shape
        kv_heads = k_new.shape[0]
        if out is None:
            out = torch.empty((q_heads, head_dim), dtype=torch.bfloat16, device=q_bf16.device)
        shape = abi.AttentionShape(q_heads, kv_heads, head_dim, 0)
        pa, pm, pl = partials if partials is not None else (None, None, None)
        spec = abi.AttentionDecodeSpec(0, position, _dp(q_bf16), _dp(k_new), _dp(v_new), _dp(cache_k), _dp(cache_v),
                                       DevicePtr(0), _dp(out), shape, kv_cache_dtype, _dp(position_device),
                                       _dp(pa), _dp(pm), _dp(pl), decode_n_splits, split_timesteps_per_block)
        _check("attention_decode", self.lib.qwen36_attention_decode(C.byref(spec)))
        return out

    @staticmethod
    def attention_verify_splits(tokens: int, q_heads: int, kv_heads: int, sms: int = 148) -> int:
        """Split count that gives the verify kernel one CTA per SM: a CTA covers one kv head and up to 64
        (token, q head) rows of it, so the grid is kv_heads x ceil(rows / 64) x n_splits."""
        rows = tokens * (q_heads // kv_heads)
        return max(1, sms // (kv_heads * ((rows + 63) // 64)))

    def attention_flash_splitk_prefill(self, q_bf16, cache_k, cache_v, start_position: int, kv_cache_dtype: int,
                                       n_splits: int, partials=None, start_position_device=None, out=None):
        """Speculative-verify attention (qwen36_attention_flash_splitk_prefill_bf16): q [tokens <= 32, q_heads,
        256] over cache rows [0, start + tokens), causal inside the chunk.  `partials` = (acc [tokens, q_heads,
        n_splits, 256], max, denom [tokens, q_heads, n_splits]) or None for the library's own scratch."""
        tokens, q_heads, head_dim = q_bf16.shape
        if out is None:
            out = torch.empty((tokens, q_heads, head_dim), dtype=torch.bfloat16, device=q_bf16.device)
        pa, pm, pl = partials if partials is not None else (None, None, None)
        spec = abi.AttentionPrefillSpec(0, start_position, tokens, _dp(q_bf16), DevicePtr(0), DevicePtr(0), _dp(cache_k),
                                        _dp(cache_v), DevicePtr(0), _dp(out),
                                        abi.AttentionShape(q_heads, cache_k.shape[1], head_dim, 0), kv_cache_dtype,
                                        _dp(start_position_device), _dp(pa), _dp(pm), _dp(pl), 0, 0, DevicePtr(0), 0)
        _check("attention_flash_splitk_prefill_bf16",
               self.lib.qwen36_attention_flash_splitk_prefill_bf16(C.byref(spec), n_splits))
        return out

    def turboquant_attention_static(self, q_bf16, kq, vq, meta, position: int, out=None) -> torch.Tensor:
        """Same result as turboquant_attention, but the split-KV partials live in a fixed buffer
        inside the library, so no scratch is passed and nothing is allocated by the call."""
        q_heads, head_dim = q_bf16.shape
        kv_heads = kq.shape[1]
        if out is None:
            out = torch.empty((q_heads, head_dim), dtype=torch.bfloat16, device=q_bf16.device)
        shape = abi.AttentionShape(q_heads, kv_heads, head_dim, 0)
        spec = abi.TurboquantAttentionSpec(0, position, _dp(q_bf16), _dp(kq), _dp(vq), _dp(meta), _dp(out),
                                           DevicePtr(0), 0, shape, 0)
        _check("turboquant_attention_static", self.lib.qwen36_turboquant_attention_static(C.byref(spec)))
        return out

    def turboquant_attention_partial(self, q_bf16, kq, vq, meta, t_begin: int, t_end: int, workspace,
                                     part_o=None, part_m=None, part_l=None):
        q_heads, head_dim = q_bf16.shape
        kv_heads = kq.shape[1]
        dev = q_bf16.device
        if part_o is None:
            part_o = torch.empty((q_heads, head_dim), dtype=torch.float32, device=dev)
            part_m = torch.empty(q_heads, dtype=torch.float32, device=dev)
            part_l = torch.empty(q_heads, dtype=torch.float32, device=dev)
        shape = abi.AttentionShape(q_heads, kv_heads, head_dim, 0)
        spec = abi.TurboquantAttentionPartialSpec(t_begin, t_end, _dp(q_bf16), _dp(kq), _dp(vq), _dp(meta),
                                                  _dp(part_o), _dp(part_m), _dp(part_l), _dp(workspace),
                                                  workspace.numel(), shape)
        _check("turboquant_attention_partial", self.lib.qwen36_turboquant_attention_partial(C.byref(spec)))
        return part_m, part_l, part_o

    def attention_merge_partials(self, part_m, part_l, part_o, out=None) -> torch.Tensor:
        """part_m/l [q_heads, n_parts], part_o [q_heads, n_parts, head_dim] -> bf16 [q_heads, head_dim]."""
        q_heads, n_parts, head_dim = part_o.shape
        if out is None:
            out = torch.empty((q_heads, head_dim), dtype=torch.bfloat16, device=part_o.device)
        spec = abi.AttentionMergeSpec(q_heads, head_dim, n_parts, _dp(part_o), _dp(part_m), _dp(part_l), _dp(out))
        _check("attention_merge_partials", self.lib.qwen36_attention_merge_partials(C.byref(spec)))
        return out
