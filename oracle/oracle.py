"""ctypes binding of the CPU oracle (oracle/oracle.c).

TEST INFRASTRUCTURE ONLY.  Imported by ``tests/``, by ``__graft_entry__.smoke``
and by the CPU-baseline legs of ``bench.py``; never by the package.  All
tensors are numpy arrays: bf16 travels as ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")

_u8p = C.POINTER(C.c_uint8)
_u16p = C.POINTER(C.c_uint16)
_u32p = C.POINTER(C.c_uint32)
_i8p = C.POINTER(C.c_int8)
_f32p = C.POINTER(C.c_float)
_sz = C.c_size_t


def reference_dir() -> str:
    """Where the reference checkout lives on the build machine: QWEN36_REFERENCE_DIR, else the
    default location.  The one place that names it; nothing that runs on a GPU box reads it."""
    return os.environ.get("QWEN36_REFERENCE_DIR", "/root/reference")


def build(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile beside this file."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        L = _lib
        L.orc_e4m3_decode.restype = C.c_float
        L.orc_e4m3_decode.argtypes = [C.c_uint8]
        L.orc_ue4m3_encode.restype = C.c_uint8
        L.orc_ue4m3_encode.argtypes = [C.c_float]
        L.orc_e2m1_encode.restype = C.c_uint8
        L.orc_e2m1_encode.argtypes = [C.c_float]
        L.orc_e2m1_value.restype = C.c_float
        L.orc_e2m1_value.argtypes = [C.c_uint8]
        L.orc_fp8_e4m3_to_f32.restype = C.c_float
        L.orc_fp8_e4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_f32_to_fp8_e4m3.restype = C.c_uint8
        L.orc_f32_to_fp8_e4m3.argtypes = [C.c_float]
        L.orc_sf_offset.restype = _sz
        L.orc_sf_offset.argtypes = [_sz, _sz, _sz]
        L.orc_sf_bytes.restype = _sz
        L.orc_sf_bytes.argtypes = [_sz, _sz]
        L.orc_nvfp4_count_e2m1_ties.restype = _sz
        L.orc_num_threads.restype = C.c_int
        L.orc_kv_e4m3_decode.restype = C.c_float
        L.orc_kv_e4m3_decode.argtypes = [C.c_uint8]
        L.orc_kv_e4m3_encode.restype = C.c_uint8
        L.orc_kv_e4m3_encode.argtypes = [C.c_float]
    return _lib


def _p(a: np.ndarray, t):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(t)


# ----------------------------------------------------------------------------
# bf16 helpers (numpy has no bf16: uint16 bit patterns throughout)
# ----------------------------------------------------------------------------

def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = 0x7FFF
    return r


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ----------------------------------------------------------------------------
# scalar codecs
# ----------------------------------------------------------------------------

def e4m3_decode(code: int) -> float:
    return float(lib().orc_e4m3_decode(code & 0xFF))


def ue4m3_encode(v: float) -> int:
    return int(lib().orc_ue4m3_encode(np.float32(v)))


def e2m1_encode(v: float) -> int:
    return int(lib().orc_e2m1_encode(np.float32(v)))


def e2m1_value(code: int) -> float:
    return float(lib().orc_e2m1_value(code & 0xF))


def fp8_e4m3_to_f32(code: int) -> float:
    return float(lib().orc_fp8_e4m3_to_f32(code & 0xFF))


def f32_to_fp8_e4m3(v: float) -> int:
    return int(lib().orc_f32_to_fp8_e4m3(np.float32(v)))


def sf_offset(inner: int, outer: int, sf_inner_dim: int) -> int:
    return int(lib().orc_sf_offset(inner, outer, sf_inner_dim))


def sf_bytes(inner_groups: int, outer: int) -> int:
    return int(lib().orc_sf_bytes(inner_groups, outer))


# ----------------------------------------------------------------------------
# tensor functions
# ----------------------------------------------------------------------------

def retile_scales(sf_row_major: np.ndarray) -> np.ndarray:
    rows, groups = sf_row_major.shape
    out = np.zeros(sf_bytes(groups, rows), dtype=np.uint8)
    lib().orc_retile_scales(_p(sf_row_major, _u8p), _p(out, _u8p), _sz(rows), _sz(groups))
    return out


def nvfp4_quantize_rows(x_bf16: np.ndarray, input_tensor_scale: float = 0.0):
    """-> (fp4 [rows, ceil(values/2)], swizzled sf bytes (zero-initialised), tensor scale)."""
    rows, values = x_bf16.shape
    groups = (values + 15) // 16
    fp4 = np.zeros((rows, (values + 1) // 2), dtype=np.uint8)
    sf = np.zeros(sf_bytes(groups, rows), dtype=np.uint8)
    ts = np.zeros(1, dtype=np.float32)
    lib().orc_nvfp4_quantize_rows(_p(x_bf16, _u16p), _sz(rows), _sz(values),
                                  C.c_float(input_tensor_scale), _p(fp4, _u8p),
                                  _p(sf, _u8p), _p(ts, _f32p))
    return fp4, sf, float(ts[0])


def rmsnorm_nvfp4_quantize(x_bf16: np.ndarray, weight_bf16: np.ndarray, residual_bf16=None, eps: float = 1e-6,
                           input_tensor_scale: float = 0.0):
    """One vector.  -> dict(out_bf16, residual_out, fp4, sf (zero-initialised), ts, weighted_f32)."""
    hidden = x_bf16.shape[0]
    groups = (hidden + 15) // 16
    out = np.zeros(hidden, dtype=np.uint16)
    res_out = np.zeros(hidden, dtype=np.uint16)
    fp4 = np.zeros((hidden + 1) // 2, dtype=np.uint8)
    sf = np.zeros(sf_bytes(groups, 1), dtype=np.uint8)
    ts = np.zeros(1, dtype=np.float32)
    weighted = np.zeros(hidden, dtype=np.float32)
    lib().orc_rmsnorm_nvfp4_quantize(_p(x_bf16, _u16p), _p(weight_bf16, _u16p),
                                     None if residual_bf16 is None else _p(residual_bf16, _u16p), _sz(hidden),
                                     C.c_float(eps), C.c_float(input_tensor_scale), _p(out, _u16p),
                                     _p(res_out, _u16p), _p(fp4, _u8p), _p(sf, _u8p), _p(ts, _f32p),
                                     _p(weighted, _f32p))
    return {"out_bf16": out, "residual_out": res_out, "fp4": fp4, "sf": sf, "ts": float(ts[0]),
            "weighted_f32": weighted}


def swiglu_nvfp4_quantize(gate_bf16: np.ndarray, up_bf16: np.ndarray, input_tensor_scale: float = 0.0):
    """One vector.  -> dict(fp4, sf (zero-initialised), ts, y_f32)."""
    values = gate_bf16.shape[0]
    groups = (values + 15) // 16
    fp4 = np.zeros((values + 1) // 2, dtype=np.uint8)
    sf = np.zeros(sf_bytes(groups, 1), dtype=np.uint8)
    ts = np.zeros(1, dtype=np.float32)
    y = np.zeros(values, dtype=np.float32)
    lib().orc_swiglu_nvfp4_quantize(_p(gate_bf16, _u16p), _p(up_bf16, _u16p), _sz(values),
                                    C.c_float(input_tensor_scale), _p(fp4, _u8p), _p(sf, _u8p), _p(ts, _f32p),
                                    _p(y, _f32p))
    return {"fp4": fp4, "sf": sf, "ts": float(ts[0]), "y_f32": y}


def lm_head_top2_margin(logits_bf16: np.ndarray, eps: float):
    """[rows, vocab] bf16 bits -> (tokens u32, flags u32, rows whose guard failed)."""
    rows, vocab = logits_bf16.shape
    tokens = np.zeros(rows, dtype=np.uint32)
    flags = np.zeros(rows, dtype=np.uint32)
    L = lib()
    L.orc_lm_head_top2_margin.restype = C.c_uint32
    fb = L.orc_lm_head_top2_margin(_p(logits_bf16, _u16p), _sz(rows), _sz(vocab), C.c_float(eps),
                                   _p(tokens, C.POINTER(C.c_uint32)), _p(flags, C.POINTER(C.c_uint32)))
    return tokens, flags, int(fb)


def lm_head_top8_rescore(logits_bf16: np.ndarray, weight_bf16: np.ndarray, input_bf16: np.ndarray, eps: float):
    rows, vocab = logits_bf16.shape
    cols = weight_bf16.shape[1]
    tokens = np.zeros(rows, dtype=np.uint32)
    flags = np.zeros(rows, dtype=np.uint32)
    L = lib()
    L.orc_lm_head_top8_rescore.restype = C.c_uint32
    fb = L.orc_lm_head_top8_rescore(_p(logits_bf16, _u16p), _p(weight_bf16, _u16p), _p(input_bf16, _u16p), _sz(rows),
                                    _sz(vocab), _sz(cols), C.c_float(eps), _p(tokens, C.POINTER(C.c_uint32)),
                                    _p(flags, C.POINTER(C.c_uint32)))
    return tokens, flags, int(fb)


def bf16_matvec_argmax_rows(input_bf16: np.ndarray, weight_bf16: np.ndarray, skip_flags=None, tokens_in=None):
    """input [rows, in], weight [out, in] -> tokens u32 [rows]; flagged rows keep tokens_in."""
    rows, in_features = input_bf16.shape
    out_features = weight_bf16.shape[0]
    tokens = np.zeros(rows, dtype=np.uint32) if tokens_in is None else tokens_in.astype(np.uint32).copy()
    lib().orc_bf16_matvec_argmax_rows(_p(input_bf16, _u16p), _p(weight_bf16, _u16p),
                                      None if skip_flags is None else _p(skip_flags, C.POINTER(C.c_uint32)),
                                      _sz(rows), _sz(out_features), _sz(in_features),
                                      _p(tokens, C.POINTER(C.c_uint32)))
    return tokens


def nvfp4_count_e2m1_ties(x_bf16: np.ndarray, input_tensor_scale: float = 0.0) -> int:
    rows, values = x_bf16.shape
    return int(lib().orc_nvfp4_count_e2m1_ties(_p(x_bf16, _u16p), _sz(rows), _sz(values),
                                               C.c_float(input_tensor_scale)))


def nvfp4_dequant(weight: np.ndarray, sf_swizzled: np.ndarray, global_scale: float,
                  in_features: int) -> np.ndarray:
    out_features = weight.shape[0]
    out = np.empty((out_features, in_features), dtype=np.float32)
    lib().orc_nvfp4_dequant(_p(weight, _u8p), _p(sf_swizzled, _u8p), C.c_float(global_scale),
                            _sz(out_features), _sz(in_features), _p(out, _f32p))
    return out


def nvfp4_matvec(x_bf16: np.ndarray, weight: np.ndarray, sf_swizzled: np.ndarray,
                 tensor_scale, in_features: int) -> np.ndarray:
    """tensor_scale=None models a NULL tensor_scale pointer."""
    out_features = weight.shape[0]
    out = np.empty(out_features, dtype=np.uint16)
    lib().orc_nvfp4_matvec(_p(x_bf16, _u16p), _p(weight, _u8p), _p(sf_swizzled, _u8p),
                           C.c_int(0 if tensor_scale is None else 1),
                           C.c_float(0.0 if tensor_scale is None else tensor_scale),
                           _sz(in_features), _sz(out_features), _p(out, _u16p))
    return out


def nvfp4_gemm(a, a_sf, b, b_sf, alpha: float, m: int, n: int, k: int) -> np.ndarray:
    out = np.empty((n, m), dtype=np.uint16)
    lib().orc_nvfp4_gemm(_p(a, _u8p), _p(a_sf, _u8p), _p(b, _u8p), _p(b_sf, _u8p),
                         C.c_float(alpha), _sz(m), _sz(n), _sz(k), _p(out, _u16p))
    return out


def nvfp4_gemm_sampled(a, a_sf, b, b_sf, alpha: float, m: int, n: int, k: int,
                       tok: np.ndarray, feat: np.ndarray) -> np.ndarray:
    tok = np.ascontiguousarray(tok, dtype=np.uint32)
    feat = np.ascontiguousarray(feat, dtype=np.uint32)
    out = np.empty(tok.shape[0], dtype=np.float32)
    lib().orc_nvfp4_gemm_sampled(_p(a, _u8p), _p(a_sf, _u8p), _p(b, _u8p), _p(b_sf, _u8p),
                                 C.c_float(alpha), _sz(m), _sz(n), _sz(k), _p(tok, _u32p),
                                 _p(feat, _u32p), _sz(tok.shape[0]), _p(out, _f32p))
    return out


def lm_head_fp8_quantize(w_bf16: np.ndarray):
    rows, cols = w_bf16.shape
    q = np.empty((rows, cols), dtype=np.uint8)
    s = np.empty(rows, dtype=np.float32)
    lib().orc_lm_head_fp8_quantize(_p(w_bf16, _u16p), _sz(rows), _sz(cols), _p(q, _u8p),
                                   _p(s, _f32p))
    return q, s


def lm_head_fp8_gemv(w_e4m3: np.ndarray, row_scales: np.ndarray, x_bf16: np.ndarray) -> np.ndarray:
    rows, cols = w_e4m3.shape
    n = x_bf16.shape[0]
    y = np.empty((n, rows), dtype=np.uint16)
    lib().orc_lm_head_fp8_gemv(_p(w_e4m3, _u8p), _p(row_scales, _f32p), _p(x_bf16, _u16p),
                               _sz(rows), _sz(cols), _sz(n), _p(y, _u16p))
    return y


def argmax_rows(logits_bf16: np.ndarray, temperature: float = 1.0) -> np.ndarray:
    rows, vocab = logits_bf16.shape
    out = np.empty(rows, dtype=np.uint32)
    lib().orc_argmax_rows(_p(logits_bf16, _u16p), _sz(rows), _sz(vocab), C.c_float(temperature),
                          _p(out, _u32p))
    return out


def kv_encode(k_bf16: np.ndarray, v_bf16: np.ndarray, position: int, kq: np.ndarray,
              vq: np.ndarray, meta: np.ndarray) -> None:
    """k,v [tokens, kv_heads, head_dim]; writes cache rows [position, position+tokens)."""
    tokens, kv_heads, head_dim = k_bf16.shape
    lib().orc_kv_encode(_p(k_bf16, _u16p), _p(v_bf16, _u16p), _sz(position), _sz(tokens),
                        _sz(kv_heads), _sz(head_dim), _p(kq, _i8p), _p(vq, _i8p), _p(meta, _f32p))


def kv_attention(q_bf16: np.ndarray, kq: np.ndarray, vq: np.ndarray, meta: np.ndarray,
                 position: int) -> np.ndarray:
    q_heads, head_dim = q_bf16.shape
    kv_heads = kq.shape[1]
    scores = np.empty(q_heads * (position + 1), dtype=np.float32)
    out = np.empty((q_heads, head_dim), dtype=np.uint16)
    lib().orc_kv_attention(_p(q_bf16, _u16p), _p(kq, _i8p), _p(vq, _i8p), _p(meta, _f32p),
                           _sz(position), _sz(q_heads), _sz(kv_heads), _sz(head_dim),
                           _p(scores, _f32p), _p(out, _u16p))
    return out


def kv_attention_partial(q_bf16, kq, vq, meta, t_begin: int, t_end: int):
    q_heads, head_dim = q_bf16.shape
    kv_heads = kq.shape[1]
    pm = np.empty(q_heads, dtype=np.float32)
    pl = np.empty(q_heads, dtype=np.float32)
    po = np.empty((q_heads, head_dim), dtype=np.float32)
    lib().orc_kv_attention_partial(_p(q_bf16, _u16p), _p(kq, _i8p), _p(vq, _i8p), _p(meta, _f32p),
                                   _sz(t_begin), _sz(t_end), _sz(q_heads), _sz(kv_heads),
                                   _sz(head_dim), _p(pm, _f32p), _p(pl, _f32p), _p(po, _f32p))
    return pm, pl, po


def merge_partials(part_m: np.ndarray, part_l: np.ndarray, part_o: np.ndarray) -> np.ndarray:
    """part_m/l [q_heads, n_parts], part_o [q_heads, n_parts, head_dim] -> bf16 [q_heads, head_dim]."""
    q_heads, n_parts, head_dim = part_o.shape
    out = np.empty((q_heads, head_dim), dtype=np.uint16)
    lib().orc_merge_partials(_p(np.ascontiguousarray(part_m, dtype=np.float32), _f32p),
                             _p(np.ascontiguousarray(part_l, dtype=np.float32), _f32p),
                             _p(np.ascontiguousarray(part_o, dtype=np.float32), _f32p),
                             _sz(q_heads), _sz(n_parts), _sz(head_dim), _p(out, _u16p))
    return out


def kv_e4m3_decode(code: int) -> float:
    return float(lib().orc_kv_e4m3_decode(code))


def kv_e4m3_encode(v: float) -> int:
    return int(lib().orc_kv_e4m3_encode(float(v)))


def attention_decode(q_bf16: np.ndarray, k_new: np.ndarray, v_new: np.ndarray, cache_k: np.ndarray,
                     cache_v: np.ndarray, kv_cache_dtype: int, position: int) -> np.ndarray:
    """q [q_heads, head_dim], k_new / v_new [kv_heads, head_dim] bf16 bits; caches
    [>= position + 1, kv_heads, head_dim] of uint16 (BF16, dtype 0) or uint8 (E4M3, dtype 1).
    Returns bf16 [q_heads, head_dim] and writes cache row `position` in place."""
    q_heads, head_dim = q_bf16.shape
    kv_heads = k_new.shape[0]
    assert cache_k.dtype == (np.uint8 if kv_cache_dtype == 1 else np.uint16) and cache_k.flags.c_contiguous
    assert cache_v.dtype == cache_k.dtype and cache_v.flags.c_contiguous and cache_k.shape[0] > position
    out = np.empty((q_heads, head_dim), dtype=np.uint16)
    lib().orc_attention_decode(_p(q_bf16, _u16p), _p(k_new, _u16p), _p(v_new, _u16p),
                               cache_k.ctypes.data_as(C.c_void_p), cache_v.ctypes.data_as(C.c_void_p),
                               C.c_int(kv_cache_dtype), _sz(position), _sz(q_heads), _sz(kv_heads),
                               _sz(head_dim), _p(out, _u16p))
    return out


def attention_verify(q_bf16: np.ndarray, cache_k: np.ndarray, cache_v: np.ndarray, kv_cache_dtype: int,
                     start_position: int) -> np.ndarray:
    """Speculative-verify attention, the arithmetic of kernels-cuda/attention_flash_splitk.cu:96-420
    restated without tiles or splits: q [tokens, q_heads, 256] bf16 bits; caches [>= start + tokens,
    kv_heads, 256] of uint16 (BF16) or uint8 (E4M3, read as attention_flash_splitk.cu:54-72 reads it:
    0x7F / 0xFF are +-448); query row i attends to cache rows [0, start + i] (causal mask, lines
    243-254) with scores q.k * rsqrt(256); float64 softmax; returns float64 [tokens, q_heads, 256]
    (the kernel rounds probabilities to the operand type before P V and the result to bf16: the GPU
    test allows rel-L2 1e-2 for that)."""
    tokens, q_heads, head_dim = q_bf16.shape
    kv_heads = cache_k.shape[1]
    rows = start_position + tokens
    if kv_cache_dtype == 1:
        table = np.array([kv_e4m3_decode(c) for c in range(256)], dtype=np.float64)
        k = table[cache_k[:rows]]
        v = table[cache_v[:rows]]
    else:
        k = bf16_to_f32(cache_k[:rows]).astype(np.float64)
        v = bf16_to_f32(cache_v[:rows]).astype(np.float64)
    q = bf16_to_f32(q_bf16).astype(np.float64)
    out = np.zeros((tokens, q_heads, head_dim), dtype=np.float64)
    per = q_heads // kv_heads
    for h in range(q_heads):
        kvh = h // per
        s = q[:, h, :] @ k[:, kvh, :].T / np.sqrt(float(head_dim))          # [tokens, rows]
        t = np.arange(rows)[None, :]
        s = np.where(t <= (start_position + np.arange(tokens))[:, None], s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        pr = np.exp(s)
        pr /= pr.sum(axis=1, keepdims=True)
        out[:, h, :] = pr @ v[:, kvh, :]
    return out


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))
