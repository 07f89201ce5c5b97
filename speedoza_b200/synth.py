"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no checkpoint or dataset is involved).

numpy on the host (what the CPU oracle consumes) and torch on the device (what
the large benchmark shapes need).  bf16 host arrays are uint16 bit patterns.
"""
from __future__ import annotations

import numpy as np

# Qwen3.6-27B decode shapes (N x K) of one layer, in execution order.
DECODE_SHAPES = [
    ("attn.q_gate", 12288, 5120),
    ("attn.k", 1024, 5120),
    ("attn.v", 1024, 5120),
    ("attn.o", 5120, 6144),
    ("mlp.gate_up", 34816, 5120),
    ("mlp.down", 5120, 17408),
]
LAYERS = 64
HIDDEN = 5120
VOCAB = 248320
Q_HEADS, KV_HEADS, HEAD_DIM = 24, 4, 256
WEIGHT_GLOBAL_SCALE = 1.0 / 2688.0
SF_CODE_LO, SF_CODE_HI = 0x18, 0x58      # UE4M3 codes of 2^-4 .. 2^4, 8 codes per octave


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def nvfp4_weight(rng: np.random.Generator, n: int, k: int):
    """Packed E2M1 codes uniform over all 16 codes [n, k/2] and row-major UE4M3 block scales
    [n, k/16], log-uniform in [2^-4, 2^4]."""
    packed = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    sf = rng.integers(SF_CODE_LO, SF_CODE_HI + 1, size=(n, (k + 15) // 16), dtype=np.uint8)
    return packed, sf


def activations(rng: np.random.Generator, rows: int, k: int, outlier_frac: float = 0.0,
                outlier_gain: float = 20.0) -> np.ndarray:
    """bf16 bits of N(0,1) activations; `outlier_frac` of the channels scaled by `outlier_gain`."""
    x = rng.standard_normal((rows, k), dtype=np.float32)
    if outlier_frac > 0:
        ch = rng.choice(k, size=max(1, int(round(k * outlier_frac))), replace=False)
        x[:, ch] *= outlier_gain
    return f32_to_bf16_bits(x)


def lm_head_weight(rng: np.random.Generator, rows: int, cols: int):
    """Finite FP8 E4M3 bytes (|code| < 0x7F) and row scales log-uniform in [2^-6, 2^-2]."""
    mag = rng.integers(0, 0x7F, size=(rows, cols), dtype=np.uint8)
    sign = rng.integers(0, 2, size=(rows, cols), dtype=np.uint8) << 7
    scales = np.exp2(rng.uniform(-6.0, -2.0, size=rows)).astype(np.float32)
    return (mag | sign).astype(np.uint8), scales


def qkv(rng: np.random.Generator, tokens: int, q_heads: int = Q_HEADS, kv_heads: int = KV_HEADS,
        head_dim: int = HEAD_DIM, outliers: int = 4, gain: float = 10.0):
    """bf16 bits: q [q_heads, head_dim], k and v [tokens, kv_heads, head_dim]; `outliers` fixed channels
    per head scaled by `gain`."""
    q = rng.standard_normal((q_heads, head_dim), dtype=np.float32)
    k = rng.standard_normal((tokens, kv_heads, head_dim), dtype=np.float32)
    v = rng.standard_normal((tokens, kv_heads, head_dim), dtype=np.float32)
    ch = rng.choice(head_dim, size=outliers, replace=False)
    q[:, ch] *= gain
    k[:, :, ch] *= gain
    v[:, :, ch] *= gain
    return f32_to_bf16_bits(q), f32_to_bf16_bits(k), f32_to_bf16_bits(v)


# ---- device-side generation for the large benchmark shapes -------------------

def nvfp4_weight_device(gen, n: int, k: int, device):
    import torch
    packed = torch.randint(0, 256, (n, k // 2), generator=gen, dtype=torch.uint8, device=device)
    sf = torch.randint(SF_CODE_LO, SF_CODE_HI + 1, (n, k // 16), generator=gen, dtype=torch.uint8, device=device)
    return packed, sf
