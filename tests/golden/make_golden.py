#!/usr/bin/env python3
"""Generates tests/golden/reference_python.npz by importing the reference's own
Python decomposition of the NVFP4 path (scripts/decode_parity.py in the
reference checkout) and recording its outputs on small seeded inputs.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

The resulting .npz (a few tens of KB) is committed; tests read only the .npz.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch


def load_reference(ref_root: str):
    path = os.path.join(ref_root, "scripts", "decode_parity.py")
    spec = importlib.util.spec_from_file_location("ref_decode_parity", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.DEVICE = torch.device("cpu")
    return mod


class FakeSafetensors:
    """Stands in for the safetensors handle that dequant_nvfp4_from() reads."""

    def __init__(self, tensors):
        self.tensors = tensors

    def get_tensor(self, name):
        return self.tensors[name]


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16).copy()


def main() -> None:
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    from oracle import oracle as orc
    ref_root = sys.argv[1] if len(sys.argv) > 1 else orc.reference_dir()
    ref = load_reference(ref_root)
    out = {}

    # 1. E4M3 decode of all 256 codes.
    out["e4m3_decode_table"] = np.array([ref.decode_e4m3_value(c) for c in range(256)],
                                        dtype=np.float32)

    # 2. UE4M3 encode: every representable value, the midpoints between
    #    neighbours (ties), values one float32 ulp either side of them, the
    #    clamps, and seeded log-uniform draws.
    pos = sorted({ref.decode_e4m3_value(c) for c in range(0x7F)})
    vals = list(pos)
    for lo, hi in zip(pos[:-1], pos[1:]):
        mid = np.float32((np.float64(lo) + np.float64(hi)) / 2)
        vals += [float(mid), float(np.nextafter(mid, np.float32(0))),
                 float(np.nextafter(mid, np.float32(1e9)))]
    vals += [0.0, -1.0, 1e-9, 447.9, 448.0, 449.0, 1e6, 1.0 / 6.0, 1.0e-8]
    rng = np.random.default_rng(20260504)
    vals += list(np.exp2(rng.uniform(-12, 10, size=2000)).astype(np.float32))
    vals = np.array(vals, dtype=np.float32)
    out["ue4m3_encode_in"] = vals
    out["ue4m3_encode_out"] = np.array([ref.encode_e4m3_positive_value(float(v)) for v in vals],
                                       dtype=np.uint8)

    # 3. Activation quantise->dequantise.  Row 0: N(0,1) with outliers, row 1:
    #    exact E2M1 ties after scaling (amax 6 -> scale 1), row 2: zeros and
    #    tiny values, rows 3..5: seeded N(0,1)*{0.01, 1, 30}; one ragged width.
    g = torch.Generator().manual_seed(515151)
    x = torch.randn(6, 128, generator=g)
    x[0, ::17] *= 20.0
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0,
                         -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    x[1] = ties.repeat(8)
    x[2] = 0.0
    x[2, 16:32] = 1e-6
    x[2, 33] = -0.0
    x[3] *= 0.01
    x[5] *= 30.0
    x = x.to(torch.bfloat16)
    out["act_in_bf16"] = bf16_bits(x)
    for name, s in (("1", 1.0), ("1p25", 1.25), ("0p5", 0.5), ("0", 0.0)):
        out[f"act_dequant_scale_{name}"] = ref.nvfp4_activation_dequant_rows(
            x.float(), input_scale=s).numpy().astype(np.float32)
    xr = x[:3, :40].contiguous()   # ragged: 40 = 2 full groups + 8
    out["act_ragged_in_bf16"] = bf16_bits(xr)
    out["act_ragged_dequant"] = ref.nvfp4_activation_dequant_rows(
        xr.float(), input_scale=1.25).numpy().astype(np.float32)

    # 4. Weight dequantisation + full linear on a seeded 160 x 192 NVFP4 weight
    #    (rows cross a 128-row scale block, K/16 = 12 groups = 3 scale tiles).
    n_out, k_in = 160, 192
    packed = torch.randint(0, 256, (n_out, k_in // 2), generator=g, dtype=torch.uint8)
    sf_codes = torch.randint(0x18, 0x58, (n_out, k_in // 16), generator=g, dtype=torch.uint8)
    sf_f8 = sf_codes.view(torch.float8_e4m3fn)
    ws2 = torch.tensor(1.0 / 2688.0, dtype=torch.float32)
    in_scale = torch.tensor(1.25, dtype=torch.float32)
    f = FakeSafetensors({"L.weight": packed, "L.weight_scale": sf_f8,
                         "L.weight_scale_2": ws2, "L.input_scale": in_scale})
    out["w_packed"] = packed.numpy()
    out["w_sf_row_major"] = sf_codes.numpy()
    out["w_scale_2"] = np.array([ws2.item()], dtype=np.float32)
    out["w_dequant"] = ref.dequant_nvfp4_from(f, "L").numpy().astype(np.float32)
    xa = torch.randn(3, k_in, generator=g).to(torch.bfloat16)
    out["lin_x_bf16"] = bf16_bits(xa)
    out["lin_input_scale"] = np.array([in_scale.item()], dtype=np.float32)
    out["lin_y"] = ref.linear_nvfp4(f, "L", xa.float()).numpy().astype(np.float32)

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_python.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
