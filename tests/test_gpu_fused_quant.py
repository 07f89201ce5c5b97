"""Fused producers of NVFP4 activations (qwen36_rmsnorm_nvfp4_quantize, qwen36_swiglu_nvfp4_quantize)
through the C ABI against the CPU oracle.  The device normaliser is rsqrtf and the device exponential
CUDA's expf; the oracle uses the correctly rounded host functions, so a value within a few ulps of a
rounding boundary may land on the neighbouring bf16 / code.  These tests bound that (neighbours only,
well under 1 %); exact equality with the reference's own CUDA kernels is asserted in
test_gpu_reference_cuda.py."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from speedoza_b200 import abi, synth
from conftest import bf16_host, to_dev

pytestmark = pytest.mark.gpu


def nibbles(fp4: np.ndarray, n: int) -> np.ndarray:
    out = np.empty(fp4.size * 2, dtype=np.uint8)
    out[0::2] = fp4 & 15
    out[1::2] = fp4 >> 4
    return out[:n]


def assert_codes_close(got_fp4, got_sf, want_fp4, want_sf, n, max_frac=5e-3):
    groups = (n + 15) // 16
    sf_inner = (groups + 3) // 4 * 4
    offs = np.array([orc.sf_offset(g, 0, sf_inner) for g in range(groups)])
    same_scale = got_sf[offs] == want_sf[offs]
    assert same_scale.mean() >= 0.99, same_scale.mean()
    # bytes outside the written positions stay zero on both sides
    mask = np.ones(got_sf.size, dtype=bool)
    mask[offs] = False
    assert not got_sf[mask].any()
    g_codes, w_codes = nibbles(got_fp4, n), nibbles(want_fp4, n)
    keep = np.repeat(same_scale, 16)[:n]
    diff = (g_codes != w_codes) & keep
    assert diff.mean() <= max_frac, diff.mean()
    # a differing code is the neighbouring magnitude (or +0 / -0 at the origin)
    gi, wi = g_codes[diff] & 7, w_codes[diff] & 7
    assert np.all(np.abs(gi.astype(int) - wi.astype(int)) <= 1)


@pytest.mark.parametrize("hidden,with_residual,its", [(5120, True, 0.0), (5120, False, 1.25), (6144, True, 0.37),
                                                      (33, False, 1.25), (100, True, 0.0), (16, False, 0.0)])
def test_rmsnorm_nvfp4_quantize_vs_oracle(backend, hidden, with_residual, its):
    rng = np.random.default_rng(hidden + int(its * 100))
    x = synth.activations(rng, 1, hidden, outlier_frac=0.01)[0]
    w = synth.f32_to_bf16_bits((rng.standard_normal(hidden) * 0.1).astype(np.float32))
    res = synth.activations(rng, 1, hidden)[0] if with_residual else None
    want = orc.rmsnorm_nvfp4_quantize(x, w, res, 1e-6, its)
    out, res_out, fp4, sf, ts = backend.rmsnorm_nvfp4_quantize(
        to_dev(x), to_dev(w), None if res is None else to_dev(res), 1e-6, its, want_bf16=True, want_residual_out=True)
    assert ts.item() == np.float32(want["ts"])
    assert np.array_equal(bf16_host(res_out), want["residual_out"])          # exact arithmetic on both sides
    got_out = bf16_host(out)
    ulp = np.abs(got_out.astype(np.int32) - want["out_bf16"].astype(np.int32))
    assert ulp.max() <= 1 and (ulp != 0).mean() <= 0.02
    assert_codes_close(fp4.cpu().numpy(), sf.cpu().numpy(), want["fp4"], want["sf"], hidden)


def test_rmsnorm_known_answer_and_optional_outputs(backend):
    # kernels-cuda/smoke.cu:1187-1215
    ones = to_dev(synth.f32_to_bf16_bits(np.ones(16, np.float32)))
    zeros = to_dev(synth.f32_to_bf16_bits(np.zeros(16, np.float32)))
    out, res_out, fp4, sf, ts = backend.rmsnorm_nvfp4_quantize(ones, zeros, None, 0.0, 0.0, want_bf16=False)
    assert out is None and res_out is None
    assert torch.all(fp4 == 0x77) and sf[0].item() == 0x23 and ts.item() == 1.0
    # argument checks of the entry point (kernels-cuda/ops.cu:1009-1016)
    spec = abi.RmsnormNvfp4QuantizeSpec(0, 0.0, abi.DevicePtr(ones.data_ptr()), abi.DevicePtr(zeros.data_ptr()),
                                        abi.DevicePtr(0), abi.DevicePtr(0), abi.DevicePtr(0),
                                        abi.DevicePtr(fp4.data_ptr()), abi.DevicePtr(sf.data_ptr()), abi.DevicePtr(0), 0.0)
    import ctypes as C
    assert backend.lib.qwen36_rmsnorm_nvfp4_quantize(C.byref(spec)) == abi.INVALID_ARGUMENT
    assert backend.lib.qwen36_rmsnorm_nvfp4_quantize(None) == abi.NULL_POINTER


@pytest.mark.parametrize("n,its", [(17408, 0.0), (17408, 0.37), (33, 1.25), (16, 0.0), (1000, 0.0)])
def test_swiglu_nvfp4_quantize_vs_oracle(backend, n, its):
    rng = np.random.default_rng(n + int(its * 100))
    gate = synth.f32_to_bf16_bits((rng.standard_normal(n) * 2.0).astype(np.float32))
    up = synth.activations(rng, 1, n, outlier_frac=0.01)[0]
    want = orc.swiglu_nvfp4_quantize(gate, up, its)
    fp4, sf, ts = backend.swiglu_nvfp4_quantize(to_dev(gate), to_dev(up), its)
    assert ts.item() == np.float32(want["ts"])
    assert_codes_close(fp4.cpu().numpy(), sf.cpu().numpy(), want["fp4"], want["sf"], n)


def test_swiglu_feeds_the_down_projection(backend):
    """The fused producer's output is a valid B operand of the W4A4 product: down_proj(silu(g) * u)
    through qwen36_decode_nvfp4_gemv against the float64 product of the dequantised operands."""
    rng = np.random.default_rng(99)
    n_out, k = 256, 17408
    packed, sf_rm = synth.nvfp4_weight(rng, n_out, k)
    a_sf = orc.retile_scales(sf_rm)
    gate = synth.f32_to_bf16_bits((rng.standard_normal(k) * 2.0).astype(np.float32))
    up = synth.activations(rng, 1, k)[0]
    fp4, sf, ts = backend.swiglu_nvfp4_quantize(to_dev(gate), to_dev(up), 0.37)
    alpha = synth.WEIGHT_GLOBAL_SCALE * 0.37
    out = torch.empty((1, n_out), dtype=torch.bfloat16, device="cuda")
    assert backend.decode_nvfp4_gemv_raw(to_dev(packed), to_dev(a_sf), fp4.view(1, -1), sf, alpha, n_out, 1, k, out) == abi.SUCCESS
    want = orc.nvfp4_gemm(packed, a_sf, fp4.cpu().numpy()[None, :], sf.cpu().numpy(), alpha, n_out, 1, k)
    got = synth.bf16_bits_to_f32(bf16_host(out))
    ref = synth.bf16_bits_to_f32(want)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 1e-2


def _special_rows(rng, rows, n):
    """gate / up blocks with the values the codec treats specially planted in: all-zero groups, a
    NaN, infinities, float32-subnormal products, exact E2M1 ties, huge and tiny magnitudes."""
    gate = synth.f32_to_bf16_bits((rng.standard_normal((rows, n)) * 2.0).astype(np.float32))
    up = np.stack([synth.activations(rng, 1, n, outlier_frac=0.01)[0] for _ in range(rows)])
    f2b = lambda v: synth.f32_to_bf16_bits(np.array([v], np.float32))[0]
    gate[0, :32] = 0; up[0, 16:48] = 0                       # zero groups (either factor)
    gate[1, 40] = f2b(np.nan); up[1, 70] = f2b(np.inf); gate[1, 90] = f2b(-np.inf)
    gate[2, :16] = f2b(-80.0); up[2, :16] = f2b(1e-10); up[2, 3] = f2b(3.0)      # products far below 2^-96 beside a normal one
    gate[2, 16:32] = f2b(-87.0); up[2, 16:32] = f2b(1e-8)   # a whole group of subnormal products
    gate[3, :16] = f2b(30.0)                                 # silu(30) = 30: exact quotients, E2M1 ties
    up[3, :16] = synth.f32_to_bf16_bits(np.array([6, 0.75, 1.75, 3.5, 0.25, 1.25, 2.5, 5, -0.75, -1.75, -3.5, -6, 3, 1, 0.5, 4],
                                                 np.float32) / 30.0)
    up[min(4, rows - 1), 100:116] = f2b(3e38); gate[min(4, rows - 1), 100:116] = f2b(20.0)   # overflow to inf
    return gate, up


@pytest.mark.parametrize("rows,n,its", [(5, 17408, 0.37), (130, 1088, 0.0), (3, 16, 1.25), (257, 80, 0.0)])
def test_swiglu_rows_equal_the_single_vector_entry_row_by_row(backend, rows, n, its):
    """qwen36_swiglu_nvfp4_quantize_rows: every row's code bytes and scale bytes are those of
    qwen36_swiglu_nvfp4_quantize on that row (itself byte-identical to the reference's kernel), also
    with gate and up as the two halves of one [rows, 2 n] buffer; untouched scale bytes stay zero."""
    rng = np.random.default_rng(rows * 7 + n)
    gate, up = _special_rows(rng, rows, n) if n >= 128 else (
        synth.f32_to_bf16_bits((rng.standard_normal((rows, n)) * 2.0).astype(np.float32)),
        np.stack([synth.activations(rng, 1, n)[0] for _ in range(rows)]))
    both = to_dev(np.concatenate([gate, up], axis=1))        # [rows, 2 n]: the gate_up GEMM's output layout
    groups = n // 16
    inner = (groups + 3) // 4 * 4
    for g_d, u_d in ((to_dev(gate), to_dev(up)), (both[:, :n], both[:, n:])):
        fp4, sf, ts = backend.swiglu_nvfp4_quantize_rows(g_d, u_d, its)
        fp4_h, sf_h = fp4.cpu().numpy(), sf.cpu().numpy()
        written = np.zeros(sf_h.size, dtype=bool)
        check = range(rows) if rows <= 8 else sorted({0, 1, 2, 3, 4, 31, 32, 127, 128, 129, rows - 1} & set(range(rows)))
        for r in check:
            f1, s1, t1 = backend.swiglu_nvfp4_quantize(g_d[r].contiguous(), u_d[r].contiguous(), its)
            assert ts.item() == t1.item()
            assert np.array_equal(fp4_h[r], f1.cpu().numpy()), r
            s1_h = s1.cpu().numpy()
            for g in range(groups):
                assert sf_h[orc.sf_offset(g, r, inner)] == s1_h[orc.sf_offset(g, 0, inner)], (r, g)
        for r in range(rows):
            for g in range(groups):
                written[orc.sf_offset(g, r, inner)] = True
        assert not sf_h[~written].any()


def test_swiglu_rows_vs_oracle_and_down_projection(backend):
    """Against the host oracle row by row (neighbouring codes only where libm and the device differ in
    the last place), and as the activation operand of the down projection's GEMM."""
    rng = np.random.default_rng(2025)
    rows, n, n_out = 48, 2048, 256
    gate = synth.f32_to_bf16_bits((rng.standard_normal((rows, n)) * 2.0).astype(np.float32))
    up = np.stack([synth.activations(rng, 1, n, outlier_frac=0.01)[0] for _ in range(rows)])
    fp4, sf, ts = backend.swiglu_nvfp4_quantize_rows(to_dev(gate), to_dev(up), 0.37)
    fp4_h, sf_h = fp4.cpu().numpy(), sf.cpu().numpy()
    groups, inner = n // 16, n // 16
    for r in (0, 17, 47):
        want = orc.swiglu_nvfp4_quantize(gate[r], up[r], 0.37)
        row_sf = np.zeros_like(want["sf"])
        for g in range(groups):
            row_sf[orc.sf_offset(g, 0, inner)] = sf_h[orc.sf_offset(g, r, inner)]
        assert_codes_close(fp4_h[r], row_sf, want["fp4"], want["sf"], n)
    packed, sf_rm = synth.nvfp4_weight(rng, n_out, n)
    a_sf = orc.retile_scales(sf_rm)
    alpha = synth.WEIGHT_GLOBAL_SCALE * 0.37
    c = backend.nvfp4_gemm(to_dev(packed), to_dev(a_sf), fp4, sf, alpha, n_out, rows, n)
    want = synth.bf16_bits_to_f32(orc.nvfp4_gemm(packed, a_sf, fp4_h, sf_h, alpha, n_out, rows, n))
    got = synth.bf16_bits_to_f32(bf16_host(c))
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-2


def test_swiglu_rows_argument_checks(backend):
    import ctypes as C
    lib = backend.lib
    g = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    fp4 = torch.zeros((4, 32), dtype=torch.uint8, device="cuda")
    sf = torch.zeros(512, dtype=torch.uint8, device="cuda")
    dp = lambda t: abi.DevicePtr(0 if t is None else t.data_ptr())

    def spec(rows=4, n=64, stride=64, gate=g, up=g, out=fp4, scales=sf):
        return abi.SwigluNvfp4QuantizeRowsSpec(rows, n, stride, dp(gate), dp(up), dp(out), dp(scales), dp(None), 0.0)
    assert lib.qwen36_swiglu_nvfp4_quantize_rows(None) == abi.NULL_POINTER
    assert lib.qwen36_swiglu_nvfp4_quantize_rows(C.byref(spec())) == abi.SUCCESS
    for bad in (spec(rows=0), spec(n=0), spec(n=40), spec(stride=48), spec(stride=68), spec(gate=None), spec(up=None),
                spec(out=None), spec(scales=None), spec(gate=g.view(-1)[4:].view(-1))):
        assert lib.qwen36_swiglu_nvfp4_quantize_rows(C.byref(bad)) == abi.INVALID_ARGUMENT
