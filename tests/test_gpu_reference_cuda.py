"""Pins the CPU oracle to the reference itself: the reference's own CUDA kernels (compiled for
sm_100a from the reference checkout into oracle/_ref by oracle/Makefile, never copied) run on
the GPU and their outputs are compared with the oracle on the same seeded inputs.  Skipped when
that library has not been built.  The reference's sm_120-only decode GEMV is not part of it."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from speedoza_b200 import abi, synth
from conftest import bf16_host, to_dev

pytestmark = pytest.mark.gpu

REF_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                      "libqwen36_ref.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_SO) or not torch.cuda.is_available():
        pytest.skip("oracle/_ref/libqwen36_ref.so not built")
    torch.zeros(1, device="cuda")
    return C.CDLL(REF_SO, mode=os.RTLD_LOCAL | os.RTLD_DEEPBIND)


def dp(t):
    return abi.DevicePtr(0 if t is None else t.data_ptr())


def test_reference_quantize_and_retile_equal_oracle(ref):
    rng = np.random.default_rng(11)
    x = synth.activations(rng, 37, 5120, outlier_frac=0.01)
    x[1, :16] = synth.f32_to_bf16_bits(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 2, np.float32))
    # amax/6 exactly between subnormal UE4M3 codes (float32 tie behaviour of the encoder)
    x[2, ::16] = synth.f32_to_bf16_bits(np.resize(np.array([(c + 0.5) * 2.0 ** -9 * 6 for c in range(1, 7)], np.float32), 320))
    for its in (0.0, 1.25, 0.37):
        xd = to_dev(x)
        fp4 = torch.zeros((37, 2560), dtype=torch.uint8, device="cuda")
        sf = torch.zeros(orc.sf_bytes(320, 37), dtype=torch.uint8, device="cuda")
        ts = torch.zeros(1, dtype=torch.float32, device="cuda")
        spec = abi.Nvfp4QuantizeRowsSpec(37, 5120, dp(xd), dp(fp4), dp(sf), dp(ts), its)
        assert ref.qwen36_nvfp4_quantize_rows(C.byref(spec)) == 0
        torch.cuda.synchronize()
        w_fp4, w_sf, w_ts = orc.nvfp4_quantize_rows(x, its)
        assert np.array_equal(fp4.cpu().numpy(), w_fp4)
        assert np.array_equal(sf.cpu().numpy(), w_sf)
        assert ts.item() == np.float32(w_ts)
    sf_rm = rng.integers(0, 256, size=(300, 13), dtype=np.uint8)
    out = torch.full((orc.sf_bytes(13, 300),), 0xAA, dtype=torch.uint8, device="cuda")
    sf_rm_d = to_dev(sf_rm)
    spec = abi.Nvfp4RetileScalesSpec(300, 13, dp(sf_rm_d), dp(out))
    assert ref.qwen36_nvfp4_retile_scales(C.byref(spec)) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), orc.retile_scales(sf_rm))


def test_reference_matvec_equals_oracle_bitwise(ref):
    """The reference's scalar matvec has two input paths.  Its vector path reads sixteen bf16
    activations through a 16-byte `uint4` (kernels-cuda/ops.cu:597-604: eight bf16 pairs are
    indexed out of a value that holds four), so half of every group's activations are
    indeterminate there.  Its element-wise path (taken when the activation pointer is not
    16-byte aligned) is the documented arithmetic, and that is what the oracle is pinned to."""
    rng = np.random.default_rng(12)
    n, k = 1024, 5120
    packed, sf_rm = synth.nvfp4_weight(rng, n, k)
    sf = orc.retile_scales(sf_rm)
    x = synth.activations(rng, 1, k)[0]
    ts = torch.tensor([synth.WEIGHT_GLOBAL_SCALE], dtype=torch.float32, device="cuda")
    y = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    x_pad = torch.zeros(k + 8, dtype=torch.bfloat16, device="cuda")
    x_pad[1:k + 1] = to_dev(x)
    x_unaligned = x_pad[1:k + 1]                     # 2 bytes past a 16-byte boundary
    assert x_unaligned.data_ptr() % 16 == 2
    pd, sd = to_dev(packed), to_dev(sf)              # keep the buffers alive across the call
    spec = abi.Nvfp4MatvecSpec(n, k, dp(x_unaligned), dp(pd), dp(sd), dp(ts), dp(y))
    assert ref.qwen36_nvfp4_matvec(C.byref(spec)) == 0
    torch.cuda.synchronize()
    want = orc.nvfp4_matvec(x, packed, sf, synth.WEIGHT_GLOBAL_SCALE, k)
    assert np.array_equal(bf16_host(y), want)      # same summation order, same fused multiply-adds


def test_reference_lm_head_equals_oracle_bitwise(ref):
    rng = np.random.default_rng(13)
    rows, cols, n = 1500, 5120, 4
    wb = synth.f32_to_bf16_bits((rng.standard_normal((rows, cols)) * 0.05).astype(np.float32))
    wd = to_dev(wb)
    q = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
    s = torch.zeros(rows, dtype=torch.float32, device="cuda")
    spec = abi.LmHeadFp8QuantizeSpec(rows, cols, dp(wd), dp(q), dp(s))
    assert ref.qwen36_lm_head_fp8_quantize(C.byref(spec)) == 0
    torch.cuda.synchronize()
    oq, os_ = orc.lm_head_fp8_quantize(wb)
    assert np.array_equal(q.cpu().numpy(), oq) and np.array_equal(s.cpu().numpy().view(np.uint32), os_.view(np.uint32))
    x = synth.activations(rng, n, cols)
    y = torch.zeros((n, rows), dtype=torch.bfloat16, device="cuda")
    xd = to_dev(x)
    spec = abi.LmHeadFp8GemvSpec(rows, cols, n, dp(q), dp(s), dp(xd), dp(y))
    assert ref.qwen36_lm_head_fp8_gemv(C.byref(spec)) == 0
    torch.cuda.synchronize()
    want = orc.lm_head_fp8_gemv(oq, os_, x)
    assert np.array_equal(bf16_host(y), want)
    tok = torch.zeros(n, dtype=torch.int32, device="cuda")
    spec = abi.SamplingRowsSpec(n, rows, dp(y), dp(tok), abi.DevicePtr(0), 1.0)
    assert ref.qwen36_sample_rows(C.byref(spec)) == 0
    torch.cuda.synchronize()
    assert np.array_equal(tok.cpu().numpy().astype(np.uint32), orc.argmax_rows(want))


def test_reference_int8_kv_equals_oracle(ref):
    rng = np.random.default_rng(14)
    T = 40
    q, k, v = synth.qkv(rng, T)
    kq = torch.zeros((T, 4, 256), dtype=torch.int8, device="cuda"); vq = torch.zeros_like(kq)
    meta = torch.zeros((T, 4, 2), dtype=torch.float32, device="cuda")
    shape = abi.AttentionShape(24, 4, 256, 0)
    kd, vd = to_dev(k), to_dev(v)
    for t in range(T):
        spec = abi.TurboquantEncodeSpec(0, t, dp(kd[t]), dp(vd[t]), dp(kq), dp(vq), dp(meta), shape)
        assert ref.qwen36_turboquant_encode_kv(C.byref(spec)) == 0
    torch.cuda.synchronize()
    kq_o = np.zeros((T, 4, 256), np.int8); vq_o = np.zeros_like(kq_o); meta_o = np.zeros((T, 4, 2), np.float32)
    orc.kv_encode(k, v, 0, kq_o, vq_o, meta_o)
    assert np.array_equal(kq.cpu().numpy(), kq_o) and np.array_equal(vq.cpu().numpy(), vq_o)
    assert np.array_equal(meta.cpu().numpy().view(np.uint32), meta_o.view(np.uint32))
    out = torch.zeros((24, 256), dtype=torch.bfloat16, device="cuda")
    qd = to_dev(q)
    spec = abi.TurboquantAttentionSpec(0, T - 1, dp(qd), dp(kq), dp(vq), dp(meta), dp(out),
                                       abi.DevicePtr(0), 0, shape, 0)
    assert ref.qwen36_turboquant_attention(C.byref(spec)) == 0
    torch.cuda.synchronize()
    want = synth.bf16_bits_to_f32(orc.kv_attention(q, kq_o, vq_o, meta_o, T - 1)).astype(np.float64)
    got = synth.bf16_bits_to_f32(bf16_host(out)).astype(np.float64)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 2e-3     # expf differs by an ulp or two


@pytest.mark.parametrize("hidden,with_residual,its", [(5120, True, 0.0), (5120, False, 0.37), (6144, True, 1.25),
                                                      (33, True, 1.25), (100, False, 0.0)])
def test_rmsnorm_nvfp4_quantize_equals_reference_bitwise(ref, backend, hidden, with_residual, its):
    """This library's fused RMSNorm + quantise against the reference's own kernel, both on the GPU:
    every output byte equal (bf16 copy, residual, codes, tiled scale bytes, tensor scale)."""
    rng = np.random.default_rng(31 * hidden + int(its * 100))
    x = to_dev(synth.activations(rng, 1, hidden, outlier_frac=0.01)[0])
    w = to_dev(synth.f32_to_bf16_bits((rng.standard_normal(hidden) * 0.1).astype(np.float32)))
    res = to_dev(synth.activations(rng, 1, hidden)[0]) if with_residual else None
    outs = []
    for entry in (ref.qwen36_rmsnorm_nvfp4_quantize, backend.lib.qwen36_rmsnorm_nvfp4_quantize):
        out = torch.zeros(hidden, dtype=torch.bfloat16, device="cuda")
        res_out = torch.zeros(hidden, dtype=torch.bfloat16, device="cuda")
        fp4 = torch.zeros((hidden + 1) // 2, dtype=torch.uint8, device="cuda")
        sf = torch.zeros(orc.sf_bytes((hidden + 15) // 16, 1), dtype=torch.uint8, device="cuda")
        ts = torch.zeros(1, dtype=torch.float32, device="cuda")
        spec = abi.RmsnormNvfp4QuantizeSpec(hidden, 1e-6, dp(x), dp(w), dp(res), dp(res_out), dp(out), dp(fp4), dp(sf),
                                            dp(ts), its)
        assert entry(C.byref(spec)) == 0
        torch.cuda.synchronize()
        outs.append([t.cpu().numpy() for t in (out.view(torch.int16), res_out.view(torch.int16), fp4, sf, ts)])
    for a, b in zip(*outs):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("n,its", [(17408, 0.0), (17408, 0.37), (33, 1.25), (1000, 0.0)])
def test_swiglu_nvfp4_quantize_equals_reference_bitwise(ref, backend, n, its):
    rng = np.random.default_rng(17 * n + int(its * 100))
    gate = to_dev(synth.f32_to_bf16_bits((rng.standard_normal(n) * 2.0).astype(np.float32)))
    up = to_dev(synth.activations(rng, 1, n, outlier_frac=0.01)[0])
    outs = []
    for entry in (ref.qwen36_swiglu_nvfp4_quantize, backend.lib.qwen36_swiglu_nvfp4_quantize):
        fp4 = torch.zeros((n + 1) // 2, dtype=torch.uint8, device="cuda")
        sf = torch.zeros(orc.sf_bytes((n + 15) // 16, 1), dtype=torch.uint8, device="cuda")
        ts = torch.zeros(1, dtype=torch.float32, device="cuda")
        spec = abi.SwigluNvfp4QuantizeSpec(n, dp(gate), dp(up), dp(fp4), dp(sf), dp(ts), its)
        assert entry(C.byref(spec)) == 0
        torch.cuda.synchronize()
        outs.append([t.cpu().numpy() for t in (fp4, sf, ts)])
    for a, b in zip(*outs):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("position,n_splits", [(0, 0), (37, 0), (700, 0), (2100, 8), (5000, 64)])
def test_reference_attention_decode_equals_oracle_and_this_library(ref, backend, dtype, position, n_splits):
    """qwen36_attention_decode over a BF16 / FP8 cache: the reference's kernels (its one-block-per-head
    kernel without partial buffers, its GQA split / register-tiled kernels with them), the oracle and
    this library on the same inputs.  Outputs within rel-L2 1e-2 of the oracle; the cache after the
    call (append side effect) is byte-identical in all three."""
    from test_gpu_kv_decode import make_case, cache_to_dev, cache_host, partial_buffers, rel_l2
    q, k_new, v_new, ck, cv = make_case(900 + position + dtype, position + 1, 24, 4, 256, dtype)
    qd, kd, vd = to_dev(q), to_dev(k_new), to_dev(v_new)
    ck_o, cv_o = ck.copy(), cv.copy()
    want = synth.bf16_bits_to_f32(orc.attention_decode(q, k_new, v_new, ck_o, cv_o, dtype, position))

    ck_r, cv_r = cache_to_dev(ck), cache_to_dev(cv)
    out_r = torch.zeros((24, 256), dtype=torch.bfloat16, device="cuda")
    parts = partial_buffers(24, n_splits, 256) if n_splits else (None, None, None)
    spec = abi.AttentionDecodeSpec(0, position, dp(qd), dp(kd), dp(vd), dp(ck_r), dp(cv_r), dp(None), dp(out_r),
                                   abi.AttentionShape(24, 4, 256, 0), dtype, dp(None), dp(parts[0]), dp(parts[1]),
                                   dp(parts[2]), n_splits, 0)
    torch.cuda.synchronize()
    assert ref.qwen36_attention_decode(C.byref(spec)) == 0
    torch.cuda.synchronize()
    assert rel_l2(synth.bf16_bits_to_f32(bf16_host(out_r)), want) <= 1e-2
    assert np.array_equal(cache_host(ck_r), ck_o) and np.array_equal(cache_host(cv_r), cv_o)

    ck_m, cv_m = cache_to_dev(ck), cache_to_dev(cv)
    out_m = backend.attention_decode(qd, kd, vd, ck_m, cv_m, position, dtype,
                                     partial_buffers(24, n_splits, 256) if n_splits else None, n_splits)
    torch.cuda.synchronize()
    assert rel_l2(synth.bf16_bits_to_f32(bf16_host(out_m)), want) <= 1e-2
    assert torch.equal(ck_m, ck_r) and torch.equal(cv_m, cv_r)
    # the two GPU implementations against each other
    assert rel_l2(synth.bf16_bits_to_f32(bf16_host(out_m)),
                  synth.bf16_bits_to_f32(bf16_host(out_r)).astype(np.float64)) <= 1e-2


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("start,tokens,n_splits", [(0, 16, 1), (100, 5, 3), (1000, 16, 16), (4093, 32, 48), (700, 9, 64)])
def test_reference_verify_attention_equals_oracle_and_this_library(ref, backend, dtype, start, tokens, n_splits):
    """qwen36_attention_flash_splitk_prefill_bf16: the reference's wmma kernel + reduce, this library's
    kernel + reduce and the oracle on the same seeded inputs (seed 515151 as in the reference's own
    kernel-vs-kernel gate, kernels-cuda/smoke.cu:3614-3773).  Outputs within rel-L2 1e-2 of the oracle
    and of each other; the per-split partials (same partition, same token-major layout) agree too:
    max within 1e-3, denominator and accumulator within rel 5e-3 (both round P to the operand type)."""
    from test_gpu_attention_verify import make_verify_case, rel_l2
    from test_gpu_kv_decode import cache_to_dev
    q, ck, cv = make_verify_case(515151 + start + tokens + dtype, start, tokens, 24, 4, dtype)
    want = orc.attention_verify(q, ck, cv, dtype, start)
    qd, ckd, cvd = to_dev(q), cache_to_dev(ck), cache_to_dev(cv)
    results = []
    for lib in (ref, backend.lib):
        out = torch.zeros((tokens, 24, 256), dtype=torch.bfloat16, device="cuda")
        pa = torch.zeros((tokens, 24, n_splits, 256), device="cuda")
        pm = torch.zeros((tokens, 24, n_splits), device="cuda")
        pl = torch.zeros((tokens, 24, n_splits), device="cuda")
        spec = abi.AttentionPrefillSpec(0, start, tokens, dp(qd), dp(None), dp(None), dp(ckd), dp(cvd), dp(None), dp(out),
                                        abi.AttentionShape(24, 4, 256, 0), dtype, dp(None), dp(pa), dp(pm), dp(pl), 0, 0,
                                        dp(None), 0)
        torch.cuda.synchronize()
        assert lib.qwen36_attention_flash_splitk_prefill_bf16(C.byref(spec), n_splits) == 0
        torch.cuda.synchronize()
        got = synth.bf16_bits_to_f32(bf16_host(out))
        assert rel_l2(got, want) <= 1e-2
        results.append((got, pa.cpu().numpy(), pm.cpu().numpy(), pl.cpu().numpy()))
    (o_r, pa_r, pm_r, pl_r), (o_m, pa_m, pm_m, pl_m) = results
    assert rel_l2(o_m, o_r) <= 1e-2
    assert np.array_equal(np.isneginf(pm_r), np.isneginf(pm_m))
    live = ~np.isneginf(pm_r)
    assert np.allclose(pm_m[live], pm_r[live], rtol=0, atol=1e-3)
    assert np.allclose(pl_m[live], pl_r[live], rtol=5e-3)
    assert rel_l2(pa_m, pa_r) <= 5e-3


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("position,block", [(0, 64), (513, 64), (3000, 128), (2049, 8)])
def test_reference_decode_split_tiled_equals_this_library(ref, backend, dtype, position, block):
    """qwen36_attention_decode_split_tiled: partials of the reference's register-tiled kernel and of this
    library for the same fixed-size splits, and the cache after the call (append by the owning split)
    byte-identical."""
    from test_gpu_kv_decode import make_case, cache_to_dev, cache_host, partial_buffers
    q, k_new, v_new, ck, cv = make_case(626262 + position + dtype, position + 1, 24, 4, 256, dtype)
    qd, kd, vd = to_dev(q), to_dev(k_new), to_dev(v_new)
    n_splits = position // block + 2
    results = []
    for lib in (ref, backend.lib):
        ckd, cvd = cache_to_dev(ck), cache_to_dev(cv)
        pa, pm, pl = partial_buffers(24, n_splits, 256)
        out = torch.zeros((24, 256), dtype=torch.bfloat16, device="cuda")
        spec = abi.AttentionDecodeSpec(0, position, dp(qd), dp(kd), dp(vd), dp(ckd), dp(cvd), dp(None), dp(out),
                                       abi.AttentionShape(24, 4, 256, 0), dtype, dp(None), dp(pa), dp(pm), dp(pl),
                                       n_splits, block)
        torch.cuda.synchronize()
        assert lib.qwen36_attention_decode_split_tiled(C.byref(spec), n_splits, block) == 0
        torch.cuda.synchronize()
        results.append((pa.cpu().numpy(), pm.cpu().numpy(), pl.cpu().numpy(), cache_host(ckd), cache_host(cvd)))
    (pa_r, pm_r, pl_r, ck_r, cv_r), (pa_m, pm_m, pl_m, ck_m, cv_m) = results
    assert np.array_equal(ck_r, ck_m) and np.array_equal(cv_r, cv_m)
    assert np.array_equal(np.isneginf(pm_r), np.isneginf(pm_m))
    live = ~np.isneginf(pm_r)
    assert np.allclose(pm_m[live], pm_r[live], rtol=0, atol=2e-3)
    assert np.allclose(pl_m[live], pl_r[live], rtol=1e-2)
    assert np.linalg.norm(pa_m - pa_r) / np.linalg.norm(pa_r) <= 1e-2


@pytest.mark.parametrize("m_out,k,tokens", [(1024, 5120, 1), (1024, 5120, 5), (2048, 5120, 128), (1024, 17408, 512),
                                            (4096, 5120, 2048)])
def test_nvfp4_gemm_equals_reference_cublaslt(ref, backend, m_out, k, tokens):
    """The reference's prefill path (qwen36_nvfp4_gemm -> cuBLASLt block-scaled NVFP4, kernels-cuda/
    nvfp4_gemm.cu:341-409) and this library's tcgen05 kernels on the same quantised operands: both
    accumulate exact FP4 x FP4 x scale products in float32 and round once to bf16, so they agree to
    the last bits of the accumulation order (rel-L2 <= 1e-3 asserted; the share of identical bf16
    outputs is checked too), and both sit within rel-L2 1e-2 of the float64 oracle."""
    rng = np.random.default_rng(m_out + k + tokens)
    packed, sf_rm = synth.nvfp4_weight(rng, m_out, k)
    sfa = orc.retile_scales(sf_rm)
    x = synth.activations(rng, tokens, k, outlier_frac=0.01)
    fp4, sfb, ts = orc.nvfp4_quantize_rows(x, 0.37)
    alpha = float(np.float32(ts) * np.float32(synth.WEIGHT_GLOBAL_SCALE))
    a_d, sfa_d, b_d, sfb_d = to_dev(packed), to_dev(sfa), to_dev(fp4), to_dev(sfb)
    c_ref = torch.zeros((tokens, m_out), dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    spec = abi.Nvfp4GemmSpec(m_out, tokens, k, dp(a_d), dp(sfa_d), dp(None), dp(b_d), dp(sfb_d), dp(None), dp(c_ref),
                             dp(ws), ws.numel(), alpha)
    torch.cuda.synchronize()
    rc = ref.qwen36_nvfp4_gemm(C.byref(spec))
    torch.cuda.synchronize()
    if rc != 0:
        pytest.skip(f"this cuBLASLt has no block-scaled NVFP4 plan for the shape (status {rc})")
    c_our = torch.zeros_like(c_ref)
    assert backend.nvfp4_gemm_raw(a_d, sfa_d, b_d, sfb_d, alpha, m_out, tokens, k, c_our) == 0
    torch.cuda.synchronize()
    got, want = synth.bf16_bits_to_f32(bf16_host(c_our)).astype(np.float64), synth.bf16_bits_to_f32(bf16_host(c_ref)).astype(np.float64)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3
    assert (bf16_host(c_our) == bf16_host(c_ref)).mean() >= 0.99
    if tokens <= 128:
        exact = orc.nvfp4_gemm(packed, sfa, fp4, sfb, alpha, m_out, tokens, k)
        exact = synth.bf16_bits_to_f32(exact).astype(np.float64) if exact.dtype == np.uint16 else exact.astype(np.float64)
        assert np.linalg.norm(want - exact.reshape(want.shape)) / np.linalg.norm(exact) <= 1e-2
