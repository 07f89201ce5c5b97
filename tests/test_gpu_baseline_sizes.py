"""Parity at the benchmark configurations' own sizes (the other GPU test files use sizes the
oracle finishes in milliseconds):

* prefill chain (config 2): quantize_rows codes and scale bytes bit-exact against the oracle at the
  full [M, K] size, and 4096 sampled (token, feature) outputs of the GEMM against the oracle's
  float64 dequantise-and-dot, rel-L2 <= 1e-2, on gate_up 34816 x 5120 and down 5120 x 17408 for
  M in {512, 2048, 8192}; where the reference's own CUDA library has been built, the whole output
  also against the reference's cuBLASLt call;
* int8 KV attention (config 4) at 32768 and 131072 tokens and the BF16 / FP8 decode attention at
  32768 tokens against the oracle, rel-L2 <= 1e-2;
* fused lm_head argmax (config 3) over the whole 248320-row vocabulary, M in {1, 4}: indices equal
  to the oracle's argmax over all logits.
"""
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


def rel_l2(got, want):
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    return np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)


def outlier_activations(gen, rows, k):
    """bf16 ~ N(0, 1) with 1 % of the channels scaled by 20 (config 2)."""
    x = torch.randn((rows, k), generator=gen, device="cuda")
    ch = torch.randperm(k, generator=gen, device="cuda")[: k // 100]
    x[:, ch] *= 20.0
    return x.to(torch.bfloat16)


# ------------------------------------------------------------------ config 2: prefill chain

@pytest.fixture(scope="module")
def prefill_weights():
    gen = torch.Generator(device="cuda").manual_seed(4242)
    out = {}
    for name, n_out, k in (("gate_up", 34816, 5120), ("down", 5120, 17408)):
        packed, sf_rm = synth.nvfp4_weight_device(gen, n_out, k, "cuda")
        out[name] = (n_out, k, packed, sf_rm)
    return out


@pytest.mark.parametrize("shape", ["gate_up", "down"])
@pytest.mark.parametrize("tokens", [512, 2048, 8192])
def test_prefill_chain_at_config_sizes(backend, prefill_weights, shape, tokens):
    n_out, k, packed, sf_rm = prefill_weights[shape]
    sfa = backend.nvfp4_retile_scales(sf_rm)
    gen = torch.Generator(device="cuda").manual_seed(tokens + k)
    x = outlier_activations(gen, tokens, k)
    its = 0.37
    fp4, sfb, ts = backend.nvfp4_quantize_rows(x, its)
    x_h = bf16_host(x)
    w_fp4, w_sf, w_ts = orc.nvfp4_quantize_rows(x_h, its)
    assert float(ts.item()) == np.float32(w_ts)
    assert np.array_equal(fp4.cpu().numpy(), w_fp4), "packed activation codes"
    assert np.array_equal(sfb.cpu().numpy(), w_sf), "activation scale bytes"
    del x_h
    alpha = float(np.float32(synth.WEIGHT_GLOBAL_SCALE) * np.float32(w_ts))
    c = torch.zeros((tokens, n_out), dtype=torch.bfloat16, device="cuda")
    assert backend.nvfp4_gemm_raw(packed, sfa, fp4, sfb, alpha, n_out, tokens, k, c) == abi.SUCCESS
    torch.cuda.synchronize()
    assert backend.lib.qwen36_nvfp4_gemm_last_error() == 0
    rng = np.random.default_rng(tokens + n_out)
    tok = rng.integers(0, tokens, 4096).astype(np.uint32)
    feat = rng.integers(0, n_out, 4096).astype(np.uint32)
    # corners and tile borders are the likeliest places for an addressing slip
    tok[:8] = [0, 0, tokens - 1, tokens - 1, 127, 128, 255, 256]
    feat[:8] = [0, n_out - 1, 0, n_out - 1, 127, 128, n_out - 129, n_out - 128]
    want = orc.nvfp4_gemm_sampled(packed.cpu().numpy(), sfa.cpu().numpy(), w_fp4, w_sf, alpha, n_out, tokens, k, tok, feat)
    got = c[torch.from_numpy(tok.astype(np.int64)).cuda(), torch.from_numpy(feat.astype(np.int64)).cuda()].float().cpu().numpy()
    err = rel_l2(got, want)
    assert err <= 1e-2, err
    # every sampled output within bf16 rounding of the float64 value
    assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -7 + 1e-6)
    if os.path.exists(REF_SO):
        ref = C.CDLL(REF_SO, mode=os.RTLD_LOCAL | os.RTLD_DEEPBIND)
        dp = lambda t: abi.DevicePtr(0 if t is None else t.data_ptr())
        c_ref = torch.zeros_like(c)
        ws = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
        spec = abi.Nvfp4GemmSpec(n_out, tokens, k, dp(packed), dp(sfa), dp(None), dp(fp4), dp(sfb), dp(None), dp(c_ref),
                                 dp(ws), ws.numel(), alpha)
        torch.cuda.synchronize()
        rc = ref.qwen36_nvfp4_gemm(C.byref(spec))
        torch.cuda.synchronize()
        if rc == 0:
            same = (c.view(torch.int16) == c_ref.view(torch.int16)).float().mean().item()
            diff = (c.float() - c_ref.float()).norm().item() / c_ref.float().norm().item()
            assert diff <= 1e-3 and same >= 0.99, (diff, same)


# ------------------------------------------------------------------ NVFP4 lm_head scan

@pytest.fixture(scope="module")
def nvfp4_lm_head_weight(backend):
    gen = torch.Generator(device="cuda").manual_seed(777)
    packed, sf_rm = synth.nvfp4_weight_device(gen, synth.VOCAB, synth.HIDDEN, "cuda")
    sfa = backend.nvfp4_retile_scales(sf_rm)
    return packed, sfa, packed.cpu().numpy(), sfa.cpu().numpy()


@pytest.mark.parametrize("tokens", [1, 4, 16])
def test_nvfp4_lm_head_scan_shape_vs_oracle(backend, nvfp4_lm_head_weight, tokens):
    """The reference's NVFP4 lm_head is its W4A4 GEMM at m = vocabulary, n <= 16 tokens, k = hidden
    (crates/runtime/src/engine.rs:11609-11663; one token goes to the decode GEMV first, as
    crates/kernels/src/backend.rs:213-233 routes it).  4096 sampled logits, corners and tile borders
    included, against the float64 dequantise-and-dot of the oracle."""
    n_out, k = synth.VOCAB, synth.HIDDEN
    packed, sfa, packed_h, sfa_h = nvfp4_lm_head_weight
    gen = torch.Generator(device="cuda").manual_seed(tokens + 99)
    x = torch.randn((tokens, k), generator=gen, device="cuda").to(torch.bfloat16)
    its = 0.37
    fp4, sfb, ts = backend.nvfp4_quantize_rows(x, its)
    w_fp4, w_sf, w_ts = orc.nvfp4_quantize_rows(bf16_host(x), its)
    assert np.array_equal(fp4.cpu().numpy(), w_fp4) and np.array_equal(sfb.cpu().numpy(), w_sf)
    alpha = float(np.float32(synth.WEIGHT_GLOBAL_SCALE) * np.float32(w_ts))
    c = backend.nvfp4_gemm(packed, sfa, fp4, sfb, alpha, n_out, tokens, k)
    torch.cuda.synchronize()
    assert backend.lib.qwen36_nvfp4_gemm_last_error() == 0
    rng = np.random.default_rng(tokens + n_out)
    tok = rng.integers(0, tokens, 4096).astype(np.uint32)
    feat = rng.integers(0, n_out, 4096).astype(np.uint32)
    tok[:4] = [0, 0, tokens - 1, tokens - 1]
    feat[:8] = [0, n_out - 1, 0, n_out - 1, 127, 128, n_out - 129, n_out - 128]
    want = orc.nvfp4_gemm_sampled(packed_h, sfa_h, w_fp4, w_sf, alpha, n_out, tokens, k, tok, feat)
    got = c[torch.from_numpy(tok.astype(np.int64)).cuda(), torch.from_numpy(feat.astype(np.int64)).cuda()].float().cpu().numpy()
    assert rel_l2(got, want) <= 1e-2
    assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -7 + 1e-6)


# ------------------------------------------------------------------ config 4: long contexts

@pytest.fixture(scope="module")
def long_cache():
    rng = np.random.default_rng(20260)
    T = 131072
    q, k, v = synth.qkv(rng, T)                      # 4 outlier channels per head scaled by 10
    kq = np.zeros((T, 4, 256), np.int8); vq = np.zeros_like(kq)
    meta = np.zeros((T, 4, 2), np.float32)
    orc.kv_encode(k, v, 0, kq, vq, meta)
    return q, k, v, kq, vq, meta


@pytest.mark.parametrize("ctx", [32768, 131072])
def test_int8_attention_long_context_vs_oracle(backend, long_cache, ctx):
    q, k, v, kq_o, vq_o, meta_o = long_cache
    kq = torch.zeros((ctx, 4, 256), dtype=torch.int8, device="cuda"); vq = torch.zeros_like(kq)
    meta = torch.zeros((ctx, 4, 2), dtype=torch.float32, device="cuda")
    backend.turboquant_encode_kv_rows(to_dev(k[:ctx]), to_dev(v[:ctx]), kq, vq, meta, 0)
    assert np.array_equal(kq.cpu().numpy(), kq_o[:ctx]) and np.array_equal(vq.cpu().numpy(), vq_o[:ctx])
    assert np.array_equal(meta.cpu().numpy().view(np.uint32), meta_o[:ctx].view(np.uint32))
    ws = backend.attention_workspace(24, 256, "cuda")
    out = backend.turboquant_attention(to_dev(q), kq, vq, meta, ctx - 1, ws)
    want = synth.bf16_bits_to_f32(orc.kv_attention(q, kq_o, vq_o, meta_o, ctx - 1))
    err = rel_l2(synth.bf16_bits_to_f32(bf16_host(out)), want)
    assert err <= 1e-2, err
    # the allocation-free entry on the same inputs, against the oracle too
    got = torch.full((24, 256), float("nan"), dtype=torch.bfloat16, device="cuda")
    got = backend.turboquant_attention_static(to_dev(q), kq, vq, meta, ctx - 1, got)
    assert rel_l2(synth.bf16_bits_to_f32(bf16_host(got)), want) <= 1e-2


@pytest.mark.parametrize("dtype", [0, 1])
def test_decode_attention_32768_vs_oracle(backend, long_cache, dtype):
    from test_gpu_kv_decode import cache_to_dev, cache_host, e4m3_encode_bits, partial_buffers
    q, k, v = long_cache[:3]
    ctx = 32768
    ck = e4m3_encode_bits(k[:ctx]) if dtype == 1 else k[:ctx].copy()
    cv = e4m3_encode_bits(v[:ctx]) if dtype == 1 else v[:ctx].copy()
    k_new, v_new = k[ctx], v[ctx]
    ck_d, cv_d = cache_to_dev(ck), cache_to_dev(cv)
    out = backend.attention_decode(to_dev(q), to_dev(k_new), to_dev(v_new), ck_d, cv_d, ctx - 1, dtype,
                                   partial_buffers(24, 256, 256), 256)
    torch.cuda.synchronize()
    want = synth.bf16_bits_to_f32(orc.attention_decode(q, k_new, v_new, ck, cv, dtype, ctx - 1))
    err = rel_l2(synth.bf16_bits_to_f32(bf16_host(out)), want)
    assert err <= 1e-2, err
    assert np.array_equal(cache_host(ck_d), ck) and np.array_equal(cache_host(cv_d), cv)


# ------------------------------------------------------------------ config 3: whole vocabulary

@pytest.mark.parametrize("tokens", [1, 4])
def test_fused_lm_head_argmax_whole_vocab_vs_oracle(backend, tokens):
    gen = torch.Generator(device="cuda").manual_seed(50 + tokens)
    rows, cols = synth.VOCAB, synth.HIDDEN
    w = torch.randint(0, 0x7F, (rows, cols), generator=gen, dtype=torch.uint8, device="cuda")
    w |= (torch.randint(0, 2, (rows, cols), generator=gen, dtype=torch.uint8, device="cuda") << 7)
    s = torch.exp2(torch.rand(rows, generator=gen, device="cuda") * 4 - 6)
    x = torch.randn((tokens, cols), generator=gen, device="cuda").to(torch.bfloat16)
    ws = backend.lm_head_argmax_workspace(rows, tokens, "cuda")
    tok, best = backend.lm_head_fp8_gemv_argmax(w, s, x, ws)
    logits = backend.lm_head_fp8_gemv(w, s, x)
    want_logits = orc.lm_head_fp8_gemv(w.cpu().numpy(), s.cpu().numpy(), bf16_host(x))
    want = orc.argmax_rows(want_logits)
    assert np.array_equal(tok.cpu().numpy().astype(np.uint32), want)
    assert np.array_equal(best.cpu().numpy(), synth.bf16_bits_to_f32(want_logits[np.arange(tokens), want]))
    assert np.array_equal(bf16_host(logits), want_logits)          # all 248320 logits per token, bit for bit
