"""GPU parity of the FP8 lm_head path: quantise bytes and scales, bf16 logits and greedy
argmax indices are all bit-exact against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from speedoza_b200 import synth
from conftest import bf16_host, to_dev

pytestmark = pytest.mark.gpu


def test_quantize_bit_exact(backend):
    rng = np.random.default_rng(1)
    w = synth.f32_to_bf16_bits((rng.standard_normal((300, 512)) * np.exp2(rng.uniform(-8, 8, (300, 1)))).astype(np.float32))
    w[7] = 0
    q, s = backend.lm_head_fp8_quantize(to_dev(w))
    wq, ws = orc.lm_head_fp8_quantize(w)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), ws.view(np.uint32))
    assert np.array_equal(q.cpu().numpy(), wq)


@pytest.mark.parametrize("rows,cols,n", [(1000, 5120, 1), (1003, 5120, 4), (517, 1024, 5), (64, 528, 2),
                                         (33, 16, 1), (200, 5120, 16), (9, 2048, 8), (700, 5120, 11)])
def test_gemv_logits_bit_exact(backend, rows, cols, n):
    rng = np.random.default_rng(rows + cols + n)
    w, s = synth.lm_head_weight(rng, rows, cols)
    x = synth.activations(rng, n, cols)
    got = bf16_host(backend.lm_head_fp8_gemv(to_dev(w), to_dev(s), to_dev(x)))
    want = orc.lm_head_fp8_gemv(w, s, x)
    assert np.array_equal(got, want)


def test_argmax_rows_rule(backend):
    # kernels-cuda/smoke.cu:126-200: ties -> lowest index; NaN never wins; all-bad row -> 0
    logits = np.array([[1, 5, 2, 3, 5, 0], [7, 1, 1, 1, 1, 1], [np.nan, -np.inf, 3, np.nan, 3, 0],
                       [np.nan, -np.inf, np.nan, -np.inf, np.nan, np.nan]], dtype=np.float32)
    lb = synth.f32_to_bf16_bits(logits); lb[2, 0] = 0x7FC0; lb[2, 3] = 0xFFC0; lb[3, 0] = 0x7FC0
    mirror = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = backend.sample_rows(to_dev(lb), 1.0, mirror).cpu().numpy()
    assert list(got) == [1, 0, 2, 0] and mirror.item() == 0
    assert backend.sample(to_dev(lb[0]), 0.7).item() == 1


@pytest.mark.parametrize("rows,vocab,temp", [(1, 248320, 1.0), (4, 248320, 0.0), (3, 1001, 0.6), (2, 7, 1.0)])
def test_argmax_rows_vs_oracle(backend, rows, vocab, temp):
    rng = np.random.default_rng(vocab + rows)
    logits = synth.f32_to_bf16_bits(rng.standard_normal((rows, vocab)).astype(np.float32) * 4)
    # plant exact ties of the maximum at several places
    for r in range(rows):
        top = logits[r].view(np.int16).max()
        logits[r, rng.integers(0, vocab, 3)] = np.uint16(top)
    got = backend.sample_rows(to_dev(logits), temp).cpu().numpy().astype(np.uint32)
    assert np.array_equal(got, orc.argmax_rows(logits, temp))
    # unaligned row start (odd vocab rows handled above); also offset base pointer by one element
    if vocab > 16:
        t = to_dev(logits[0])
        assert backend.sample(t[1:], temp).item() == orc.argmax_rows(logits[0:1, 1:].copy(), temp)[0]


@pytest.mark.parametrize("rows,n", [(4096, 1), (5003, 4), (777, 2), (31040, 4), (3001, 9), (2000, 16)])
def test_fused_gemv_argmax_bit_exact(backend, rows, n):
    cols = 5120 if rows != 777 else 1024
    rng = np.random.default_rng(rows + n)
    w, s = synth.lm_head_weight(rng, rows, cols)
    # duplicate some rows so that exact bf16 ties of the maximum exist
    w[rows // 2] = w[rows // 3]; s[rows // 2] = s[rows // 3]
    x = synth.activations(rng, n, cols)
    ws = backend.lm_head_argmax_workspace(rows, n, "cuda")
    wd, sd, xd = to_dev(w), to_dev(s), to_dev(x)
    for rep in range(2):          # second call checks that the workspace was left clean
        tok, best = backend.lm_head_fp8_gemv_argmax(wd, sd, xd, ws, row_offset=1000)
    logits = orc.lm_head_fp8_gemv(w, s, x)
    want = orc.argmax_rows(logits)
    assert np.array_equal(tok.cpu().numpy().astype(np.uint32), want + 1000)
    best_want = synth.bf16_bits_to_f32(logits[np.arange(n), want])
    assert np.array_equal(best.cpu().numpy(), best_want)
    # and equals the unfused device path
    unfused = backend.sample_rows(backend.lm_head_fp8_gemv(wd, sd, xd)).cpu().numpy()
    assert np.array_equal(unfused.astype(np.uint32), want)


def wide_range_activations(rng, n, cols, kind):
    """Token rows that the float16 route must take (a few octaves), must decline (values 2^40 apart, an
    infinity, a bf16 subnormal) or that are all zero."""
    x = rng.standard_normal((n, cols)).astype(np.float32)
    if kind == "octaves":
        x *= np.exp2(rng.integers(-12, 13, (n, cols))).astype(np.float32)
        x *= np.exp2(rng.integers(-60, 60, (n, 1))).astype(np.float32)      # every token on its own scale
    elif kind == "too_wide":
        x[0, ::7] *= np.float32(2.0 ** 40)
    elif kind == "infinity":
        x[n - 1, 5] = np.inf
    elif kind == "subnormal":
        x[0, 3] = np.float32(2.0 ** -130)
    elif kind == "zero_token":
        x[1] = 0.0
    elif kind == "huge":
        x *= np.float32(2.0 ** 110)
    return synth.f32_to_bf16_bits(x)


@pytest.mark.parametrize("n", [2, 3, 4, 5, 8])
@pytest.mark.parametrize("kind", ["octaves", "too_wide", "infinity", "subnormal", "zero_token", "huge"])
def test_float16_route_keeps_every_bit(backend, n, kind):
    """3..8 tokens go through the float16-staged kernel when the activations allow it and through the
    float32-staged one otherwise; both must give the oracle's logits and tokens bit for bit."""
    rows, cols = 1500, 5120
    rng = np.random.default_rng(n * 31 + len(kind))
    w, s = synth.lm_head_weight(rng, rows, cols)
    x = wide_range_activations(rng, n, cols, kind)
    wd, sd, xd = to_dev(w), to_dev(s), to_dev(x)
    want = orc.lm_head_fp8_gemv(w, s, x)
    ws = backend.lm_head_argmax_workspace(rows, n, "cuda")
    try:
        for route in (0, 1):
            backend.lib.qwen36_lm_head_fp8_gemv_set_route(route)
            got = bf16_host(backend.lm_head_fp8_gemv(wd, sd, xd))
            assert np.array_equal(got, want), f"route {route}"
            tok, _ = backend.lm_head_fp8_gemv_argmax(wd, sd, xd, ws)
            assert np.array_equal(tok.cpu().numpy().astype(np.uint32), orc.argmax_rows(want)), f"route {route}"
    finally:
        backend.lib.qwen36_lm_head_fp8_gemv_set_route(0)


def test_lm_head_checksum_full_vocab(backend):
    """Full config-3 size (248320 x 5120, M = 4): fused argmax == unfused device argmax, and a
    sample of 2048 logits is bit-identical to the oracle (the oracle over the whole vocab is
    too slow for a unit test)."""
    gen = torch.Generator(device="cuda").manual_seed(5)
    rows, cols, n = synth.VOCAB, synth.HIDDEN, 4
    w = torch.randint(0, 0x7F, (rows, cols), generator=gen, dtype=torch.uint8, device="cuda")
    w |= (torch.randint(0, 2, (rows, cols), generator=gen, dtype=torch.uint8, device="cuda") << 7)
    s = torch.exp2(torch.rand(rows, generator=gen, device="cuda") * 4 - 6)
    x = torch.randn((n, cols), generator=gen, device="cuda").to(torch.bfloat16)
    logits = backend.lm_head_fp8_gemv(w, s, x)
    ws = backend.lm_head_argmax_workspace(rows, n, "cuda")
    tok, _ = backend.lm_head_fp8_gemv_argmax(w, s, x, ws)
    assert torch.equal(tok, backend.sample_rows(logits))
    idx = torch.randint(0, rows, (2048,), generator=gen, device="cuda")
    want = orc.lm_head_fp8_gemv(w[idx].cpu().numpy(), s[idx].cpu().numpy(), bf16_host(x))
    assert np.array_equal(bf16_host(logits[:, idx]), want)
