"""Exact-argmax guards through the C ABI: top-2 margin, top-8 float64 rescore, predicated bf16
lm_head + argmax.  Tokens and flags are integers: compared exactly with the oracle, and (when the
reference's own CUDA library was built) exactly with the reference kernels on the same inputs."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from speedoza_b200 import abi, synth
from conftest import to_dev
from test_oracle_golden import planted_logits

pytestmark = pytest.mark.gpu

REF_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                      "libqwen36_ref.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_SO):
        return None
    torch.zeros(1, device="cuda")
    return C.CDLL(REF_SO, mode=os.RTLD_LOCAL | os.RTLD_DEEPBIND)


def dp(t):
    return abi.DevicePtr(0 if t is None else t.data_ptr())


def u32(t):
    return t.cpu().numpy().view(np.uint32)


def test_top2_margin_known_answers_and_counters(backend):
    # kernels-cuda/smoke.cu:202-262
    logits = to_dev(planted_logits())
    fb = torch.zeros(1, dtype=torch.int32, device="cuda")
    mirror = torch.zeros(1, dtype=torch.int32, device="cuda")
    tokens, flags = backend.lm_head_top2_margin(logits, 1.0, fb, mirror)
    assert u32(tokens).tolist() == [123456, 99] and u32(flags).tolist() == [1, 0]
    assert mirror.item() == 99 and fb.item() == 1
    tokens, flags = backend.lm_head_top2_margin(logits, 0.1, fb, mirror)
    assert u32(flags).tolist() == [1, 1] and fb.item() == 1            # the counter only ever grows
    assert backend.lib.qwen36_lm_head_top2_margin(None) == abi.INVALID_ARGUMENT   # as the reference: not NULL_POINTER


@pytest.mark.parametrize("rows,vocab", [(4, 248320), (1, 1000), (3, 61441), (2, 7)])
def test_top2_margin_vs_oracle(backend, rows, vocab):
    rng = np.random.default_rng(rows * 7 + vocab)
    logits = synth.f32_to_bf16_bits((rng.standard_normal((rows, vocab)) * 3).astype(np.float32))
    if vocab > 10:
        logits[rows - 1, 5] = synth.f32_to_bf16_bits(np.array([40.0], np.float32))[0]      # a tie for first place
        logits[rows - 1, vocab - 3] = logits[rows - 1, 5]
    for eps in (0.0, 0.25, 2.0):
        want_t, want_f, _ = orc.lm_head_top2_margin(logits, eps)
        tokens, flags = backend.lm_head_top2_margin(to_dev(logits), eps)
        assert np.array_equal(u32(tokens), want_t) and np.array_equal(u32(flags), want_f)


def make_head(rng, vocab, cols, rows, noise):
    w = synth.f32_to_bf16_bits(rng.standard_normal((vocab, cols)).astype(np.float32))
    x = synth.f32_to_bf16_bits(rng.standard_normal((rows, cols)).astype(np.float32))
    exact = synth.bf16_bits_to_f32(x) @ synth.bf16_bits_to_f32(w).T
    logits = synth.f32_to_bf16_bits((exact + rng.standard_normal(exact.shape).astype(np.float32) * noise))
    return w, x, logits


@pytest.mark.parametrize("rows,vocab,cols", [(3, 20000, 512), (2, 300, 96), (1, 70000, 1024)])
def test_top8_rescore_vs_oracle(backend, rows, vocab, cols):
    rng = np.random.default_rng(vocab + cols)
    w, x, logits = make_head(rng, vocab, cols, rows, 0.3)
    for eps in (0.0, 0.5, 50.0):
        want_t, want_f, want_fb = orc.lm_head_top8_rescore(logits, w, x, eps)
        fb = torch.zeros(1, dtype=torch.int32, device="cuda")
        tokens, flags = backend.lm_head_top8_rescore(to_dev(logits), to_dev(w), to_dev(x), eps, fb)
        assert np.array_equal(u32(tokens), want_t) and np.array_equal(u32(flags), want_f) and fb.item() == want_fb


def test_top8_rescore_special_logits_vs_oracle(backend):
    """Block winners that are NaN, infinite or tied: NaN and -inf are never candidates, +inf is, equal
    values go to the smaller token; rows with fewer than eight (or no) candidates."""
    rows, vocab, cols = 5, 70000, 512
    rng = np.random.default_rng(99)
    w, x, logits = make_head(rng, vocab, cols, rows, 0.3)
    bits = lambda v: synth.f32_to_bf16_bits(np.array([v], np.float32))[0]
    logits[0, rng.integers(0, vocab, 4000)] = bits(np.nan)
    logits[0, rng.integers(0, vocab, 4000)] = bits(-np.inf)
    logits[1, [7, 40000, 69999]] = bits(np.inf)                       # three ties at the top
    logits[2, :] = bits(-np.inf)                                      # no candidate at all
    logits[2, [123, 50000]] = bits(3.0)                               # ... but two
    logits[3, :] = bits(1.5)                                          # every block winner tied
    logits[4, :] = bits(np.nan)                                       # nothing comparable
    for eps in (0.0, 0.5):
        want_t, want_f, want_fb = orc.lm_head_top8_rescore(logits, w, x, eps)
        fb = torch.zeros(1, dtype=torch.int32, device="cuda")
        tokens, flags = backend.lm_head_top8_rescore(to_dev(logits), to_dev(w), to_dev(x), eps, fb)
        assert np.array_equal(u32(tokens), want_t) and np.array_equal(u32(flags), want_f) and fb.item() == want_fb


@pytest.mark.parametrize("rows,vocab,cols", [(1, 5000, 5120), (4, 3000, 512), (11, 1000, 96), (3, 257, 33)])
def test_bf16_matvec_argmax_rows_vs_oracle(backend, rows, vocab, cols):
    rng = np.random.default_rng(rows + vocab + cols)
    w, x, _ = make_head(rng, vocab, cols, rows, 0.0)
    want = orc.bf16_matvec_argmax_rows(x, w)
    got = backend.bf16_matvec_argmax_rows(to_dev(x), to_dev(w))
    assert np.array_equal(u32(got), want)
    # predicated: flagged rows keep the token they came with, mirror follows the last row only if it ran
    skip = (np.arange(rows) % 2).astype(np.uint32)
    start = np.arange(100, 100 + rows, dtype=np.uint32)
    want = orc.bf16_matvec_argmax_rows(x, w, skip, start)
    tokens = to_dev(start.view(np.int32).copy())
    mirror = torch.full((1,), -5, dtype=torch.int32, device="cuda")
    backend.bf16_matvec_argmax_rows(to_dev(x), to_dev(w), tokens, to_dev(skip.view(np.int32).copy()), mirror)
    assert np.array_equal(u32(tokens), want)
    assert mirror.item() == (-5 if skip[rows - 1] else int(want[rows - 1]))


def test_two_stage_pipeline_equals_full_bf16_argmax(backend):
    """Stage 1 (guard over FP8-like logits) + stage 2 (predicated bf16 rescore of the failed rows)
    gives the bf16 argmax for every row."""
    rng = np.random.default_rng(5)
    rows, vocab, cols = 6, 30000, 256
    w, x, logits = make_head(rng, vocab, cols, rows, 0.05)
    full = orc.bf16_matvec_argmax_rows(x, w)
    wd, xd = to_dev(w), to_dev(x)
    tokens, flags = backend.lm_head_top8_rescore(to_dev(logits), wd, xd, 0.3)
    backend.bf16_matvec_argmax_rows(xd, wd, tokens, flags)
    assert np.array_equal(u32(tokens), full)


def test_guards_equal_reference_cuda(backend, ref):
    if ref is None:
        pytest.skip("oracle/_ref/libqwen36_ref.so not built")
    rng = np.random.default_rng(77)
    rows, vocab, cols = 3, 50000, 256
    w, x, logits = make_head(rng, vocab, cols, rows, 0.3)
    ld, wd, xd = to_dev(logits), to_dev(w), to_dev(x)
    outs = []
    for lib in (ref, backend.lib):
        res = []
        ws = torch.zeros(rows * 240 * 16, dtype=torch.uint8, device="cuda")
        for eps in (0.0, 0.5):
            tokens = torch.zeros(rows, dtype=torch.int32, device="cuda")
            flags = torch.zeros(rows, dtype=torch.int32, device="cuda")
            s2 = abi.LmHeadTop2MarginSpec(rows, vocab, eps, dp(ld), dp(tokens), dp(flags), dp(None), dp(None), dp(ws), ws.numel())
            assert lib.qwen36_lm_head_top2_margin(C.byref(s2)) == 0
            torch.cuda.synchronize()
            res += [u32(tokens).copy(), u32(flags).copy()]
            s8 = abi.LmHeadTop8RescoreSpec(rows, vocab, cols, eps, dp(ld), dp(wd), dp(xd), dp(tokens), dp(flags), dp(None),
                                           dp(None), dp(ws), ws.numel())
            assert lib.qwen36_lm_head_top8_rescore(C.byref(s8)) == 0
            torch.cuda.synchronize()
            res += [u32(tokens).copy(), u32(flags).copy()]
        tokens = torch.zeros(rows, dtype=torch.int32, device="cuda")
        ws8 = torch.zeros(rows * 8, dtype=torch.uint8, device="cuda")
        sb = abi.Bf16MatvecArgmaxRowsSpec(rows, vocab, cols, dp(xd), dp(wd), dp(tokens), dp(None), dp(ws8), ws8.numel(), dp(None))
        assert lib.qwen36_bf16_matvec_argmax_rows(C.byref(sb)) == 0
        torch.cuda.synchronize()
        res.append(u32(tokens).copy())
        outs.append(res)
    for a, b in zip(*outs):
        assert np.array_equal(a, b)
