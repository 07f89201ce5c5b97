"""GPU parity of the split-KV tensor-core attention behind qwen36_attention_flash_splitk_prefill_bf16
(speculative verify: a short query chunk over a long BF16 / FP8 cache) and
qwen36_attention_decode_split_tiled (one decode token, fixed-size splits, partials + cache append).
Outputs rel-L2 <= 1e-2 against the oracle (the test generator follows kernels-cuda/smoke.cu:3614-3773:
same shapes and split counts, seeded normal data); the partial contract (layout, empty splits, split
boundaries) is checked through the library's own merge."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from speedoza_b200 import abi, synth
from conftest import bf16_host, to_dev
from test_gpu_kv_decode import cache_host, cache_to_dev, e4m3_encode_bits, partial_buffers

pytestmark = pytest.mark.gpu
BF16, FP8 = 0, 1


def rel_l2(got, want):
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    return np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)


def dp(t):
    return abi.DevicePtr(0 if t is None else t.data_ptr())


def make_verify_case(seed, start, tokens, q_heads, kv_heads, dtype):
    rng = np.random.default_rng(seed)
    rows = start + tokens
    q = synth.f32_to_bf16_bits(rng.standard_normal((tokens, q_heads, 256), dtype=np.float32))
    k = synth.f32_to_bf16_bits(rng.standard_normal((rows, kv_heads, 256), dtype=np.float32))
    v = synth.f32_to_bf16_bits(rng.standard_normal((rows, kv_heads, 256), dtype=np.float32))
    if dtype == FP8:
        k, v = e4m3_encode_bits(k), e4m3_encode_bits(v)
    return q, np.ascontiguousarray(k), np.ascontiguousarray(v)


def run_verify(backend, q, ck, cv, dtype, start, n_splits, own_partials=True, start_device=False):
    tokens, q_heads, _ = q.shape
    kv_heads = ck.shape[1]
    qd, ckd, cvd = to_dev(q), cache_to_dev(ck), cache_to_dev(cv)
    out = torch.full((tokens, q_heads, 256), float("nan"), dtype=torch.bfloat16, device="cuda")
    pa = torch.full((tokens, q_heads, n_splits, 256), float("nan"), device="cuda") if own_partials else None
    pm = torch.full((tokens, q_heads, n_splits), float("nan"), device="cuda") if own_partials else None
    pl = torch.full((tokens, q_heads, n_splits), float("nan"), device="cuda") if own_partials else None
    pos = torch.tensor([start], dtype=torch.int32, device="cuda") if start_device else None
    spec = abi.AttentionPrefillSpec(0, 0xdead if start_device else start, tokens, dp(qd), dp(None), dp(None), dp(ckd),
                                    dp(cvd), dp(None), dp(out), abi.AttentionShape(q_heads, kv_heads, 256, 0), dtype,
                                    dp(pos), dp(pa), dp(pm), dp(pl), 0, 0, dp(None), 0)
    assert backend.lib.qwen36_attention_flash_splitk_prefill_bf16(C.byref(spec), n_splits) == abi.SUCCESS
    torch.cuda.synchronize()
    return out, pa, pm, pl


@pytest.mark.parametrize("dtype", [BF16, FP8])
@pytest.mark.parametrize("start,tokens,n_splits", [
    (0, 1, 1), (0, 16, 1), (0, 32, 3), (5, 4, 2), (63, 2, 1), (64, 16, 4), (100, 5, 1), (100, 5, 7),
    (1000, 16, 16), (1000, 32, 5), (4093, 9, 48), (8192, 16, 48), (300, 11, 64)])
def test_verify_vs_oracle(backend, dtype, start, tokens, n_splits):
    """Chunk sizes and split counts of the reference's kernel-vs-kernel gate (1..32 rows, 1..48 splits,
    more splits than K iterations included: the surplus splits must publish (-inf, 0, 0))."""
    q, ck, cv = make_verify_case(start * 7 + tokens + dtype, start, tokens, 24, 4, dtype)
    out, pa, pm, pl = run_verify(backend, q, ck, cv, dtype, start, n_splits)
    want = orc.attention_verify(q, ck, cv, dtype, start)
    got = synth.bf16_bits_to_f32(bf16_host(out))
    assert rel_l2(got, want) <= 1e-2
    # cosine per (token, head) row, the reference's own gate (>= 0.998)
    g, w = got.reshape(-1, 256).astype(np.float64), want.reshape(-1, 256)
    cos = (g * w).sum(1) / (np.linalg.norm(g, axis=1) * np.linalg.norm(w, axis=1))
    assert cos.min() >= 0.998
    # partial contract: every (token, head, split) was written; splits past the last K iteration are empty
    iters = (start + tokens + 63) // 64
    per = (iters + n_splits - 1) // n_splits
    used = (iters + per - 1) // per
    pmh, plh = pm.cpu().numpy(), pl.cpu().numpy()
    assert not np.isnan(pmh).any() and not np.isnan(plh).any() and not torch.isnan(pa).any()
    assert np.isneginf(pmh[:, :, used:]).all() and (plh[:, :, used:] == 0).all()
    # and the library's merge of those partials reproduces the output
    for tok in (0, tokens - 1):
        merged = backend.attention_merge_partials(pm[tok].contiguous(), pl[tok].contiguous(), pa[tok].contiguous())
        assert rel_l2(merged.float().cpu().numpy(), got[tok]) <= 2e-3


@pytest.mark.parametrize("dtype", [BF16, FP8])
def test_verify_other_head_groupings_and_device_position(backend, dtype):
    """8 q heads on 8 kv heads (no sharing), 16 on 2 (eight per kv head: two 64-row chunks per kv head
    at 16 tokens), the start position read from device memory, and the library-owned scratch when the
    spec carries no partial buffers."""
    for q_heads, kv_heads, tokens, start in ((8, 8, 7, 130), (16, 2, 16, 700), (24, 4, 32, 513)):
        q, ck, cv = make_verify_case(q_heads + tokens + dtype, start, tokens, q_heads, kv_heads, dtype)
        want = orc.attention_verify(q, ck, cv, dtype, start)
        for own, dev in ((True, True), (False, False)):
            out, *_ = run_verify(backend, q, ck, cv, dtype, start, 6, own_partials=own, start_device=dev)
            assert rel_l2(synth.bf16_bits_to_f32(bf16_host(out)), want) <= 1e-2


def test_verify_fp8_cache_with_every_byte_value(backend):
    """0x7F / 0xFF read as +-448, 0x80 as zero, subnormal codes: q kept small so the softmax stays spread."""
    rng = np.random.default_rng(3)
    start, tokens = 600, 8
    q = synth.f32_to_bf16_bits(rng.standard_normal((tokens, 24, 256), dtype=np.float32) * 2.0 ** -10)
    ck = rng.integers(0, 256, size=(start + tokens, 4, 256), dtype=np.uint8)
    cv = rng.integers(0, 256, size=(start + tokens, 4, 256), dtype=np.uint8)
    out, *_ = run_verify(backend, q, ck, cv, FP8, start, 5)
    assert rel_l2(synth.bf16_bits_to_f32(bf16_host(out)), orc.attention_verify(q, ck, cv, FP8, start)) <= 1e-2


def test_verify_argument_checks(backend):
    """Status codes of kernels-cuda/attention_flash_splitk.cu:509-520."""
    lib = backend.lib
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = dp(buf)
    def spec(tokens=4, head_dim=256, q_heads=24, kv_heads=4, dtype=0, q=p):
        return abi.AttentionPrefillSpec(0, 0, tokens, q, dp(None), dp(None), p, p, dp(None), p,
                                        abi.AttentionShape(q_heads, kv_heads, head_dim, 0), dtype, dp(None), p, p, p,
                                        0, 0, dp(None), 0)
    assert lib.qwen36_attention_flash_splitk_prefill_bf16(None, 2) == abi.NULL_POINTER
    for bad in (spec(tokens=0), spec(tokens=33), spec(head_dim=128), spec(q_heads=25), spec(dtype=2), spec(q=dp(None))):
        assert lib.qwen36_attention_flash_splitk_prefill_bf16(C.byref(bad), 2) == abi.INVALID_ARGUMENT
    assert lib.qwen36_attention_flash_splitk_prefill_bf16(C.byref(spec()), 0) == abi.INVALID_ARGUMENT


@pytest.mark.parametrize("dtype", [BF16, FP8])
@pytest.mark.parametrize("position,q_heads,kv_heads,block", [(0, 24, 4, 64), (63, 24, 4, 64), (64, 24, 4, 64),
                                                             (513, 24, 4, 64), (3000, 24, 4, 128), (777, 16, 2, 8),
                                                             (2500, 8, 4, 256)])
def test_decode_split_tiled_partials_and_append(backend, dtype, position, q_heads, kv_heads, block):
    """The tiled split entry writes partials for fixed-size splits (more splits than needed: the rest are
    empty) and appends the new row; merged, the partials give the oracle's decode output, and the cache
    afterwards equals the oracle's cache byte for byte."""
    from test_gpu_kv_decode import make_case
    q, k_new, v_new, ck, cv = make_case(position * 3 + q_heads + dtype, position + 1, q_heads, kv_heads, 256, dtype)
    ck_o, cv_o = ck.copy(), cv.copy()
    want = synth.bf16_bits_to_f32(orc.attention_decode(q, k_new, v_new, ck_o, cv_o, dtype, position))
    n_splits = position // block + 3
    ckd, cvd = cache_to_dev(ck), cache_to_dev(cv)
    pa, pm, pl = partial_buffers(q_heads, n_splits, 256)
    out = torch.empty((q_heads, 256), dtype=torch.bfloat16, device="cuda")
    qd, kd, vd = to_dev(q), to_dev(k_new), to_dev(v_new)
    spec = abi.AttentionDecodeSpec(0, position, dp(qd), dp(kd), dp(vd), dp(ckd), dp(cvd), dp(None), dp(out),
                                   abi.AttentionShape(q_heads, kv_heads, 256, 0), dtype, dp(None), dp(pa), dp(pm), dp(pl),
                                   n_splits, block)
    assert backend.lib.qwen36_attention_decode_split_tiled(C.byref(spec), n_splits, block) == abi.SUCCESS
    torch.cuda.synchronize()
    used = position // block + 1
    assert torch.isneginf(pm[:, used:]).all() and (pl[:, used:] == 0).all() and (pa[:, used:] == 0).all()
    merged = backend.attention_merge_partials(pm, pl, pa)
    assert rel_l2(merged.float().cpu().numpy(), want) <= 1e-2
    assert np.array_equal(cache_host(ckd), ck_o) and np.array_equal(cache_host(cvd), cv_o)
    # shapes outside the entry's range decline softly, as the reference's do
    bad = abi.AttentionDecodeSpec(0, position, dp(qd), dp(kd), dp(vd), dp(ckd), dp(cvd), dp(None), dp(out),
                                  abi.AttentionShape(q_heads, kv_heads, 128, 0), dtype, dp(None), dp(pa), dp(pm), dp(pl),
                                  n_splits, block)
    assert backend.lib.qwen36_attention_decode_split_tiled(C.byref(bad), n_splits, block) == abi.NOT_IMPLEMENTED
    assert backend.lib.qwen36_attention_decode_split_tiled(C.byref(spec), n_splits, 12) == abi.NOT_IMPLEMENTED
