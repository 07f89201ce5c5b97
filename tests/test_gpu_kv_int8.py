"""GPU parity of the int8 KV path: codes and scales bit-exact; attention output rel-L2 <= 1e-2
against the oracle (which restates the reference's two-pass float32 softmax)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from speedoza_b200 import synth
from conftest import bf16_host, to_dev

pytestmark = pytest.mark.gpu


def rel_l2(got, want):
    return np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30)


def encode_both(backend, k, v, tokens, kv_heads, head_dim):
    kq = torch.zeros((tokens, kv_heads, head_dim), dtype=torch.int8, device="cuda")
    vq = torch.zeros_like(kq)
    meta = torch.zeros((tokens, kv_heads, 2), dtype=torch.float32, device="cuda")
    backend.turboquant_encode_kv_rows(to_dev(k), to_dev(v), kq, vq, meta, 0)
    kq_o = np.zeros((tokens, kv_heads, head_dim), np.int8); vq_o = np.zeros_like(kq_o)
    meta_o = np.zeros((tokens, kv_heads, 2), np.float32)
    orc.kv_encode(k, v, 0, kq_o, vq_o, meta_o)
    return (kq, vq, meta), (kq_o, vq_o, meta_o)


@pytest.mark.parametrize("tokens,kv_heads,head_dim", [(1, 4, 256), (300, 4, 256), (17, 2, 128), (9, 3, 40)])
def test_encode_bit_exact(backend, tokens, kv_heads, head_dim):
    rng = np.random.default_rng(tokens + head_dim)
    _, k, v = synth.qkv(rng, tokens, 2 * kv_heads, kv_heads, head_dim, outliers=min(4, head_dim))
    k[0, 0] = 0                                             # zero vector: scale 0, codes 0
    # exact .5 ties after scaling: amax 127 -> scale 1
    k[-1, -1] = synth.f32_to_bf16_bits(np.resize(np.array([127, 0.5, 1.5, 2.5, -0.5, -1.5, 126.5, -126.5], np.float32), head_dim))
    (kq, vq, meta), (kq_o, vq_o, meta_o) = encode_both(backend, k, v, tokens, kv_heads, head_dim)
    assert np.array_equal(meta.cpu().numpy().view(np.uint32), meta_o.view(np.uint32))
    assert np.array_equal(kq.cpu().numpy(), kq_o) and np.array_equal(vq.cpu().numpy(), vq_o)


def test_encode_bulk_rows_bit_exact_with_special_vectors(backend):
    """The many-vector route of qwen36_turboquant_encode_kv_rows (head_dim 256, 4096 vectors or more):
    codes and scales equal the oracle's, with vectors planted that leave its fast arithmetic: zero, exact
    ties at scale 1 and at other scales, NaN, infinity, magnitudes near both ends of the bf16 range, and
    a power-of-two ladder whose quotients sit on or next to half-integers."""
    rng = np.random.default_rng(77)
    tokens, kv_heads, head_dim = 1536, 4, 256
    _, k, v = synth.qkv(rng, tokens, 2 * kv_heads, kv_heads, head_dim, outliers=4)
    f2b = lambda a: synth.f32_to_bf16_bits(np.asarray(a, np.float32))
    ties = np.resize(np.array([127, 0.5, 1.5, 2.5, -0.5, -1.5, 126.5, -126.5, 63.5, -63.5, 3.5, 100.5], np.float32), head_dim)
    k[0, 0] = 0
    k[1, 1] = f2b(ties)                                     # scale 1
    v[2, 2] = f2b(ties * 0.25)                              # scale 2^-2: the same ties
    v[3, 0] = f2b(ties * 3.0)                               # scale 3: quotients next to, not on, half-integers
    k[4, 3] = f2b(np.resize(np.array([1e-38, -3e-39, 2e-38, 5e-39], np.float32), head_dim))      # tiny: scale < 2^-60
    v[5, 1] = f2b(np.resize(np.array([3e38, -1e38, 2e37, 1e30], np.float32), head_dim))          # huge: scale > 2^60
    k[8, 0] = f2b(np.resize(127.0 * 2.0 ** -np.arange(0, 20, dtype=np.float32), head_dim))       # 127, 63.5, 31.75, ...
    ladder = (np.arange(head_dim, dtype=np.float32) - 128.0) * 0.5                                # every half-integer in [-64, 63.5]
    ladder[0] = 127.0
    v[9, 2] = f2b(ladder)
    (kq, vq, meta), (kq_o, vq_o, meta_o) = encode_both(backend, k, v, tokens, kv_heads, head_dim)
    assert np.array_equal(meta.cpu().numpy().view(np.uint32), meta_o.view(np.uint32))
    assert np.array_equal(kq.cpu().numpy(), kq_o) and np.array_equal(vq.cpu().numpy(), vq_o)
    # and the few-vector route gives the same bytes (500 tokens per call stay below the switch), also for
    # NaN and infinity, whose conversion to an integer the host leaves undefined (the device gives 0)
    k[6, 2, 7] = f2b([np.nan])[0]
    v[7, 3, 9] = f2b([np.inf])[0]
    v[10, 1, 3] = f2b([-np.inf])[0]
    k[10, 1, 200] = f2b([np.nan])[0]
    backend.turboquant_encode_kv_rows(to_dev(k), to_dev(v), kq, vq, meta, 0)
    kq2 = torch.zeros_like(kq); vq2 = torch.zeros_like(vq); meta2 = torch.zeros_like(meta)
    for t0 in range(0, tokens, 500):
        t1 = min(t0 + 500, tokens)
        backend.turboquant_encode_kv_rows(to_dev(k[t0:t1]), to_dev(v[t0:t1]), kq2, vq2, meta2, t0)
    assert torch.equal(kq, kq2) and torch.equal(vq, vq2) and torch.equal(meta.view(torch.int32), meta2.view(torch.int32))


def test_encode_single_position_entry_appends(backend):
    rng = np.random.default_rng(4)
    _, k, v = synth.qkv(rng, 6, 8, 4, 256)
    kq = torch.zeros((6, 4, 256), dtype=torch.int8, device="cuda"); vq = torch.zeros_like(kq)
    meta = torch.zeros((6, 4, 2), dtype=torch.float32, device="cuda")
    for t in range(6):
        backend.turboquant_encode_kv(to_dev(k[t]), to_dev(v[t]), kq, vq, meta, t, q_heads=8)
    (kq2, vq2, meta2), _ = encode_both(backend, k, v, 6, 4, 256)
    assert torch.equal(kq, kq2) and torch.equal(vq, vq2) and torch.equal(meta, meta2)


@pytest.mark.parametrize("tokens,q_heads,kv_heads,head_dim", [
    (1, 24, 4, 256), (63, 24, 4, 256), (513, 24, 4, 256), (8192, 24, 4, 256),
    (200, 8, 8, 128), (100, 6, 2, 64), (77, 10, 2, 256), (50, 4, 2, 40)])
def test_attention_vs_oracle(backend, tokens, q_heads, kv_heads, head_dim):
    rng = np.random.default_rng(tokens * 3 + q_heads)
    q, k, v = synth.qkv(rng, tokens, q_heads, kv_heads, head_dim, outliers=min(4, head_dim))
    (kq, vq, meta), (kq_o, vq_o, meta_o) = encode_both(backend, k, v, tokens, kv_heads, head_dim)
    ws = backend.attention_workspace(q_heads, head_dim, "cuda")
    out = backend.turboquant_attention(to_dev(q), kq, vq, meta, tokens - 1, ws)
    want = synth.bf16_bits_to_f32(orc.kv_attention(q, kq_o, vq_o, meta_o, tokens - 1))
    err = rel_l2(synth.bf16_bits_to_f32(bf16_host(out)), want)
    assert err <= 1e-2, err


def test_attention_position_inside_longer_cache(backend):
    """position < cache length: rows after `position` must not be read into the result."""
    rng = np.random.default_rng(12)
    q, k, v = synth.qkv(rng, 400)
    (kq, vq, meta), (kq_o, vq_o, meta_o) = encode_both(backend, k, v, 400, 4, 256)
    ws = backend.attention_workspace(24, 256, "cuda")
    out = backend.turboquant_attention(to_dev(q), kq, vq, meta, 249, ws)
    want = synth.bf16_bits_to_f32(orc.kv_attention(q, kq_o, vq_o, meta_o, 249))
    assert rel_l2(synth.bf16_bits_to_f32(bf16_host(out)), want) <= 1e-2


def test_partials_and_merge_equal_whole(backend):
    """KV-range sharding: partials over disjoint ranges (one empty) merged == single call."""
    rng = np.random.default_rng(21)
    T = 3000
    q, k, v = synth.qkv(rng, T)
    (kq, vq, meta), (kq_o, vq_o, meta_o) = encode_both(backend, k, v, T, 4, 256)
    ws = backend.attention_workspace(24, 256, "cuda")
    qd = to_dev(q)
    whole = backend.turboquant_attention(qd, kq, vq, meta, T - 1, ws)
    ranges = [(0, 1000), (1000, 1000), (1000, 2500), (2500, T)]
    pm = torch.empty((24, len(ranges)), dtype=torch.float32, device="cuda")
    pl = torch.empty_like(pm)
    po = torch.empty((24, len(ranges), 256), dtype=torch.float32, device="cuda")
    for i, (a, b) in enumerate(ranges):
        m_, l_, o_ = backend.turboquant_attention_partial(qd, kq, vq, meta, a, b, ws)
        pm[:, i], pl[:, i], po[:, i] = m_, l_, o_
    assert torch.isneginf(pm[:, 1]).all() and (pl[:, 1] == 0).all() and (po[:, 1] == 0).all()
    merged = backend.attention_merge_partials(pm, pl, po)
    a = merged.float().cpu().numpy(); b = whole.float().cpu().numpy()
    assert rel_l2(a, b.astype(np.float64)) <= 2e-3
    # oracle partial contract: same (m, l, o) up to float rounding
    om, ol, oo = orc.kv_attention_partial(q, kq_o, vq_o, meta_o, 1000, 2500)
    assert np.allclose(pm[:, 2].cpu().numpy(), om, rtol=1e-4, atol=1e-4)
    assert np.allclose(pl[:, 2].cpu().numpy(), ol, rtol=2e-3)
    assert rel_l2(po[:, 2].cpu().numpy(), oo.astype(np.float64)) <= 2e-3
    want = synth.bf16_bits_to_f32(orc.merge_partials(pm.cpu().numpy(), pl.cpu().numpy(), po.cpu().numpy()))
    assert rel_l2(a, want.astype(np.float64)) <= 1e-2


def test_attention_missing_workspace_is_an_error(backend):
    from speedoza_b200.abi import KernelError
    rng = np.random.default_rng(2)
    q, k, v = synth.qkv(rng, 8)
    (kq, vq, meta), _ = encode_both(backend, k, v, 8, 4, 256)
    with pytest.raises(KernelError):
        backend.turboquant_attention(to_dev(q), kq, vq, meta, 7, None)


def test_long_context_softmax_property(backend):
    """ctx 131072 (config-4 maximum): with V rows all equal to one vector the output must be that
    vector (softmax weights sum to 1) whatever the scores are."""
    T = 131072
    gen = torch.Generator(device="cuda").manual_seed(8)
    k = torch.randn((T, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
    vrow = torch.randn((1, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
    v = vrow.expand(T, 4, 256).contiguous()
    q = torch.randn((24, 256), generator=gen, device="cuda").to(torch.bfloat16)
    kq = torch.empty((T, 4, 256), dtype=torch.int8, device="cuda"); vq = torch.empty_like(kq)
    meta = torch.empty((T, 4, 2), dtype=torch.float32, device="cuda")
    backend.turboquant_encode_kv_rows(k, v, kq, vq, meta, 0)
    ws = backend.attention_workspace(24, 256, "cuda")
    out = backend.turboquant_attention(q, kq, vq, meta, T - 1, ws).float()
    vd = (vq[0].float() * meta[0, :, 1:2]).repeat_interleave(6, dim=0)
    assert torch.allclose(out, vd, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("tokens", [1, 7, 16, 17, 300, 1500, 5000])
def test_all_attention_kernels_agree(backend, tokens):
    """head_dim 256 has a tensor-core form fed through shared memory (mode 3, the default) or from
    registers (2), a 4-token SIMT path (1) and the general kernel (0): each must match the oracle, for
    contexts that end inside a 16-token group."""
    rng = np.random.default_rng(33 + tokens)
    q, k, v = synth.qkv(rng, tokens)
    (kq, vq, meta), (kq_o, vq_o, meta_o) = encode_both(backend, k, v, tokens, 4, 256)
    ws = backend.attention_workspace(24, 256, "cuda")
    qd = to_dev(q)
    want = synth.bf16_bits_to_f32(orc.kv_attention(q, kq_o, vq_o, meta_o, tokens - 1))
    try:
        for mode in (3, 2, 1, 0):
            backend.lib.qwen36_turboquant_attention_set_fast(mode)
            got = backend.turboquant_attention(qd, kq, vq, meta, tokens - 1, ws).clone()
            err = rel_l2(synth.bf16_bits_to_f32(bf16_host(got)), want)
            assert err <= (3e-3 if mode >= 2 else 1e-2), (mode, err)
    finally:
        backend.lib.qwen36_turboquant_attention_set_fast(3)
