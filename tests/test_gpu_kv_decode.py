"""GPU parity of qwen36_attention_decode (BF16 / FP8 E4M3 KV cache): output rel-L2 <= 1e-2
against the oracle's restatement of the reference's float32 online softmax, cache append
byte-exact (the appended row and nothing else changes)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from speedoza_b200 import synth
from conftest import bf16_host, to_dev

pytestmark = pytest.mark.gpu

BF16, FP8 = 0, 1
DEFAULT_MODE = 1          # qwen36_attention_decode_set_mode: 1 = tensor-core kernels where they apply (the library's default)


def rel_l2(got, want):
    return np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30)


E4M3_ENCODE = None


def e4m3_encode_bits(bits):
    """bf16 bit patterns -> E4M3 bytes with the oracle's encoder (table over all 65536 patterns)."""
    global E4M3_ENCODE
    if E4M3_ENCODE is None:
        vals = synth.bf16_bits_to_f32(np.arange(65536, dtype=np.uint16))
        E4M3_ENCODE = np.array([orc.kv_e4m3_encode(float(v)) for v in vals], np.uint8)
    return E4M3_ENCODE[bits]


def make_case(seed, rows, q_heads, kv_heads, head_dim, dtype, q_gain=1.0):
    """q, new k / v row, and a cache of `rows` rows (the last one is scratch for the append)."""
    rng = np.random.default_rng(seed)
    q, k, v = synth.qkv(rng, rows + 1, q_heads, kv_heads, head_dim, outliers=min(4, head_dim))
    if q_gain != 1.0:
        q = synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(q) * q_gain)
    k_new, v_new = k[rows].copy(), v[rows].copy()
    if dtype == FP8:
        ck, cv = e4m3_encode_bits(k[:rows]), e4m3_encode_bits(v[:rows])
    else:
        ck, cv = k[:rows].copy(), v[:rows].copy()
    return q, k_new, v_new, np.ascontiguousarray(ck), np.ascontiguousarray(cv)


def cache_to_dev(c):
    return to_dev(c) if c.dtype == np.uint16 else torch.from_numpy(c).cuda()


def cache_host(t):
    return bf16_host(t) if t.dtype == torch.bfloat16 else t.cpu().numpy()


def partial_buffers(q_heads, n, head_dim):
    return (torch.full((q_heads, n, head_dim), float("nan"), device="cuda"),
            torch.full((q_heads, n), float("nan"), device="cuda"),
            torch.full((q_heads, n), float("nan"), device="cuda"))


def run_and_check(backend, case, dtype, position, n_splits=0, position_device=False, tol=1e-2):
    q, k_new, v_new, ck, cv = case
    q_heads, head_dim = q.shape
    ck_d, cv_d = cache_to_dev(ck), cache_to_dev(cv)
    parts = partial_buffers(q_heads, n_splits, head_dim) if n_splits >= 2 else None
    pos_d = torch.tensor([position], dtype=torch.int32, device="cuda") if position_device else None
    out = backend.attention_decode(to_dev(q), to_dev(k_new), to_dev(v_new), ck_d, cv_d,
                                   0xdead if position_device else position, dtype, parts, n_splits, pos_d)
    torch.cuda.synchronize()
    ck_o, cv_o = ck.copy(), cv.copy()
    want = synth.bf16_bits_to_f32(orc.attention_decode(q, k_new, v_new, ck_o, cv_o, dtype, position))
    err = rel_l2(synth.bf16_bits_to_f32(bf16_host(out)), want)
    assert err <= tol, err
    assert np.array_equal(cache_host(ck_d), ck_o) and np.array_equal(cache_host(cv_d), cv_o)
    return err


def test_reference_known_answers(backend):
    """kernels-cuda/smoke.cu:508-532 (position 0 -> v_new, cache row 0 written), 619-650 (513 cached
    rows of K = 0.5, V = 1.0 through the split path with 2 splits -> 1.0 +- 0.02)."""
    def full(shape, val):
        return to_dev(synth.f32_to_bf16_bits(np.full(shape, val, np.float32)))
    q, k, v = full((2, 8), 0.25), full((1, 8), 0.5), full((1, 8), 1.0)
    ck, cv = full((1, 1, 8), 0.0), full((1, 1, 8), 0.0)
    out = backend.attention_decode(q, k, v, ck, cv, 0, BF16)
    assert torch.all(out.float() == 1.0) and torch.equal(ck[0], k) and torch.equal(cv[0], v)
    ck, cv = full((514, 1, 8), 0.5), full((514, 1, 8), 1.0)
    out = backend.attention_decode(q, k, v, ck, cv, 513, BF16, partial_buffers(2, 2, 8), 2)
    assert torch.all((out.float() - 1.0).abs() <= 0.02)


@pytest.mark.parametrize("dtype", [BF16, FP8])
@pytest.mark.parametrize("position,q_heads,kv_heads,head_dim,n_splits", [
    (0, 24, 4, 256, 0), (0, 24, 4, 256, 16), (1, 24, 4, 256, 16), (63, 24, 4, 256, 0), (513, 24, 4, 256, 2),
    (3000, 24, 4, 256, 64), (8192, 24, 4, 256, 256), (200, 8, 8, 128, 8), (100, 6, 2, 64, 0),
    (777, 10, 2, 256, 5), (50, 4, 2, 40, 3), (1500, 16, 2, 256, 300), (900, 8, 8, 256, 40), (640, 8, 4, 256, 4)])
def test_decode_vs_oracle(backend, dtype, position, q_heads, kv_heads, head_dim, n_splits):
    case = make_case(position * 7 + q_heads + dtype, position + 1, q_heads, kv_heads, head_dim, dtype)
    run_and_check(backend, case, dtype, position, n_splits)


@pytest.mark.parametrize("dtype", [BF16, FP8])
def test_device_position_and_rows_past_it(backend, dtype):
    """The position comes from device memory (the scalar is ignored); rows after it are neither read
    nor written."""
    case = make_case(31 + dtype, 2000, 24, 4, 256, dtype)
    run_and_check(backend, case, dtype, 1234, 32, position_device=True)
    run_and_check(backend, case, dtype, 5, 32, position_device=True)
    run_and_check(backend, case, dtype, 77, 0, position_device=True)


@pytest.mark.parametrize("dtype", [BF16, FP8])
def test_general_kernel_and_forced_splits(backend, dtype):
    """Every kernel form and odd split counts give the same answer within tolerance."""
    case = make_case(57 + dtype, 2301, 24, 4, 256, dtype)
    try:
        for mode in (0, 1):
            backend.lib.qwen36_attention_decode_set_mode(mode)
            for forced in (1, 3, 37):
                backend.lib.qwen36_attention_decode_force_splits(forced)
                run_and_check(backend, case, dtype, 2300, 64)
    finally:
        backend.lib.qwen36_attention_decode_set_mode(DEFAULT_MODE)
        backend.lib.qwen36_attention_decode_force_splits(0)


def test_fp8_cache_with_every_byte_value(backend):
    """A cache holding all 256 byte values, 0x7F / 0xFF (read as +-448) and 0x80 included; q is kept
    small so that the softmax stays spread over many rows."""
    rng = np.random.default_rng(91)
    q, k_new, v_new, _, _ = make_case(92, 1, 24, 4, 256, FP8, q_gain=2.0 ** -10)
    ck = rng.integers(0, 256, size=(1025, 4, 256), dtype=np.uint8)
    cv = rng.integers(0, 256, size=(1025, 4, 256), dtype=np.uint8)
    for mode in (0, 1):
        backend.lib.qwen36_attention_decode_set_mode(mode)
        try:
            run_and_check(backend, (q, k_new, v_new, ck, cv), FP8, 1024, 8)
        finally:
            backend.lib.qwen36_attention_decode_set_mode(DEFAULT_MODE)


@pytest.mark.parametrize("dtype", [BF16, FP8])
def test_append_values_bit_exact_on_adversarial_row(backend, dtype):
    """The appended row alone (NaN / inf in it would poison the output on both sides alike): ties of
    the E4M3 grid (which round up), saturation, zeros of both signs, subnormals, non-finite values."""
    q, k_new, v_new, ck, cv = make_case(5 + dtype, 301, 24, 4, 256, dtype)
    specials = np.array([0.0, -0.0, 448.0, 464.0, -1e9, 2.0 ** -10, 1.5 * 2.0 ** -9, 2.5 * 2.0 ** -9, 7.5 * 2.0 ** -9,
                         1.0625, 1.1875, -1.0625, 17.0, 19.0, 2.0 ** -12, 3e-5, 440.0, 447.0, np.inf, -np.inf],
                        np.float32)
    k_new[0, :specials.size] = synth.f32_to_bf16_bits(specials)
    v_new[3, 100:100 + specials.size] = synth.f32_to_bf16_bits(-specials)
    k_new[1, :4] = np.array([0x7FC0, 0xFFC0, 0x0001, 0x8001], np.uint16)            # NaNs, bf16 subnormals
    ck_d, cv_d = cache_to_dev(ck), cache_to_dev(cv)
    for n_splits in (8, 0):
        parts = partial_buffers(24, n_splits, 256) if n_splits else None
        ck_d[300].zero_(); cv_d[300].zero_()
        backend.attention_decode(to_dev(q), to_dev(k_new), to_dev(v_new), ck_d, cv_d, 300, dtype, parts, n_splits)
        want_k = e4m3_encode_bits(k_new) if dtype == FP8 else k_new
        want_v = e4m3_encode_bits(v_new) if dtype == FP8 else v_new
        assert np.array_equal(cache_host(ck_d)[300], want_k) and np.array_equal(cache_host(cv_d)[300], want_v)
        assert np.array_equal(cache_host(ck_d)[:300], ck[:300]) and np.array_equal(cache_host(cv_d)[:300], cv[:300])


@pytest.mark.parametrize("dtype", [BF16, FP8])
def test_chained_steps_grow_the_cache(backend, dtype):
    """Four decode steps in a row, the position advancing on the device (qwen36_increment_i32):
    every step sees the rows the earlier steps appended."""
    rng = np.random.default_rng(77 + dtype)
    q_heads, kv_heads, head_dim, start, steps = 24, 4, 256, 600, 4
    _, _, _, ck, cv = make_case(78 + dtype, start + steps, q_heads, kv_heads, head_dim, dtype)
    ck_d, cv_d = cache_to_dev(ck), cache_to_dev(cv)
    pos_d = torch.tensor([start], dtype=torch.int32, device="cuda")
    parts = partial_buffers(q_heads, 16, head_dim)
    from speedoza_b200 import abi
    for step in range(steps):
        q, k, v = synth.qkv(rng, 1, q_heads, kv_heads, head_dim)
        out = backend.attention_decode(to_dev(q), to_dev(k[0]), to_dev(v[0]), ck_d, cv_d, 0, dtype, parts, 16, pos_d)
        assert backend.lib.qwen36_increment_i32(abi.DevicePtr(pos_d.data_ptr())) == 0
        want = synth.bf16_bits_to_f32(orc.attention_decode(q, k[0], v[0], ck, cv, dtype, start + step))
        assert rel_l2(synth.bf16_bits_to_f32(bf16_host(out)), want) <= 1e-2
    assert pos_d.item() == start + steps
    assert np.array_equal(cache_host(ck_d), ck) and np.array_equal(cache_host(cv_d), cv)


def test_argument_checks(backend):
    """Status codes of kernels-cuda/attention.cu:2716-2754; TurboQuant3 caches are not built."""
    from speedoza_b200.abi import KernelError
    q = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    k = torch.zeros((2, 64), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((4, 2, 64), dtype=torch.bfloat16, device="cuda")
    assert backend.lib.qwen36_attention_decode(None) == 1
    with pytest.raises(KernelError):
        backend.attention_decode(q, k, k, None, c, 0, BF16)
    with pytest.raises(KernelError):
        backend.attention_decode(q, k, k, c, c, 0, 7)
    with pytest.raises(KernelError):
        backend.attention_decode(q, torch.zeros((3, 64), dtype=torch.bfloat16, device="cuda"), k, c, c, 0, BF16)
    with pytest.raises(KernelError):
        backend.attention_decode(q, k, k, c, c, 0, BF16, partial_buffers(4, 4, 64), 4, split_timesteps_per_block=32)
    with pytest.raises(KernelError) as e:
        backend.attention_decode(q, k, k, c, c, 0, 2)                   # TurboQuant3 without its metadata
    assert e.value.code == 2
