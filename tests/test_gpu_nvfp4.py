"""GPU parity of the NVFP4 kernels against the CPU oracle, through the C ABI.

Bit-exact: quantised codes, packing, scale bytes, retiled scales, dequantised
weights.  Floating-point outputs: rel-L2 against the oracle with the tolerance
stated in each test (1e-3 for the W4A16 GEMV, 1e-2 for the W4A4 product)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from speedoza_b200 import abi, synth
from conftest import bf16_host, to_dev

pytestmark = pytest.mark.gpu


def rel_l2(got, want):
    got = got.astype(np.float64); want = want.astype(np.float64)
    return np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)


def make_weight(rng, n, k):
    packed, sf_rm = synth.nvfp4_weight(rng, n, k)
    return packed, sf_rm, orc.retile_scales(sf_rm)


# ---------------------------------------------------------------- retile / quantise

@pytest.mark.parametrize("rows,groups", [(1, 1), (5, 3), (128, 4), (130, 12), (257, 7), (5120, 320)])
def test_retile_scales_bit_exact(backend, rows, groups):
    rng = np.random.default_rng(rows * 1000 + groups)
    sf = rng.integers(0, 256, size=(rows, groups), dtype=np.uint8)
    got = backend.nvfp4_retile_scales(to_dev(sf)).cpu().numpy()
    assert np.array_equal(got, orc.retile_scales(sf))


def adversarial_activations(rng, rows, k):
    x = rng.standard_normal((rows, k)).astype(np.float32)
    x[:, ::37] *= 20.0                       # outlier channels
    if rows > 1:
        ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], dtype=np.float32)
        x[1, :16] = np.concatenate([ties, -ties])          # amax 6 -> scale 1 -> exact ties
    if rows > 2:
        x[2] = 0.0
        x[2, 5] = 1e-3                        # scale code underflows to 0
        x[2, 17] = -1e-30
    if rows > 3:
        x[3] *= 1e-4
    if rows > 4:
        x[4] *= 3000.0                        # scales near the UE4M3 clamp
    return synth.f32_to_bf16_bits(x)


@pytest.mark.parametrize("general", [0, 1])
@pytest.mark.parametrize("rows,k,its", [(1, 128, 0.0), (5, 5120, 0.0), (7, 40, 1.25), (130, 192, 0.5),
                                        (3, 33, 1.25), (64, 17408, 1.0 / 2688.0), (512, 5120, 0.37),
                                        (37, 6144, 37.0), (9, 1040, 1e-3), (300, 48, 2.0 ** 12)])
def test_quantize_rows_bit_exact(backend, rows, k, its, general):
    """`general` = 1 forces the kernel that takes every shape; 0 lets widths that are multiples of 16
    take the streamlined kernel (branch-free scale arithmetic for normal UE4M3 scales, the reference's
    own arithmetic for the rest).  The large and tiny tensor scales push whole rows into the
    subnormal, saturated and clamped scale ranges."""
    rng = np.random.default_rng(rows * 7 + k)
    x = adversarial_activations(rng, rows, k)
    w_fp4, w_sf, w_ts = orc.nvfp4_quantize_rows(x, its)
    backend.lib.qwen36_nvfp4_quantize_set_path(general)
    try:
        fp4, sf, ts = backend.nvfp4_quantize_rows(to_dev(x), its)
    finally:
        backend.lib.qwen36_nvfp4_quantize_set_path(0)
    assert float(ts.item()) == np.float32(w_ts)
    assert np.array_equal(fp4.cpu().numpy(), w_fp4), "packed codes"
    assert np.array_equal(sf.cpu().numpy(), w_sf), "scale bytes"


def test_quantize_scale_bytes_at_every_ue4m3_boundary(backend):
    """Group maxima placed on, just below and just above every rounding boundary of the UE4M3 scale
    (amax = 6 * boundary, which bf16 holds exactly or within one step): the streamlined kernel's
    reciprocal-multiply quotient must land on the reference's byte, ties included."""
    vals = []
    for code in range(0x08, 0x7E):
        a = orc.e4m3_decode(code); b = orc.e4m3_decode(code + 1)
        mid = np.float32((a + b) * 0.5 * 6.0)
        bits = int(synth.f32_to_bf16_bits(np.array([mid], np.float32))[0])
        vals += [bits - 1, bits, bits + 1]
    vals = np.array(vals, dtype=np.uint16)
    x = np.zeros((len(vals), 16), dtype=np.uint16)
    x[:, 3] = vals
    x[:, 7] = vals | 0x8000
    for its in (0.0, 1.0 / 3.0, 0.37, 7.0):
        w_fp4, w_sf, _ = orc.nvfp4_quantize_rows(x, its)
        fp4, sf, _ = backend.nvfp4_quantize_rows(to_dev(x), its)
        assert np.array_equal(sf.cpu().numpy(), w_sf), its
        assert np.array_equal(fp4.cpu().numpy(), w_fp4), its


def test_quantize_single_row_entry_and_known_answer(backend):
    # kernels-cuda/smoke.cu:2140-2180: ones -> scale byte 0x23, codes 0x77
    x = synth.f32_to_bf16_bits(np.ones((1, 128), dtype=np.float32))
    fp4, sf, ts = backend.nvfp4_quantize_bf16(to_dev(x).reshape(-1))
    assert float(ts.item()) == 1.0
    assert np.all(fp4.cpu().numpy() == 0x77)
    sfh = sf.cpu().numpy()
    assert all(sfh[orc.sf_offset(g, 0, 8)] == 0x23 for g in range(8))
    rng = np.random.default_rng(9)
    x = adversarial_activations(rng, 1, 5120)
    w_fp4, w_sf, _ = orc.nvfp4_quantize_rows(x, 1.25)
    fp4, sf, _ = backend.nvfp4_quantize_bf16(to_dev(x).reshape(-1), 1.25)
    assert np.array_equal(fp4.cpu().numpy(), w_fp4.reshape(-1)) and np.array_equal(sf.cpu().numpy(), w_sf)


def test_quantize_subnormal_scale_ties(backend):
    """amax/6 landing exactly between two subnormal UE4M3 codes: the float32 expression of
    kernels-cuda/ops.cu:96 rounds those up."""
    vals = np.array([(c + 0.5) * 2.0 ** -9 * 6.0 for c in range(1, 7)], dtype=np.float32)
    x = np.zeros((1, 16 * len(vals)), dtype=np.float32)
    x[0, ::16] = vals
    xb = synth.f32_to_bf16_bits(x)
    assert np.array_equal(synth.bf16_bits_to_f32(xb), x)       # exactly representable
    w_fp4, w_sf, _ = orc.nvfp4_quantize_rows(xb, 0.0)
    fp4, sf, _ = backend.nvfp4_quantize_rows(to_dev(xb), 0.0)
    assert np.array_equal(sf.cpu().numpy(), w_sf) and np.array_equal(fp4.cpu().numpy(), w_fp4)
    assert [int(w_sf[orc.sf_offset(g, 0, 8)]) for g in range(6)] == [2, 3, 4, 5, 6, 7]


def test_quantize_round_trip_property_large(backend):
    """At full prefill size (M = 8192, K = 5120): requantising the dequantised tensor gives the
    same bytes (idempotence), checked on the device without the oracle."""
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((8192, 5120), generator=g, device="cuda", dtype=torch.float32)
    x[:, ::97] *= 20
    x = x.to(torch.bfloat16)
    fp4, sf, ts = backend.nvfp4_quantize_rows(x, 0.5)
    deq = backend.nvfp4_dequantize(fp4, sf, ts, 5120).to(torch.bfloat16)
    fp4b, sfb, _ = backend.nvfp4_quantize_rows(deq, 0.5)
    assert torch.equal(sf, sfb)
    assert torch.equal(fp4 & 0x77, fp4b & 0x77)      # magnitudes; a -0 code may lose its sign bit


# ---------------------------------------------------------------- dequantise / W4A16 GEMV

@pytest.mark.parametrize("n,k", [(1, 4), (160, 192), (5120, 5120), (130, 40)])
def test_dequantised_weights_bit_exact(backend, n, k):
    rng = np.random.default_rng(n + k)
    packed = rng.integers(0, 256, size=(n, (k + 1) // 2), dtype=np.uint8)
    sf_rm = rng.integers(0, 256, size=(n, (k + 15) // 16), dtype=np.uint8)      # every byte value
    sf = orc.retile_scales(sf_rm)
    ts = torch.tensor([synth.WEIGHT_GLOBAL_SCALE], dtype=torch.float32, device="cuda")
    got = backend.nvfp4_dequantize(to_dev(packed), to_dev(sf), ts, k).cpu().numpy()
    want = orc.nvfp4_dequant(packed, sf, synth.WEIGHT_GLOBAL_SCALE, k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_matvec_known_answer(backend):
    # kernels-cuda/smoke.cu:2114-2138
    w = to_dev(np.array([[0x42, 0xA1]], dtype=np.uint8))
    sf = backend.nvfp4_retile_scales(to_dev(np.array([[0x38]], dtype=np.uint8)))
    assert sf.numel() == 512
    x = to_dev(synth.f32_to_bf16_bits(np.array([1, 2, 3, 4], dtype=np.float32)))
    one = torch.ones(1, dtype=torch.float32, device="cuda")
    assert backend.nvfp4_matvec(x, w, sf, one).float().item() == 2.5
    assert backend.nvfp4_matvec(x, w, sf, None).float().item() == 2.5


@pytest.mark.parametrize("quads", [0, 8, 2])
@pytest.mark.parametrize("n,k", [(5120, 5120), (1024, 5120), (5120, 6144), (12288, 5120), (5120, 17408),
                                 (34816, 5120), (130, 96), (40, 2080), (7, 33), (256, 32768), (384, 8224)])
def test_matvec_w4a16_vs_oracle(backend, n, k, quads):
    """Config-0 bar: rel-L2 <= 1e-3 on the bf16 output against the reference's scalar semantics.
    `quads` forces the work-unit size of the pipelined kernel (0 = the library's own choice)."""
    rng = np.random.default_rng(n * 3 + k + 1)
    packed = rng.integers(0, 256, size=(n, (k + 1) // 2), dtype=np.uint8)
    sf_rm = rng.integers(synth.SF_CODE_LO, synth.SF_CODE_HI + 1, size=(n, (k + 15) // 16), dtype=np.uint8)
    sf = orc.retile_scales(sf_rm)
    x = synth.activations(rng, 1, k)[0]
    ts = torch.tensor([synth.WEIGHT_GLOBAL_SCALE], dtype=torch.float32, device="cuda")
    backend.lib.qwen36_nvfp4_matvec_force_quads(quads)
    try:
        got = bf16_host(backend.nvfp4_matvec(to_dev(x), to_dev(packed), to_dev(sf), ts))
    finally:
        backend.lib.qwen36_nvfp4_matvec_force_quads(0)
    assert backend.lib.qwen36_nvfp4_matvec_last_error() == 0
    want = orc.nvfp4_matvec(x, packed, sf, synth.WEIGHT_GLOBAL_SCALE, k)
    err = rel_l2(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(want))
    assert err <= 1e-3, err
    assert (got == want).mean() > 0.98       # nearly every bf16 output identical


@pytest.mark.parametrize("n,k", [(128, 256), (128, 1024), (256, 1280), (384, 7424), (640, 2048), (1152, 3328)])
def test_matvec_tensor_core_path_small_shapes(backend, n, k):
    """Shapes the tensor-core GEMV takes (rows % 128 == 0, columns % 256 == 0), chosen so that the
    last pipeline stage is partial, a unit's 32 rows straddle every quarter of a 128-row block, and
    a CTA walks several units; every UE4M3 byte value occurs among the block scales, including the
    subnormal codes, 0x80 (zero) and 0x7F / 0xFF, which the reference reads as 448 (rows that hold
    one are recomputed by the kernel's scalar fallback)."""
    rng = np.random.default_rng(n * 5 + k)
    packed = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    sf_rm = rng.integers(0, 256, size=(n, k // 16), dtype=np.uint8)
    sf_rm[::3] &= 0x7F                         # a third of the rows without negative scales
    sf_rm[1::2][sf_rm[1::2] == 0x7F] = 0x30    # half of the rows free of the 448 codes
    sf_rm[1::2][sf_rm[1::2] == 0xFF] = 0x31
    sf = orc.retile_scales(sf_rm)
    x = synth.activations(rng, 1, k)[0]
    ts = torch.tensor([0.37], dtype=torch.float32, device="cuda")
    got = bf16_host(backend.nvfp4_matvec(to_dev(x), to_dev(packed), to_dev(sf), ts))
    assert backend.lib.qwen36_nvfp4_gemv_mma_last_error() == 0
    want = orc.nvfp4_matvec(x, packed, sf, 0.37, k)
    assert rel_l2(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(want)) <= 1e-3
    assert (got == want).mean() > 0.98


def test_matvec_group_equals_single_calls(backend):
    """qwen36_nvfp4_matvec_group over the q / k / v projections of a decode layer (one launch) gives
    what three qwen36_nvfp4_matvec calls give, and the oracle's result; a group the one-launch
    kernel declines (ragged rows) still returns the right answers; mismatched inputs are refused."""
    import ctypes as C
    rng = np.random.default_rng(606)
    k = 5120
    x = synth.activations(rng, 1, k)[0]
    xd = to_dev(x)
    mats, wants = [], []
    for i, n in enumerate((12288, 1024, 1024, 256)):
        packed, sf_rm, sf = make_weight(rng, n, k)
        g = synth.WEIGHT_GLOBAL_SCALE * (i + 1)
        ts = torch.tensor([g], dtype=torch.float32, device="cuda") if i != 3 else None
        out = torch.full((n,), float("nan"), dtype=torch.bfloat16, device="cuda")
        mats.append((to_dev(packed), to_dev(sf), ts, out))
        wants.append(orc.nvfp4_matvec(x, packed, sf, g if i != 3 else None, k))
    backend.nvfp4_matvec_group(xd, mats)
    assert backend.lib.qwen36_nvfp4_gemv_mma_last_error() == 0
    for (w, sf, ts, out), want in zip(mats, wants):
        got = bf16_host(out)
        assert rel_l2(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(want)) <= 1e-3
        assert np.array_equal(got, bf16_host(backend.nvfp4_matvec(xd, w, sf, ts)))
    # a group with a ragged matrix falls back to one launch per matrix
    packed, sf_rm, sf = make_weight(rng, 130, k)
    out = torch.empty(130, dtype=torch.bfloat16, device="cuda")
    backend.nvfp4_matvec_group(xd, [mats[1], (to_dev(packed), to_dev(sf), None, out)])
    want = orc.nvfp4_matvec(x, packed, sf, None, k)
    assert rel_l2(synth.bf16_bits_to_f32(bf16_host(out)), synth.bf16_bits_to_f32(want)) <= 1e-3
    # specs that do not share their input are an error
    specs = (abi.Nvfp4MatvecSpec * 2)()
    for i in range(2):
        w, sf, ts, out = mats[i]
        other = to_dev(x.copy())
        specs[i] = abi.Nvfp4MatvecSpec(w.shape[0], k, abi.DevicePtr((xd if i == 0 else other).data_ptr()),
                                       abi.DevicePtr(w.data_ptr()), abi.DevicePtr(sf.data_ptr()),
                                       abi.DevicePtr(ts.data_ptr()), abi.DevicePtr(out.data_ptr()))
    assert backend.lib.qwen36_nvfp4_matvec_group(specs, 2) == abi.INVALID_ARGUMENT
    assert backend.lib.qwen36_nvfp4_matvec_group(specs, 5) == abi.INVALID_ARGUMENT
    assert backend.lib.qwen36_nvfp4_matvec_group(None, 1) == abi.NULL_POINTER


def test_matvec_non_finite_activations(backend):
    """inf or NaN among the activations: rows whose reference result is NaN / inf come out NaN / inf
    here too, all other outputs keep their tolerance (the kernel redoes NaN rows with the scalar
    arithmetic of the reference)."""
    rng = np.random.default_rng(88)
    n, k = 256, 2048
    packed, sf_rm, sf = make_weight(rng, n, k)
    packed[7, :] = 0                            # a row of zero weights: inf * 0 = NaN
    ts = torch.ones(1, dtype=torch.float32, device="cuda")
    x = synth.activations(rng, 1, k)[0]
    x[100] = 0x7F80                             # +inf
    got = synth.bf16_bits_to_f32(bf16_host(backend.nvfp4_matvec(to_dev(x), to_dev(packed), to_dev(sf), ts)))
    want = synth.bf16_bits_to_f32(orc.nvfp4_matvec(x, packed, sf, 1.0, k))
    assert np.array_equal(np.isnan(got), np.isnan(want))
    fin = np.isfinite(want)
    assert np.array_equal(got[~fin & ~np.isnan(want)], want[~fin & ~np.isnan(want)])
    assert rel_l2(got[fin], want[fin]) <= 1e-3


def test_matvec_extreme_activation_ranges(backend):
    """Scaled-float16 activation path: tiny, huge and mixed magnitudes stay within tolerance."""
    rng = np.random.default_rng(77)
    n, k = 256, 1024
    packed, sf_rm, sf = make_weight(rng, n, k)
    ts = torch.ones(1, dtype=torch.float32, device="cuda")
    for gain in (1e-30, 1e-12, 1.0, 1e12, 1e30):
        x = (rng.standard_normal(k) * gain).astype(np.float32)
        x[::50] *= 1e-6
        xb = synth.f32_to_bf16_bits(x)
        got = synth.bf16_bits_to_f32(bf16_host(backend.nvfp4_matvec(to_dev(xb), to_dev(packed), to_dev(sf), ts)))
        want = synth.bf16_bits_to_f32(orc.nvfp4_matvec(xb, packed, sf, 1.0, k))
        assert rel_l2(got, want) <= 1e-3, gain


def test_matvec_linearity_full_size(backend):
    """Size-independent property at the largest decode shape: W(2x) == 2 W(x) exactly in bf16."""
    gen = torch.Generator(device="cuda").manual_seed(1)
    n, k = 34816, 5120
    packed, sf_rm = synth.nvfp4_weight_device(gen, n, k, "cuda")
    sf = backend.nvfp4_retile_scales(sf_rm)
    x = torch.randn(k, generator=gen, device="cuda").to(torch.bfloat16)
    ts = torch.tensor([synth.WEIGHT_GLOBAL_SCALE], dtype=torch.float32, device="cuda")
    y1 = backend.nvfp4_matvec(x, packed, sf, ts)
    y2 = backend.nvfp4_matvec(x * 2, packed, sf, ts)
    assert torch.equal(y1.float() * 2, y2.float())


def test_quantize_codes_at_every_rounding_boundary(backend):
    """The device encoder (hardware e2m1 conversion + explicit tie handling) against the oracle's
    threshold chain on inputs placed exactly on, one bf16 step below and one step above each of the
    seven rounding boundaries, both signs, for several power-of-two scales (so the quotient is exact),
    plus zeros of both signs, NaN, infinities and subnormals."""
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    rows = []
    for d in (2.0 ** -10, 0.25, 1.0, 8.0, 2.0 ** 20):
        vals = []
        for t in ties:
            b = int(synth.f32_to_bf16_bits(np.array([t * d], np.float32))[0])
            for step in (-2, -1, 0, 1, 2):
                vals += [b + step, (b + step) | 0x8000]
        vals += [0x0000, 0x8000, 0x7FC0, 0xFFC0, 0x7F80, 0xFF80, 0x0001, 0x8001, 0x0080, 0x8080]
        vals = np.array(vals, dtype=np.uint16)
        anchor = synth.f32_to_bf16_bits(np.array([6.0 * d], np.float32))[0]      # fixes the group scale at d
        for i in range(0, len(vals), 15):
            chunk = vals[i:i + 15]
            group = np.full(16, 0, dtype=np.uint16)
            group[0] = anchor
            group[1:1 + len(chunk)] = chunk
            rows.append(group)
    rows.append(np.zeros(16, dtype=np.uint16))                                   # all +0
    rows.append(np.full(16, 0x8000, dtype=np.uint16))                            # all -0
    rows.append(np.array([0, 0x7FC0] + [0] * 14, dtype=np.uint16))               # zeros and one NaN
    rows.append(np.array([0x8000, 0x3F80] + [0] * 14, dtype=np.uint16))          # zeros mixed with a value
    x = np.stack(rows)
    # groups that hold NaN or inf take their scale from that value: still compared, only the finite
    # anchor groups exercise the boundaries
    for its in (0.0, 2.0):
        want_fp4, want_sf, _ = orc.nvfp4_quantize_rows(x, its)
        fp4, sf, _ = backend.nvfp4_quantize_rows(to_dev(x), its)
        assert np.array_equal(fp4.cpu().numpy(), want_fp4)
        assert np.array_equal(sf.cpu().numpy(), want_sf)


# ---------------------------------------------------------------- W4A4 product

def w4a4_case(rng, m, n, k, its=1.25):
    packed, sf_rm, a_sf = make_weight(rng, m, k)
    x = synth.activations(rng, n, k, outlier_frac=0.01)
    b, b_sf, ts = orc.nvfp4_quantize_rows(x, its)
    return packed, a_sf, x, b, b_sf, synth.WEIGHT_GLOBAL_SCALE * ts


@pytest.mark.parametrize("m,n,k", [(128, 1, 128), (256, 1, 5120), (40, 3, 96), (384, 5, 1024), (256, 8, 512),
                                   (128, 17, 256), (256, 130, 512), (384, 512, 768)])
def test_w4a4_gemm_vs_oracle(backend, m, n, k):
    """rel-L2 <= 1e-2 against the double-precision dequantise-and-multiply oracle."""
    rng = np.random.default_rng(m + 31 * n + k)
    a, a_sf, x, b, b_sf, alpha = w4a4_case(rng, m, n, k)
    got = bf16_host(backend.nvfp4_gemm(to_dev(a), to_dev(a_sf), to_dev(b), to_dev(b_sf), alpha, m, n, k))
    want = orc.nvfp4_gemm(a, a_sf, b, b_sf, alpha, m, n, k)
    err = rel_l2(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(want))
    assert err <= 1e-2, err


@pytest.mark.parametrize("m,n,k", [(256, 130, 512), (512, 300, 1024), (384, 257, 768), (256, 1000, 8192),
                                   (1024, 640, 2560)])
def test_w4a4_gemm_tile_variants(backend, m, n, k):
    """Every tile form of the tcgen05 kernel (128- and 256-token single-CTA tiles, 256 x 256 CTA
    pairs with five combined stages, and with six operand stages + the scale tiles on a pipeline of
    their own; the pair forms step aside when m is not a multiple of 256) gives the oracle's
    result, and all forms agree bit for bit: they accumulate K in the same order."""
    rng = np.random.default_rng(7 * m + n + k)
    a, a_sf, x, b, b_sf, alpha = w4a4_case(rng, m, n, k)
    want = synth.bf16_bits_to_f32(orc.nvfp4_gemm(a, a_sf, b, b_sf, alpha, m, n, k))
    dev = [to_dev(t) for t in (a, a_sf, b, b_sf)]
    outs = []
    try:
        backend.lib.qwen36_nvfp4_gemm_stream_k(1)          # whole tiles only: the stream-K form regroups the K sum
        for tile in (0, 128, 256, 512, 768):
            backend.lib.qwen36_nvfp4_gemm_force_bn(tile)
            got = bf16_host(backend.nvfp4_gemm(*dev, alpha, m, n, k))
            assert rel_l2(synth.bf16_bits_to_f32(got), want) <= 1e-2, tile
            outs.append(got)
    finally:
        backend.lib.qwen36_nvfp4_gemm_force_bn(0)
        backend.lib.qwen36_nvfp4_gemm_stream_k(0)
    assert backend.lib.qwen36_nvfp4_gemm_last_error() == 0
    for got in outs[1:]:
        assert np.array_equal(got, outs[0])


@pytest.mark.parametrize("m,n,k", [(256, 1000, 8192), (512, 600, 4096), (1024, 512, 8704), (256, 512, 2560)])
def test_w4a4_gemm_stream_k(backend, m, n, k):
    """Stream-K form of the CTA-pair kernel (tiles cut along K so that every pair gets the same number of
    K-blocks; partial tiles meet in the caller's workspace, added in K order): the oracle's result, the
    whole-tile form's result up to the regrouping of float32 additions, the same bits on every run (a
    second launch finds the first one's flags in the workspace), and the whole-tile form when no
    workspace is passed.  Shapes: a tile shared by up to eighteen pairs, ragged token counts, fewer
    K-blocks per pair than a tile has."""
    rng = np.random.default_rng(11 * m + n + k)
    a, a_sf, x, b, b_sf, alpha = w4a4_case(rng, m, n, k)
    want = synth.bf16_bits_to_f32(orc.nvfp4_gemm(a, a_sf, b, b_sf, alpha, m, n, k))
    dev = [to_dev(t) for t in (a, a_sf, b, b_sf)]
    try:
        backend.lib.qwen36_nvfp4_gemm_force_bn(768)
        backend.lib.qwen36_nvfp4_gemm_stream_k(1)
        whole = bf16_host(backend.nvfp4_gemm(*dev, alpha, m, n, k))
        backend.lib.qwen36_nvfp4_gemm_stream_k(2)
        cut = [bf16_host(backend.nvfp4_gemm(*dev, alpha, m, n, k)) for _ in range(3)]
        out = torch.zeros((n, m), dtype=torch.bfloat16, device="cuda")
        spec = abi.Nvfp4GemmSpec(m, n, k, *[abi.DevicePtr(t.data_ptr()) for t in dev[:2]], abi.DevicePtr(0),
                                 *[abi.DevicePtr(t.data_ptr()) for t in dev[2:]], abi.DevicePtr(0),
                                 abi.DevicePtr(out.data_ptr()), abi.DevicePtr(0), 0, alpha)
        import ctypes as C
        assert backend.lib.qwen36_nvfp4_gemm(C.byref(spec)) == abi.SUCCESS
        no_ws = bf16_host(out)
    finally:
        backend.lib.qwen36_nvfp4_gemm_force_bn(0)
        backend.lib.qwen36_nvfp4_gemm_stream_k(0)
    assert backend.lib.qwen36_nvfp4_gemm_last_error() == 0
    assert np.array_equal(no_ws, whole)
    assert np.array_equal(cut[1], cut[0]) and np.array_equal(cut[2], cut[0])
    got, ref = synth.bf16_bits_to_f32(cut[0]), synth.bf16_bits_to_f32(whole)
    assert rel_l2(got, want) <= 1e-2
    assert rel_l2(got, ref) <= 2e-4
    assert (cut[0] == whole).mean() >= 0.995
    assert not np.array_equal(cut[0], whole) or k <= 2560     # the cut really happened where the shape is large enough


@pytest.mark.parametrize("m,n,k", [(1024, 1, 5120), (640, 8, 6144), (256, 3, 17408), (384, 16, 1024), (128, 5, 512),
                                   (384, 24, 2048), (256, 32, 17408), (640, 33, 6144), (256, 64, 4096)])
def test_w4a4_decode_split_k(backend, m, n, k):
    """Few tokens, few row blocks: clusters of CTAs split K and add their partial sums through
    distributed shared memory.  Every split factor matches the oracle; split and unsplit results
    differ only by float32 summation order."""
    rng = np.random.default_rng(11 * m + n + k)
    a, a_sf, x, b, b_sf, alpha = w4a4_case(rng, m, n, k)
    want = synth.bf16_bits_to_f32(orc.nvfp4_gemm(a, a_sf, b, b_sf, alpha, m, n, k))
    dev = [to_dev(t) for t in (a, a_sf, b, b_sf)]
    try:
        for split in (0, 1, 2, 3, 8):
            backend.lib.qwen36_nvfp4_gemm_force_split(split)
            out = torch.full((n, m), float("nan"), dtype=torch.bfloat16, device="cuda")
            entry = backend.decode_nvfp4_gemv_raw if n <= 8 else backend.nvfp4_gemm_raw   # the decode entry takes n <= 8
            assert entry(*dev, alpha, m, n, k, out) == abi.SUCCESS
            got = synth.bf16_bits_to_f32(bf16_host(out))
            assert rel_l2(got, want) <= 1e-2, split
    finally:
        backend.lib.qwen36_nvfp4_gemm_force_split(0)
    assert backend.lib.qwen36_nvfp4_gemm_last_error() == 0


@pytest.mark.parametrize("m,k", [(1024, 5120), (5120, 6144), (5120, 17408), (12288, 5120), (128, 256), (384, 1280)])
def test_w4a4_one_token_decode_vs_oracle(backend, m, k):
    """One token through qwen36_decode_nvfp4_gemv and qwen36_nvfp4_gemm (the route of the
    5120 x 17408 down projection): the tensor-core GEMV with the activation dequantised to float16
    (exact).  rel-L2 <= 1e-2 against the float64 oracle (in fact ~1e-3: bf16 rounding of the output)."""
    rng = np.random.default_rng(m + k)
    a, a_sf, x, b, b_sf, alpha = w4a4_case(rng, m, 1, k)
    want = synth.bf16_bits_to_f32(orc.nvfp4_gemm(a, a_sf, b, b_sf, alpha, m, 1, k))
    dev = [to_dev(t) for t in (a, a_sf, b, b_sf)]
    for entry in (backend.decode_nvfp4_gemv_raw, backend.nvfp4_gemm_raw):
        out = torch.full((1, m), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert entry(*dev, alpha, m, 1, k, out) == abi.SUCCESS
        got = synth.bf16_bits_to_f32(bf16_host(out))
        assert rel_l2(got, want) <= 3e-3
    assert backend.lib.qwen36_nvfp4_gemv_mma_last_error() == 0


def test_w4a4_known_answer_132_and_alpha_zero(backend):
    # kernels-cuda/smoke.cu:2140-2180
    k = m = 128
    x = to_dev(synth.f32_to_bf16_bits(np.ones((1, k), dtype=np.float32)))
    fp4, sf, _ = backend.nvfp4_quantize_rows(x)
    a = torch.full((m, k // 2), 0x22, dtype=torch.uint8, device="cuda")
    a_sf = torch.full((m * k // 16,), 0x38, dtype=torch.uint8, device="cuda")
    out = torch.empty((1, m), dtype=torch.bfloat16, device="cuda")
    assert backend.nvfp4_gemm_raw(a, a_sf, fp4, sf, 1.0, m, 1, k, out) == abi.SUCCESS
    assert torch.all(out.float() == 132.0)
    assert backend.nvfp4_gemm_raw(a, a_sf, fp4, sf, 0.0, m, 1, k, out) == abi.SUCCESS      # alpha 0 -> 1
    assert torch.all(out.float() == 132.0)


def test_quantise_then_gemm_end_to_end(backend):
    """The prefill chain on the device: quantize_rows -> nvfp4_gemm, against oracle of the same chain."""
    rng = np.random.default_rng(2024)
    m, n, k = 512, 160, 1024
    packed, sf_rm, a_sf = make_weight(rng, m, k)
    x = synth.activations(rng, n, k, outlier_frac=0.01)
    fp4, sf, ts = backend.nvfp4_quantize_rows(to_dev(x), 0.37)
    alpha = synth.WEIGHT_GLOBAL_SCALE * float(ts.item())
    got = bf16_host(backend.nvfp4_gemm(to_dev(packed), to_dev(a_sf), fp4, sf, alpha, m, n, k))
    b, b_sf, ts_o = orc.nvfp4_quantize_rows(x, 0.37)
    want = orc.nvfp4_gemm(packed, a_sf, b, b_sf, synth.WEIGHT_GLOBAL_SCALE * ts_o, m, n, k)
    assert rel_l2(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(want)) <= 1e-2


@pytest.mark.parametrize("m,n", [(1280, 2048), (2560, 512), (1280, 8192)])
def test_w4a4_gemm_stream_k_on_row_shards_of_down(backend, m, n):
    """The down projection split by rows over two or four GPUs (K = 17408) at prefill token counts: the
    library's own choice with a workspace (stream-K: few tiles, long K) against the whole-tile form,
    which other tests pin to the oracle."""
    k = 17408
    gen = torch.Generator(device="cuda").manual_seed(m + n)
    packed, sf_rm = synth.nvfp4_weight_device(gen, m, k, "cuda")
    sfa = backend.nvfp4_retile_scales(sf_rm)
    x = torch.randn((n, k), generator=gen, device="cuda").to(torch.bfloat16)
    fp4, sfb, ts = backend.nvfp4_quantize_rows(x, 0.37)
    alpha = float(np.float32(synth.WEIGHT_GLOBAL_SCALE) * np.float32(ts.item()))
    try:
        backend.lib.qwen36_nvfp4_gemm_stream_k(1)
        whole = backend.nvfp4_gemm(packed, sfa, fp4, sfb, alpha, m, n, k).clone()
        backend.lib.qwen36_nvfp4_gemm_stream_k(0)
        chosen = [backend.nvfp4_gemm(packed, sfa, fp4, sfb, alpha, m, n, k).clone() for _ in range(2)]
    finally:
        backend.lib.qwen36_nvfp4_gemm_stream_k(0)
    torch.cuda.synchronize()
    assert backend.lib.qwen36_nvfp4_gemm_last_error() == 0
    assert torch.equal(chosen[0], chosen[1])
    diff = (chosen[0].float() - whole.float()).norm().item() / whole.float().norm().item()
    same = (chosen[0].view(torch.int16) == whole.view(torch.int16)).float().mean().item()
    assert diff <= 2e-4 and same >= 0.995, (diff, same)
    assert same < 1.0              # the cut really happened: some float32 sums were regrouped


def test_w4a4_gemm_stream_k_under_graph_replay(backend):
    """A captured stream-K launch replays with the same tag: the flags of one replay must not satisfy the
    next.  Three replays on fresh activations, each against the eager result for the same operands."""
    m, n, k = 256, 1000, 8192
    rng = np.random.default_rng(5)
    a, a_sf, x, b, b_sf, alpha = w4a4_case(rng, m, n, k)
    a_d, sfa_d = to_dev(a), to_dev(a_sf)
    cases = [(to_dev(b), to_dev(b_sf))]
    for _ in range(2):
        _, _, _, b2, b2_sf, _ = w4a4_case(rng, m, n, k)
        cases.append((to_dev(b2), to_dev(b2_sf)))
    try:
        backend.lib.qwen36_nvfp4_gemm_force_bn(768)
        backend.lib.qwen36_nvfp4_gemm_stream_k(2)
        eager = [backend.nvfp4_gemm(a_d, sfa_d, bb, bs, alpha, m, n, k).clone() for bb, bs in cases]
        torch.cuda.synchronize()
        b_buf, s_buf = cases[0][0].clone(), cases[0][1].clone()
        out = torch.zeros((n, m), dtype=torch.bfloat16, device="cuda")
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            backend.sync_stream()
            backend.nvfp4_gemm(a_d, sfa_d, b_buf, s_buf, alpha, m, n, k, out)
        backend.sync_stream()
        for (bb, bs), want in zip(cases, eager):
            b_buf.copy_(bb); s_buf.copy_(bs)
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, want)
    finally:
        backend.lib.qwen36_nvfp4_gemm_force_bn(0)
        backend.lib.qwen36_nvfp4_gemm_stream_k(0)
        backend.sync_stream()
    assert backend.lib.qwen36_nvfp4_gemm_last_error() == 0
