"""The CPU oracle against what the reference itself pins: fixtures recorded
from the reference's Python decomposition (tests/golden/make_golden.py) and the
known-answer vectors of the reference's kernel smoke test
(kernels-cuda/smoke.cu:126-200, 2114-2180)."""
import numpy as np

from oracle import oracle as orc
from speedoza_b200 import synth

LUT = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


def dequant_activation(fp4, sf, rows, values, g):
    """lut(code) * max(decode(sf) * g, 1e-8) from oracle-quantised bytes."""
    groups = (values + 15) // 16
    sf_inner = (groups + 3) // 4 * 4
    out = np.zeros((rows, values), dtype=np.float32)
    for r in range(rows):
        for c in range(values):
            b = fp4[r, c // 2]
            code = (b >> 4) if (c & 1) else (b & 15)
            ds = max(np.float32(orc.e4m3_decode(int(sf[orc.sf_offset(c // 16, r, sf_inner)]))) *
                     np.float32(g), np.float32(1e-8))
            out[r, c] = LUT[code] * np.float32(ds)
    return out


def test_e4m3_decode_all_codes(golden):
    got = np.array([orc.e4m3_decode(c) for c in range(256)], dtype=np.float32)
    assert np.array_equal(got, golden["e4m3_decode_table"])


def test_ue4m3_encode_matches_reference(golden):
    vals = golden["ue4m3_encode_in"]
    got = np.array([orc.ue4m3_encode(v) for v in vals], dtype=np.uint8)
    want = golden["ue4m3_encode_out"]
    diff = np.nonzero(got != want)[0]
    # The only disagreements allowed are exact (or one-ulp-near) ties on the
    # SUBNORMAL grid: there the reference CUDA evaluates
    # floorf(v / 2^-9 + 0.49999994f) in float32 (kernels-cuda/ops.cu:96), where
    # the sum rounds up to the next integer, while the reference's Python
    # script evaluates the same expression in float64.  The oracle follows the
    # CUDA source, so on those inputs it must give the Python answer + 1.
    for i in diff:
        steps = np.float64(vals[i]) / 2.0 ** -9
        assert vals[i] < 2.0 ** -6 and abs(steps - np.floor(steps) - 0.5) < 1e-6, vals[i]
        assert got[i] == want[i] + 1
    assert len(diff) <= 8


def test_activation_quantise_dequant_bit_exact(golden):
    x = golden["act_in_bf16"]
    for name, s in (("1", 1.0), ("1p25", 1.25), ("0p5", 0.5), ("0", 0.0)):
        fp4, sf, ts = orc.nvfp4_quantize_rows(x, s)
        g = s if s > 0 else 1.0
        assert ts == np.float32(g)
        got = dequant_activation(fp4, sf, *x.shape, g)
        want = golden[f"act_dequant_scale_{name}"]
        assert np.array_equal(got.view(np.uint32) & 0x7FFFFFFF, want.view(np.uint32) & 0x7FFFFFFF), name
        # signs agree wherever the value is non-zero (the reference Python
        # drops the sign of a zero code, the byte keeps it)
        nz = want != 0
        assert np.array_equal(np.signbit(got[nz]), np.signbit(want[nz]))


def test_activation_quantise_ragged(golden):
    x = golden["act_ragged_in_bf16"]
    fp4, sf, _ = orc.nvfp4_quantize_rows(x, 1.25)
    got = dequant_activation(fp4, sf, *x.shape, 1.25)
    assert np.array_equal(np.abs(got), np.abs(golden["act_ragged_dequant"]))


def test_e2m1_ties_go_toward_zero():
    for v, code in ((0.25, 0), (0.75, 1), (1.25, 2), (1.75, 3), (2.5, 4), (3.5, 5), (5.0, 6),
                    (-0.75, 9), (-0.0, 0), (7.0, 7), (float("nan"), 7), (-100.0, 15)):
        assert orc.e2m1_encode(v) == code, v


def test_weight_dequant_bit_exact(golden):
    sf = orc.retile_scales(golden["w_sf_row_major"])
    got = orc.nvfp4_dequant(golden["w_packed"], sf, float(golden["w_scale_2"][0]), 192)
    want = golden["w_dequant"]
    # The reference Python forms (lut * sf) * ws2 (one rounding); the reference
    # CUDA forms lut * (sf * ws2) (kernels-cuda/ops.cu:574-575,631: the scale is
    # rounded first, then the product).  The oracle follows the CUDA order, so
    # against the Python fixture it may differ by the last float32 bit only.
    ulp = np.abs(got.view(np.int32) - want.view(np.int32))
    assert ulp.max() <= 1
    assert (ulp == 0).mean() > 0.5
    # and the oracle equals the CUDA order restated in numpy float32
    sfd = np.array([orc.e4m3_decode(int(c)) for c in range(256)], dtype=np.float32)
    scale = sfd[golden["w_sf_row_major"]] * np.float32(golden["w_scale_2"][0])
    w = golden["w_packed"]
    codes = np.stack([w & 15, w >> 4], -1).reshape(160, 192)
    assert np.array_equal(got, LUT[codes] * np.repeat(scale, 16, axis=1))


def test_linear_w4a4_against_reference_python(golden):
    sf = orc.retile_scales(golden["w_sf_row_major"])
    x = golden["lin_x_bf16"]
    in_scale = float(golden["lin_input_scale"][0])
    b, b_sf, ts = orc.nvfp4_quantize_rows(x, in_scale)
    alpha = float(golden["w_scale_2"][0]) * ts
    y = orc.bf16_to_f32(orc.nvfp4_gemm(golden["w_packed"], sf, b, b_sf, alpha, 160, 3, 192))
    want = golden["lin_y"]
    rel = np.linalg.norm(y - want) / np.linalg.norm(want)
    assert rel < 2e-3, rel


def test_smoke_known_answer_matvec_2p5():
    # kernels-cuda/smoke.cu:2114-2138
    w = np.array([[0x42, 0xA1]], dtype=np.uint8)
    sf = orc.retile_scales(np.array([[0x38]], dtype=np.uint8))
    assert sf.shape == (512,)
    x = orc.f32_to_bf16(np.array([1, 2, 3, 4], dtype=np.float32))
    y = orc.nvfp4_matvec(x, w, sf, 1.0, 4)
    assert orc.bf16_to_f32(y)[0] == 2.5
    assert orc.bf16_to_f32(orc.nvfp4_matvec(x, w, sf, None, 4))[0] == 2.5


def test_smoke_known_answer_quantise_ones_and_gemm_132():
    # kernels-cuda/smoke.cu:2140-2180
    k, m = 128, 128
    x = orc.f32_to_bf16(np.ones((1, k), dtype=np.float32))
    fp4, sf, ts = orc.nvfp4_quantize_rows(x, 0.0)
    assert ts == 1.0
    assert np.all(fp4 == 0x77)
    assert all(sf[orc.sf_offset(g, 0, 8)] == 0x23 for g in range(8))
    a = np.full((m, k // 2), 0x22, dtype=np.uint8)
    a_sf = np.full(m * k // 16, 0x38, dtype=np.uint8)
    y = orc.bf16_to_f32(orc.nvfp4_gemm(a, a_sf, fp4, sf, 1.0, m, 1, k))
    assert np.all(y == 132.0)
    # alpha == 0 is read as 1 (kernels-cuda/nvfp4_gemm.cu:380)
    assert np.all(orc.bf16_to_f32(orc.nvfp4_gemm(a, a_sf, fp4, sf, 0.0, m, 1, k)) == 132.0)


def test_quantise_zero_group_and_saturation():
    x = np.zeros((1, 32), dtype=np.float32)
    x[0, 16] = 1e-3           # amax/6 encodes to scale code 0: the decoded scale clamps
    x[0, 17] = -1e-3          # to 1e-8 and every value above 5e-8 saturates to +-6
    x[0, 18] = -1e-30         # ... a tiny negative keeps its sign bit on a zero magnitude
    fp4, sf, _ = orc.nvfp4_quantize_rows(orc.f32_to_bf16(x), 0.0)
    assert sf[orc.sf_offset(0, 0, 4)] == 0x38 and np.all(fp4[0, :8] == 0)
    assert sf[orc.sf_offset(1, 0, 4)] == 0x00
    assert fp4[0, 8] == 0xF7 and fp4[0, 9] == 0x08 and np.all(fp4[0, 10:] == 0)


def test_argmax_ties_and_nan():
    # kernels-cuda/smoke.cu:126-200: rows 1 and 4 tie at 5.0 -> lowest index
    logits = np.array([[1, 5, 2, 3, 5, 0], [7, 1, 1, 1, 1, 1]], dtype=np.float32)
    assert list(orc.argmax_rows(orc.f32_to_bf16(logits))) == [1, 0]
    nanrow = np.array([[np.nan, -np.inf, 3.0, np.nan]], dtype=np.float32)
    assert list(orc.argmax_rows(orc.f32_to_bf16(nanrow))) == [2]
    allbad = np.array([[np.nan, -np.inf, np.nan]], dtype=np.float32)
    assert list(orc.argmax_rows(orc.f32_to_bf16(allbad))) == [0]


def test_fp8_e4m3_roundtrip_and_rne():
    for c in range(256):
        v = orc.fp8_e4m3_to_f32(c)
        if np.isnan(v):
            assert (c & 0x7F) == 0x7F
            continue
        assert orc.f32_to_fp8_e4m3(v) == c or v == 0.0
    # against torch's float8_e4m3fn cast (round-to-nearest-even, saturating inputs in range)
    import torch
    rng = np.random.default_rng(7)
    vals = np.concatenate([rng.normal(size=4000) * 100, rng.normal(size=2000) * 0.01,
                           [0.0, 448.0, -448.0, 2 ** -9, 2 ** -10, 3 * 2 ** -10]]).astype(np.float32)
    vals = np.clip(vals, -448, 448)
    want = torch.from_numpy(vals).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([orc.f32_to_fp8_e4m3(v) for v in vals], dtype=np.uint8)
    # +0/-0 inputs aside, codes agree bit for bit
    assert np.array_equal(got & 0x7F, want & 0x7F)
    assert orc.f32_to_fp8_e4m3(1e9) == 0x7E and orc.f32_to_fp8_e4m3(-1e9) == 0xFE


def test_lm_head_quantise_and_gemv_small():
    rng = np.random.default_rng(3)
    w = orc.f32_to_bf16(rng.normal(size=(40, 64)).astype(np.float32))
    w[5] = 0
    q, s = orc.lm_head_fp8_quantize(w)
    assert s[5] == 1.0 and np.all(q[5] == 0)
    wf = orc.bf16_to_f32(w)
    assert np.allclose(s[0], np.abs(wf[0]).max() / 448.0)
    x = orc.f32_to_bf16(rng.normal(size=(2, 64)).astype(np.float32))
    y = orc.bf16_to_f32(orc.lm_head_fp8_gemv(q, s, x))
    deq = np.array([[orc.fp8_e4m3_to_f32(int(c)) for c in row] for row in q], dtype=np.float64) * s[:, None]
    want = orc.bf16_to_f32(x).astype(np.float64) @ deq.T
    assert np.allclose(y, want, rtol=1e-2, atol=1e-3)


def test_kv_encode_attention_and_split_merge():
    rng = np.random.default_rng(11)
    T, H, KV, D = 37, 6, 2, 32
    k = orc.f32_to_bf16(rng.normal(size=(T, KV, D)).astype(np.float32))
    v = orc.f32_to_bf16(rng.normal(size=(T, KV, D)).astype(np.float32))
    k[3, 1] = 0     # zero vector: scale 0, codes 0
    kq = np.zeros((T, KV, D), np.int8); vq = np.zeros((T, KV, D), np.int8)
    meta = np.zeros((T, KV, 2), np.float32)
    orc.kv_encode(k, v, 0, kq, vq, meta)
    kf = orc.bf16_to_f32(k)
    assert meta[3, 1, 0] == 0 and np.all(kq[3, 1] == 0)
    assert np.allclose(meta[..., 0], np.abs(kf).max(-1) / np.float32(127))
    assert np.abs(kq).max() == 127
    q = orc.f32_to_bf16(rng.normal(size=(H, D)).astype(np.float32))
    out = orc.bf16_to_f32(orc.kv_attention(q, kq, vq, meta, T - 1))
    # numpy float64 restatement
    kd = kq.astype(np.float64) * meta[..., 0:1]; vd = vq.astype(np.float64) * meta[..., 1:2]
    qf = orc.bf16_to_f32(q).astype(np.float64)
    want = np.zeros((H, D))
    for h in range(H):
        s = kd[:, h // (H // KV)] @ qf[h] / np.sqrt(D)
        p = np.exp(s - s.max()); p /= p.sum()
        want[h] = p @ vd[:, h // (H // KV)]
    assert np.allclose(out, want, rtol=2e-2, atol=2e-3)
    # split into 3 ranges (one empty) + merge == whole
    parts = [orc.kv_attention_partial(q, kq, vq, meta, a, b) for a, b in ((0, 10), (10, 10), (10, T))]
    pm = np.stack([p[0] for p in parts], 1); pl = np.stack([p[1] for p in parts], 1)
    po = np.stack([p[2] for p in parts], 1)
    assert np.isneginf(pm[:, 1]).all() and (pl[:, 1] == 0).all()
    merged = orc.bf16_to_f32(orc.merge_partials(pm, pl, po))
    assert np.allclose(merged, want, rtol=2e-2, atol=2e-3)


def test_fused_producers_known_answers():
    """kernels-cuda/smoke.cu:1187-1215: RMSNorm + quantise of sixteen ones with zero weight gives bf16
    1.0, scale byte 0x23 and codes 0x77.  SwiGLU + quantise equals the plain row quantiser applied
    to the float32 product (same codec), checked on values that are exact in bf16."""
    ones = synth.f32_to_bf16_bits(np.ones(16, np.float32))
    zeros = synth.f32_to_bf16_bits(np.zeros(16, np.float32))
    r = orc.rmsnorm_nvfp4_quantize(ones, zeros, None, 1e-6, 0.0)
    assert np.all(r["fp4"] == 0x77) and r["sf"][0] == 0x23 and r["ts"] == 1.0
    assert np.all(synth.bf16_bits_to_f32(r["out_bf16"]) == 1.0)
    # residual path: input + residual is what gets normalised and what residual_out carries
    half = synth.f32_to_bf16_bits(np.full(16, 0.5, np.float32))
    r2 = orc.rmsnorm_nvfp4_quantize(half, zeros, half, 1e-6, 0.0)
    assert np.array_equal(r2["fp4"], r["fp4"]) and np.array_equal(r2["residual_out"], ones)
    # ragged vector (33 values), global-scale branch
    x = synth.f32_to_bf16_bits(((np.arange(33) % 13) - 6).astype(np.float32) * 0.1875)
    w = synth.f32_to_bf16_bits(np.linspace(-0.5, 0.5, 33).astype(np.float32))
    r3 = orc.rmsnorm_nvfp4_quantize(x, w, None, 1e-6, 1.25)
    assert r3["ts"] == 1.25 and r3["fp4"].shape == (17,) and (r3["fp4"][16] >> 4) == 0
    # swiglu: gate = 0 gives silu = 0 -> all-zero codes and the amax == 0 scale byte 0x38
    g0 = synth.f32_to_bf16_bits(np.zeros(32, np.float32))
    up = synth.f32_to_bf16_bits(np.arange(32, dtype=np.float32))
    s0 = orc.swiglu_nvfp4_quantize(g0, up, 0.0)
    assert np.all(s0["fp4"] == 0) and s0["sf"][0] == 0x38 and s0["sf"][1] == 0x38
    # the codes follow from y exactly as the row quantiser would produce them from bf16(y) when y is exact in bf16
    g = synth.f32_to_bf16_bits(np.full(32, 40.0, np.float32))      # silu(40) == 40 in float32
    s1 = orc.swiglu_nvfp4_quantize(g, up, 0.0)
    want_fp4, want_sf, _ = orc.nvfp4_quantize_rows(synth.f32_to_bf16_bits(40.0 * np.arange(32, dtype=np.float32))[None, :], 0.0)
    assert np.array_equal(s1["fp4"], want_fp4[0]) and np.array_equal(s1["sf"], want_sf)


def planted_logits():
    """The reference's own known-answer construction (kernels-cuda/smoke.cu:202-219): a pattern that
    depends only on the indices, with two planted leaders per row.  Row 0 margin 2.0, row 1 margin 0.25."""
    rows, vocab = 2, 250000
    i = np.arange(vocab, dtype=np.int64)
    logits = np.stack([-2.0 + ((r * 911 + i * 37) % 997).astype(np.float32) / 1000.0 for r in range(rows)]).astype(np.float32)
    logits[0, 123456] = 7.0
    logits[0, 7] = 5.0
    logits[1, 99] = 3.25
    logits[1, vocab - 1] = 3.0
    return synth.f32_to_bf16_bits(logits)


def test_top2_margin_known_answers():
    # kernels-cuda/smoke.cu:237-262
    logits = planted_logits()
    tokens, flags, fb = orc.lm_head_top2_margin(logits, 1.0)
    assert tokens.tolist() == [123456, 99] and flags.tolist() == [1, 0] and fb == 1
    tokens, flags, fb = orc.lm_head_top2_margin(logits, 0.1)
    assert tokens.tolist() == [123456, 99] and flags.tolist() == [1, 1] and fb == 0
    # a tie for first place: lowest index wins, margin 0 fails any positive eps; NaN never wins
    small = synth.f32_to_bf16_bits(np.array([[1.0, 5.0, np.nan, 5.0, -1.0]], np.float32))
    tokens, flags, fb = orc.lm_head_top2_margin(small, 0.5)
    assert tokens.tolist() == [1] and flags.tolist() == [0] and fb == 1
    tokens, flags, _ = orc.lm_head_top2_margin(small, 0.0)
    assert flags.tolist() == [1]


def test_top8_rescore_and_bf16_argmax_small():
    """Float64 rescore of the eight best block winners picks the bf16-exact leader even when the
    (perturbed) first-stage logits rank another token first; the bf16 matvec argmax agrees with a
    float64 dot product wherever the top two are clearly apart, and honours skip flags."""
    rng = np.random.default_rng(3)
    vocab, cols, rows = 3000, 256, 3
    w = synth.f32_to_bf16_bits(rng.standard_normal((vocab, cols)).astype(np.float32))
    x = synth.f32_to_bf16_bits(rng.standard_normal((rows, cols)).astype(np.float32))
    exact = synth.bf16_bits_to_f32(x).astype(np.float64) @ synth.bf16_bits_to_f32(w).astype(np.float64).T
    noisy = exact + rng.standard_normal(exact.shape) * 0.3          # stands in for the FP8 logits
    logits = synth.f32_to_bf16_bits(noisy.astype(np.float32))
    tokens, flags, fb = orc.lm_head_top8_rescore(logits, w, x, 0.5)
    order = np.argsort(-exact, axis=1)
    for r in range(rows):
        # the rescored winner is the best exact logit among the eight candidates; when the guard
        # certifies the row it is the global bf16 argmax
        if flags[r]:
            assert tokens[r] == order[r, 0]
    assert fb == int((flags == 0).sum())
    full = orc.bf16_matvec_argmax_rows(x, w)
    for r in range(rows):
        if exact[r, order[r, 0]] - exact[r, order[r, 1]] > 1e-3:
            assert full[r] == order[r, 0]
    skip = np.array([0, 1, 0], dtype=np.uint32)
    kept = orc.bf16_matvec_argmax_rows(x, w, skip, np.array([11, 22, 33], dtype=np.uint32))
    assert kept[1] == 22 and kept[0] == full[0] and kept[2] == full[2]


def _e4m3_magnitudes():
    """The 127 finite E4M3 magnitudes by the format's definition (code 0x7F excluded)."""
    mags = []
    for code in range(0x7F):
        e, m = code >> 3, code & 7
        mags.append(m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7))
    return np.array(mags, np.float64)


def test_kv_cache_e4m3_codec_all_values():
    """The FP8 KV cache codec (kernels-cuda/attention.cu:101-160) against the format's definition:
    decode of all 256 bytes (0x7F / 0xFF read as +-448), and the append's encoder on every bf16 bit
    pattern: nearest magnitude with ties going UP, saturation at 0x7E, zero and non-finite -> 0."""
    mags = _e4m3_magnitudes()
    for code in range(256):
        want = 448.0 if (code & 0x7F) == 0x7F else mags[code & 0x7F]
        got = orc.kv_e4m3_decode(code)
        assert got == (-want if code & 0x80 else want), code
    bits = np.arange(65536, dtype=np.uint16)
    vals = synth.bf16_bits_to_f32(bits)
    mids = (mags[:-1] + mags[1:]) / 2
    for b, v in zip(bits.tolist(), vals.tolist()):
        got = orc.kv_e4m3_encode(v)
        if v == 0 or not np.isfinite(v):
            want = 0
        else:
            a = abs(v)
            idx = 0x7E if a >= 448 else int(np.searchsorted(mids, a, side="right"))   # a == midpoint -> upper code
            want = (0x80 if v < 0 else 0) | idx
        assert got == want, (hex(b), v, got, want)


def _decode_case(position, q_val, k_val, v_val, ck_val, cv_val, fp8=False):
    """The reference's smoke shape (kernels-cuda/smoke.cu:508-532): 2 q heads, 1 kv head, 8 dims."""
    q = synth.f32_to_bf16_bits(np.full((2, 8), q_val, np.float32))
    k = synth.f32_to_bf16_bits(np.full((1, 8), k_val, np.float32))
    v = synth.f32_to_bf16_bits(np.full((1, 8), v_val, np.float32))
    if fp8:
        ck = np.full((position + 1, 1, 8), orc.kv_e4m3_encode(ck_val), np.uint8)
        cv = np.full((position + 1, 1, 8), orc.kv_e4m3_encode(cv_val), np.uint8)
    else:
        ck = synth.f32_to_bf16_bits(np.full((position + 1, 1, 8), ck_val, np.float32))
        cv = synth.f32_to_bf16_bits(np.full((position + 1, 1, 8), cv_val, np.float32))
    return q, k, v, ck, cv


def test_attention_decode_known_answers():
    # kernels-cuda/smoke.cu:519-532: position 0 -> the output is v_new and row 0 of the cache is k / v
    q, k, v, ck, cv = _decode_case(0, 0.25, 0.5, 1.0, 0.0, 0.0)
    out = synth.bf16_bits_to_f32(orc.attention_decode(q, k, v, ck, cv, 0, 0))
    assert np.all(out == 1.0) and np.array_equal(ck[0], k) and np.array_equal(cv[0], v)
    # kernels-cuda/smoke.cu:619-650: 513 cached rows of K = 0.5, V = 1.0 -> 1.0 +- 0.02
    q, k, v, ck, cv = _decode_case(513, 0.25, 0.5, 1.0, 0.5, 1.0)
    out = synth.bf16_bits_to_f32(orc.attention_decode(q, k, v, ck, cv, 0, 513))
    assert np.all(np.abs(out - 1.0) <= 0.02)
    # kernels-cuda/smoke.cu:546-566: one cached row (K 0.25, V 0.75) + the new row (0.5, 1.0)
    for fp8 in (False, True):
        q, k, v, ck, cv = _decode_case(1, 0.25, 0.5, 1.0, 0.25, 0.75, fp8)
        before = ck[0].copy()
        out = synth.bf16_bits_to_f32(orc.attention_decode(q, k, v, ck, cv, int(fp8), 1))
        s_old, s_new = 8 * 0.25 * 0.25 / np.sqrt(8), 8 * 0.25 * 0.5 / np.sqrt(8)
        want = (np.exp(s_old) * 0.75 + np.exp(s_new) * 1.0) / (np.exp(s_old) + np.exp(s_new))
        assert np.all(np.abs(out - want) <= 4e-3)
        assert np.array_equal(ck[0], before)
        if fp8:
            assert np.all(ck[1] == 0x30) and np.all(cv[1] == 0x38)      # 0.5 and 1.0 in E4M3
        else:
            assert np.array_equal(ck[1], k) and np.array_equal(cv[1], v)
