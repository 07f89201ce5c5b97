// The arithmetic of one NVFP4 group (16 float32 values -> 8 code bytes + one UE4M3 scale byte), shared
// by the row quantiser and the fused producers that quantise rows.  Bit for bit the reference's
// rule (kernels-cuda/ops.cu:81-139, 704-761: scale = amax / (6 g) in IEEE float32, UE4M3 ties
// down, IEEE division by the decoded scale, E2M1 ties toward zero) by the branch-free route where
// that is provably the same and by the reference's own arithmetic elsewhere.
#pragma once
#include "common.cuh"

namespace q36 {

// x: the group; amax: max |x| with NaNs ignored (fmaxf from 0); any_nonzero: some value is not +-0
// (NaN counts); g: tensor scale (> 0), six_g = 6 g, rcp6 = 1 / six_g, both correctly rounded.
// force_exact: take the reference's divisions for the codes whatever the scale (callers whose values are
// not bf16 pass it for groups holding magnitudes below 2^-96, whose quotients may underflow: there
// the multiplication by a reciprocal and the division can fall on different sides of zero).
// lo / hi: codes of values 0..7 / 8..15, low nibble first.
__device__ __forceinline__ void nvfp4_quantize_group(const float (&x)[16], float amax, bool any_nonzero,
                                                     bool force_exact, float g, float six_g, float rcp6,
                                                     uint32_t &lo, uint32_t &hi, uint32_t &sf_code) {
  lo = 0u;
  hi = 0u;
  if (amax > 0.0f) {
    // sv = max(amax / (6 g), 1e-8)
    float sv = __fmul_rn(amax, rcp6);
    sv = fmaf(fmaf(-sv, six_g, amax), rcp6, sv);
    const uint32_t sbits = __float_as_uint(sv);
    const bool scale_fast = sv >= 0x1p-6f && sv < 448.0f;
    if (!scale_fast || ((sbits + 2u - 0x80000u) & 0xfffffu) < 5u) sv = __fdiv_rn(amax, six_g);   // also when sv is not finite
    sv = fmaxf(sv, 1.0e-8f);
    float dec;
    if (scale_fast) {
      sf_code = min(((__float_as_uint(sv) + 0x7ffffu) >> 20) - 960u, 0x7eu);
      dec = __uint_as_float((sf_code << 20) + 0x3c000000u);
    } else {
      sf_code = q36::encode_ue4m3(sv);
      dec = q36::decode_e4m3(sf_code);
    }
    const float ds = fmaxf(__fmul_rn(dec, g), 1.0e-8f);
    // ds with an all-ones mantissa is the one case in which reciprocal + two FMAs may miss the
    // correctly rounded quotient; a very large ds could underflow a negative quotient to -0
    const bool exact = force_exact || !scale_fast || sf_code < 8u || ds > 65536.0f || (__float_as_uint(ds) & 0x7fffffu) == 0x7fffffu;
    if (!exact) {
      const float rcp = __frcp_rn(ds), nds = -ds;
      // Four pairs per word: x * rcp (within 2 ulps of the IEEE quotient) through the hardware
      // e2m1x2 conversion.  That is the reference's code unless the quotient lies within 2 ulps of
      // a value with at most three significant bits: all seven rounding boundaries are such values
      // (the approximate quotient may sit on the wrong side of one, and the hardware breaks exact
      // ties to even where the reference breaks them toward zero: 0.75, 1.75, 3.5), and so is -0,
      // which the reference encodes as +0.  One masked compare per pair finds these; the pair is
      // then redone from the correctly rounded quotient (reciprocal + two FMAs, Markstein).  Exactly
      // representable quotients are common, about 0.2 % of all values when bf16 inputs meet a short
      // scale, so this patch stays per pair: redoing whole groups would put most warps on it.
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = __fmul_rn(x[8 * h + i], rcp);
        uint32_t word;
        asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t"
            "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n\t"
            "cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n\t"
            "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n\t"
            "cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n\t"
            "mov.b32 %0, {t0, t1, t2, t3};\n\t}"
            : "=r"(word)
            : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t b0 = __float_as_uint(q[2 * i]), b1 = __float_as_uint(q[2 * i + 1]);
          if (min((b0 + 2u) & 0x001ffffcu, (b1 + 2u) & 0x001ffffcu) == 0u) {
            const float x0 = x[8 * h + 2 * i], x1 = x[8 * h + 2 * i + 1];
            const float e0 = fmaf(fmaf(q[2 * i], nds, x0), rcp, q[2 * i]);
            const float e1 = fmaf(fmaf(q[2 * i + 1], nds, x1), rcp, q[2 * i + 1]);
            uint32_t byte;
            asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}"
                : "=r"(byte) : "f"(e1), "f"(e0));
            const uint32_t a0 = __float_as_uint(e0) & 0x7fffffffu, a1 = __float_as_uint(e1) & 0x7fffffffu;
            if (a0 == 0x3f400000u || a0 == 0x3fe00000u || a0 == 0x40600000u) byte -= 1u;
            if (a1 == 0x3f400000u || a1 == 0x3fe00000u || a1 == 0x40600000u) byte -= 16u;
            if (a0 == 0u) byte &= 0xf0u;
            if (a1 == 0u) byte &= 0x0fu;
            word = (word & ~(0xffu << (8 * i))) | (byte << (8 * i));
          }
        }
        if (h == 0) lo = word; else hi = word;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        lo |= q36::encode_e2m1x2(__fdiv_rn(x[2 * i], ds), __fdiv_rn(x[2 * i + 1], ds)) << (8 * i);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        hi |= q36::encode_e2m1x2(__fdiv_rn(x[8 + 2 * i], ds), __fdiv_rn(x[9 + 2 * i], ds)) << (8 * i);
    }
  } else {
    // amax is 0 (all zeros) or every value is NaN (fmaxf never picks NaN): the reference's scale is
    // 1.0 either way; zeros encode to 0, NaNs to +6
    sf_code = 0x38u;
    if (any_nonzero) {
#pragma unroll
      for (int i = 0; i < 4; ++i) lo |= q36::encode_e2m1x2(x[2 * i], x[2 * i + 1]) << (8 * i);
#pragma unroll
      for (int i = 0; i < 4; ++i) hi |= q36::encode_e2m1x2(x[8 + 2 * i], x[9 + 2 * i]) << (8 * i);
    }
  }
}

}  // namespace q36
