// Scalar numerics shared by the CUDA routing kernels and the host code (and, through an
// include, by the CPU oracle that checks them): exp/sigmoid with a fixed operation sequence
// that is bit-identical under g++ and nvcc, the fp8/fp4/bf16 codecs, and the NVFP4 / FP8
// quantiser primitives.
//
// Why a private exp: routing weights must be bit-equal between the device and the CPU
// check.  The reference (crates/colibri-engine/src/moe.rs:1066, math.rs:122-132) calls Rust
// std `f32::exp`, i.e. the platform libm, which cannot be linked into a device kernel.
// `coli_expf` evaluates exp in f64 with explicit fma steps (IEEE on both sides, so the f64
// result is the same bit pattern on host and device) and rounds once to f32; the f64 result
// is accurate to <1e-15 relative, so the f32 value is the correctly rounded one except in
// ~1e-8 of inputs — the same value a correctly rounded libm expf returns.
//
// Every f32 operation that must not be contracted or reordered is spelled through the
// CF_* wrappers: on the device they are the round-to-nearest intrinsics (never fused by
// nvcc), on the host they are plain operators and the translation unit is compiled with
// -ffp-contract=off.
#ifndef COLI_MATH_H
#define COLI_MATH_H

#include <stdint.h>
#include <string.h>
#include <math.h>

#if defined(__CUDACC__)
#define CF_HD __host__ __device__ __forceinline__
#else
#define CF_HD static inline
#endif

#if defined(__CUDA_ARCH__)
#define CF_ADD(a, b) __fadd_rn((a), (b))
#define CF_SUB(a, b) __fsub_rn((a), (b))
#define CF_MUL(a, b) __fmul_rn((a), (b))
#define CF_DIV(a, b) __fdiv_rn((a), (b))
#define CF_DFMA(a, b, c) __fma_rn((a), (b), (c))
#define CF_DMUL(a, b) __dmul_rn((a), (b))
#else
#define CF_ADD(a, b) ((a) + (b))
#define CF_SUB(a, b) ((a) - (b))
#define CF_MUL(a, b) ((a) * (b))
#define CF_DIV(a, b) ((a) / (b))
#define CF_DFMA(a, b, c) fma((a), (b), (c))
#define CF_DMUL(a, b) ((a) * (b))
#endif

CF_HD uint32_t cf_f32_bits(float v) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(v);
#else
  uint32_t u;
  memcpy(&u, &v, 4);
  return u;
#endif
}
CF_HD float cf_bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float v;
  memcpy(&v, &u, 4);
  return v;
#endif
}
CF_HD double cf_bits_f64(uint64_t u) {
#if defined(__CUDA_ARCH__)
  return __longlong_as_double((long long)u);
#else
  double v;
  memcpy(&v, &u, 8);
  return v;
#endif
}

// exp(x) for f32 x, evaluated in f64 and rounded once.  n = rint(x*log2e); r = x - n*ln2 in
// two fma steps (hi/lo split of ln2); Taylor polynomial of degree 13 by Horner with fma
// (|r| <= 0.3466, truncation error 1.7e-16); scale by 2^n built from exponent bits.
CF_HD float coli_expf(float xf) {
  if (xf != xf) return xf;
  if (xf > 88.8f) return cf_bits_f32(0x7f800000u);  // +inf; the f64->f32 round gives inf above 88.7228
  if (xf < -104.0f) return 0.0f;                    // below half the smallest f32 subnormal
  const double x = (double)xf;
  const double n = rint(CF_DMUL(x, 1.4426950408889634074));
  double r = CF_DFMA(n, -6.93147180369123816490e-01, x);
  r = CF_DFMA(n, -1.90821492927058770002e-10, r);
  double p = 1.0 / 6227020800.0;
  p = CF_DFMA(p, r, 1.0 / 479001600.0);
  p = CF_DFMA(p, r, 1.0 / 39916800.0);
  p = CF_DFMA(p, r, 1.0 / 3628800.0);
  p = CF_DFMA(p, r, 1.0 / 362880.0);
  p = CF_DFMA(p, r, 1.0 / 40320.0);
  p = CF_DFMA(p, r, 1.0 / 5040.0);
  p = CF_DFMA(p, r, 1.0 / 720.0);
  p = CF_DFMA(p, r, 1.0 / 120.0);
  p = CF_DFMA(p, r, 1.0 / 24.0);
  p = CF_DFMA(p, r, 1.0 / 6.0);
  p = CF_DFMA(p, r, 0.5);
  p = CF_DFMA(p, r, 1.0);
  p = CF_DFMA(p, r, 1.0);
  const int64_t ni = (int64_t)n;  // |n| <= 151, 2^n is a normal f64
  const double s = cf_bits_f64((uint64_t)(ni + 1023) << 52);
  return (float)CF_DMUL(p, s);
}

// 1/(1+exp(-x)) — crates/colibri-engine/src/math.rs:122-125.
CF_HD float coli_sigmoidf(float x) { return CF_DIV(1.0f, CF_ADD(1.0f, coli_expf(-x))); }

// x/(1+exp(-x)) — crates/colibri-engine/src/math.rs:129-132.
CF_HD float coli_siluf(float x) { return CF_DIV(x, CF_ADD(1.0f, coli_expf(-x))); }

// Gate/up combine of one element under the process-wide activation setting
// (crates/colibri-backend/cuda/backend_cuda.cu:380-392 selects the same three ways):
//   oai != 0            clamped OpenAI-SwiGLU, crates/colibri-engine/src/math.rs:143-148:
//                       g = min(gate, limit), u = clamp(up, -limit, limit),
//                       out = g / (1 + exp(-alpha g)) * (u + 1)
//   oai == 0, limit > 0 SwiGLU under the asymmetric clamp, crates/colibri-engine/src/dsv4.rs:738-742:
//                       out = silu(min(gate, limit)) * clamp(up, -limit, limit)
//   otherwise           plain SwiGLU, silu(gate) * up (moe.rs:1187-1230)
CF_HD float coli_act_combine(float gate, float up, int oai, float alpha, float limit) {
  if (oai) {
    const float g = gate < limit ? gate : limit;
    const float u = up < -limit ? -limit : (up > limit ? limit : up);
    return CF_MUL(CF_DIV(g, CF_ADD(1.0f, coli_expf(-CF_MUL(alpha, g)))), CF_ADD(u, 1.0f));
  }
  if (limit > 0.0f) {
    const float g = gate < limit ? gate : limit;
    const float u = up < -limit ? -limit : (up > limit ? limit : up);
    return CF_MUL(coli_siluf(g), u);
  }
  return CF_MUL(coli_siluf(gate), up);
}

// bf16 <-> f32 — crates/colibri-core/src/dtype.rs:165-194 (RNE, NaN kept a NaN).
CF_HD float coli_bf16_to_f32(uint16_t h) { return cf_bits_f32((uint32_t)h << 16); }
CF_HD uint16_t coli_f32_to_bf16(float v) {
  const uint32_t bits = cf_f32_bits(v);
  if (v != v) return (uint16_t)((bits >> 16) | 0x0040u);
  const uint32_t rounded = bits + 0x7fffu + ((bits >> 16) & 1u);
  return (uint16_t)(rounded >> 16);
}

// e4m3 (OCP e4m3fn) decode — crates/colibri-engine/src/linear.rs:188-197.  Codes 0x7F/0xFF
// (NaN in the container format) decode as 480 here exactly as that arm does; the quantisers
// below never emit them.
CF_HD float coli_e4m3_to_f32(uint8_t b) {
  const uint32_t e = (b >> 3) & 0x0fu;
  const uint32_t m = b & 0x07u;
  uint32_t bits;
  if (e == 0) {
    // subnormal m * 2^-9: exact via integer -> float, then exponent shift
    const float v = (float)m * (1.0f / 512.0f);
    bits = cf_f32_bits(v);
  } else {
    bits = ((e - 7u + 127u) << 23) | (m << 20);
  }
  return cf_bits_f32(bits | ((uint32_t)(b & 0x80u) << 24));
}

// f32 -> e4m3, round-to-nearest-even on the mantissa, saturate to 448, NaN/0 -> signed zero —
// crates/colibri-engine/src/convert.rs:1006-1036.  The exponent is taken from the f32 bits
// (exact) where that code takes floor(log2(a)); the two agree on every input because an `a`
// that log2 misplaces by one binade is within 1 ulp of a power of two, which either choice
// encodes as that power of two.
CF_HD uint8_t coli_f32_to_e4m3(float x) {
  const uint32_t xb = cf_f32_bits(x);
  const uint8_t sign = (uint8_t)((xb >> 24) & 0x80u);
  const float a = cf_bits_f32(xb & 0x7fffffffu);
  if (!(a > 0.0f)) return sign;
  if (a >= 448.0f) return (uint8_t)(sign | 0x7Eu);
  int e = (int)((xb >> 23) & 0xffu) - 127;  // floor(log2 a) for normal a; subnormal f32 gives -127
  if (e < -6) {
    int m = (int)rintf(CF_MUL(a, 512.0f));
    if (m >= 8) return (uint8_t)(sign | 0x08u);
    if (m < 0) m = 0;
    return (uint8_t)(sign | (uint8_t)m);
  }
  const float scale = cf_bits_f32((uint32_t)(127 - e) << 23);  // 2^-e, e in [-6, 8]
  int m = (int)rintf(CF_MUL(CF_SUB(CF_MUL(a, scale), 1.0f), 8.0f));
  int eb = e + 7;
  if (m >= 8) {
    m = 0;
    eb += 1;
  }
  if (eb >= 15 && m > 6) return (uint8_t)(sign | 0x7Eu);
  return (uint8_t)(sign | (uint8_t)(eb << 3) | (uint8_t)(m & 7));
}

// E2M1 magnitude levels — crates/colibri-engine/src/convert.rs:1631, linear.rs:182-184.
CF_HD float coli_e2m1_level(int idx) {
  // 0, .5, 1, 1.5, 2, 3, 4, 6 without a memory table (usable in device code)
  const uint32_t packed[8] = {0x00000000u, 0x3f000000u, 0x3f800000u, 0x3fc00000u,
                              0x40000000u, 0x40400000u, 0x40800000u, 0x40c00000u};
  return cf_bits_f32(packed[idx & 7]);
}
CF_HD float coli_e2m1_to_f32(uint8_t nib) {
  const float v = coli_e2m1_level(nib & 7);
  return (nib & 8) ? -v : v;
}

// Nearest E2M1 code, first minimum wins a tie — crates/colibri-engine/src/convert.rs:1078-1090.
CF_HD uint8_t coli_e2m1_code(float t) {
  const float a = fabsf(t);
  int best = 0;
  float bd = cf_bits_f32(0x7f800000u);
  for (int idx = 0; idx < 8; ++idx) {
    const float d = fabsf(CF_SUB(a, coli_e2m1_level(idx)));
    if (d < bd) {
      bd = d;
      best = idx;
    }
  }
  return (uint8_t)(((cf_f32_bits(t) >> 31) ? 8u : 0u) | (uint32_t)best);
}

// NVFP4 per-tensor scale from the tensor's absolute maximum —
// crates/colibri-engine/src/convert.rs:1108-1109 (amax/(6*448), floored at f32::MIN_POSITIVE).
CF_HD float coli_nvfp4_global(float amax) {
  const float g = CF_DIV(amax, CF_MUL(6.0f, 448.0f));
  const float tiny = cf_bits_f32(0x00800000u);
  return g > tiny ? g : tiny;
}
// Block-scale code for a 16-wide block with absolute maximum bmax —
// crates/colibri-engine/src/convert.rs:1119-1120.
CF_HD uint8_t coli_nvfp4_block_code(float bmax, float global) {
  return coli_f32_to_e4m3(CF_DIV(CF_DIV(bmax, 6.0f), global));
}
// Nibble for one weight given its block's code — crates/colibri-engine/src/convert.rs:1122-1124.
CF_HD uint8_t coli_nvfp4_nibble(float v, uint8_t code, float global) {
  const float eff = CF_MUL(coli_e4m3_to_f32(code), global);
  return eff > 0.0f ? coli_e2m1_code(CF_DIV(v, eff)) : (uint8_t)0;
}

// FP8 with one f32 scale per 128x128 block.  The reference only DEcodes this form
// (crates/colibri-engine/src/convert.rs:731-741: W = e4m3 * scale[block]); the encoder is
// defined here: scale = amax/448 (1.0 for an all-zero block), code = e4m3(w * (1/scale)),
// the same rule as the per-row quantiser at convert.rs:1042-1054 applied per block.
CF_HD float coli_fp8_block_scale(float amax) { return amax > 0.0f ? CF_DIV(amax, 448.0f) : 1.0f; }
CF_HD uint8_t coli_fp8_block_code(float v, float scale) {
  return coli_f32_to_e4m3(CF_MUL(v, CF_DIV(1.0f, scale)));
}

#endif  // COLI_MATH_H
