// Arithmetic shared verbatim by the CUDA kernels and the C++ CPU library, so that decisions
// which must agree bit for bit on both sides (which token a sampler picks, where a top-p
// cut falls) are taken from identical numbers. Only IEEE-754 operations that round the same
// way on host and device are used: +, *, fma, float<->int conversion.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define KA_HD __host__ __device__ __forceinline__
#else
#define KA_HD inline
#endif

namespace ka {

KA_HD float bits_to_float(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  std::memcpy(&f, &u, 4);
  return f;
#endif
}

KA_HD uint32_t float_to_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
#endif
}

KA_HD float fma_rn(float a, float b, float c) {
#if defined(__CUDA_ARCH__)
  return __fmaf_rn(a, b, c);
#else
  return std::fmaf(a, b, c);
#endif
}

KA_HD float mul_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);
#else
  return a * b;
#endif
}

KA_HD float sub_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fsub_rn(a, b);
#else
  return a - b;
#endif
}

// Order-preserving map from float to uint32: a < b  <=>  key(a) < key(b). NaN sorts lowest.
KA_HD uint32_t float_to_key(float f) {
  if (f != f) return 0u;
  const uint32_t u = float_to_bits(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

KA_HD float key_to_float(uint32_t k) {
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return bits_to_float(u);
}

// exp(d) for d <= 0, reproducible across host and device (about 2 ulp).
// 2^t with t = d * log2(e): split t into a rounded integer and a fraction in [-0.5, 0.5],
// degree-6 polynomial for 2^fraction, exponent added by integer arithmetic on the bits.
KA_HD float exp_det(float d) {
  const float t = mul_rn(d, 1.4426950408889634f);
  if (!(t > -125.0f)) return 0.0f;  // also catches -inf and NaN
  if (t >= 0.0f) return 1.0f;
  const float n = rintf(t);
  const float f = sub_rn(t, n);
  float p = 1.5403530393381609e-4f;
  p = fma_rn(p, f, 1.3333558146428443e-3f);
  p = fma_rn(p, f, 9.6181291076284772e-3f);
  p = fma_rn(p, f, 5.5504108664821580e-2f);
  p = fma_rn(p, f, 2.4022650695910071e-1f);
  p = fma_rn(p, f, 6.9314718055994531e-1f);
  p = fma_rn(p, f, 1.0f);
  const int e = static_cast<int>(n);
  const uint32_t scale_bits = static_cast<uint32_t>(e + 127) << 23;
  return mul_rn(p, bits_to_float(scale_bits));
}

// Probability mass as a 32.32-style fixed-point integer: sums of these are exact and
// independent of the order of addition, which makes parallel reductions reproducible.
KA_HD uint64_t mass_fixed(float e) {
  // e in [0, 1]; e * 2^32 is exact in float (power-of-two scaling), truncation is exact too
  return static_cast<uint64_t>(e * 4294967296.0f);
}

// floor(frac * total) for frac in [0, 1], identical on host and device (IEEE double).
KA_HD uint64_t mass_fraction(double frac, uint64_t total) {
  const double v = frac * static_cast<double>(total);
  if (!(v > 0.0)) return 0;
  const uint64_t r = static_cast<uint64_t>(v);
  return r > total ? total : r;
}

// floor(u24 * total / 2^24) without overflowing 64 bits.
KA_HD uint64_t mass_scale_u24(uint32_t u24, uint64_t total) {
  const uint64_t hi = (total >> 24) * u24;
  const uint64_t lo = ((total & 0xFFFFFFull) * u24) >> 24;
  return hi + lo;
}

// Philox4x32-10 counter-based generator. Counter = (row id lo, row id hi, step lo, step hi),
// key = (seed lo, seed hi): the draw for a row depends only on (seed, row id, step), never on
// the batch the row was sampled in.
struct Philox4 {
  uint32_t x, y, z, w;
};

KA_HD void philox_mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
  const uint64_t p = static_cast<uint64_t>(a) * b;
  hi = static_cast<uint32_t>(p >> 32);
  lo = static_cast<uint32_t>(p);
}

KA_HD Philox4 philox4x32_10(uint64_t seed, uint64_t row, uint64_t step) {
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  Philox4 c{static_cast<uint32_t>(row), static_cast<uint32_t>(row >> 32), static_cast<uint32_t>(step),
            static_cast<uint32_t>(step >> 32)};
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    philox_mulhilo(0xD2511F53u, c.x, hi0, lo0);
    philox_mulhilo(0xCD9E8D57u, c.z, hi1, lo1);
    Philox4 n{hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0};
    c = n;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c;
}

// 24 uniform bits for (seed, row, step).
KA_HD uint32_t uniform_u24(uint64_t seed, uint64_t row, uint64_t step) {
  return philox4x32_10(seed, row, step).x >> 8;
}

}  // namespace ka
