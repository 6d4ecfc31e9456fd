// Scalar arithmetic of the per-token-group quantiser, shared by the device kernels and by the
// host-side exhaustive check (tests/csrc/check_quant_math.cpp compiles this header with g++).
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define SGLB_HD __host__ __device__ __forceinline__
#else
#include <math.h>
#define SGLB_HD inline
#endif

namespace sglb {

SGLB_HD float bits_to_float(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}
SGLB_HD uint32_t float_to_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
#endif
}

SGLB_HD float div_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fdiv_rn(a, b);
#else
  return a / b;
#endif
}
SGLB_HD float rcp_rn(float a) {
#if defined(__CUDA_ARCH__)
  return __frcp_rn(a);
#else
  return 1.0f / a;
#endif
}
SGLB_HD float fma_rn(float a, float b, float c) {
#if defined(__CUDA_ARCH__)
  return __fmaf_rn(a, b, c);
#else
  return fmaf(a, b, c);
#endif
}

// Scale of one group from its absolute maximum: amax / fp8_max as an IEEE division, and for the
// power-of-two variant the smallest power of two that is >= that quotient (taken from the bits
// of the quotient, so 7 * 2^k / 448 stays exactly 2^(k-6)).
SGLB_HD float group_scale(float amax, float fp8_max, bool ue8m0) {
  float s = div_rn(amax, fp8_max);
  if (ue8m0) {
    uint32_t u = float_to_bits(s);
    uint32_t e = (u >> 23) & 0xffu;
    if (e == 0) {
      e = 1;  // sub-normal quotient: clamp to the smallest normal power of two
    } else if (u & 0x7fffffu) {
      e += 1;
    }
    s = bits_to_float(e << 23);
  }
  return s;
}

SGLB_HD float mul_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);
#else
  return a * b;
#endif
}

// group_scale without the division routine: with c = RN(1 / fp8_max), q0 = amax*c,
// rem = amax - q0*fp8_max (exact, one FMA), s = q0 + rem*c is the correctly rounded quotient
// whenever it is a normal number (checked on the host for fp8_max = 448 over every 16-bit-float
// amax and a long run of random fp32 ones); tiny maxima, which need eps < 2^-100, take the division.
SGLB_HD float group_scale_fast(float amax, float fp8_max, float inv_max, bool ue8m0) {
  float s;
  if (amax >= 7.888609e-31f) {
    const float q0 = mul_rn(amax, inv_max);
    const float rem = fma_rn(-q0, fp8_max, amax);
    s = fma_rn(rem, inv_max, q0);
  } else {
    s = div_rn(amax, fp8_max);
  }
  if (ue8m0) {
    uint32_t u = float_to_bits(s);
    uint32_t e = (u >> 23) & 0xffu;
    if (e == 0) {
      e = 1;
    } else if (u & 0x7fffffu) {
      e += 1;
    }
    s = bits_to_float(e << 23);
  }
  return s;
}

// The divisor is shared by a whole group, so the per-element quotient uses one correctly
// rounded reciprocal and two FMAs (a Markstein step): q0 = x*r; rem = x - q0*s; q = q0 + rem*r.
// For s in [2^-100, 2^100] and 16-bit-float x this equals RN(x / s) wherever the e4m3 result
// is not zero (checked exhaustively on the host); outside that range fall back to the division.
struct GroupDivisor {
  float s;
  float r;
  bool fast;
};
SGLB_HD GroupDivisor make_divisor(float s, bool allow_fast) {
  GroupDivisor d;
  d.s = s;
  d.fast = allow_fast && (s >= 7.888609e-31f) && (s <= 1.2676506e30f);
  d.r = rcp_rn(s);
  return d;
}
SGLB_HD float quotient(float x, const GroupDivisor& d) {
  if (d.fast) {
    float q0 = mul_rn(x, d.r);
    float rem = fma_rn(-q0, d.s, x);
    float q = fma_rn(rem, d.r, q0);
    // s > 0, so the quotient carries x's sign; restoring it keeps -0 / s = -0 (the FMA chain gives +0)
    return bits_to_float((float_to_bits(q) & 0x7fffffffu) | (float_to_bits(x) & 0x80000000u));
  }
  return div_rn(x, d.s);
}

}  // namespace sglb
