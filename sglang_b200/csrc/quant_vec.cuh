// Vector arithmetic of the per-token-group quantiser that more than one kernel uses: the element traits of the
// input types, the packed quotient step and the e4m3 pair conversion (device only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "quant_math.cuh"

namespace sglb {

// ---- element traits: E = elements per 16-byte vector -----------------------------------------
template <typename T>
struct Elem;

template <>
struct Elem<__nv_bfloat16> {
  static constexpr int E = 8;
  // |.| maximum over the 8 packed values of a vector, as fp32
  static __device__ __forceinline__ float vec_absmax(const uint4& u) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    __nv_bfloat162 m = __hmax2(__habs2(h[0]), __habs2(h[1]));
    m = __hmax2(m, __hmax2(__habs2(h[2]), __habs2(h[3])));
    const float2 f = __bfloat1622float2(m);
    return fmaxf(f.x, f.y);
  }
  static __device__ __forceinline__ float2 pair(uint32_t w) {  // two bf16 -> two fp32 (exact)
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  }
  static __device__ __forceinline__ uint32_t sign_bytes(uint32_t w0, uint32_t w1) {  // bytes 1,3 of each word
    return __byte_perm(w0, w1, 0x7531);
  }
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

template <>
struct Elem<__half> {
  static constexpr int E = 8;
  static __device__ __forceinline__ float vec_absmax(const uint4& u) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
    __half2 m = __hmax2(__habs2(h[0]), __habs2(h[1]));
    m = __hmax2(m, __hmax2(__habs2(h[2]), __habs2(h[3])));
    const float2 f = __half22float2(m);
    return fmaxf(f.x, f.y);
  }
  static __device__ __forceinline__ float2 pair(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
  }
  static __device__ __forceinline__ uint32_t sign_bytes(uint32_t w0, uint32_t w1) {
    return __byte_perm(w0, w1, 0x7531);
  }
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

template <>
struct Elem<float> {
  static constexpr int E = 4;
  static __device__ __forceinline__ float vec_absmax(const uint4& u) {
    return fmaxf(fmaxf(fabsf(__uint_as_float(u.x)), fabsf(__uint_as_float(u.y))),
                 fmaxf(fabsf(__uint_as_float(u.z)), fabsf(__uint_as_float(u.w))));
  }
  static __device__ __forceinline__ float round(float x) { return x; }
};

__device__ __forceinline__ float silu_f32(float x) { return __fdiv_rn(x, 1.0f + expf(-x)); }

// Two quotients x / s with the shared reciprocal r = RN(1/s): packed Markstein step.
__device__ __forceinline__ float2 quotient2(float2 x, float2 rr, float2 neg_ss) {
  const float2 q0 = __fmul2_rn(x, rr);
  const float2 rem = __ffma2_rn(q0, neg_ss, x);
  return __ffma2_rn(rem, rr, q0);
}

__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}

// Sixteen consecutive 16-bit inputs (two 16-byte vectors) divided by the group's scale and converted to e4m3 with the
// e4m3 limits (the saturating conversion clamps): the same operations, in the same order, as group_quant16_kernel.
template <typename T>
__device__ __forceinline__ uint4 encode16_e4m3(const uint4& v0, const uint4& v1, float s) {
  const bool fast = (s >= 7.888609e-31f) && (s <= 1.2676506e30f);
  const float r = __frcp_rn(s);
  const float2 rr = make_float2(r, r), nss = make_float2(-s, -s);
  uint32_t packed[4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(h == 0 ? &v0 : &v1);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float2 qa, qb;
      const float2 xa = Elem<T>::pair(w[2 * j]), xb = Elem<T>::pair(w[2 * j + 1]);
      if (fast) {
        qa = quotient2(xa, rr, nss);
        qb = quotient2(xb, rr, nss);
      } else {
        qa = make_float2(__fdiv_rn(xa.x, s), __fdiv_rn(xa.y, s));
        qb = make_float2(__fdiv_rn(xb.x, s), __fdiv_rn(xb.y, s));
      }
      const uint32_t codes = cvt_e4m3x2(qa.x, qa.y) | (cvt_e4m3x2(qb.x, qb.y) << 16);
      const uint32_t signs = Elem<T>::sign_bytes(w[2 * j], w[2 * j + 1]);
      packed[2 * h + j] = (codes & 0x7f7f7f7fu) | (signs & 0x80808080u);
    }
  }
  return make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

}  // namespace sglb
