// Host-side exhaustive check of the group quotient used by the quantiser: for every finite
// positive 16-bit-float amax and every same-format x with |x| <= amax, the two-FMA quotient of
// sglang_b200/csrc/quant_math.cuh must give the same e4m3 code as the IEEE division x / s.
// Usage: check_quant_math <bf16|f16> <stride>   (stride 1 = every amax; larger = sample)
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include "../../sglang_b200/csrc/quant_math.cuh"

static float from16(uint16_t h, bool bf16) {
  if (bf16) return sglb::bits_to_float((uint32_t)h << 16);
  uint32_t s = (h >> 15) & 1, e = (h >> 10) & 0x1f, m = h & 0x3ff;
  float v;
  if (e == 0) v = ldexpf((float)m, -24);
  else if (e == 31) v = m ? NAN : INFINITY;
  else v = ldexpf((float)(m | 0x400), (int)e - 25);
  return s ? -v : v;
}

// fp32 -> e4m3 (fn variant), round to nearest even, saturating to +-448.
static uint8_t to_e4m3(float f) {
  uint32_t u = sglb::float_to_bits(f);
  uint8_t sign = (u >> 24) & 0x80;
  float a = fabsf(f);
  if (a != a) return sign | 0x7f;
  if (a >= 448.0f) return sign | 0x7e;
  if (a < ldexpf(1.0f, -6)) {  // sub-normal target: multiples of 2^-9
    float r = nearbyintf(a * 512.0f);
    return sign | (uint8_t)r;  // r in 0..8; 8 encodes the smallest normal
  }
  int e;
  float m = frexpf(a, &e);          // a = m * 2^e, m in [0.5, 1)
  float r = nearbyintf(m * 16.0f);  // 4 significant bits
  if (r == 16.0f) { r = 8.0f; e += 1; }
  int be = e - 1 + 7;
  uint8_t code = (uint8_t)((be << 3) | ((int)r - 8));
  return sign | (code > 0x7e ? 0x7e : code);
}

int main(int argc, char** argv) {
  bool bf16 = argc < 2 || strcmp(argv[1], "bf16") == 0;
  int stride = argc > 2 ? atoi(argv[2]) : 1;
  unsigned top = bf16 ? 0x7f80u : 0x7c00u;
  long long bad_code = 0, bad_f32 = 0, n = 0, n_fast = 0;
#pragma omp parallel for schedule(dynamic, 64) reduction(+ : bad_code, bad_f32, n, n_fast)
  for (unsigned ia = 1; ia < top; ia += stride) {
    float amax = from16((uint16_t)ia, bf16);
    for (int mode = 0; mode < 2; ++mode) {
      float s = sglb::group_scale(amax, 448.0f, mode == 1);
      sglb::GroupDivisor d = sglb::make_divisor(s, true);
      n_fast += d.fast;
      for (unsigned ix = 0; ix <= ia; ++ix) {
        float x = from16((uint16_t)ix, bf16);
        float q = sglb::quotient(x, d), ref = x / s;
        float qc = fminf(fmaxf(q, -448.f), 448.f), rc = fminf(fmaxf(ref, -448.f), 448.f);
        bad_f32 += (sglb::float_to_bits(q) != sglb::float_to_bits(ref));
        bad_code += (to_e4m3(qc) != to_e4m3(rc));
        float qn = sglb::quotient(-x, d), refn = -x / s;
        bad_code += (to_e4m3(fmaxf(qn, -448.f)) != to_e4m3(fmaxf(refn, -448.f)));
        n += 2;
      }
    }
  }
  // the FMA-based scale against the IEEE division: every 16-bit amax, then random fp32 amax
  long long bad_scale = 0;
  const float inv448 = 1.0f / 448.0f;
  for (unsigned ia = 1; ia < top; ++ia) {
    float amax = from16((uint16_t)ia, bf16);
    for (int mode = 0; mode < 2; ++mode)
      bad_scale += sglb::float_to_bits(sglb::group_scale_fast(amax, 448.0f, inv448, mode == 1)) !=
                   sglb::float_to_bits(sglb::group_scale(amax, 448.0f, mode == 1));
  }
  unsigned long long rng = 0x9E3779B97F4A7C15ull;
  for (long long i = 0; i < 200000000ll / stride; ++i) {
    rng = rng * 6364136223846793005ull + 1442695040888963407ull;
    uint32_t u = (uint32_t)(rng >> 33) & 0x7fffffffu;
    float amax = sglb::bits_to_float(u);
    if (!(amax >= 1e-37f && amax < 3e38f)) continue;
    bad_scale += sglb::float_to_bits(sglb::group_scale_fast(amax, 448.0f, inv448, false)) !=
                 sglb::float_to_bits(sglb::group_scale(amax, 448.0f, false));
  }
  bad_code += bad_scale;
  printf("scale_mismatch=%lld ", bad_scale);
  printf("format=%s stride=%d pairs=%lld fast_divisors=%lld fp32_mismatch=%lld code_mismatch=%lld\n",
         bf16 ? "bf16" : "f16", stride, n, n_fast, bad_f32, bad_code);
  return bad_code == 0 ? 0 : 1;
}
