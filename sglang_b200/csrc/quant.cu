// Per-token-group quantisation to e4m3 (and the fused SiLU-and-mul variant).
//
// HBM-bound, one pass: every thread loads 8 consecutive elements (16 bytes of bf16/f16) of
// UNROLL different groups up front, so a 256-thread block has UNROLL * 4 KiB in flight; the
// group maximum is a butterfly of __shfl_xor over the group's lanes; codes leave as one
// 8-byte store per thread.  The input is read once.  Algorithmic bytes per group of 128 bf16:
// 256 read + 128 written + 4 (float scale) or 1 (UE8M0 byte).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "quant_math.cuh"

namespace sglb {
namespace {

constexpr int kThreads = 256;

template <typename T>
struct Vec8;

template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};

template <>
struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};

template <>
struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    float4 a = __ldcs(reinterpret_cast<const float4*>(p));
    float4 b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ float round(float x) { return x; }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
};

__device__ __forceinline__ float silu_f32(float x) { return __fdiv_rn(x, 1.0f + expf(-x)); }

struct QuantParams {
  const void* in;
  uint8_t* out_q;
  void* out_s;
  void* out_act;  // fused variant only, may be null
  uint32_t num_groups;  // rows * groups_per_row
  uint32_t groups_per_row;
  uint32_t hidden;  // elements per output row
  float eps, fp8_min, fp8_max;
  int64_t s_stride_row, s_stride_group;
};

// TPG = lanes per group (group_size / 8); UNROLL = groups per thread.
template <typename T, int TPG, int UNROLL, bool UE8M0, bool FUSE_SILU>
__global__ void __launch_bounds__(kThreads) group_quant_kernel(const QuantParams p) {
  constexpr int kGroupsPerIter = kThreads / TPG;
  const uint32_t tg = threadIdx.x / TPG;
  const uint32_t lane = threadIdx.x % TPG;
  const uint32_t base = blockIdx.x * (uint32_t)(kGroupsPerIter * UNROLL) + tg;

  float v[UNROLL][8];
  uint32_t row[UNROLL], grp[UNROLL];
  bool live[UNROLL];

#pragma unroll
  for (int i = 0; i < UNROLL; ++i) {
    const uint32_t t = base + (uint32_t)i * kGroupsPerIter;
    live[i] = t < p.num_groups;
    row[i] = live[i] ? t / p.groups_per_row : 0u;
    grp[i] = live[i] ? t - row[i] * p.groups_per_row : 0u;
    if (live[i]) {
      const size_t col = (size_t)grp[i] * (TPG * 8) + lane * 8;
      if constexpr (FUSE_SILU) {
        const T* g = static_cast<const T*>(p.in) + (size_t)row[i] * p.hidden * 2 + col;
        float u[8];
        Vec8<T>::load(g, v[i]);
        Vec8<T>::load(g + p.hidden, u);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = Vec8<T>::round(Vec8<T>::round(silu_f32(v[i][j])) * u[j]);
      } else {
        Vec8<T>::load(static_cast<const T*>(p.in) + (size_t)row[i] * p.hidden + col, v[i]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
    }
  }

#pragma unroll
  for (int i = 0; i < UNROLL; ++i) {
    float amax = p.eps;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
#pragma unroll
    for (int m = TPG / 2; m >= 1; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));

    const float s = group_scale(amax, p.fp8_max, UE8M0);
    const GroupDivisor d = make_divisor(s, sizeof(T) == 2);

    if (!live[i]) continue;  // after the shuffles: every lane of the warp takes part in them

    uint32_t packed[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float q[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) q[j] = fminf(fmaxf(quotient(v[i][4 * h + j], d), p.fp8_min), p.fp8_max);
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q[0], q[1]), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q[2], q[3]), __NV_SATFINITE, __NV_E4M3);
      packed[h] = lo | (hi << 16);
    }
    const size_t off = (size_t)row[i] * p.hidden + (size_t)grp[i] * (TPG * 8) + lane * 8;
    __stcs(reinterpret_cast<uint2*>(p.out_q + off), make_uint2(packed[0], packed[1]));
    if constexpr (FUSE_SILU) {
      if (p.out_act != nullptr) Vec8<T>::store(static_cast<T*>(p.out_act) + off, v[i]);
    }

    if (lane == 0) {
      if constexpr (UE8M0) {
        uint8_t* w = reinterpret_cast<uint8_t*>(p.out_s) +
                     4 * ((int64_t)row[i] * p.s_stride_row + (int64_t)(grp[i] >> 2) * p.s_stride_group);
        const uint32_t b = grp[i] & 3u;
        w[b] = (uint8_t)(float_to_bits(s) >> 23);
        if (grp[i] + 1 == p.groups_per_row) {
          for (uint32_t z = b + 1; z < 4; ++z) w[z] = 0;  // bytes of the word past the last group
        }
      } else {
        static_cast<float*>(p.out_s)[(int64_t)row[i] * p.s_stride_row + (int64_t)grp[i] * p.s_stride_group] = s;
      }
    }
  }
}

template <typename T, int TPG, bool FUSE>
int launch_tpg(const QuantParams& p, bool ue8m0, cudaStream_t stream) {
  constexpr int UNROLL = 4;
  constexpr int kGroupsPerBlock = (kThreads / TPG) * UNROLL;
  const uint32_t blocks = (p.num_groups + kGroupsPerBlock - 1) / kGroupsPerBlock;
  if (ue8m0) {
    group_quant_kernel<T, TPG, UNROLL, true, FUSE><<<blocks, kThreads, 0, stream>>>(p);
  } else {
    group_quant_kernel<T, TPG, UNROLL, false, FUSE><<<blocks, kThreads, 0, stream>>>(p);
  }
  SGLB_CHECK_LAUNCH("group_quant_kernel");
  return SGLB200_OK;
}

template <typename T, bool FUSE>
int launch_t(const QuantParams& p, int group_size, bool ue8m0, cudaStream_t stream) {
  switch (group_size) {
    case 128: return launch_tpg<T, 16, FUSE>(p, ue8m0, stream);
    case 64: return launch_tpg<T, 8, FUSE>(p, ue8m0, stream);
    case 32: return launch_tpg<T, 4, FUSE>(p, ue8m0, stream);
    case 16: return launch_tpg<T, 2, FUSE>(p, ue8m0, stream);
  }
  return fail(SGLB200_ERR_SHAPE, "group_size=%d: must be 16, 32, 64 or 128", group_size);
}

template <bool FUSE>
int quant_entry(const void* input, int in_dtype, void* out_q, void* out_s, void* out_act, int64_t num_rows,
                int64_t hidden, int group_size, float eps, float fp8_min, float fp8_max, int scale_ue8m0,
                int64_t s_stride_row, int64_t s_stride_group, void* stream) {
  SGLB_REQUIRE(num_rows >= 0 && hidden >= 0, SGLB200_ERR_SHAPE, "num_rows=%lld hidden=%lld: negative size",
               (long long)num_rows, (long long)hidden);
  SGLB_REQUIRE(group_size == 16 || group_size == 32 || group_size == 64 || group_size == 128, SGLB200_ERR_SHAPE,
               "group_size=%d: must be 16, 32, 64 or 128", group_size);
  SGLB_REQUIRE(hidden % group_size == 0, SGLB200_ERR_SHAPE, "hidden=%lld is not a multiple of group_size=%d",
               (long long)hidden, group_size);
  SGLB_REQUIRE(in_dtype == SGLB200_BF16 || in_dtype == SGLB200_F16 || in_dtype == SGLB200_F32, SGLB200_ERR_DTYPE,
               "in_dtype=%d", in_dtype);
  if (num_rows == 0 || hidden == 0) return SGLB200_OK;
  SGLB_REQUIRE(input && out_q && out_s, SGLB200_ERR_NULL, "input/out_q/out_s must not be NULL");
  const int64_t G = hidden / group_size;
  SGLB_REQUIRE(num_rows * G < (int64_t)1 << 31, SGLB200_ERR_SHAPE, "rows*groups=%lld exceeds 2^31",
               (long long)(num_rows * G));
  SGLB_REQUIRE(aligned(input, 16), SGLB200_ERR_ALIGN, "input pointer must be 16-byte aligned");
  SGLB_REQUIRE(aligned(out_q, 8), SGLB200_ERR_ALIGN, "out_q pointer must be 8-byte aligned");
  SGLB_REQUIRE(aligned(out_s, 4), SGLB200_ERR_ALIGN, "out_s pointer must be 4-byte aligned");
  if (FUSE && out_act) SGLB_REQUIRE(aligned(out_act, 16), SGLB200_ERR_ALIGN, "out_act pointer must be 16-byte aligned");
  SGLB_REQUIRE(fp8_max > 0.f && fp8_min < fp8_max, SGLB200_ERR_SHAPE, "fp8_min/fp8_max out of order");
  SGLB_REQUIRE(eps >= 0.f, SGLB200_ERR_SHAPE, "eps must be >= 0");
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  SGLB_REQUIRE(di.cc_major == 10, SGLB200_ERR_ARCH, "compute capability %d.%d: this library is built for sm_100a only",
               di.cc_major, di.cc_minor);

  QuantParams p;
  p.in = input;
  p.out_q = static_cast<uint8_t*>(out_q);
  p.out_s = out_s;
  p.out_act = out_act;
  p.num_groups = (uint32_t)(num_rows * G);
  p.groups_per_row = (uint32_t)G;
  p.hidden = (uint32_t)hidden;
  p.eps = eps;
  p.fp8_min = fp8_min;
  p.fp8_max = fp8_max;
  p.s_stride_row = s_stride_row;
  p.s_stride_group = s_stride_group;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (in_dtype) {
    case SGLB200_BF16: return launch_t<__nv_bfloat16, FUSE>(p, group_size, scale_ue8m0 != 0, st);
    case SGLB200_F16: return launch_t<__half, FUSE>(p, group_size, scale_ue8m0 != 0, st);
    default: return launch_t<float, FUSE>(p, group_size, scale_ue8m0 != 0, st);
  }
}

}  // namespace
}  // namespace sglb

extern "C" int sglb200_per_token_group_quant_fp8(const void* input, int in_dtype, void* out_q, void* out_s,
                                                 int64_t num_rows, int64_t hidden, int group_size, float eps,
                                                 float fp8_min, float fp8_max, int scale_ue8m0,
                                                 int64_t s_stride_row, int64_t s_stride_group, void* stream) {
  return sglb::quant_entry<false>(input, in_dtype, out_q, out_s, nullptr, num_rows, hidden, group_size, eps, fp8_min,
                                  fp8_max, scale_ue8m0, s_stride_row, s_stride_group, stream);
}

extern "C" int sglb200_silu_mul_group_quant_fp8(const void* input, int in_dtype, void* out_q, void* out_s,
                                                void* out_act, int64_t num_rows, int64_t hidden, int group_size,
                                                float eps, float fp8_min, float fp8_max, int scale_ue8m0,
                                                int64_t s_stride_row, int64_t s_stride_group, void* stream) {
  return sglb::quant_entry<true>(input, in_dtype, out_q, out_s, out_act, num_rows, hidden, group_size, eps, fp8_min,
                                 fp8_max, scale_ue8m0, s_stride_row, s_stride_group, stream);
}
