// Per-token-group quantisation to e4m3 (and the fused SiLU-and-mul variant).
//
// HBM-bound, one pass, written to keep the instruction count per element low enough that the
// issue slots do not become the limit (about 8 instructions per element for bf16 input):
//   * a thread owns 16 consecutive-in-pairs elements of a group (two 16-byte loads), so a group of
//     128 is 8 lanes and the scale arithmetic is shared by 16 elements;
//   * the group maximum is taken on packed 16-bit pairs and finished with a 3-step butterfly;
//   * the scale amax/448 and the per-element quotients use FMA-based correctly rounded divisions
//     (quant_math.cuh), evaluated two lanes at a time with the packed fp32x2 FMA of sm_100;
//   * codes are converted two at a time (cvt.rn.satfinite.e4m3x2.f32) and the sign bit is taken
//     from the input so that -0 stays -0.
// Every thread has UNROLL groups (4 x 16 B) in flight.  Algorithmic bytes per group of 128 bf16:
// 256 read + 128 written + 4 (float scale) or 1 (UE8M0 byte).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "ptx.cuh"
#include "quant_math.cuh"
#include "quant_vec.cuh"

namespace sglb {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 2;

struct QuantParams {
  const void* in;
  uint8_t* out_q;
  void* out_s;
  void* out_act;  // fused variant only, may be null
  uint32_t num_groups;  // rows * groups_per_row
  uint32_t groups_per_row;
  uint32_t div_mul, div_shift;  // t / groups_per_row == (uint64(t) * div_mul) >> div_shift for t < 2^31
  uint32_t hidden;              // elements per output row
  float eps, fp8_min, fp8_max;
  int64_t s_stride_row, s_stride_group;
  // batched / masked layout (rows_per_batch > 0; 16-bit inputs only): row = batch * rows_per_batch + local, scales at
  // batch * s_stride_batch + local * s_stride_row, and with masked_m only local < masked_m[batch] is processed
  const int32_t* masked_m;
  uint32_t rows_per_batch, bdiv_mul, bdiv_shift;
  int64_t s_stride_batch;
};

// 16-bit input types.  LPG = lanes per group = group_size / 16; each lane owns vectors `lane` and
// `lane + LPG` of its group (group_size 16: one lane, both vectors).
template <typename T, int LPG, bool UE8M0, bool FUSE_SILU, bool CLAMP>
__global__ void __launch_bounds__(kThreads) group_quant16_kernel(const QuantParams p) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  constexpr int kGroupsPerIter = kThreads / LPG;
  constexpr int kGroupSize = LPG * 16;
  constexpr int kSecond = (LPG == 1 && kGroupSize == 16) ? 1 : LPG;  // vector index of the second load
  const uint32_t tg = threadIdx.x / LPG;
  const uint32_t lane = threadIdx.x % LPG;
  const uint32_t base = blockIdx.x * (uint32_t)(kGroupsPerIter * kUnroll) + tg;
  const float inv_max = __frcp_rn(p.fp8_max);
  const bool fast_scale = p.fp8_max == 448.0f;
  // programmatic dependent launch: the GEMM that follows may begin its set-up and stream its weights beside this
  // kernel; this kernel's own input comes from the kernel before it
  ptx::grid_dep_launch();
  ptx::grid_dep_wait();

  uint4 raw[kUnroll][2];
  uint32_t row[kUnroll], grp[kUnroll];
  int64_t s_off[kUnroll];  // offset of the row's scales
  bool live[kUnroll];

#pragma unroll
  for (int i = 0; i < kUnroll; ++i) {
    const uint32_t t = base + (uint32_t)i * kGroupsPerIter;
    live[i] = t < p.num_groups;
    const uint32_t tt = live[i] ? t : 0u;
    row[i] = (uint32_t)(((uint64_t)tt * p.div_mul) >> p.div_shift);
    grp[i] = tt - row[i] * p.groups_per_row;
    s_off[i] = (int64_t)row[i] * p.s_stride_row;
    if (p.rows_per_batch != 0) {
      const uint32_t b = (uint32_t)(((uint64_t)row[i] * p.bdiv_mul) >> p.bdiv_shift);
      const uint32_t local = row[i] - b * p.rows_per_batch;
      s_off[i] = (int64_t)b * p.s_stride_batch + (int64_t)local * p.s_stride_row;
      if (p.masked_m != nullptr && (int32_t)local >= __ldg(p.masked_m + b)) live[i] = false;
    }
    raw[i][0] = raw[i][1] = make_uint4(0, 0, 0, 0);
    if (live[i]) {
      if constexpr (FUSE_SILU) {
        const T* g = static_cast<const T*>(p.in) + (size_t)row[i] * p.hidden * 2 + (size_t)grp[i] * kGroupSize;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t vec = lane + h * kSecond;
          const uint4 gv = __ldcs(reinterpret_cast<const uint4*>(g) + vec);
          const uint4 uv = __ldcs(reinterpret_cast<const uint4*>(g + p.hidden) + vec);
          const uint32_t* gw = reinterpret_cast<const uint32_t*>(&gv);
          const uint32_t* uw = reinterpret_cast<const uint32_t*>(&uv);
          uint32_t* ow = reinterpret_cast<uint32_t*>(&raw[i][h]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 gf = Elem<T>::pair(gw[j]), uf = Elem<T>::pair(uw[j]);
            ow[j] = Elem<T>::pack(Elem<T>::round(silu_f32(gf.x)) * uf.x, Elem<T>::round(silu_f32(gf.y)) * uf.y);
          }
        }
      } else {
        const uint4* g = reinterpret_cast<const uint4*>(static_cast<const T*>(p.in) + (size_t)tt * kGroupSize);
        raw[i][0] = __ldcs(g + lane);
        raw[i][1] = __ldcs(g + lane + kSecond);
      }
    }
  }

#pragma unroll
  for (int i = 0; i < kUnroll; ++i) {
    float amax = fmaxf(p.eps, fmaxf(Elem<T>::vec_absmax(raw[i][0]), Elem<T>::vec_absmax(raw[i][1])));
#pragma unroll
    for (int m = LPG / 2; m >= 1; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));

    const float s = fast_scale ? group_scale_fast(amax, p.fp8_max, inv_max, UE8M0) : group_scale(amax, p.fp8_max, UE8M0);
    if (!live[i]) continue;  // after the shuffles: every lane of the warp takes part in them
    const bool fast = (s >= 7.888609e-31f) && (s <= 1.2676506e30f);
    const float r = __frcp_rn(s);
    const float2 rr = make_float2(r, r), nss = make_float2(-s, -s);

    const size_t off = (size_t)row[i] * p.hidden + (size_t)grp[i] * kGroupSize;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw[i][h]);
      uint32_t packed[2];
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
        if constexpr (CLAMP) {
          qa.x = fminf(fmaxf(qa.x, p.fp8_min), p.fp8_max);
          qa.y = fminf(fmaxf(qa.y, p.fp8_min), p.fp8_max);
          qb.x = fminf(fmaxf(qb.x, p.fp8_min), p.fp8_max);
          qb.y = fminf(fmaxf(qb.y, p.fp8_min), p.fp8_max);
        }
        const uint32_t codes = cvt_e4m3x2(qa.x, qa.y) | (cvt_e4m3x2(qb.x, qb.y) << 16);
        // the quotient carries x's sign (s > 0): take bit 7 of every code from the input, so -0 / s = -0
        const uint32_t signs = Elem<T>::sign_bytes(w[2 * j], w[2 * j + 1]);
        packed[j] = (codes & 0x7f7f7f7fu) | (signs & 0x80808080u);
      }
      const uint32_t vec = lane + h * kSecond;
      __stcs(reinterpret_cast<uint2*>(p.out_q + off) + vec, make_uint2(packed[0], packed[1]));
      if constexpr (FUSE_SILU) {
        if (p.out_act != nullptr) reinterpret_cast<uint4*>(static_cast<T*>(p.out_act) + off)[vec] = raw[i][h];
      }
    }

    if (lane == 0) {
      if constexpr (UE8M0) {
        uint8_t* wp = reinterpret_cast<uint8_t*>(p.out_s) + 4 * (s_off[i] + (int64_t)(grp[i] >> 2) * p.s_stride_group);
        const uint32_t b = grp[i] & 3u;
        wp[b] = (uint8_t)(__float_as_uint(s) >> 23);
        if (grp[i] + 1 == p.groups_per_row) {
          for (uint32_t z = b + 1; z < 4; ++z) wp[z] = 0;  // bytes of the word past the last group
        }
      } else {
        static_cast<float*>(p.out_s)[s_off[i] + (int64_t)grp[i] * p.s_stride_group] = s;
      }
    }
  }
}

// fp32 input (rare): 8 elements per lane, plain IEEE divisions.
template <int LPG, bool UE8M0, bool FUSE_SILU>
__global__ void __launch_bounds__(kThreads) group_quant32_kernel(const QuantParams p) {
  constexpr int kGroupsPerIter = kThreads / LPG;
  constexpr int kGroupSize = LPG * 8;
  const uint32_t tg = threadIdx.x / LPG;
  const uint32_t lane = threadIdx.x % LPG;
  const uint32_t t = blockIdx.x * (uint32_t)kGroupsPerIter + tg;
  const bool live = t < p.num_groups;
  const uint32_t tt = live ? t : 0u;
  const uint32_t row = (uint32_t)(((uint64_t)tt * p.div_mul) >> p.div_shift);
  const uint32_t grp = tt - row * p.groups_per_row;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = 0.f;
  if (live) {
    if constexpr (FUSE_SILU) {
      const float* g = static_cast<const float*>(p.in) + (size_t)row * p.hidden * 2 + (size_t)grp * kGroupSize + lane * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = silu_f32(__ldcs(g + j)) * __ldcs(g + p.hidden + j);
    } else {
      const float4* g = reinterpret_cast<const float4*>(static_cast<const float*>(p.in) + (size_t)tt * kGroupSize) + lane * 2;
      const float4 a = __ldcs(g), b = __ldcs(g + 1);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
  }
  float amax = p.eps;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
  for (int m = LPG / 2; m >= 1; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
  const float s = group_scale(amax, p.fp8_max, UE8M0);
  if (!live) return;
  uint32_t packed[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = fminf(fmaxf(__fdiv_rn(v[4 * h + j], s), p.fp8_min), p.fp8_max);
    packed[h] = cvt_e4m3x2(q[0], q[1]) | (cvt_e4m3x2(q[2], q[3]) << 16);
  }
  const size_t off = (size_t)row * p.hidden + (size_t)grp * kGroupSize + lane * 8;
  __stcs(reinterpret_cast<uint2*>(p.out_q + off), make_uint2(packed[0], packed[1]));
  if constexpr (FUSE_SILU) {
    if (p.out_act != nullptr) {
      float* o = static_cast<float*>(p.out_act) + off;
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[j];
    }
  }
  if (lane == 0) {
    if constexpr (UE8M0) {
      uint8_t* wp = reinterpret_cast<uint8_t*>(p.out_s) +
                    4 * ((int64_t)row * p.s_stride_row + (int64_t)(grp >> 2) * p.s_stride_group);
      const uint32_t b = grp & 3u;
      wp[b] = (uint8_t)(__float_as_uint(s) >> 23);
      if (grp + 1 == p.groups_per_row) {
        for (uint32_t z = b + 1; z < 4; ++z) wp[z] = 0;
      }
    } else {
      static_cast<float*>(p.out_s)[(int64_t)row * p.s_stride_row + (int64_t)grp * p.s_stride_group] = s;
    }
  }
}

template <typename T, int LPG, bool FUSE>
int launch16(const QuantParams& p, bool ue8m0, bool clamp, cudaStream_t stream) {
  constexpr int kGroupsPerBlock = (kThreads / LPG) * kUnroll;
  const uint32_t blocks = (p.num_groups + kGroupsPerBlock - 1) / kGroupsPerBlock;
  if (ue8m0) {
    if (clamp) launch_pdl(group_quant16_kernel<T, LPG, true, FUSE, true>, dim3(blocks), dim3(kThreads), 0, stream, p);
    else launch_pdl(group_quant16_kernel<T, LPG, true, FUSE, false>, dim3(blocks), dim3(kThreads), 0, stream, p);
  } else {
    if (clamp) launch_pdl(group_quant16_kernel<T, LPG, false, FUSE, true>, dim3(blocks), dim3(kThreads), 0, stream, p);
    else launch_pdl(group_quant16_kernel<T, LPG, false, FUSE, false>, dim3(blocks), dim3(kThreads), 0, stream, p);
  }
  SGLB_CHECK_LAUNCH("group_quant16_kernel");
  return SGLB200_OK;
}

template <typename T, bool FUSE>
int launch_t16(const QuantParams& p, int group_size, bool ue8m0, bool clamp, cudaStream_t stream) {
  switch (group_size) {
    case 128: return launch16<T, 8, FUSE>(p, ue8m0, clamp, stream);
    case 64: return launch16<T, 4, FUSE>(p, ue8m0, clamp, stream);
    case 32: return launch16<T, 2, FUSE>(p, ue8m0, clamp, stream);
    default: return launch16<T, 1, FUSE>(p, ue8m0, clamp, stream);
  }
}

template <int LPG, bool FUSE>
int launch32(const QuantParams& p, bool ue8m0, cudaStream_t stream) {
  constexpr int kGroupsPerBlock = kThreads / LPG;
  const uint32_t blocks = (p.num_groups + kGroupsPerBlock - 1) / kGroupsPerBlock;
  if (ue8m0) group_quant32_kernel<LPG, true, FUSE><<<blocks, kThreads, 0, stream>>>(p);
  else group_quant32_kernel<LPG, false, FUSE><<<blocks, kThreads, 0, stream>>>(p);
  SGLB_CHECK_LAUNCH("group_quant32_kernel");
  return SGLB200_OK;
}

template <bool FUSE>
int launch_t32(const QuantParams& p, int group_size, bool ue8m0, cudaStream_t stream) {
  switch (group_size) {
    case 128: return launch32<16, FUSE>(p, ue8m0, stream);
    case 64: return launch32<8, FUSE>(p, ue8m0, stream);
    case 32: return launch32<4, FUSE>(p, ue8m0, stream);
    default: return launch32<2, FUSE>(p, ue8m0, stream);
  }
}

template <bool FUSE>
int quant_entry(const void* input, int in_dtype, void* out_q, void* out_s, void* out_act, int64_t num_rows,
                int64_t hidden, int group_size, float eps, float fp8_min, float fp8_max, int scale_ue8m0,
                int64_t s_stride_row, int64_t s_stride_group, void* stream, int64_t rows_per_batch = 0,
                int64_t s_stride_batch = 0, const int32_t* masked_m = nullptr) {
  SGLB_REQUIRE(rows_per_batch == 0 || (in_dtype != SGLB200_F32 && rows_per_batch > 0 && num_rows % rows_per_batch == 0),
               SGLB200_ERR_SHAPE, "batched layout: 16-bit input and num_rows a multiple of rows_per_batch=%lld",
               (long long)rows_per_batch);
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
  {  // round-up magic number: with s = ceil(log2 G), m = ceil(2^(31+s) / G) < 2^32 and
     // floor(t / G) == (t * m) >> (31 + s) for every t < 2^31
    uint32_t sh = 0;
    while (((uint64_t)1 << sh) < (uint64_t)G) ++sh;
    p.div_shift = 31 + sh;
    p.div_mul = (uint32_t)((((uint64_t)1 << (31 + sh)) + (uint64_t)G - 1) / (uint64_t)G);
  }
  p.hidden = (uint32_t)hidden;
  p.eps = eps;
  p.fp8_min = fp8_min;
  p.fp8_max = fp8_max;
  p.s_stride_row = s_stride_row;
  p.s_stride_group = s_stride_group;
  p.masked_m = masked_m;
  p.rows_per_batch = (uint32_t)rows_per_batch;
  p.bdiv_mul = p.bdiv_shift = 0;
  p.s_stride_batch = s_stride_batch;
  if (rows_per_batch > 0) {  // same round-up magic number as for the groups
    uint32_t sh = 0;
    while (((uint64_t)1 << sh) < (uint64_t)rows_per_batch) ++sh;
    p.bdiv_shift = 31 + sh;
    p.bdiv_mul = (uint32_t)((((uint64_t)1 << (31 + sh)) + (uint64_t)rows_per_batch - 1) / (uint64_t)rows_per_batch);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // with the e4m3 limits the saturating conversion already clamps; other limits need the explicit clamp
  const bool clamp = !(fp8_max == 448.0f && fp8_min == -448.0f);
  switch (in_dtype) {
    case SGLB200_BF16: return launch_t16<__nv_bfloat16, FUSE>(p, group_size, scale_ue8m0 != 0, clamp, st);
    case SGLB200_F16: return launch_t16<__half, FUSE>(p, group_size, scale_ue8m0 != 0, clamp, st);
    default: return launch_t32<FUSE>(p, group_size, scale_ue8m0 != 0, st);
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

extern "C" int sglb200_group_quant_fp8_batched(const void* input, int in_dtype, void* out_q, void* out_s,
                                               int64_t num_batches, int64_t rows_per_batch, int64_t hidden,
                                               int group_size, float eps, float fp8_min, float fp8_max,
                                               int scale_ue8m0, int fuse_silu_and_mul, const int32_t* masked_m,
                                               int64_t s_stride_batch, int64_t s_stride_row, int64_t s_stride_group,
                                               void* stream) {
  SGLB_REQUIRE(num_batches >= 0 && rows_per_batch >= 1, SGLB200_ERR_SHAPE, "num_batches=%lld rows_per_batch=%lld",
               (long long)num_batches, (long long)rows_per_batch);
  const int64_t rows = num_batches * rows_per_batch;
  if (fuse_silu_and_mul)
    return sglb::quant_entry<true>(input, in_dtype, out_q, out_s, nullptr, rows, hidden, group_size, eps, fp8_min,
                                   fp8_max, scale_ue8m0, s_stride_row, s_stride_group, stream, rows_per_batch,
                                   s_stride_batch, masked_m);
  return sglb::quant_entry<false>(input, in_dtype, out_q, out_s, nullptr, rows, hidden, group_size, eps, fp8_min, fp8_max,
                                  scale_ue8m0, s_stride_row, s_stride_group, stream, rows_per_batch, s_stride_batch,
                                  masked_m);
}
