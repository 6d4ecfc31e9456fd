// Integer routing tables and the HBM-bound row movers around the grouped GEMMs:
// prepare_moe_input (stable counting sort by expert), shuffle_rows (row gather),
// apply_shuffle_mul_sum (weighted top-k combine) and silu_and_mul.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace sglb {
namespace {

// ------------------------------------------------------------------------------------------
// prepare_moe_input: one block of 1024 threads.  Warp w owns the contiguous slice
// [w*chunk, (w+1)*chunk) of the flattened topk_ids.  Pass 1 counts (warp, expert) occurrences in
// shared memory; a block scan turns them into per-expert offsets and per-(warp, expert) bases;
// pass 2 walks each slice in order and ranks equal ids inside a 32-lane batch with
// __match_any_sync, which keeps rows of one expert in ascending slot order (a stable sort).
// ------------------------------------------------------------------------------------------
constexpr int kPrepThreads = 1024;
constexpr int kPrepWarps = kPrepThreads / 32;

__global__ void __launch_bounds__(kPrepThreads)
prepare_moe_input_kernel(const int32_t* __restrict__ topk_ids, int32_t* __restrict__ expert_offsets,
                         int32_t* __restrict__ ps1, int32_t* __restrict__ ps2, int32_t* __restrict__ a_map,
                         int32_t* __restrict__ c_map, int32_t len, int32_t topk, int32_t E, int32_t n, int32_t k) {
  extern __shared__ int32_t sm[];
  int32_t* wcnt = sm;                     // [kPrepWarps][E] counts, then running bases
  int32_t* scan = sm + kPrepWarps * E;    // [kPrepThreads] scratch for the block scan
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int32_t chunk = ((len + kPrepWarps - 1) / kPrepWarps + 31) / 32 * 32;
  const int32_t c0 = warp * chunk, c1 = min(c0 + chunk, len);

  for (int i = threadIdx.x; i < kPrepWarps * E; i += kPrepThreads) wcnt[i] = 0;
  __syncthreads();

  for (int32_t i = c0 + lane; i < c1; i += 32) {
    const int32_t e = topk_ids[i];
    if (e >= 0 && e < E) atomicAdd(&wcnt[warp * E + e], 1);
  }
  __syncthreads();

  // per-expert totals and exclusive scan over experts (E <= 1024: one expert per thread)
  int32_t total = 0;
  if ((int)threadIdx.x < E) {
    for (int w = 0; w < kPrepWarps; ++w) total += wcnt[w * E + threadIdx.x];
  }
  scan[threadIdx.x] = total;
  __syncthreads();
  for (int d = 1; d < kPrepThreads; d <<= 1) {
    int32_t v = 0;
    if ((int)threadIdx.x >= d) v = scan[threadIdx.x - d];
    __syncthreads();
    scan[threadIdx.x] += v;
    __syncthreads();
  }
  const int32_t grand_total = scan[kPrepThreads - 1];
  if ((int)threadIdx.x < E) {
    const int32_t e = threadIdx.x;
    const int32_t start = scan[e] - total;
    if (e == 0) expert_offsets[0] = 0;
    expert_offsets[e + 1] = scan[e];
    if (ps1) { ps1[e * 3] = total; ps1[e * 3 + 1] = 2 * n; ps1[e * 3 + 2] = k; }
    if (ps2) { ps2[e * 3] = total; ps2[e * 3 + 1] = k; ps2[e * 3 + 2] = n; }
    int32_t run = start;
    for (int w = 0; w < kPrepWarps; ++w) {
      const int32_t c = wcnt[w * E + e];
      wcnt[w * E + e] = run;
      run += c;
    }
  }
  __syncthreads();

  for (int32_t i0 = c0; i0 < c1; i0 += 32) {
    const int32_t i = i0 + lane;
    int32_t e = -1;
    if (i < c1) e = topk_ids[i];
    const bool valid = e >= 0 && e < E;
    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? e : -1 - lane);
    if (valid) {
      const int32_t rank = __popc(peers & ((1u << lane) - 1u));
      const int32_t pos = wcnt[warp * E + e] + rank;
      a_map[pos] = i / topk;
      c_map[i] = pos;
    } else if (i < c1) {
      c_map[i] = -1;
    }
    __syncwarp();
    if (valid && (peers & ((1u << lane) - 1u)) == 0) wcnt[warp * E + e] += __popc(peers);
    __syncwarp();
  }
  // rows past the last routed one (only when some ids were out of range)
  for (int32_t i = grand_total + threadIdx.x; i < len; i += kPrepThreads) a_map[i] = 0;
}

// ------------------------------------------------------------------------------------------
// shuffle_rows: one warp per destination row, 16-byte (or 4-byte) pieces
// ------------------------------------------------------------------------------------------
template <typename V>
__global__ void __launch_bounds__(256)
shuffle_rows_kernel(const V* __restrict__ in, const int32_t* __restrict__ map, V* __restrict__ out, int64_t n_dst,
                    int64_t row_vecs) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * 8;
  for (int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); r < n_dst; r += warps) {
    const V* src = in + (int64_t)map[r] * row_vecs;
    V* dst = out + r * row_vecs;
    for (int64_t c = lane; c < row_vecs; c += 32) dst[c] = __ldg(src + c);
  }
}

// ------------------------------------------------------------------------------------------
// apply_shuffle_mul_sum and silu_and_mul
// ------------------------------------------------------------------------------------------
template <typename T>
struct Cvt;
template <>
struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 t(float x) { return __float2bfloat16_rn(x); }
};
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half t(float x) { return __float2half_rn(x); }
};

// ROUND: each product is rounded to T before it is added (the torch-native expert-MLP reference sums
// bf16 products); otherwise products stay in fp32 (the reference's CUDA combine kernel).
template <typename T, bool ROUND>
__global__ void __launch_bounds__(256)
combine_kernel(const T* __restrict__ in, T* __restrict__ out, const int32_t* __restrict__ perm,
               const T* __restrict__ factors, int32_t topk, int32_t hidden) {
  const int64_t i = blockIdx.x;
  const int32_t vecs = hidden / 8;
  for (int32_t c = threadIdx.x; c < vecs; c += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int x = 0; x < 8; ++x) acc[x] = 0.f;
    for (int32_t j = 0; j < topk; ++j) {
      const int32_t src = __ldg(perm + i * topk + j);
      if (src < 0) continue;
      const float w = factors ? Cvt<T>::f(factors[i * topk + j]) : 1.f;
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(in + (int64_t)src * hidden) + c);
      const T* h = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        if constexpr (ROUND) {
          acc[x] += Cvt<T>::f(Cvt<T>::t(w * Cvt<T>::f(h[x])));
        } else {
          acc[x] = fmaf(w, Cvt<T>::f(h[x]), acc[x]);
        }
      }
    }
    uint4 o;
    T* oh = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int x = 0; x < 8; ++x) oh[x] = Cvt<T>::t(acc[x]);
    reinterpret_cast<uint4*>(out + i * hidden)[c] = o;
  }
  for (int32_t d = vecs * 8 + threadIdx.x; d < hidden; d += blockDim.x) {
    float acc = 0.f;
    for (int32_t j = 0; j < topk; ++j) {
      const int32_t src = perm[i * topk + j];
      if (src < 0) continue;
      const float w = factors ? Cvt<T>::f(factors[i * topk + j]) : 1.f;
      if constexpr (ROUND) {
        acc += Cvt<T>::f(Cvt<T>::t(w * Cvt<T>::f(in[(int64_t)src * hidden + d])));
      } else {
        acc = fmaf(w, Cvt<T>::f(in[(int64_t)src * hidden + d]), acc);
      }
    }
    out[i * hidden + d] = Cvt<T>::t(acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
silu_and_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t rows, int32_t hidden) {
  const int32_t vecs = hidden / 8;
  const int64_t total = rows * vecs;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / vecs;
    const int32_t c = (int32_t)(idx - r * vecs);
    const uint4 g = __ldg(reinterpret_cast<const uint4*>(in + r * 2 * hidden) + c);
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(in + r * 2 * hidden + hidden) + c);
    const T* gh = reinterpret_cast<const T*>(&g);
    const T* uh = reinterpret_cast<const T*>(&u);
    uint4 o;
    T* oh = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      const float gv = Cvt<T>::f(gh[x]);
      const T s = Cvt<T>::t(__fdiv_rn(gv, 1.0f + expf(-gv)));
      oh[x] = Cvt<T>::t(Cvt<T>::f(s) * Cvt<T>::f(uh[x]));
    }
    reinterpret_cast<uint4*>(out + r * hidden)[c] = o;
  }
}

int check_arch() {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  SGLB_REQUIRE(di.cc_major == 10, SGLB200_ERR_ARCH, "compute capability %d.%d: this library is built for sm_100a only",
               di.cc_major, di.cc_minor);
  return SGLB200_OK;
}

}  // namespace
}  // namespace sglb

using namespace sglb;

extern "C" int sglb200_prepare_moe_input(const int32_t* topk_ids, int32_t* expert_offsets, int32_t* problem_sizes1,
                                         int32_t* problem_sizes2, int32_t* a_map, int32_t* c_map, int64_t num_tokens,
                                         int64_t topk, int64_t num_experts, int64_t n, int64_t k, void* stream) {
  SGLB_REQUIRE(num_tokens >= 0 && topk >= 1, SGLB200_ERR_SHAPE, "num_tokens=%lld topk=%lld", (long long)num_tokens,
               (long long)topk);
  SGLB_REQUIRE(num_experts >= 1 && num_experts <= 1024, SGLB200_ERR_SHAPE, "num_experts=%lld: 1..1024",
               (long long)num_experts);
  SGLB_REQUIRE(num_tokens * topk <= (1 << 24), SGLB200_ERR_SHAPE, "num_tokens*topk=%lld exceeds 2^24",
               (long long)(num_tokens * topk));
  SGLB_REQUIRE(expert_offsets && a_map && c_map && (topk_ids || num_tokens == 0), SGLB200_ERR_NULL,
               "topk_ids/expert_offsets/a_map/c_map must not be NULL");
  if (int rc = check_arch()) return rc;
  const size_t smem = ((size_t)kPrepWarps * num_experts + kPrepThreads) * sizeof(int32_t);
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(prepare_moe_input_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(((size_t)kPrepWarps * 1024 + kPrepThreads) * sizeof(int32_t)));
    if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done[dev] = true;
  }
  prepare_moe_input_kernel<<<1, kPrepThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      topk_ids, expert_offsets, problem_sizes1, problem_sizes2, a_map, c_map, (int32_t)(num_tokens * topk),
      (int32_t)topk, (int32_t)num_experts, (int32_t)n, (int32_t)k);
  SGLB_CHECK_LAUNCH("prepare_moe_input_kernel");
  return SGLB200_OK;
}

extern "C" int sglb200_shuffle_rows(const void* input, const int32_t* dst2src, void* output, int64_t num_dst_rows,
                                    int64_t row_bytes, void* stream) {
  SGLB_REQUIRE(num_dst_rows >= 0 && row_bytes >= 0 && row_bytes % 4 == 0, SGLB200_ERR_SHAPE,
               "num_dst_rows=%lld row_bytes=%lld (must be a multiple of 4)", (long long)num_dst_rows,
               (long long)row_bytes);
  if (num_dst_rows == 0 || row_bytes == 0) return SGLB200_OK;
  SGLB_REQUIRE(input && dst2src && output, SGLB200_ERR_NULL, "input/dst2src/output must not be NULL");
  if (int rc = check_arch()) return rc;
  DeviceInfo di;
  device_info(&di);
  int64_t blocks = (num_dst_rows + 7) / 8;
  const int64_t cap = (int64_t)di.sm_count * 32;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (row_bytes % 16 == 0 && aligned(input, 16) && aligned(output, 16)) {
    shuffle_rows_kernel<uint4><<<(int)blocks, 256, 0, st>>>(static_cast<const uint4*>(input), dst2src,
                                                            static_cast<uint4*>(output), num_dst_rows, row_bytes / 16);
  } else {
    SGLB_REQUIRE(aligned(input, 4) && aligned(output, 4), SGLB200_ERR_ALIGN, "input/output must be 4-byte aligned");
    shuffle_rows_kernel<uint32_t><<<(int)blocks, 256, 0, st>>>(static_cast<const uint32_t*>(input), dst2src,
                                                               static_cast<uint32_t*>(output), num_dst_rows,
                                                               row_bytes / 4);
  }
  SGLB_CHECK_LAUNCH("shuffle_rows_kernel");
  return SGLB200_OK;
}

extern "C" int sglb200_apply_shuffle_mul_sum(const void* input, void* output, const int32_t* perm, const void* factors,
                                             int64_t m, int64_t topk, int64_t hidden, int dtype, int round_products,
                                             void* stream) {
  SGLB_REQUIRE(m >= 0 && topk >= 1 && hidden >= 0, SGLB200_ERR_SHAPE, "m=%lld topk=%lld hidden=%lld", (long long)m,
               (long long)topk, (long long)hidden);
  SGLB_REQUIRE(dtype == SGLB200_BF16 || dtype == SGLB200_F16, SGLB200_ERR_DTYPE, "dtype=%d", dtype);
  if (m == 0 || hidden == 0) return SGLB200_OK;
  SGLB_REQUIRE(input && output && perm, SGLB200_ERR_NULL, "input/output/perm must not be NULL");
  SGLB_REQUIRE(hidden % 8 == 0 ? (aligned(input, 16) && aligned(output, 16)) : true, SGLB200_ERR_ALIGN,
               "input/output must be 16-byte aligned");
  SGLB_REQUIRE(hidden % 8 == 0 || hidden < 8, SGLB200_ERR_SHAPE,
               "hidden=%lld: rows must be a multiple of 8 elements (16-byte rows)", (long long)hidden);
  SGLB_REQUIRE(m < ((int64_t)1 << 31), SGLB200_ERR_SHAPE, "m too large");
  if (int rc = check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int threads = (int)(hidden / 8 < 32 ? 32 : (hidden / 8 > 256 ? 256 : (hidden / 8 + 31) / 32 * 32));
#define SGLB_COMBINE(T, R)                                                                                   \
  combine_kernel<T, R><<<(int)m, threads, 0, st>>>(static_cast<const T*>(input), static_cast<T*>(output), perm, \
                                                   static_cast<const T*>(factors), (int32_t)topk, (int32_t)hidden)
  if (dtype == SGLB200_BF16) {
    if (round_products) SGLB_COMBINE(__nv_bfloat16, true); else SGLB_COMBINE(__nv_bfloat16, false);
  } else {
    if (round_products) SGLB_COMBINE(__half, true); else SGLB_COMBINE(__half, false);
  }
#undef SGLB_COMBINE
  SGLB_CHECK_LAUNCH("combine_kernel");
  return SGLB200_OK;
}

extern "C" int sglb200_silu_and_mul(const void* input, void* output, int64_t num_rows, int64_t hidden, int dtype,
                                    void* stream) {
  SGLB_REQUIRE(num_rows >= 0 && hidden >= 0, SGLB200_ERR_SHAPE, "num_rows=%lld hidden=%lld", (long long)num_rows,
               (long long)hidden);
  SGLB_REQUIRE(dtype == SGLB200_BF16 || dtype == SGLB200_F16, SGLB200_ERR_DTYPE, "dtype=%d", dtype);
  SGLB_REQUIRE(hidden % 8 == 0, SGLB200_ERR_SHAPE, "hidden=%lld must be a multiple of 8", (long long)hidden);
  if (num_rows == 0 || hidden == 0) return SGLB200_OK;
  SGLB_REQUIRE(input && output, SGLB200_ERR_NULL, "input/output must not be NULL");
  SGLB_REQUIRE(aligned(input, 16) && aligned(output, 16), SGLB200_ERR_ALIGN, "input/output must be 16-byte aligned");
  if (int rc = check_arch()) return rc;
  DeviceInfo di;
  device_info(&di);
  const int64_t total = num_rows * (hidden / 8);
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)di.sm_count * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == SGLB200_BF16) {
    silu_and_mul_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(input),
                                                                   static_cast<__nv_bfloat16*>(output), num_rows,
                                                                   (int32_t)hidden);
  } else {
    silu_and_mul_kernel<__half><<<(int)blocks, 256, 0, st>>>(static_cast<const __half*>(input),
                                                            static_cast<__half*>(output), num_rows, (int32_t)hidden);
  }
  SGLB_CHECK_LAUNCH("silu_and_mul_kernel");
  return SGLB200_OK;
}
