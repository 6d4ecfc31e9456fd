// Routing-side helpers of the MoE path: softmax + top-k selection, the block-aligned counting sort used by the
// tile-gather MoE runner, and the top-k sum.  Integer work and HBM-bound row sums; no tensor cores.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <float.h>

#include "common.cuh"

namespace sglb {
namespace {

// ------------------------------------------------------------------------------------------
// topk_softmax: one warp per token.  probabilities = softmax(logits) in fp32; the k largest are taken
// in descending order, ties to the lower expert index; optional renormalisation by their sum.
// ------------------------------------------------------------------------------------------
constexpr int kMaxPerLane = 32;  // experts per lane: up to 1024 experts

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T, int PER_LANE>
__global__ void __launch_bounds__(256)
topk_softmax_kernel(const T* __restrict__ logits, float* __restrict__ weights, int32_t* __restrict__ ids,
                    int32_t num_tokens, int32_t E, int32_t topk, int renormalize) {
  const int lane = threadIdx.x & 31;
  const int64_t token = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= num_tokens) return;
  const T* row = logits + token * E;
  float v[PER_LANE];
  float mx = -FLT_MAX;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? to_f32<T>(row[e]) : -FLT_MAX;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) v[i] = (i * 32 + lane < E) ? v[i] * inv : -1.f;  // probabilities are >= 0

  float picked_sum = 0.f;
  float my_w = 0.f;
  int32_t my_id = 0;
  for (int32_t j = 0; j < topk; ++j) {
    float best = -2.f;
    int32_t best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > best) { best = v[i]; best_e = e; }  // ascending e inside a lane: first maximum wins
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, d);
      const int32_t oe = __shfl_xor_sync(0xffffffffu, best_e, d);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i)
        if (i == (best_e >> 5)) v[i] = -1.f;  // taken
    }
    picked_sum += best;
    if (lane == (j & 31)) { my_w = best; my_id = best_e; }
    if ((j & 31) == 31 || j + 1 == topk) {  // flush up to 32 results
      const int32_t base = j & ~31;
      if (base + lane <= j) {
        weights[token * topk + base + lane] = my_w;
        ids[token * topk + base + lane] = my_id;
      }
    }
  }
  if (renormalize) {
    __syncwarp();
    const float r = __fdiv_rn(1.0f, picked_sum);
    for (int32_t j = lane; j < topk; j += 32) weights[token * topk + j] *= r;
  }
}

// ------------------------------------------------------------------------------------------
// moe_fused_gate: sigmoid router with a selection bias and two-level (group, then expert) top-k, one warp per
// token.  s = sigmoid(x), b = s + bias (both rounded to the input type); a group's score is the sum of its two
// largest b; the topk_group best groups stay (ties: lower group); inside them the topk best b (ties: lower
// expert) are taken and weighted by s; weights are divided by their sum.
// ------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float round_to(float x);
template <>
__device__ __forceinline__ float round_to<float>(float x) { return x; }
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
template <>
__device__ __forceinline__ float round_to<__half>(float x) { return __half2float(__float2half_rn(x)); }

template <typename T, int PER_LANE>
__global__ void __launch_bounds__(256)
fused_gate_kernel(const T* __restrict__ logits, const T* __restrict__ bias, float* __restrict__ weights,
                  int32_t* __restrict__ ids, int32_t num_tokens, int32_t E, int32_t G, int32_t topk_group,
                  int32_t topk, int32_t n_shared, float rsf, int apply_rsf) {
  extern __shared__ float gate_sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t token = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (token >= num_tokens) return;
  float* sb = gate_sm + (size_t)warp * E;
  const T* row = logits + token * E;
  float s[PER_LANE], b[PER_LANE];
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = i * 32 + lane;
    s[i] = 0.f;
    b[i] = -INFINITY;
    if (e < E) {
      s[i] = round_to<T>(__fdiv_rn(1.0f, 1.0f + expf(-to_f32<T>(row[e]))));
      b[i] = round_to<T>(s[i] + to_f32<T>(bias[e]));
      sb[e] = b[i];
    }
  }
  __syncwarp();
  const int gsz = E / G;
  float gscore = -INFINITY;
  if (lane < G) {
    float m1 = -FLT_MAX, m2 = -FLT_MAX;
    for (int j = 0; j < gsz; ++j) {
      const float v = sb[lane * gsz + j];
      if (v > m1) { m2 = m1; m1 = v; }
      else if (v > m2) m2 = v;
    }
    gscore = round_to<T>(m1 + m2);
  }
  uint32_t keep = 0;
  for (int t = 0; t < topk_group; ++t) {
    float best = gscore;
    int who = lane;
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, d);
      const int ow = __shfl_xor_sync(0xffffffffu, who, d);
      if (ob > best || (ob == best && ow < who)) { best = ob; who = ow; }
    }
    keep |= 1u << who;
    if (lane == who) gscore = -INFINITY;
  }
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = i * 32 + lane;
    if (e < E && !((keep >> (e / gsz)) & 1u)) b[i] = -INFINITY;
  }
  const int32_t topk_real = topk - n_shared;
  float sum = 0.f, my_w = 0.f;
  int32_t my_id = 0;
  for (int32_t j = 0; j < topk_real; ++j) {
    float best = -INFINITY;
    int32_t best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = i * 32 + lane;
      if (b[i] > best) { best = b[i]; best_e = e; }  // taken and masked entries sit at -INFINITY and never win
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, d);
      const int32_t oe = __shfl_xor_sync(0xffffffffu, best_e, d);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    float sw = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i)
      if (i == (best_e >> 5)) { sw = s[i]; if ((best_e & 31) == lane) b[i] = -INFINITY; }
    sw = __shfl_sync(0xffffffffu, sw, best_e & 31);
    sum += sw;
    if (lane == j) { my_w = sw; my_id = best_e; }
  }
  if (lane >= topk_real && lane < topk) {
    my_w = __fdiv_rn(sum, rsf);
    my_id = E + (lane - topk_real);
  }
  if (lane < topk) {
    float r = __fdiv_rn(my_w, sum);
    if (apply_rsf) r *= rsf;
    weights[token * topk + lane] = r;
    ids[token * topk + lane] = my_id;
  }
}

// ------------------------------------------------------------------------------------------
// moe_align_block_size: stable counting sort of the flattened expert ids into buckets padded to a multiple of
// block_size.  Bucket b holds id b - 1 (bucket 0 = id -1, the experts another rank owns).  One block.
// ------------------------------------------------------------------------------------------
constexpr int kAlignThreads = 1024;
constexpr int kAlignWarps = kAlignThreads / 32;

__global__ void __launch_bounds__(kAlignThreads)
moe_align_kernel(const int32_t* __restrict__ topk_ids, int32_t* __restrict__ sorted_ids, int32_t* __restrict__ expert_ids,
                 int32_t* __restrict__ num_post_pad, int32_t* __restrict__ cumsum, int32_t numel, int32_t B,
                 int32_t block_size, int pad_sorted) {
  extern __shared__ int32_t sm[];
  int32_t* wcnt = sm;                  // [kAlignWarps][B]
  int32_t* scan = sm + kAlignWarps * B;  // [kAlignThreads]
  int32_t* prefix = scan + kAlignThreads;  // [B + 1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int32_t chunk = ((numel + kAlignWarps - 1) / kAlignWarps + 31) / 32 * 32;
  const int32_t c0 = warp * chunk, c1 = min(c0 + chunk, numel);
  for (int i = threadIdx.x; i < kAlignWarps * B; i += kAlignThreads) wcnt[i] = 0;
  __syncthreads();
  for (int32_t i = c0 + lane; i < c1; i += 32) {
    const int32_t b = topk_ids[i] + 1;
    if (b >= 0 && b < B) atomicAdd(&wcnt[warp * B + b], 1);
  }
  __syncthreads();
  int32_t total = 0, padded = 0;
  if ((int)threadIdx.x < B) {
    for (int w = 0; w < kAlignWarps; ++w) total += wcnt[w * B + threadIdx.x];
    padded = (total + block_size - 1) / block_size * block_size;
  }
  scan[threadIdx.x] = padded;
  __syncthreads();
  for (int d = 1; d < kAlignThreads; d <<= 1) {
    int32_t v = 0;
    if ((int)threadIdx.x >= d) v = scan[threadIdx.x - d];
    __syncthreads();
    scan[threadIdx.x] += v;
    __syncthreads();
  }
  const int32_t post_pad = scan[kAlignThreads - 1];
  if ((int)threadIdx.x < B) {
    const int32_t start = scan[threadIdx.x] - padded;
    prefix[threadIdx.x] = start;
    if (cumsum) cumsum[threadIdx.x] = start;
    int32_t run = start;
    for (int w = 0; w < kAlignWarps; ++w) {
      const int32_t c = wcnt[w * B + threadIdx.x];
      wcnt[w * B + threadIdx.x] = run;
      run += c;
    }
  }
  if (threadIdx.x == 0) {
    prefix[B] = post_pad;
    if (cumsum) cumsum[B] = post_pad;
    *num_post_pad = post_pad;
  }
  __syncthreads();
  if (pad_sorted) {
    for (int32_t i = threadIdx.x; i < post_pad; i += kAlignThreads) sorted_ids[i] = numel;
  }
  for (int32_t i = threadIdx.x; i < post_pad / block_size; i += kAlignThreads) {
    const int32_t bs = i * block_size;
    int lo = 0, hi = B;  // last bucket with prefix <= bs
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (prefix[mid] <= bs) lo = mid; else hi = mid;
    }
    // empty buckets share their start with the next one: take the last bucket that starts here
    expert_ids[i] = lo - 1;
  }
  __syncthreads();
  for (int32_t i0 = c0; i0 < c1; i0 += 32) {
    const int32_t i = i0 + lane;
    int32_t b = -1;
    if (i < c1) b = topk_ids[i] + 1;
    const bool valid = b >= 0 && b < B;
    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? b : -1 - lane);
    if (valid) sorted_ids[wcnt[warp * B + b] + __popc(peers & ((1u << lane) - 1u))] = i;
    __syncwarp();
    if (valid && (peers & ((1u << lane) - 1u)) == 0) wcnt[warp * B + b] += __popc(peers);
    __syncwarp();
  }
}

// ------------------------------------------------------------------------------------------
// moe_sum_reduce: out[m, :] = cast( scale * sum_j in[m, j, :] ), fp32 sum in ascending j
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
moe_sum_reduce_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t tokens, int32_t topk, int32_t hidden,
                      float scale) {
  const int32_t vecs = hidden / 8;
  const int64_t total = tokens * vecs;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = idx / vecs;
    const int32_t c = (int32_t)(idx - m * vecs);
    float acc[8];
#pragma unroll
    for (int x = 0; x < 8; ++x) acc[x] = 0.f;
    for (int32_t j = 0; j < topk; ++j) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(in + (m * topk + j) * hidden) + c);
      const T* h = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int x = 0; x < 8; ++x) acc[x] += to_f32<T>(h[x]);
    }
    uint4 o;
    T* oh = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      const float r = acc[x] * scale;
      if constexpr (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) oh[x] = __float2bfloat16_rn(r);
      else oh[x] = __float2half_rn(r);
    }
    reinterpret_cast<uint4*>(out + m * hidden)[c] = o;
  }
}

int arch_ok() {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  SGLB_REQUIRE(di.cc_major == 10, SGLB200_ERR_ARCH, "compute capability %d.%d: this library is built for sm_100a only",
               di.cc_major, di.cc_minor);
  return SGLB200_OK;
}

template <typename T>
int launch_topk(const void* logits, float* w, int32_t* ids, int64_t tokens, int32_t E, int32_t topk, int renorm,
                cudaStream_t st) {
  const int per_lane = (E + 31) / 32;
  const int blocks = (int)((tokens + 7) / 8);
#define SGLB_TOPK(P)                                                                                            \
  topk_softmax_kernel<T, P><<<blocks, 256, 0, st>>>(static_cast<const T*>(logits), w, ids, (int32_t)tokens, E, topk, \
                                                    renorm)
  if (per_lane <= 1) SGLB_TOPK(1);
  else if (per_lane <= 2) SGLB_TOPK(2);
  else if (per_lane <= 4) SGLB_TOPK(4);
  else if (per_lane <= 8) SGLB_TOPK(8);
  else if (per_lane <= 16) SGLB_TOPK(16);
  else SGLB_TOPK(32);
#undef SGLB_TOPK
  SGLB_CHECK_LAUNCH("topk_softmax_kernel");
  return SGLB200_OK;
}

template <typename T>
int launch_gate(const void* logits, const void* bias, float* w, int32_t* ids, int64_t tokens, int32_t E, int32_t G,
                int32_t topk_group, int32_t topk, int32_t n_shared, float rsf, int apply_rsf, cudaStream_t st) {
  const int per_lane = (E + 31) / 32;
  const int blocks = (int)((tokens + 7) / 8);
  const size_t smem = (size_t)8 * E * sizeof(float);
#define SGLB_GATE(P)                                                                                        \
  fused_gate_kernel<T, P><<<blocks, 256, smem, st>>>(static_cast<const T*>(logits), static_cast<const T*>(bias), w, \
                                                     ids, (int32_t)tokens, E, G, topk_group, topk, n_shared, rsf,  \
                                                     apply_rsf)
  if (per_lane <= 1) SGLB_GATE(1);
  else if (per_lane <= 2) SGLB_GATE(2);
  else if (per_lane <= 4) SGLB_GATE(4);
  else if (per_lane <= 8) SGLB_GATE(8);
  else if (per_lane <= 16) SGLB_GATE(16);
  else SGLB_GATE(32);
#undef SGLB_GATE
  SGLB_CHECK_LAUNCH("fused_gate_kernel");
  return SGLB200_OK;
}

}  // namespace
}  // namespace sglb

using namespace sglb;

extern "C" int sglb200_topk_softmax(const void* gating_output, int dtype, float* topk_weights, int32_t* topk_ids,
                                    int64_t num_tokens, int64_t num_experts, int64_t topk, int renormalize,
                                    void* stream) {
  SGLB_REQUIRE(num_tokens >= 0 && num_experts >= 1 && num_experts <= 32 * kMaxPerLane, SGLB200_ERR_SHAPE,
               "num_tokens=%lld num_experts=%lld (1..1024)", (long long)num_tokens, (long long)num_experts);
  SGLB_REQUIRE(topk >= 1 && topk <= num_experts, SGLB200_ERR_SHAPE, "topk=%lld must be in 1..num_experts",
               (long long)topk);
  SGLB_REQUIRE(dtype == SGLB200_BF16 || dtype == SGLB200_F16 || dtype == SGLB200_F32, SGLB200_ERR_DTYPE, "dtype=%d",
               dtype);
  if (num_tokens == 0) return SGLB200_OK;
  SGLB_REQUIRE(gating_output && topk_weights && topk_ids, SGLB200_ERR_NULL, "pointers must not be NULL");
  SGLB_REQUIRE(num_tokens < ((int64_t)1 << 31), SGLB200_ERR_SHAPE, "num_tokens too large");
  if (int rc = arch_ok()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SGLB200_BF16:
      return launch_topk<__nv_bfloat16>(gating_output, topk_weights, topk_ids, num_tokens, (int32_t)num_experts,
                                        (int32_t)topk, renormalize, st);
    case SGLB200_F16:
      return launch_topk<__half>(gating_output, topk_weights, topk_ids, num_tokens, (int32_t)num_experts,
                                 (int32_t)topk, renormalize, st);
    default:
      return launch_topk<float>(gating_output, topk_weights, topk_ids, num_tokens, (int32_t)num_experts, (int32_t)topk,
                                renormalize, st);
  }
}

extern "C" int sglb200_moe_fused_gate(const void* input, const void* bias, int dtype, float* topk_weights,
                                      int32_t* topk_ids, int64_t num_tokens, int64_t num_experts,
                                      int64_t num_expert_group, int64_t topk_group, int64_t topk,
                                      int64_t num_fused_shared_experts, float routed_scaling_factor,
                                      int apply_routed_scaling_factor_on_output, void* stream) {
  SGLB_REQUIRE(num_tokens >= 0 && num_tokens < ((int64_t)1 << 31), SGLB200_ERR_SHAPE, "num_tokens=%lld",
               (long long)num_tokens);
  SGLB_REQUIRE(num_experts >= 2 && num_experts <= 1024, SGLB200_ERR_SHAPE, "num_experts=%lld (2..1024)",
               (long long)num_experts);
  SGLB_REQUIRE(num_expert_group >= 1 && num_expert_group <= 32 && num_experts % num_expert_group == 0 &&
                   num_experts / num_expert_group >= 2,
               SGLB200_ERR_SHAPE, "num_expert_group=%lld must be 1..32, divide num_experts=%lld, and leave >= 2 experts per group",
               (long long)num_expert_group, (long long)num_experts);
  SGLB_REQUIRE(topk_group >= 1 && topk_group <= num_expert_group, SGLB200_ERR_SHAPE, "topk_group=%lld (1..%lld)",
               (long long)topk_group, (long long)num_expert_group);
  SGLB_REQUIRE(num_fused_shared_experts >= 0 && num_fused_shared_experts < topk, SGLB200_ERR_SHAPE,
               "num_fused_shared_experts=%lld must be in 0..topk-1", (long long)num_fused_shared_experts);
  SGLB_REQUIRE(topk >= 1 && topk <= 32 &&
                   topk - num_fused_shared_experts <= topk_group * (num_experts / num_expert_group),
               SGLB200_ERR_SHAPE, "topk=%lld must be 1..32 and fit into the selected groups", (long long)topk);
  SGLB_REQUIRE(num_fused_shared_experts == 0 || routed_scaling_factor != 0.f, SGLB200_ERR_SHAPE,
               "routed_scaling_factor must not be 0 with fused shared experts");
  SGLB_REQUIRE(dtype == SGLB200_BF16 || dtype == SGLB200_F16 || dtype == SGLB200_F32, SGLB200_ERR_DTYPE, "dtype=%d",
               dtype);
  if (num_tokens == 0) return SGLB200_OK;
  SGLB_REQUIRE(input && bias && topk_weights && topk_ids, SGLB200_ERR_NULL, "pointers must not be NULL");
  if (int rc = arch_ok()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int32_t E = (int32_t)num_experts, G = (int32_t)num_expert_group, tg = (int32_t)topk_group, k = (int32_t)topk,
                ns = (int32_t)num_fused_shared_experts;
  switch (dtype) {
    case SGLB200_BF16:
      return launch_gate<__nv_bfloat16>(input, bias, topk_weights, topk_ids, num_tokens, E, G, tg, k, ns,
                                        routed_scaling_factor, apply_routed_scaling_factor_on_output, st);
    case SGLB200_F16:
      return launch_gate<__half>(input, bias, topk_weights, topk_ids, num_tokens, E, G, tg, k, ns,
                                 routed_scaling_factor, apply_routed_scaling_factor_on_output, st);
    default:
      return launch_gate<float>(input, bias, topk_weights, topk_ids, num_tokens, E, G, tg, k, ns,
                                routed_scaling_factor, apply_routed_scaling_factor_on_output, st);
  }
}

extern "C" int sglb200_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int64_t num_buckets,
                                            int64_t block_size, int32_t* sorted_token_ids, int32_t* expert_ids,
                                            int32_t* num_tokens_post_pad, int32_t* cumsum, int pad_sorted_token_ids,
                                            void* stream) {
  SGLB_REQUIRE(numel >= 0 && numel <= (1 << 24), SGLB200_ERR_SHAPE, "numel=%lld (0..2^24)", (long long)numel);
  SGLB_REQUIRE(num_buckets >= 1 && num_buckets <= 1024, SGLB200_ERR_SHAPE, "num_buckets=%lld (1..1024)",
               (long long)num_buckets);
  SGLB_REQUIRE(block_size >= 1 && block_size <= 4096, SGLB200_ERR_SHAPE, "block_size=%lld", (long long)block_size);
  SGLB_REQUIRE(sorted_token_ids && expert_ids && num_tokens_post_pad && (topk_ids || numel == 0), SGLB200_ERR_NULL,
               "pointers must not be NULL");
  if (int rc = arch_ok()) return rc;
  const size_t smem = ((size_t)kAlignWarps * num_buckets + kAlignThreads + num_buckets + 1) * sizeof(int32_t);
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(moe_align_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(((size_t)kAlignWarps * 1024 + kAlignThreads + 1025) * sizeof(int32_t)));
    if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done[dev] = true;
  }
  moe_align_kernel<<<1, kAlignThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      topk_ids, sorted_token_ids, expert_ids, num_tokens_post_pad, cumsum, (int32_t)numel, (int32_t)num_buckets,
      (int32_t)block_size, pad_sorted_token_ids);
  SGLB_CHECK_LAUNCH("moe_align_kernel");
  return SGLB200_OK;
}

extern "C" int sglb200_moe_sum_reduce(const void* input, void* output, int64_t num_tokens, int64_t topk,
                                      int64_t hidden, int dtype, float routed_scaling_factor, void* stream) {
  SGLB_REQUIRE(num_tokens >= 0 && topk >= 1 && hidden >= 0, SGLB200_ERR_SHAPE, "num_tokens=%lld topk=%lld hidden=%lld",
               (long long)num_tokens, (long long)topk, (long long)hidden);
  SGLB_REQUIRE(dtype == SGLB200_BF16 || dtype == SGLB200_F16, SGLB200_ERR_DTYPE, "dtype=%d", dtype);
  SGLB_REQUIRE(hidden % 8 == 0, SGLB200_ERR_SHAPE, "hidden=%lld must be a multiple of 8", (long long)hidden);
  if (num_tokens == 0 || hidden == 0) return SGLB200_OK;
  SGLB_REQUIRE(input && output, SGLB200_ERR_NULL, "input/output must not be NULL");
  SGLB_REQUIRE(aligned(input, 16) && aligned(output, 16), SGLB200_ERR_ALIGN, "input/output must be 16-byte aligned");
  if (int rc = arch_ok()) return rc;
  DeviceInfo di;
  device_info(&di);
  const int64_t total = num_tokens * (hidden / 8);
  int64_t blocks = (total + 255) / 256;
  if (blocks > (int64_t)di.sm_count * 16) blocks = (int64_t)di.sm_count * 16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == SGLB200_BF16) {
    moe_sum_reduce_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(input), static_cast<__nv_bfloat16*>(output), num_tokens, (int32_t)topk,
        (int32_t)hidden, routed_scaling_factor);
  } else {
    moe_sum_reduce_kernel<__half><<<(int)blocks, 256, 0, st>>>(static_cast<const __half*>(input),
                                                              static_cast<__half*>(output), num_tokens, (int32_t)topk,
                                                              (int32_t)hidden, routed_scaling_factor);
  }
  SGLB_CHECK_LAUNCH("moe_sum_reduce_kernel");
  return SGLB200_OK;
}
