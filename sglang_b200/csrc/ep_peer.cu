// Expert-parallel token dispatch and combine over peer memory (CUDA-IPC mapped buffers, NVLink): no collective
// library call and no host round trip for the row counts.
//
// Every rank owns one exchange buffer that all ranks map:
//   recv_q    [capacity][H]        e4m3 rows received for this rank's experts
//   recv_s    [capacity][H / 128]  their group scales
//   recv_meta [capacity][2]        (source rank, token index at the source)
//   recv_ids  [capacity][topk]     expert ids relative to this rank's first expert, -1 = not here
//   recv_w    [capacity][topk]     routing weights
//   comb      [world][m_max][H]    partial output rows coming back: comb[r][t] = what rank r's experts add to my token t
//   ctl       row counters (one per epoch parity), completion flags per source rank, block tickets, and the number of
//             exchanges this rank has completed: the epoch of an exchange is that number + 1, read by all four kernels
//             and advanced by the last block of the combine-reduce kernel, so a captured CUDA graph of the layer can be
//             replayed
// dispatch:        one warp per token; for every rank that owns one of the token's experts it reserves a row there with
//                  a remote atomic and stores the quantised row, scales, ids and weights; the last block raises this
//                  rank's "done" flag on every peer.
// receive:         waits (bounded) for all done flags, then marks the rows past the received count as empty (ids -1).
// combine push:    one warp per received row: the partial output row goes to comb[this rank][token] at its source; the
//                  last block raises this rank's "returned" flag on every peer.
// combine reduce:  waits (bounded) for all returned flags, then out[t] = sum over the ranks that own an expert of t, in
//                  ascending rank order, fp32.
// The order in which rows arrive at an expert rank depends on timing; the result does not (rows are independent in the
// expert MLP and the sums are taken in a fixed order).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"
#include "quant_vec.cuh"

namespace sglb {

__device__ int g_ep_status = 0;

int ep_take_device_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_ep_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (v != 0) {
    const int z = 0;
    cudaMemcpyToSymbol(g_ep_status, &z, sizeof(int));
  }
  return v;
}

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxTopk = 32;
// control words (uint32)
constexpr int kCtlCount = 0;      // [2]   rows received, per epoch parity
constexpr int kCtlTicket = 2;     // [3]   block tickets of the dispatch / combine-push / combine-reduce kernels
constexpr int kCtlEpoch = 5;      //       exchanges completed by this rank; the epoch in flight is this + 1
constexpr int kCtlFailed = 6;     //       a block of the combine-reduce kernel gave up waiting
constexpr int kCtlDone = 8;       // [2][8] source rank r finished dispatching epoch e
constexpr int kCtlReturned = 24;  // [2][8] expert rank r finished returning partial rows of epoch e
constexpr int kCtlWords = 64;

struct Layout {
  int64_t q, s, meta, ids, w, comb, ctl, total;
};

__host__ __device__ inline int64_t up16(int64_t x) { return (x + 15) / 16 * 16; }

__host__ __device__ inline Layout make_layout(int64_t capacity, int64_t H, int64_t topk, int64_t world, int64_t m_max) {
  Layout l;
  l.q = 0;
  l.s = up16(l.q + capacity * H);
  l.meta = up16(l.s + capacity * (H / 128) * 4);
  l.ids = up16(l.meta + capacity * 2 * 4);
  l.w = up16(l.ids + capacity * topk * 4);
  l.comb = up16(l.w + capacity * topk * 4);
  l.ctl = up16(l.comb + world * m_max * H * 2);
  l.total = l.ctl + kCtlWords * 4;
  return l;
}

struct EpParams {
  char* peer[kMaxRanks];  // every rank's buffer as mapped here; peer[rank] is this rank's own
  Layout lay;
  int32_t rank, world, H, topk, e_local, capacity, m_max;
  uint64_t limit_ns;
};

__device__ __forceinline__ uint32_t epoch_of(const EpParams& p) {
  return *reinterpret_cast<volatile uint32_t*>(reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.lay.ctl) + kCtlEpoch) + 1u;
}

__device__ __forceinline__ uint32_t* ctl_of(const EpParams& p, int r) {
  return reinterpret_cast<uint32_t*>(p.peer[r] + p.lay.ctl);
}

// last-block pattern: every block calls this after its stores; the last one raises flag word `which` + parity * 8 +
// rank on every peer
__device__ __forceinline__ void finish_and_flag(const EpParams& p, uint32_t epoch, int ticket_idx, int which) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* my = ctl_of(p, p.rank);
    if (atomicAdd(&my[kCtlTicket + ticket_idx], 1u) == gridDim.x - 1) {
      my[kCtlTicket + ticket_idx] = 0;
      __threadfence_system();
      const uint32_t par = epoch & 1u;
      for (int r = 0; r < p.world; ++r) ptx::st_release_sys_u32(ctl_of(p, r) + which + par * 8 + p.rank, epoch);
    }
  }
}

// block-wide bounded wait until word base[r] reached the epoch for every r < world; false on time-out
__device__ __forceinline__ bool wait_flags(const EpParams& p, uint32_t epoch, const uint32_t* base, int code) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < p.world) {
    uint64_t t0 = 0;
    uint32_t polls = 0;
    while ((int32_t)(ptx::ld_acquire_sys_u32(base + threadIdx.x) - epoch) < 0) {
      if ((++polls & 255u) == 0) {
        const uint64_t now = ptx::global_timer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if ((int64_t)(now - t0) > (int64_t)p.limit_ns) {
          s_ok = 0;
          atomicCAS(&g_ep_status, 0, code);
          break;
        }
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const EpParams p, const uint8_t* __restrict__ q, const float* __restrict__ s, int64_t s_stride_m,
                   int64_t s_stride_k, const int32_t* __restrict__ topk_ids, const float* __restrict__ topk_w,
                   int32_t M) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t epoch = epoch_of(p), par = epoch & 1u;
  const int G = p.H / 128, vecs = p.H / 16;
  for (int32_t t = blockIdx.x * 8 + warp; t < M; t += gridDim.x * 8) {
    int32_t id = -1;
    float w = 0.f;
    if (lane < p.topk) {
      id = __ldg(topk_ids + (int64_t)t * p.topk + lane);
      w = __ldg(topk_w + (int64_t)t * p.topk + lane);
    }
    const int owner = (id >= 0 && id / p.e_local < p.world) ? id / p.e_local : -1;
    for (int r = 0; r < p.world; ++r) {
      if (!__any_sync(0xffffffffu, owner == r)) continue;
      uint32_t slot = 0;
      if (lane == 0) slot = atomicAdd_system(ctl_of(p, r) + kCtlCount + par, 1u);
      slot = __shfl_sync(0xffffffffu, slot, 0);
      if (slot >= (uint32_t)p.capacity) {
        if (lane == 0) atomicCAS(&g_ep_status, 0, 23);  // receive buffer of rank r is full: the row is dropped
        continue;
      }
      char* dst = p.peer[r];
      const uint4* src = reinterpret_cast<const uint4*>(q + (int64_t)t * p.H);
      uint4* dq = reinterpret_cast<uint4*>(dst + p.lay.q + (int64_t)slot * p.H);
      for (int v = lane; v < vecs; v += 32) dq[v] = __ldg(src + v);
      float* ds = reinterpret_cast<float*>(dst + p.lay.s) + (int64_t)slot * G;
      for (int g = lane; g < G; g += 32) ds[g] = __ldg(s + (int64_t)t * s_stride_m + (int64_t)g * s_stride_k);
      if (lane < p.topk) {
        reinterpret_cast<int32_t*>(dst + p.lay.ids)[(int64_t)slot * p.topk + lane] = owner == r ? id - r * p.e_local : -1;
        reinterpret_cast<float*>(dst + p.lay.w)[(int64_t)slot * p.topk + lane] = w;
      }
      if (lane == 0) {
        int32_t* dm = reinterpret_cast<int32_t*>(dst + p.lay.meta) + (int64_t)slot * 2;
        dm[0] = p.rank;
        dm[1] = t;
      }
    }
  }
  finish_and_flag(p, epoch, 0, kCtlDone);
}

// Dispatch with the activation quantiser in front of it: one warp per token reads the 16-bit row once, reserves the
// token's rows on the owning ranks (lane r asks rank r, so the remote atomics overlap), and per 128-wide group takes
// the maximum, derives the scale and stores the sixteen codes of each lane (16 bytes) straight into every owner's
// receive row.  Group size 128, e4m3 limits, fp32 scales: codes and scales are bit-identical to
// sglb200_per_token_group_quant_fp8 followed by ep_dispatch_kernel, without the [M, H] e4m3 round trip through HBM.
template <typename T>
__global__ void __launch_bounds__(256)
ep_dispatch_quant_kernel(const EpParams p, const T* __restrict__ x, int64_t ldx, const int32_t* __restrict__ topk_ids,
                         const float* __restrict__ topk_w, int32_t M, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t epoch = epoch_of(p), par = epoch & 1u;
  const int G = p.H / 128;
  const int sub = lane & 7, gsel = lane >> 3;
  const float inv_max = __frcp_rn(448.0f);
  for (int32_t t = blockIdx.x * 8 + warp; t < M; t += gridDim.x * 8) {
    int32_t id = -1;
    float w = 0.f;
    if (lane < p.topk) {
      id = __ldg(topk_ids + (int64_t)t * p.topk + lane);
      w = __ldg(topk_w + (int64_t)t * p.topk + lane);
    }
    const int owner = (id >= 0 && id / p.e_local < p.world) ? id / p.e_local : -1;
    uint32_t mask = 0;
    for (int r = 0; r < p.world; ++r)
      if (__any_sync(0xffffffffu, owner == r)) mask |= 1u << r;
    uint32_t my_slot = 0xffffffffu;
    if (lane < p.world && ((mask >> lane) & 1u)) {
      my_slot = atomicAdd_system(ctl_of(p, lane) + kCtlCount + par, 1u);
      if (my_slot >= (uint32_t)p.capacity) {
        atomicCAS(&g_ep_status, 0, 23);  // receive buffer of that rank is full: the row is dropped
        my_slot = 0xffffffffu;
      }
    }
    uint32_t slot[kMaxRanks];  // 0xffffffff: rank r gets no copy of this token
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      slot[r] = __shfl_sync(0xffffffffu, my_slot, r);
      if (slot[r] == 0xffffffffu) continue;
      char* dst = p.peer[r];
      if (lane < p.topk) {
        reinterpret_cast<int32_t*>(dst + p.lay.ids)[(int64_t)slot[r] * p.topk + lane] =
            owner == r ? id - r * p.e_local : -1;
        reinterpret_cast<float*>(dst + p.lay.w)[(int64_t)slot[r] * p.topk + lane] = w;
      }
      if (lane == 0) {
        int32_t* dm = reinterpret_cast<int32_t*>(dst + p.lay.meta) + (int64_t)slot[r] * 2;
        dm[0] = p.rank;
        dm[1] = t;
      }
    }
    const uint4* row = reinterpret_cast<const uint4*>(x + (int64_t)t * ldx);
#pragma unroll 2
    for (int g0 = 0; g0 < G; g0 += 4) {
      const int g = g0 + gsel;
      const bool live = g < G;
      uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
      if (live) {
        v0 = __ldcs(row + g * 16 + sub * 2);
        v1 = __ldcs(row + g * 16 + sub * 2 + 1);
      }
      float amax = fmaxf(eps, fmaxf(Elem<T>::vec_absmax(v0), Elem<T>::vec_absmax(v1)));
#pragma unroll
      for (int m = 4; m >= 1; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
      const float s = group_scale_fast(amax, 448.0f, inv_max, false);
      const uint4 codes = encode16_e4m3<T>(v0, v1, s);
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (slot[r] == 0xffffffffu || !live) continue;
        char* dst = p.peer[r];
        reinterpret_cast<uint4*>(dst + p.lay.q + (int64_t)slot[r] * p.H)[g * 8 + sub] = codes;
        if (sub == 0) reinterpret_cast<float*>(dst + p.lay.s)[(int64_t)slot[r] * G + g] = s;
      }
    }
  }
  finish_and_flag(p, epoch, 0, kCtlDone);
}

__global__ void __launch_bounds__(256) ep_receive_kernel(const EpParams p, int32_t* __restrict__ count_out) {
  uint32_t* my = ctl_of(p, p.rank);
  const uint32_t epoch = epoch_of(p), par = epoch & 1u;
  if (!wait_flags(p, epoch, my + kCtlDone + par * 8, 21)) return;
  const uint32_t n = min(*reinterpret_cast<volatile uint32_t*>(my + kCtlCount + par), (uint32_t)p.capacity);
  int32_t* ids = reinterpret_cast<int32_t*>(p.peer[p.rank] + p.lay.ids);
  const int64_t total = (int64_t)p.capacity * p.topk;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    if (i / p.topk >= n) ids[i] = -1;  // rows that were not received in this epoch
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (count_out) *count_out = (int32_t)n;
    my[kCtlCount + (par ^ 1u)] = 0;  // nobody dispatches the next epoch before this rank has returned this one's rows
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ep_combine_push_kernel(const EpParams p, const T* __restrict__ partial) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t epoch = epoch_of(p), par = epoch & 1u;
  const uint32_t n = min(*reinterpret_cast<volatile uint32_t*>(ctl_of(p, p.rank) + kCtlCount + par), (uint32_t)p.capacity);
  const int32_t* meta = reinterpret_cast<const int32_t*>(p.peer[p.rank] + p.lay.meta);
  const int vecs = p.H / 8;
  for (uint32_t i = blockIdx.x * 8 + warp; i < n; i += gridDim.x * 8) {
    const int32_t src = meta[2 * i], tok = meta[2 * i + 1];
    if (src < 0 || src >= p.world || tok < 0 || tok >= p.m_max) continue;
    const uint4* from = reinterpret_cast<const uint4*>(partial + (int64_t)i * p.H);
    uint4* to = reinterpret_cast<uint4*>(p.peer[src] + p.lay.comb) + ((int64_t)p.rank * p.m_max + tok) * vecs;
    for (int v = lane; v < vecs; v += 32) to[v] = __ldg(from + v);
  }
  finish_and_flag(p, epoch, 1, kCtlReturned);
}

template <typename T>
__global__ void __launch_bounds__(256)
ep_combine_reduce_kernel(const EpParams p, const int32_t* __restrict__ topk_ids, T* __restrict__ out, int32_t M) {
  const uint32_t epoch = epoch_of(p), par = epoch & 1u;
  const bool ok = wait_flags(p, epoch, ctl_of(p, p.rank) + kCtlReturned + par * 8, 22);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int vecs = p.H / 8;
  const uint4* comb = reinterpret_cast<const uint4*>(p.peer[p.rank] + p.lay.comb);
  for (int32_t t = blockIdx.x * 8 + warp; ok && t < M; t += gridDim.x * 8) {
    int owner = -1;
    if (lane < p.topk) {
      const int32_t id = __ldg(topk_ids + (int64_t)t * p.topk + lane);
      owner = (id >= 0 && id / p.e_local < p.world) ? id / p.e_local : -1;
    }
    uint32_t mask = 0;
    for (int r = 0; r < p.world; ++r)
      if (__any_sync(0xffffffffu, owner == r)) mask |= 1u << r;
    for (int v = lane; v < vecs; v += 32) {
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = 0.f;
      for (int r = 0; r < p.world; ++r) {
        if (!((mask >> r) & 1u)) continue;
        const uint4 u = __ldcv(comb + ((int64_t)r * p.m_max + t) * vecs + v);  // written by a peer: bypass L1
        const T* h = reinterpret_cast<const T*>(&u);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] += static_cast<float>(h[j]);
      }
      uint4 o;
      T* oh = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) oh[j] = static_cast<T>(a[j]);
      reinterpret_cast<uint4*>(out + (int64_t)t * p.H)[v] = o;
    }
  }
  // every block has read the epoch by now; the last one closes the exchange (not if a block gave up: the exchange can
  // then be reduced again once the missing rank has caught up)
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* my = ctl_of(p, p.rank);
    if (!ok) atomicExch(&my[kCtlFailed], 1u);
    if (atomicAdd(&my[kCtlTicket + 2], 1u) == gridDim.x - 1) {
      const uint32_t failed = atomicExch(&my[kCtlFailed], 0u);
      my[kCtlTicket + 2] = 0;
      if (!failed) *reinterpret_cast<volatile uint32_t*>(my + kCtlEpoch) = epoch;
    }
  }
}

int fill_params(EpParams* p, void* const* peer_bases, int rank, int world, int64_t H, int64_t topk, int64_t e_local,
                int64_t capacity, int64_t m_max, int64_t timeout_ns) {
  SGLB_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, SGLB200_ERR_SHAPE, "world=%d (1..%d) rank=%d",
               world, kMaxRanks, rank);
  SGLB_REQUIRE(H > 0 && H % 128 == 0, SGLB200_ERR_SHAPE, "H=%lld must be a positive multiple of 128", (long long)H);
  SGLB_REQUIRE(topk >= 1 && topk <= kMaxTopk && e_local >= 1 && capacity >= 1 && m_max >= 1, SGLB200_ERR_SHAPE,
               "topk=%lld (1..%d) e_local=%lld capacity=%lld m_max=%lld", (long long)topk, kMaxTopk, (long long)e_local,
               (long long)capacity, (long long)m_max);
  SGLB_REQUIRE(peer_bases != nullptr, SGLB200_ERR_NULL, "peer_bases must not be NULL");
  for (int r = 0; r < kMaxRanks; ++r) {
    p->peer[r] = r < world ? static_cast<char*>(peer_bases[r]) : nullptr;
    SGLB_REQUIRE(r >= world || (p->peer[r] && aligned(p->peer[r], 16)), SGLB200_ERR_NULL,
                 "peer %d: buffer missing or not 16-byte aligned", r);
  }
  p->lay = make_layout(capacity, H, topk, world, m_max);
  p->rank = rank;
  p->world = world;
  p->H = (int32_t)H;
  p->topk = (int32_t)topk;
  p->e_local = (int32_t)e_local;
  p->capacity = (int32_t)capacity;
  p->m_max = (int32_t)m_max;
  p->limit_ns = timeout_ns > 0 ? (uint64_t)timeout_ns : 2000000000ull;
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  SGLB_REQUIRE(di.cc_major == 10, SGLB200_ERR_ARCH, "compute capability %d.%d: this library is built for sm_100a only",
               di.cc_major, di.cc_minor);
  return SGLB200_OK;
}

int grid_for(int64_t warps_of_work) {
  DeviceInfo di;
  device_info(&di);
  int64_t blocks = (warps_of_work + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > (int64_t)di.sm_count * 4) blocks = (int64_t)di.sm_count * 4;
  return (int)blocks;
}

}  // namespace
}  // namespace sglb

using namespace sglb;

extern "C" int64_t sglb200_ep_buffer_bytes(int64_t capacity, int64_t H, int64_t topk, int64_t world, int64_t m_max) {
  if (capacity <= 0 || H <= 0 || topk <= 0 || world <= 0 || m_max <= 0) return 0;
  return make_layout(capacity, H, topk, world, m_max).total;
}

extern "C" int sglb200_ep_buffer_offsets(int64_t capacity, int64_t H, int64_t topk, int64_t world, int64_t m_max,
                                         int64_t* offsets7) {
  SGLB_REQUIRE(offsets7 != nullptr && capacity > 0 && H > 0 && topk > 0 && world > 0 && m_max > 0, SGLB200_ERR_SHAPE,
               "bad layout arguments");
  const Layout l = make_layout(capacity, H, topk, world, m_max);
  const int64_t v[7] = {l.q, l.s, l.meta, l.ids, l.w, l.comb, l.ctl};
  for (int i = 0; i < 7; ++i) offsets7[i] = v[i];
  return SGLB200_OK;
}

extern "C" int sglb200_ep_dispatch(const void* q, const float* s, int64_t s_stride_m, int64_t s_stride_k,
                                   const int32_t* topk_ids, const float* topk_weights, int64_t M, int64_t H,
                                   int64_t topk, int64_t num_local_experts, void* const* peer_bases, int rank, int world,
                                   int64_t capacity, int64_t m_max, void* stream) {
  EpParams p;
  if (int rc = fill_params(&p, peer_bases, rank, world, H, topk, num_local_experts, capacity, m_max, 0)) return rc;
  SGLB_REQUIRE(M >= 0 && M <= m_max, SGLB200_ERR_SHAPE, "M=%lld must be in 0..m_max=%lld", (long long)M, (long long)m_max);
  SGLB_REQUIRE(M == 0 || (q && s && topk_ids && topk_weights && aligned(q, 16)), SGLB200_ERR_NULL,
               "q (16-byte aligned), s, topk_ids and topk_weights must be given");
  ep_dispatch_kernel<<<grid_for(M), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      p, static_cast<const uint8_t*>(q), s, s_stride_m, s_stride_k, topk_ids, topk_weights, (int32_t)M);
  SGLB_CHECK_LAUNCH("ep_dispatch_kernel");
  return SGLB200_OK;
}

extern "C" int sglb200_ep_dispatch_quant(const void* x, int in_dtype, int64_t ldx, const int32_t* topk_ids,
                                         const float* topk_weights, int64_t M, int64_t H, int64_t topk,
                                         int64_t num_local_experts, void* const* peer_bases, int rank, int world,
                                         int64_t capacity, int64_t m_max, float eps, void* stream) {
  SGLB_REQUIRE(in_dtype == SGLB200_BF16 || in_dtype == SGLB200_F16, SGLB200_ERR_DTYPE, "in_dtype=%d: bf16 or f16", in_dtype);
  SGLB_REQUIRE(ldx >= H && ldx % 8 == 0, SGLB200_ERR_SHAPE, "ldx=%lld must be >= H and a multiple of 8", (long long)ldx);
  SGLB_REQUIRE(eps >= 0.f, SGLB200_ERR_SHAPE, "eps must be >= 0");
  EpParams p;
  if (int rc = fill_params(&p, peer_bases, rank, world, H, topk, num_local_experts, capacity, m_max, 0)) return rc;
  SGLB_REQUIRE(M >= 0 && M <= m_max, SGLB200_ERR_SHAPE, "M=%lld must be in 0..m_max=%lld", (long long)M, (long long)m_max);
  SGLB_REQUIRE(M == 0 || (x && topk_ids && topk_weights), SGLB200_ERR_NULL, "x, topk_ids and topk_weights must be given");
  SGLB_REQUIRE(M == 0 || aligned(x, 16), SGLB200_ERR_ALIGN, "x must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(M);
  if (in_dtype == SGLB200_BF16)
    ep_dispatch_quant_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, static_cast<const __nv_bfloat16*>(x), ldx, topk_ids,
                                                                    topk_weights, (int32_t)M, eps);
  else
    ep_dispatch_quant_kernel<__half><<<grid, 256, 0, st>>>(p, static_cast<const __half*>(x), ldx, topk_ids, topk_weights,
                                                             (int32_t)M, eps);
  SGLB_CHECK_LAUNCH("ep_dispatch_quant_kernel");
  return SGLB200_OK;
}

extern "C" int sglb200_ep_receive(void* const* peer_bases, int rank, int world, int64_t H, int64_t topk,
                                  int64_t num_local_experts, int64_t capacity, int64_t m_max, int32_t* count_out,
                                  int64_t timeout_ns, void* stream) {
  EpParams p;
  if (int rc = fill_params(&p, peer_bases, rank, world, H, topk, num_local_experts, capacity, m_max, timeout_ns))
    return rc;
  ep_receive_kernel<<<grid_for(capacity * topk / 256 + 1), 256, 0, static_cast<cudaStream_t>(stream)>>>(p, count_out);
  SGLB_CHECK_LAUNCH("ep_receive_kernel");
  return SGLB200_OK;
}

extern "C" int sglb200_ep_combine_push(const void* partial, int dtype, void* const* peer_bases, int rank, int world,
                                       int64_t H, int64_t topk, int64_t num_local_experts, int64_t capacity,
                                       int64_t m_max, void* stream) {
  EpParams p;
  if (int rc = fill_params(&p, peer_bases, rank, world, H, topk, num_local_experts, capacity, m_max, 0)) return rc;
  SGLB_REQUIRE(dtype == SGLB200_BF16 || dtype == SGLB200_F16, SGLB200_ERR_DTYPE, "dtype=%d", dtype);
  SGLB_REQUIRE(partial && aligned(partial, 16), SGLB200_ERR_NULL, "partial must be given, 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(capacity);
  if (dtype == SGLB200_BF16)
    ep_combine_push_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, static_cast<const __nv_bfloat16*>(partial));
  else
    ep_combine_push_kernel<__half><<<grid, 256, 0, st>>>(p, static_cast<const __half*>(partial));
  SGLB_CHECK_LAUNCH("ep_combine_push_kernel");
  return SGLB200_OK;
}

extern "C" int sglb200_ep_combine_reduce(void* const* peer_bases, int rank, int world, const int32_t* topk_ids,
                                         void* out, int dtype, int64_t M, int64_t H, int64_t topk,
                                         int64_t num_local_experts, int64_t capacity, int64_t m_max, int64_t timeout_ns,
                                         void* stream) {
  EpParams p;
  if (int rc = fill_params(&p, peer_bases, rank, world, H, topk, num_local_experts, capacity, m_max, timeout_ns))
    return rc;
  SGLB_REQUIRE(dtype == SGLB200_BF16 || dtype == SGLB200_F16, SGLB200_ERR_DTYPE, "dtype=%d", dtype);
  SGLB_REQUIRE(M >= 0 && M <= m_max, SGLB200_ERR_SHAPE, "M=%lld must be in 0..m_max=%lld", (long long)M, (long long)m_max);
  SGLB_REQUIRE(M == 0 || (topk_ids && out && aligned(out, 16)), SGLB200_ERR_NULL, "topk_ids and out must be given");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(M);
  if (dtype == SGLB200_BF16)
    ep_combine_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, topk_ids, static_cast<__nv_bfloat16*>(out), (int32_t)M);
  else
    ep_combine_reduce_kernel<__half><<<grid, 256, 0, st>>>(p, topk_ids, static_cast<__half*>(out), (int32_t)M);
  SGLB_CHECK_LAUNCH("ep_combine_reduce_kernel");
  return SGLB200_OK;
}

extern "C" int sglb200_ep_completed(const void* local_base, int64_t capacity, int64_t H, int64_t topk, int64_t world,
                                    int64_t m_max, int64_t* completed) {
  SGLB_REQUIRE(local_base && completed && capacity > 0 && H > 0 && topk > 0 && world > 0 && m_max > 0, SGLB200_ERR_NULL,
               "local_base, completed and the layout arguments must be given");
  const Layout l = make_layout(capacity, H, topk, world, m_max);
  uint32_t v = 0;
  cudaError_t e = cudaMemcpy(&v, static_cast<const char*>(local_base) + l.ctl + kCtlEpoch * 4, sizeof(v),
                             cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaMemcpy: %s", cudaGetErrorString(e));
  *completed = v;
  return SGLB200_OK;
}
