// Pieces shared by the multicast (NVSwitch) all-reduce kernel (nvls.cu) and the GEMM whose extra CTAs run the same
// reduction on finished row blocks (gemm.cu): flag-block layout, the cross-rank barrier and the multimem accessors.
#pragma once
#include <cstdint>

#include "ptx.cuh"

namespace sglb {
namespace nvls {

constexpr int kBlocks = 128;  // most blocks a launch may use (the flag block has a word per block and source rank)
constexpr int kMaxRanks = 8;
// flag block of a rank, in 32-bit words: [2 barriers][kMaxRanks sources][kBlocks] flags, then [kBlocks] epochs
constexpr int kFlagWords = 2 * kMaxRanks * kBlocks;
constexpr int kCtlWords = kBlocks;

struct FlagPtrs {
  uint32_t* p[kMaxRanks];  // flag block of every rank, as mapped into this process
};

template <bool BF16>
__device__ __forceinline__ uint4 mm_ld_reduce(uint64_t addr) {
  uint4 v;
  if constexpr (BF16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(addr)
                 : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(addr)
                 : "memory");
  return v;
}

template <bool BF16>
__device__ __forceinline__ void mm_st(uint64_t addr, uint4 v) {
  if constexpr (BF16)
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
  else
    asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}

// Barrier between block `block` of every rank.  Threads 0 .. world-1 each signal one peer and wait for one peer.
// Returns false (uniformly over the CTA) when a wait ran out; *status (a device word of the calling translation unit)
// then holds `code` unless it was already set.
__device__ __forceinline__ bool rank_barrier(const FlagPtrs& fp, int which, int block, int rank, int world, uint32_t epoch,
                                             uint64_t limit_ns, int* s_ok, int* status, int code) {
  __syncthreads();  // everything this CTA did so far is ordered before the signal
  if ((int)threadIdx.x < world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    ptx::st_release_sys_u32(fp.p[peer] + ((which * kMaxRanks + rank) * kBlocks + block), epoch);
    const uint32_t* f = fp.p[rank] + ((which * kMaxRanks + peer) * kBlocks + block);
    uint64_t t0 = 0;
    uint32_t polls = 0;
    while ((int32_t)(ptx::ld_acquire_sys_u32(f) - epoch) < 0) {
      if ((++polls & 255u) == 0) {
        const uint64_t now = ptx::global_timer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if ((int64_t)(now - t0) > (int64_t)limit_ns) {
          *s_ok = 0;
          atomicCAS(status, 0, code);
          break;
        }
      }
    }
  }
  __syncthreads();
  return *s_ok != 0;
}

// Sum over the ranks of vectors [v0, v1) (16 bytes each) of the multicast buffer at mc_base, written back to every rank;
// the calling CTAs share the range: CTA `part` of `parts`, `threads` threads each.
template <bool BF16, int UNROLL>
__device__ __forceinline__ void reduce_range(uint64_t mc_base, int64_t v0, int64_t v1, int part, int parts, int threads) {
  const int64_t stride = (int64_t)parts * threads;
  for (int64_t v = v0 + (int64_t)part * threads + threadIdx.x; v < v1; v += stride * UNROLL) {
    uint4 r[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (v + u * stride < v1) r[u] = mm_ld_reduce<BF16>(mc_base + (uint64_t)(v + u * stride) * 16u);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (v + u * stride < v1) mm_st<BF16>(mc_base + (uint64_t)(v + u * stride) * 16u, r[u]);
  }
}

}  // namespace nvls
}  // namespace sglb
