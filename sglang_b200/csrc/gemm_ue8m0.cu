// Block-scaled FP8 GEMM with POWER-OF-TWO (UE8M0) scales, using the tensor core's own block scaling.
//
//   out[m, n] = cast( sum_k a[m,k] * 2^ea[m, k/128] * b[n,k] * 2^eb[n/128, k/128] )
//
// With power-of-two scales the scaling can be applied by tcgen05.mma kind::mxf8f6f4.block_scale itself (one UE8M0
// factor per row per 32 elements of K, exact), so the whole K loop accumulates in TMEM like an ordinary GEMM and
// there is no per-k-block promotion through registers, which is what bounds the fp32-scale kernel in gemm.cu.
// This is the arrangement the reference uses on Blackwell through DeepGEMM (UE8M0 activation scales from the
// quantiser, weights requantised to UE8M0: python/sglang/srt/layers/quantization/fp8_utils.py:416-512,
// deep_gemm_wrapper/configurer.py:24-25).
//
// One CTA per SM, 416 threads:
//   warps 0-1   TMA producers (k-blocks alternate): A tile 128 x 128 B and B tile 224 x 128 B into a 4-stage ring.
//   warp 2      the MMA issuer (one thread): per k-block four 128 x 224 x 32 block-scaled MMAs into one of TWO
//               224-column TMEM accumulators (tiles alternate, so the epilogue of a tile overlaps the next tile's
//               MMAs).  Before the first k-block of every group of four it copies that group's scale words from shared
//               memory into TMEM scale columns (tcgen05.cp; two sets, alternating).  All tensor-pipe work comes from
//               this one thread, so copies and MMAs execute in the order they were issued.
//   warp 3      idle.
//   warp 4      scale loader: per tile and per group of four k-blocks, 128 packed scale words of A (one int32 holds the
//               four exponent bytes of a row, the layout the quantiser writes) and 224 of B, written to shared memory
//               in the 32 x 16 B arrangement tcgen05.cp.32x128b.warpx4 expects (lane l: rows l, l+32, l+64, l+96).
//               The k-block inside the group picks the byte through the instruction descriptor's scale ids.
//   warps 5-12  epilogue: after the last k-block of a tile, its accumulator -> bf16/f16 rows.
// Every mbarrier wait is bounded; on time-out the CTA records a code in g_device_status and winds down.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace sglb {

// status word of this kernel's bounded waits (device variables are private to a translation unit; the public
// reader in gemm.cu collects this one through ue8m0_take_device_status)
__device__ int g_ue8m0_status = 0;
// Optional mirror of the status word in host-mapped memory (survives a lost context); set by the debug hook below.
__device__ volatile int* g_ue8m0_mirror = nullptr;
int ue8m0_take_device_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_ue8m0_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_ue8m0_status, &z, sizeof(int));
  }
  return v;
}

namespace {

constexpr int BM = 128, BN = 224, BK = 128;
constexpr int kStages = 4;
constexpr int kSfBufs = 4;
constexpr int kThreads = 13 * 32;
constexpr int kEpiWarp0 = 5, kEpiWarps = 8;
constexpr int kEpiCols = BN / 2;  // 112 columns per epilogue warp: three loads of 32 and one of 16
constexpr uint32_t kTileABytes = BM * BK, kTileBBytes = BN * BK, kStageBytes = kTileABytes + kTileBBytes;
constexpr uint32_t kSfABytes = 512, kSfBBytes = 1024, kSfBufBytes = kSfABytes + kSfBBytes;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSfTmemBase = 2 * BN;  // 448: scale columns start after the two accumulators
constexpr uint32_t kSfTmemPerSet = 12;    // 4 columns for A's scales + 8 for B's (224 rows -> two copies of 128)
constexpr int kGroupM = 16;
constexpr int kMaxExperts = 1024;
constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + (size_t)kSfBufs * kSfBufBytes + 256 +
                              (kMaxExperts + 1) * sizeof(int32_t);

struct Params {
  const int32_t* sfa;  // packed exponents of A: word (m, kg) at sfa[kg * sfa_ld + m * sfa_stride_m]
  const int32_t* sfb;  // of B: word (e, nb, kg) at sfb[e * sfb_stride_e + nb * sfb_stride_n + kg * sfb_stride_k]
  void* out;
  const int32_t* expert_offsets;  // grouped: rows of expert e are [expert_offsets[e], expert_offsets[e + 1])
  int32_t M, N, K, num_experts;   // M = total rows of a / out
  int32_t m_tiles, n_tiles, k_tiles, k_groups;
  int64_t ldc, sfa_ld, sfa_stride_m, sfb_stride_e, sfb_stride_n, sfb_stride_k;
  int32_t out_dtype;
};

struct Ctl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t sf_full[kSfBufs];
  uint64_t sf_empty[kSfBufs];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  int32_t total_tiles;
};
static_assert(sizeof(Ctl) <= 256, "control block");

struct TileUe {
  int32_t m0, row_end, n0, expert;
};

// dense: grouped-M raster; grouped: tile table of the experts (prefix sums in shared memory), n-major inside an expert
template <bool GROUPED>
__device__ __forceinline__ TileUe tile_coords(const Params& p, const int32_t* tile_start, int32_t t) {
  TileUe tl;
  if constexpr (!GROUPED) {
    const int32_t per_group = kGroupM * p.n_tiles;
    const int32_t gid = t / per_group;
    const int32_t first_m = gid * kGroupM;
    const int32_t gm = min(p.m_tiles - first_m, kGroupM);
    const int32_t local = t - gid * per_group;
    const int32_t nt = local / gm;
    tl.m0 = (first_m + (local - nt * gm)) * BM;
    tl.row_end = p.M;
    tl.n0 = nt * BN;
    tl.expert = 0;
  } else {
    int32_t lo = 0, hi = p.num_experts;  // last e with tile_start[e] <= t
    while (hi - lo > 1) {
      const int32_t mid = (lo + hi) >> 1;
      if (tile_start[mid] <= t) lo = mid; else hi = mid;
    }
    const int32_t r0 = __ldg(p.expert_offsets + lo), r1 = __ldg(p.expert_offsets + lo + 1);
    const int32_t me = (r1 - r0 + BM - 1) / BM;
    const int32_t local = t - tile_start[lo];
    const int32_t nt = local / me;
    tl.m0 = r0 + (local - nt * me) * BM;
    tl.row_end = r1;
    tl.n0 = nt * BN;
    tl.expert = lo;
  }
  return tl;
}

__device__ __forceinline__ void timeout(Ctl* ctl, int code) {
  ctl->abort_flag = 1;
  atomicCAS(&g_ue8m0_status, 0, code);
  if (g_ue8m0_mirror != nullptr) {
    g_ue8m0_mirror[0] = code;
    g_ue8m0_mirror[1] = (int)blockIdx.x;
    __threadfence_system();
  }
}

template <typename OutT>
__device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <typename OutT>
__device__ __forceinline__ void store32(const uint32_t (&a)[32], const uint32_t (&b)[32], bool use_b, OutT* dst,
                                        int32_t n_first, int32_t N) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    if (n_first + c * 8 < N) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        v[j] = __uint_as_float(a[c * 8 + j]) + (use_b ? __uint_as_float(b[c * 8 + j]) : 0.f);
      uint4 u;
      u.x = pack_pair<OutT>(v[0], v[1]);
      u.y = pack_pair<OutT>(v[2], v[3]);
      u.z = pack_pair<OutT>(v[4], v[5]);
      u.w = pack_pair<OutT>(v[6], v[7]);
      *reinterpret_cast<uint4*>(dst + c * 8) = u;
    }
  }
}

template <bool GROUPED>
__global__ void __launch_bounds__(kThreads, 1)
fp8_ue8m0_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sf_smem = smem + (size_t)kStages * kStageBytes;
  Ctl* ctl = reinterpret_cast<Ctl*>(sf_smem + (size_t)kSfBufs * kSfBufBytes);
  int32_t* tile_start = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(ctl) + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&ctl->full[i], 1);
      ptx::mbar_init(&ctl->empty[i], 1);
    }
    for (int i = 0; i < kSfBufs; ++i) {
      ptx::mbar_init(&ctl->sf_full[i], 1);
      ptx::mbar_init(&ctl->sf_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&ctl->acc_full[i], 1);
      ptx::mbar_init(&ctl->acc_empty[i], kEpiWarps);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == 2) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  if constexpr (GROUPED) {
    if (warp == 0) {  // exclusive prefix sum of tiles per expert
      int32_t running = 0;
      for (int32_t base = 0; base < p.num_experts; base += 32) {
        const int32_t e = base + lane;
        int32_t v = 0;
        if (e < p.num_experts)
          v = ((__ldg(p.expert_offsets + e + 1) - __ldg(p.expert_offsets + e) + BM - 1) / BM) * p.n_tiles;
        int32_t incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int32_t o = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += o;
        }
        if (e < p.num_experts) tile_start[e] = running + incl - v;
        running += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) {
        tile_start[p.num_experts] = running;
        ctl->total_tiles = running;
      }
    }
  } else {
    if (threadIdx.x == 0) ctl->total_tiles = p.m_tiles * p.n_tiles;
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const int32_t total_tiles = ctl->total_tiles;

  const uint32_t full0 = ptx::smem_u32(&ctl->full[0]);
  const uint32_t empty0 = ptx::smem_u32(&ctl->empty[0]);
  const uint32_t sf_full0 = ptx::smem_u32(&ctl->sf_full[0]);
  const uint32_t sf_empty0 = ptx::smem_u32(&ctl->sf_empty[0]);
  const uint32_t acc_full0 = ptx::smem_u32(&ctl->acc_full[0]);
  const uint32_t acc_empty0 = ptx::smem_u32(&ctl->acc_empty[0]);
  const uint32_t stage0 = ptx::smem_u32(smem);
  const uint32_t sf0 = ptx::smem_u32(sf_smem);

  if (warp < 2) {
    // ===== TMA producers
    uint32_t stage = 0, phase = 0, g = 0;
    for (int32_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const TileUe tl = tile_coords<GROUPED>(p, tile_start, t);
      bool ok = true;
      for (int32_t kb = 0; kb < p.k_tiles; ++kb, ++g) {
        if ((g & 1) == (uint32_t)warp) {
          if (!ptx::mbar_wait_a(empty0 + stage * 8, phase ^ 1)) {
            timeout(ctl, 11);
            ok = false;
            break;
          }
          if (lane == 0) {
            const uint32_t dst = stage0 + stage * kStageBytes;
            ptx::mbar_arrive_expect_tx_a(full0 + stage * 8, kStageBytes);
            ptx::tma_load_2d_a(dst, &map_a, full0 + stage * 8, kb * BK, tl.m0);
            ptx::tma_load_3d_a(dst + kTileABytes, &map_b, full0 + stage * 8, kb * BK, tl.n0, tl.expert);
          }
        }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (!ok || ctl->abort_flag) break;
    }
    // Tail: tcgen05.commit arrives on the `empty` barriers asynchronously.  Nobody waits for the last ones, so
    // without this the CTA could exit (and the next kernel's CTA re-initialise barriers at the same shared-memory
    // addresses) while such an arrival is still in flight.  Acquire every stage once more before leaving.
    if (warp == 0 && !ctl->abort_flag) {
      for (int i = 0; i < kStages; ++i) {
        if (!ptx::mbar_wait_a(empty0 + stage * 8, phase ^ 1)) { timeout(ctl, 17); break; }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 2) {
    // ===== MMA issuer
    const uint64_t desc0 = ptx::make_kmajor_sw128_desc(stage0);
    uint32_t stage = 0, phase = 0, q = 0, tile_i = 0;
    for (int32_t t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_i) {
      const uint32_t as = tile_i & 1;  // accumulator of this tile
      bool ok = ptx::mbar_wait_a(acc_empty0 + as * 8, ((tile_i >> 1) & 1) ^ 1);
      if (!ok) timeout(ctl, 12);
      const uint32_t d_tmem = tmem_base + as * BN;
      for (int32_t kg = 0; kg < p.k_groups && ok; ++kg, ++q) {
        const uint32_t buf = q % kSfBufs;
        if (!ptx::mbar_wait_a(sf_full0 + buf * 8, (q / kSfBufs) & 1)) {
          timeout(ctl, 13);
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t sf_col = tmem_base + kSfTmemBase + (q & 1) * kSfTmemPerSet;
        if (lane == 0) {
          const uint32_t src = sf0 + buf * kSfBufBytes;
          ptx::tmem_cp_32x128b_warpx4(sf_col, ptx::make_sf_desc(src));
          ptx::tmem_cp_32x128b_warpx4(sf_col + 4, ptx::make_sf_desc(src + kSfABytes));
          ptx::tmem_cp_32x128b_warpx4(sf_col + 8, ptx::make_sf_desc(src + kSfABytes + 512));
          ptx::mma_commit_a(sf_empty0 + buf * 8);
        }
        const int32_t kb_end = min(kg * 4 + 4, p.k_tiles);
        for (int32_t kb = kg * 4; kb < kb_end; ++kb) {
          if (!ptx::mbar_wait_a(full0 + stage * 8, phase)) {
            timeout(ctl, 14);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          if (lane == 0) {
            const uint64_t a_desc = desc0 + (uint64_t)(stage * (kStageBytes >> 4));
            const uint64_t b_desc = a_desc + (kTileABytes >> 4);
            const uint32_t idesc = ptx::make_idesc_mxf8(BM, BN, (uint32_t)(kb & 3));
            ptx::mma_mxf8_block_scaled(d_tmem, a_desc, b_desc, idesc, sf_col, sf_col + 4, kb > 0 ? 1u : 0u);
#pragma unroll
            for (uint32_t k = 1; k < BK / 32; ++k)
              ptx::mma_mxf8_block_scaled(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, sf_col, sf_col + 4, 1u);
            ptx::mma_commit_a(empty0 + stage * 8);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok || ctl->abort_flag) break;
      if (lane == 0) ptx::mma_commit_a(acc_full0 + as * 8);  // the tile is complete when everything issued so far is
    }
  } else if (warp == 4) {
    // ===== scale loader
    const int32_t nb_last = (p.N + 127) / 128 - 1;
    uint32_t q = 0;
    for (int32_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const TileUe tl = tile_coords<GROUPED>(p, tile_start, t);
      const int32_t m0 = tl.m0, n0 = tl.n0;
      bool ok = true;
      for (int32_t kg = 0; kg < p.k_groups; ++kg, ++q) {
        const uint32_t buf = q % kSfBufs;
        if (!ptx::mbar_wait_a(sf_empty0 + buf * 8, ((q / kSfBufs) & 1) ^ 1)) {
          timeout(ctl, 15);
          ok = false;
          break;
        }
        uint8_t* dst = sf_smem + (size_t)buf * kSfBufBytes;
        const int32_t* a_col = p.sfa + (int64_t)kg * p.sfa_ld;
        uint4 va;
        va.x = (uint32_t)__ldg(a_col + (int64_t)min(m0 + lane, p.M - 1) * p.sfa_stride_m);
        va.y = (uint32_t)__ldg(a_col + (int64_t)min(m0 + 32 + lane, p.M - 1) * p.sfa_stride_m);
        va.z = (uint32_t)__ldg(a_col + (int64_t)min(m0 + 64 + lane, p.M - 1) * p.sfa_stride_m);
        va.w = (uint32_t)__ldg(a_col + (int64_t)min(m0 + 96 + lane, p.M - 1) * p.sfa_stride_m);
        reinterpret_cast<uint4*>(dst)[lane] = va;
        const int32_t* b_col = p.sfb + (int64_t)tl.expert * p.sfb_stride_e + (int64_t)kg * p.sfb_stride_k;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint4 vb;
          vb.x = (uint32_t)__ldg(b_col + (int64_t)min((n0 + j * 128 + lane) / 128, nb_last) * p.sfb_stride_n);
          vb.y = (uint32_t)__ldg(b_col + (int64_t)min((n0 + j * 128 + 32 + lane) / 128, nb_last) * p.sfb_stride_n);
          vb.z = (uint32_t)__ldg(b_col + (int64_t)min((n0 + j * 128 + 64 + lane) / 128, nb_last) * p.sfb_stride_n);
          vb.w = (uint32_t)__ldg(b_col + (int64_t)min((n0 + j * 128 + 96 + lane) / 128, nb_last) * p.sfb_stride_n);
          reinterpret_cast<uint4*>(dst + kSfABytes + j * 512)[lane] = vb;
        }
        ptx::fence_proxy_async();  // the tensor core reads this block through the async proxy
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_a(sf_full0 + buf * 8);
      }
      if (!ok || ctl->abort_flag) break;
    }
    // Tail, as for the producers: wait until both issuers' commits on every scale buffer have arrived.
    if (!ctl->abort_flag) {
      for (int i = 0; i < kSfBufs; ++i, ++q) {
        if (!ptx::mbar_wait_a(sf_empty0 + (q % kSfBufs) * 8, ((q / kSfBufs) & 1) ^ 1)) { timeout(ctl, 18); break; }
      }
    }
  } else if (warp >= kEpiWarp0) {
    // ===== epilogue (warps 5..12): TMEM lane quarter = warp % 4, column half = (warp - 5) / 4
    const int qd = warp & 3;
    const int col0 = ((warp - kEpiWarp0) >> 2) * kEpiCols;
    uint32_t tile_i = 0;
    for (int32_t t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_i) {
      const TileUe tl = tile_coords<GROUPED>(p, tile_start, t);
      const int32_t m0 = tl.m0, n0 = tl.n0;
      const uint32_t as = tile_i & 1;
      if (!ptx::mbar_wait_a(acc_full0 + as * 8, (tile_i >> 1) & 1)) {
        timeout(ctl, 16);
        break;
      }
      ptx::tc_fence_after();
      const uint32_t tlane = tmem_base + ((uint32_t)(qd * 32) << 16) + as * BN + col0;
      const int32_t row = m0 + qd * 32 + lane;
      // 112 columns = 32 + 32 + 32 + 16; the last load reads 32 columns of which the first 16 are this warp's
      // (the other 16 belong to the neighbouring half or to the other accumulator and are not stored)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t va[32];
        ptx::tmem_ld_32x32(tlane + c * 32, va);
        ptx::tmem_ld_wait(va);
        if (c == 3) {
          // all TMEM reads of this tile have landed: the issuer may overwrite this accumulator
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive_a(acc_empty0 + as * 8);
        }
        if (row < tl.row_end) {
          const int32_t n_first = n0 + col0 + c * 32;
          const int32_t n_limit = min(p.N, n0 + col0 + kEpiCols);  // do not store beyond this warp's 112 columns
          if (p.out_dtype == SGLB200_BF16) {
            store32<__nv_bfloat16>(va, va, false, static_cast<__nv_bfloat16*>(p.out) + (int64_t)row * p.ldc + n_first,
                                   n_first, n_limit);
          } else {
            store32<__half>(va, va, false, static_cast<__half*>(p.out) + (int64_t)row * p.ldc + n_first, n_first,
                            n_limit);
          }
        }
      }
      if (ctl->abort_flag) break;
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace
}  // namespace sglb

using namespace sglb;

// Debug hook (not in the public header): mirror time-out codes of the UE8M0 GEMM into host-mapped memory.
extern "C" int sglb200_debug_set_status_mirror(int* device_visible_host_ptr) {
  return (int)cudaMemcpyToSymbol(g_ue8m0_mirror, &device_visible_host_ptr, sizeof(int*));
}

namespace sglb {
namespace {
int ue8m0_common(const void* a, const void* b, const int32_t* sfa, const int32_t* sfb, void* out,
                 const int32_t* expert_offsets, int64_t M, int64_t num_experts, int64_t N, int64_t K, int64_t lda,
                 int64_t ldb, int64_t ldb_e, int64_t ldc, int64_t sfa_ld, int64_t sfa_stride_m, int64_t sfb_stride_e,
                 int64_t sfb_stride_n, int64_t sfb_stride_k, int out_dtype, void* stream, float* workspace = nullptr,
                 int64_t workspace_floats = 0) {
  const bool grouped = expert_offsets != nullptr;
  SGLB_REQUIRE(M >= 0 && N >= 0 && K >= 0, SGLB200_ERR_SHAPE, "M=%lld N=%lld K=%lld: negative size", (long long)M,
               (long long)N, (long long)K);
  SGLB_REQUIRE(out_dtype == SGLB200_BF16 || out_dtype == SGLB200_F16, SGLB200_ERR_DTYPE,
               "out_dtype=%d: only bf16 (0) and f16 (1)", out_dtype);
  SGLB_REQUIRE(M < ((int64_t)1 << 31) - 256 && N < ((int64_t)1 << 31) - 256 && K < ((int64_t)1 << 31) - 256,
               SGLB200_ERR_SHAPE, "a dimension exceeds 2^31");
  SGLB_REQUIRE(K > 0 || M == 0 || N == 0, SGLB200_ERR_SHAPE, "K must be positive");
  SGLB_REQUIRE(K % 16 == 0, SGLB200_ERR_SHAPE, "K=%lld must be a multiple of 16", (long long)K);
  SGLB_REQUIRE(N % 8 == 0, SGLB200_ERR_SHAPE, "N=%lld must be a multiple of 8 (16-byte output rows)", (long long)N);
  if (grouped)
    SGLB_REQUIRE(num_experts >= 1 && num_experts <= kMaxExperts, SGLB200_ERR_SHAPE, "num_experts=%lld: 1..%d",
                 (long long)num_experts, kMaxExperts);
  if (M == 0 || N == 0) return SGLB200_OK;
  SGLB_REQUIRE(a && b && sfa && sfb && out, SGLB200_ERR_NULL, "a/b/sfa/sfb/out must not be NULL");
  SGLB_REQUIRE(lda >= K && lda % 16 == 0 && ldb >= K && ldb % 16 == 0, SGLB200_ERR_ALIGN,
               "lda=%lld / ldb=%lld must be >= K and multiples of 16", (long long)lda, (long long)ldb);
  SGLB_REQUIRE(!grouped || (ldb_e % 16 == 0 && ldb_e >= ldb), SGLB200_ERR_ALIGN,
               "ldb_e=%lld must be a multiple of 16 and >= ldb", (long long)ldb_e);
  SGLB_REQUIRE(ldc >= N && (ldc * 2) % 16 == 0, SGLB200_ERR_ALIGN, "ldc=%lld must be >= N and a multiple of 8",
               (long long)ldc);
  SGLB_REQUIRE(aligned(a, 16) && aligned(b, 16) && aligned(out, 16) && aligned(sfa, 4) && aligned(sfb, 4),
               SGLB200_ERR_ALIGN, "a, b, out must be 16-byte aligned and the scale pointers 4-byte aligned");
  SGLB_REQUIRE(sfa_stride_m >= 1 && sfa_ld >= 1, SGLB200_ERR_SHAPE, "sfa_ld=%lld sfa_stride_m=%lld", (long long)sfa_ld,
               (long long)sfa_stride_m);
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  SGLB_REQUIRE(di.cc_major == 10, SGLB200_ERR_ARCH, "compute capability %d.%d: this library is built for sm_100a only",
               di.cc_major, di.cc_minor);

  if (!grouped && M <= 64) {
    // few rows: the weight-streaming kernel with swapped operands decodes the exponent bytes itself (gemm_smallm.cu);
    // from 65 rows up the block-scaled tile kernel below, which has no promotion, is the faster one
    int splits = 1;
    if (int rc = smallm_gemm(a, b, reinterpret_cast<const float*>(sfa), reinterpret_cast<const float*>(sfb), out, M, N, K,
                             lda, ldb, ldc, sfa_stride_m, sfa_ld, sfb_stride_n, sfb_stride_k, out_dtype, workspace,
                             workspace_floats, di.sm_count, stream, &splits, false, true))
      return rc;
    if (splits > 1) launch_splitk_reduce(workspace, out, M, N, ldc, splits, out_dtype, di.sm_count, stream);
    SGLB_CHECK_LAUNCH("splitk_reduce_kernel");
    return SGLB200_OK;
  }

  if (grouped) {
    // few rows per expert: the weight-streaming kernel decodes the exponent bytes itself (gemm_smallm.cu).  In a burst
    // the block-scaled tile kernel below is as fast; sustained it runs into the board's power cap at half the clock.
    if (const int chunk = smallm_grouped_chunk(M, num_experts, 0))
      return smallm_grouped_gemm(chunk, a, b, reinterpret_cast<const float*>(sfa), reinterpret_cast<const float*>(sfb),
                                 out, expert_offsets, nullptr, 1, M, num_experts, 0, N, K, lda, ldb, ldb_e, ldc, 0,
                                 sfa_stride_m, sfa_ld, sfb_stride_e, sfb_stride_n, sfb_stride_k, out_dtype, di.sm_count,
                                 stream, true);
  }

  alignas(64) CUtensorMap map_a, map_b;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t str[1] = {(uint64_t)lda};
    if (int rc = make_map_sw128(&map_a, a, 2, dims, str, BM, CU_TENSOR_MAP_L2_PROMOTION_L2_128B)) return rc;
  }
  {
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, grouped ? (uint64_t)num_experts : 1};
    const uint64_t str[2] = {(uint64_t)ldb, grouped ? (uint64_t)ldb_e : (uint64_t)ldb * (uint64_t)N};
    if (int rc = make_map_sw128(&map_b, b, 3, dims, str, BN, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) return rc;
  }

  Params p;
  p.sfa = sfa;
  p.sfb = sfb;
  p.out = out;
  p.expert_offsets = expert_offsets;
  p.M = (int32_t)M;
  p.N = (int32_t)N;
  p.K = (int32_t)K;
  p.num_experts = grouped ? (int32_t)num_experts : 1;
  p.m_tiles = (int32_t)((M + BM - 1) / BM);
  p.n_tiles = (int32_t)((N + BN - 1) / BN);
  p.k_tiles = (int32_t)((K + BK - 1) / BK);
  p.k_groups = (p.k_tiles + 3) / 4;
  p.ldc = ldc;
  p.sfa_ld = sfa_ld;
  p.sfa_stride_m = sfa_stride_m;
  p.sfb_stride_e = grouped ? sfb_stride_e : 0;
  p.sfb_stride_n = sfb_stride_n;
  p.sfb_stride_k = sfb_stride_k;
  p.out_dtype = out_dtype;

  static bool attr_done[2][64] = {{false}};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[grouped][dev]) {
    cudaError_t e = grouped ? cudaFuncSetAttribute(fp8_ue8m0_gemm_kernel<true>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes)
                            : cudaFuncSetAttribute(fp8_ue8m0_gemm_kernel<false>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done[grouped][dev] = true;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (grouped) {
    // an upper bound on the tile count without reading the device: every expert can add one ragged m-tile
    const int64_t max_tiles = ((M + BM - 1) / BM + num_experts) * p.n_tiles;
    const int grid = (int)(max_tiles < di.sm_count ? max_tiles : di.sm_count);
    fp8_ue8m0_gemm_kernel<true><<<grid, kThreads, kSmemBytes, st>>>(map_a, map_b, p);
  } else {
    const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
    const int grid = (int)(tiles < di.sm_count ? tiles : di.sm_count);
    fp8_ue8m0_gemm_kernel<false><<<grid, kThreads, kSmemBytes, st>>>(map_a, map_b, p);
  }
  SGLB_CHECK_LAUNCH("fp8_ue8m0_gemm_kernel");
  return SGLB200_OK;
}
}  // namespace
}  // namespace sglb

extern "C" int sglb200_fp8_ue8m0_scaled_mm(const void* a, const void* b, const int32_t* sfa, const int32_t* sfb,
                                           void* out, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                           int64_t ldc, int64_t sfa_ld, int64_t sfb_stride_n, int64_t sfb_stride_k,
                                           int out_dtype, void* stream) {
  SGLB_REQUIRE(sfa_ld >= M, SGLB200_ERR_SHAPE, "sfa_ld=%lld must be >= M (scale words of a row group are contiguous)",
               (long long)sfa_ld);
  return sglb::ue8m0_common(a, b, sfa, sfb, out, nullptr, M, 1, N, K, lda, ldb, 0, ldc, sfa_ld, 1, 0, sfb_stride_n,
                            sfb_stride_k, out_dtype, stream);
}

extern "C" int sglb200_fp8_ue8m0_scaled_mm_ws(const void* a, const void* b, const int32_t* sfa, const int32_t* sfb,
                                              void* out, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                              int64_t ldc, int64_t sfa_ld, int64_t sfb_stride_n, int64_t sfb_stride_k,
                                              int out_dtype, void* workspace, int64_t workspace_bytes, void* stream) {
  SGLB_REQUIRE(sfa_ld >= M, SGLB200_ERR_SHAPE, "sfa_ld=%lld must be >= M (scale words of a row group are contiguous)",
               (long long)sfa_ld);
  SGLB_REQUIRE(workspace_bytes >= 0 && (workspace == nullptr || sglb::aligned(workspace, 16)), SGLB200_ERR_ALIGN,
               "workspace must be 16-byte aligned");
  return sglb::ue8m0_common(a, b, sfa, sfb, out, nullptr, M, 1, N, K, lda, ldb, 0, ldc, sfa_ld, 1, 0, sfb_stride_n,
                            sfb_stride_k, out_dtype, stream, static_cast<float*>(workspace),
                            workspace ? workspace_bytes / (int64_t)sizeof(float) : 0);
}

extern "C" int sglb200_fp8_ue8m0_scaled_grouped_mm(const void* a, const void* b, const int32_t* sfa, const int32_t* sfb,
                                                   void* out, const int32_t* expert_offsets, int64_t total_rows,
                                                   int64_t num_experts, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                                   int64_t ldb_e, int64_t ldc, int64_t sfa_stride_m, int64_t sfa_stride_k,
                                                   int64_t sfb_stride_e, int64_t sfb_stride_n, int64_t sfb_stride_k,
                                                   int out_dtype, void* stream) {
  SGLB_REQUIRE(expert_offsets != nullptr, SGLB200_ERR_NULL, "expert_offsets must not be NULL");
  return sglb::ue8m0_common(a, b, sfa, sfb, out, expert_offsets, total_rows, num_experts, N, K, lda, ldb, ldb_e, ldc,
                            sfa_stride_k, sfa_stride_m, sfb_stride_e, sfb_stride_n, sfb_stride_k, out_dtype, stream);
}
