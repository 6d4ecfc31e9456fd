// Block-scaled FP8 GEMM on CTA pairs (tcgen05 cta_group::2), dense, for large M.
//
//   out[m, n] = cast( sum_kb ( sum_{k in kb} a[m,k] * b[n,k] ) * sa[m,kb] * sb[n/128,kb] )
//
// Why pairs: a 128 x 128 tile needs (128 + 128) x 128 bytes of operands per k-block for 256 clocks of tensor-core work,
// 128 bytes per clock per SM from L2 at full rate.  Here two CTAs of a cluster (two SMs of one TPC) work on one
// 256 x BN tile: each CTA loads its own 128 rows of A and only HALF of the B rows, and one tcgen05.mma.cta_group::2
// issued by the even CTA reads both halves from both shared memories.  Bytes per clock of tensor work per SM:
// BN = 128: (128 + 64) x 128 / 256 = 96; BN = 256: (128 + 128) x 128 / 512 = 64; BN = 256 also halves the MMA, commit
// and barrier operations per flop.  No load is broadcast: every CTA fetches its own tiles with its own TMA copies; only
// mbarrier arrivals cross between the two CTAs.
// Measured on B200 (M = 8192, the five DeepSeek-V3 shapes): BN = 128 is level with the single-CTA kernel of gemm.cu
// (1147-1725 against 1150-1717 TFLOP/s), BN = 256 behind it on four of five shapes: with the loads removed altogether
// the single-CTA kernel gains only 15 %, so operand delivery is not what bounds this family of kernels; the per-k-block
// hand-over of partial sums through TMEM is, and BN = 256 has only two TMEM stages to hide it.  The kernel is therefore
// an explicit entry point (sglb200_fp8_blockwise_scaled_mm_pair), not the default.
//
// Per CTA, 384 threads, warp-specialised as in gemm.cu:
//   warps 0-1  TMA producers (k-blocks alternate): A [128 x 128 B] and B [BN/2 x 128 B] per k-block into a ring of
//              128-byte-swizzled stages.  The completion bytes of BOTH CTAs are counted on the even CTA's `full`
//              barrier (the even CTA's producer announces the sum).
//   warps 2-3  MMA issuers, active in the even CTA only (k-blocks alternate): four tcgen05.mma (256 x BN x 32) per
//              k-block that overwrite one TMEM accumulator stage of BN columns in both CTAs, then two commits that
//              arrive on the `empty` (smem stage) and `acc_full` (TMEM stage) barriers of both CTAs.
//   warps 4-11 promotion + epilogue for the CTA's own 128 rows: two warps per TMEM lane quarter, BN/2 columns each.
//              acc += partial * sa[m,kb] * sb[nb,kb] in fp32 registers; the TMEM stage is handed back by an arrival
//              on the even CTA's `acc_empty` barrier (16 arrivals: 8 warps x 2 CTAs).
// BN = 256 keeps 128 accumulators per thread, so its promotion warps take registers from the other warps
// (setmaxnreg); it has two TMEM stages of 256 columns, BN = 128 has four of 128.
//
// Every wait is bounded (about two seconds); on time-out the CTA records a code in the status word, stops issuing
// work and leaves through the common exit (cluster barrier, TMEM release).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace sglb {

__device__ int g_pair_status = 0;

int pair_take_device_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_pair_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_pair_status, &z, sizeof(int));
  }
  return v;
}


namespace {

constexpr int kPairThreads = 384;
constexpr int kProducers = 2, kMmaWarps = 2, kPromoWarps = 8;
constexpr int kFirstPromoWarp = kProducers + kMmaWarps;
constexpr int kScaleAhead = 4;
constexpr int kGroupM2 = 8;  // 256-row tiles per raster group

template <int BN_>
struct PairCfg {
  static constexpr int BN = BN_;
  static constexpr int kAccStages = 512 / BN;
  static constexpr int kBRows = BN / 2;  // B rows held by each CTA
  static constexpr uint32_t kTileA = 128 * 128, kTileB = kBRows * 128, kStage = kTileA + kTileB;
  static constexpr int kStages = BN == 128 ? 8 : 6;
  static constexpr int kCols = BN / 2;  // columns per promotion warp
  static constexpr bool kRealloc = true;
  static constexpr size_t kSmem = 1024 + (size_t)kStages * kStage + 512;
};

struct PairParams {
  const float* sa;
  const float* sb;
  void* out;
  int32_t M, N, K;
  int32_t m2_tiles, n_tiles, k_tiles, sb_blocks;
  int64_t ldc, sa_stride_m, sa_stride_k, sb_stride_n, sb_stride_k;
  int32_t out_dtype;
};

template <int STAGES, int ACC>
struct PairCtl {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[ACC];
  uint64_t acc_empty[ACC];
  uint32_t tmem_base;
  volatile int32_t abort_flag;
};

__device__ __forceinline__ uint32_t pack_out(float a, float b, int out_dtype) {
  if (out_dtype == SGLB200_BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void fma32p(float2* acc, const uint32_t (&v)[32], float2 scale2) {
#pragma unroll
  for (int j = 0; j < 16; ++j)
    acc[j] = __ffma2_rn(make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1])), scale2, acc[j]);
}

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
fp8_block_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const PairParams p) {
  using C = PairCfg<BN>;
  using Ctl = PairCtl<C::kStages, C::kAccStages>;
  static_assert(sizeof(Ctl) <= 512, "control block");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + (size_t)C::kStages * C::kStage);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0: issues the MMAs; 1: partner
  const int32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int32_t total_tiles = p.m2_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      ptx::mbar_init(&ctl->full[i], 1);
      ptx::mbar_init(&ctl->empty[i], 1);
    }
    for (int i = 0; i < C::kAccStages; ++i) {
      ptx::mbar_init(&ctl->acc_full[i], 1);
      ptx::mbar_init(&ctl->acc_empty[i], 2 * kPromoWarps);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == kProducers) {
    ptx::tmem_alloc_pair(&ctl->tmem_base, 512);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  ptx::cluster_sync_all();  // both CTAs' barriers are initialised before either signals the other
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  const uint32_t full0 = ptx::smem_u32(&ctl->full[0]);
  const uint32_t empty0 = ptx::smem_u32(&ctl->empty[0]);
  const uint32_t acc_full0 = ptx::smem_u32(&ctl->acc_full[0]);
  const uint32_t acc_empty0 = ptx::smem_u32(&ctl->acc_empty[0]);
  const uint32_t stage0 = ptx::smem_u32(smem);
  // the even CTA's barriers as seen from either CTA
  const uint32_t lead_full0 = ptx::mapa_shared(full0, 0);
  const uint32_t lead_acc_empty0 = ptx::mapa_shared(acc_empty0, 0);

  auto tile_of = [&](int32_t t, int32_t& row0, int32_t& n0) {
    const int32_t per_group = kGroupM2 * p.n_tiles;
    const int32_t gid = t / per_group;
    const int32_t first_m = gid * kGroupM2;
    const int32_t gm = min(p.m2_tiles - first_m, kGroupM2);
    const int32_t local = t - gid * per_group;
    const int32_t nt = local / gm;
    row0 = (first_m + (local - nt * gm)) * 256 + (int32_t)rank * 128;
    n0 = nt * BN;
  };

  // Registers move from the four producer / MMA warps (one warpgroup, one instruction) to the promotion warps.
  if constexpr (C::kRealloc) {
    if (warp < kFirstPromoWarp) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    } else {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    }
  }
  if (warp < kProducers) {
    uint32_t stage = 0, phase = 0, g = 0;
    uint32_t armed = 0, armed_phase = 0;  // bit i: this warp has armed stage i / the phase bit of its last arming
    for (int32_t t = pair; t < total_tiles; t += pairs) {
      int32_t row0, n0;
      tile_of(t, row0, n0);
      bool ok = true;
      for (int32_t kb = 0; kb < p.k_tiles; ++kb, ++g) {
        if ((g & (kProducers - 1)) == (uint32_t)warp) {
          if (!ptx::mbar_wait_inl_a(empty0 + stage * 8, phase ^ 1)) {
            ctl->abort_flag = 1;
            atomicCAS(&g_pair_status, 0, 31);
            ok = false;
            break;
          }
          armed |= 1u << stage;
          armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
          if (lane == 0) {
            const uint32_t dst = stage0 + stage * C::kStage;
            if (rank == 0) ptx::mbar_arrive_expect_tx_a(full0 + stage * 8, 2 * C::kStage);  // both CTAs' bytes
            ptx::tma_load_2d_pair(dst, &map_a, lead_full0 + stage * 8, kb * 128, row0);
            ptx::tma_load_2d_pair(dst + C::kTileA, &map_b, lead_full0 + stage * 8, kb * 128,
                                  n0 + (int32_t)rank * C::kBRows);
          }
        }
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
      if (!ok || ctl->abort_flag) break;
    }
    // After a time-out: no CTA may exit while bulk copies into its shared memory are in flight.  Both CTAs' copies
    // are counted on the even CTA's `full` barriers, so the even CTA waits (20 ms at most per stage) for the stages it
    // announced; the cluster barrier at the exit then holds the partner until that is done.
    if (ctl->abort_flag && rank == 0) {
      for (uint32_t i = 0; i < (uint32_t)C::kStages; ++i)
        if (armed & (1u << i)) ptx::mbar_wait_inl_a(full0 + i * 8, (armed_phase >> i) & 1u, 20000000ull);
    }
    // the last arrivals on `empty` come from asynchronous commits: take every stage once more before leaving
    if (warp == 0 && !ctl->abort_flag) {
      for (int i = 0; i < C::kStages; ++i) {
        if (!ptx::mbar_wait_inl_a(empty0 + stage * 8, phase ^ 1)) { atomicCAS(&g_pair_status, 0, 35); break; }
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp < kFirstPromoWarp) {
    if (rank == 0) {
      const uint32_t me = warp - kProducers;
      constexpr uint32_t idesc = ptx::make_idesc_e4m3_f32(256, BN);
      const uint64_t desc0 = ptx::make_kmajor_sw128_desc(stage0);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0, g = 0;
      for (int32_t t = pair; t < total_tiles; t += pairs) {
        bool ok = true;
        for (int32_t kb = 0; kb < p.k_tiles; ++kb, ++g) {
          if ((g & (kMmaWarps - 1)) == me) {
            if (!ptx::mbar_wait_inl_a(acc_empty0 + acc * 8, acc_phase ^ 1)) {
              ctl->abort_flag = 1;
              atomicCAS(&g_pair_status, 0, 32);
              ok = false;
              break;
            }
            if (!ptx::mbar_wait_inl_a(full0 + stage * 8, phase)) {
              ctl->abort_flag = 1;
              atomicCAS(&g_pair_status, 0, 33);
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            if (lane == 0) {
              const uint64_t a_desc = desc0 + (uint64_t)(stage * (C::kStage >> 4));
              const uint64_t b_desc = a_desc + (C::kTileA >> 4);
              const uint32_t d_tmem = tmem_base + acc * BN;
              ptx::mma_f8f6f4_pair(d_tmem, a_desc, b_desc, idesc, 0);
#pragma unroll
              for (uint32_t k = 1; k < 4; ++k) ptx::mma_f8f6f4_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, 1);
              ptx::mma_commit_pair_a(empty0 + stage * 8);
              ptx::mma_commit_pair_a(acc_full0 + acc * 8);
            }
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
          if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
        }
        if (!ok || ctl->abort_flag) break;
      }
    }
  } else {
    const int q = warp & 3;
    const int wi = warp - kFirstPromoWarp;
    const int col0 = (wi >> 2) * C::kCols;
    const int r_in_tile = q * 32 + lane;
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16) + col0;
    uint32_t acc_stage = 0, acc_phase = 0;
    float2 acc[C::kCols / 2];
    for (int32_t t = pair; t < total_tiles; t += pairs) {
      int32_t row0, n0;
      tile_of(t, row0, n0);
      const int32_t row = row0 + r_in_tile;
      const int32_t row_c = min(row, p.M - 1);
      const float* sa_row = p.sa + (int64_t)row_c * p.sa_stride_m;
      const float* sb_blk = p.sb + (int64_t)min((n0 + col0) / 128, p.sb_blocks - 1) * p.sb_stride_n;
#pragma unroll
      for (int j = 0; j < C::kCols / 2; ++j) acc[j] = make_float2(0.f, 0.f);
      float sa_ring[kScaleAhead], sb_ring[kScaleAhead];
#pragma unroll
      for (int u = 0; u < kScaleAhead; ++u) {
        const int32_t kc = min(u, p.k_tiles - 1);
        sa_ring[u] = __ldg(sa_row + (int64_t)kc * p.sa_stride_k);
        sb_ring[u] = __ldg(sb_blk + (int64_t)kc * p.sb_stride_k);
      }
      bool ok = true;
      for (int32_t kb0 = 0; kb0 < p.k_tiles && ok; kb0 += kScaleAhead) {
#pragma unroll
        for (int u = 0; u < kScaleAhead; ++u) {
          const int32_t kb = kb0 + u;
          if (kb >= p.k_tiles) break;
          const float scale = sa_ring[u] * sb_ring[u];
          {
            const int32_t kn = min(kb + kScaleAhead, p.k_tiles - 1);
            sa_ring[u] = __ldg(sa_row + (int64_t)kn * p.sa_stride_k);
            sb_ring[u] = __ldg(sb_blk + (int64_t)kn * p.sb_stride_k);
          }
          const float2 scale2 = make_float2(scale, scale);
          if (!ptx::mbar_wait_inl_a(acc_full0 + acc_stage * 8, acc_phase)) {
            ctl->abort_flag = 1;
            atomicCAS(&g_pair_status, 0, 34);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t taddr = tlane + acc_stage * BN;
          uint32_t va[32], vb[32];
          ptx::tmem_ld_32x32(taddr, va);
          ptx::tmem_ld_32x32(taddr + 32, vb);
          ptx::tmem_ld_wait(va);
          ptx::tmem_ld_wait(vb);
          if constexpr (C::kCols == 64) {
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (rank == 0) ptx::mbar_arrive_a(acc_empty0 + acc_stage * 8);
              else ptx::mbar_arrive_cluster(lead_acc_empty0 + acc_stage * 8);
            }
            fma32p(acc, va, scale2);
            fma32p(acc + 16, vb, scale2);
          } else {
            fma32p(acc, va, scale2);
            ptx::tmem_ld_32x32_reuse(taddr + 64, va);
            fma32p(acc + 16, vb, scale2);
            ptx::tmem_ld_32x32_reuse(taddr + 96, vb);
            ptx::tmem_ld_wait(va);
            ptx::tmem_ld_wait(vb);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (rank == 0) ptx::mbar_arrive_a(acc_empty0 + acc_stage * 8);
              else ptx::mbar_arrive_cluster(lead_acc_empty0 + acc_stage * 8);
            }
            fma32p(acc + 32, va, scale2);
            fma32p(acc + 48, vb, scale2);
          }
          if (++acc_stage == C::kAccStages) { acc_stage = 0; acc_phase ^= 1; }
        }
      }
      if (!ok || ctl->abort_flag) break;
      if (row < p.M) {
        const int32_t n_first = n0 + col0;
        const int esz = 2;
        char* out_row = static_cast<char*>(p.out) + ((int64_t)row * p.ldc + n_first) * esz;
#pragma unroll
        for (int c = 0; c < C::kCols / 8; ++c) {
          if (n_first + c * 8 < p.N) {
            uint4 u;
            u.x = pack_out(acc[c * 4 + 0].x, acc[c * 4 + 0].y, p.out_dtype);
            u.y = pack_out(acc[c * 4 + 1].x, acc[c * 4 + 1].y, p.out_dtype);
            u.z = pack_out(acc[c * 4 + 2].x, acc[c * 4 + 2].y, p.out_dtype);
            u.w = pack_out(acc[c * 4 + 3].x, acc[c * 4 + 3].y, p.out_dtype);
            *reinterpret_cast<uint4*>(out_row + c * 16) = u;
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- tear-down
  ptx::tc_fence_before();
  ptx::cluster_sync_all();  // neither CTA leaves while the other may still signal its barriers or read its tiles
  if (warp == kProducers) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, 512);
  }
}

template <int BN>
int launch_pair(const void* a, const void* b, const float* sa, const float* sb, void* out, int64_t M, int64_t N,
                int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t sa_stride_m, int64_t sa_stride_k,
                int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype, int sm_count, void* stream) {
  using C = PairCfg<BN>;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fp8_block_gemm_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)C::kSmem);
    if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done[dev] = true;
  }
  alignas(64) CUtensorMap map_a, map_b;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t str[1] = {(uint64_t)lda};
    if (int rc = make_map_sw128(&map_a, a, 2, dims, str, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_128B)) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    const uint64_t str[1] = {(uint64_t)ldb};
    if (int rc = make_map_sw128(&map_b, b, 2, dims, str, C::kBRows, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) return rc;
  }
  PairParams p;
  p.sa = sa;
  p.sb = sb;
  p.out = out;
  p.M = (int32_t)M;
  p.N = (int32_t)N;
  p.K = (int32_t)K;
  p.m2_tiles = (int32_t)((M + 255) / 256);
  p.n_tiles = (int32_t)((N + BN - 1) / BN);
  p.k_tiles = (int32_t)((K + 127) / 128);
  p.sb_blocks = (int32_t)((N + 127) / 128);
  p.ldc = ldc;
  p.sa_stride_m = sa_stride_m;
  p.sa_stride_k = sa_stride_k;
  p.sb_stride_n = sb_stride_n;
  p.sb_stride_k = sb_stride_k;
  p.out_dtype = out_dtype;
  const int64_t tiles = (int64_t)p.m2_tiles * p.n_tiles;
  int64_t pairs = sm_count / 2;
  if (tiles < pairs) pairs = tiles;
  fp8_block_gemm_pair_kernel<BN><<<(unsigned)(2 * pairs), kPairThreads, C::kSmem, static_cast<cudaStream_t>(stream)>>>(
      map_a, map_b, p);
  SGLB_CHECK_LAUNCH("fp8_block_gemm_pair_kernel");
  return SGLB200_OK;
}

}  // namespace

// Dense GEMM on CTA pairs; `bn` is 128 or 256.  Arguments as gemm_common's dense case (checked there).
int pair_gemm(int bn, const void* a, const void* b, const float* sa, const float* sb, void* out, int64_t M, int64_t N,
              int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t sa_stride_m, int64_t sa_stride_k,
              int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype, int sm_count, void* stream) {
  if (bn == 256)
    return launch_pair<256>(a, b, sa, sb, out, M, N, K, lda, ldb, ldc, sa_stride_m, sa_stride_k, sb_stride_n, sb_stride_k,
                            out_dtype, sm_count, stream);
  return launch_pair<128>(a, b, sa, sb, out, M, N, K, lda, ldb, ldc, sa_stride_m, sa_stride_k, sb_stride_n, sb_stride_k,
                          out_dtype, sm_count, stream);
}


}  // namespace sglb

extern "C" int sglb200_fp8_blockwise_scaled_mm_pair(const void* a, const void* b, const float* sa, const float* sb,
                                                    void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                                                    int64_t ldb, int64_t ldc, int64_t sa_stride_m, int64_t sa_stride_k,
                                                    int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype,
                                                    int tile_n, void* stream) {
  using namespace sglb;
  SGLB_REQUIRE(tile_n == 128 || tile_n == 256, SGLB200_ERR_SHAPE, "tile_n=%d: 128 or 256", tile_n);
  SGLB_REQUIRE(M >= 0 && N >= 0 && K > 0, SGLB200_ERR_SHAPE, "M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  SGLB_REQUIRE(M < ((int64_t)1 << 31) - 512 && N < ((int64_t)1 << 31) - 512 && K < ((int64_t)1 << 31) - 512,
               SGLB200_ERR_SHAPE, "a dimension exceeds 2^31");
  SGLB_REQUIRE(out_dtype == SGLB200_BF16 || out_dtype == SGLB200_F16, SGLB200_ERR_DTYPE,
               "out_dtype=%d: only bf16 (0) and f16 (1)", out_dtype);
  SGLB_REQUIRE(K % 16 == 0 && N % 8 == 0, SGLB200_ERR_SHAPE, "K=%lld must be a multiple of 16, N=%lld of 8", (long long)K,
               (long long)N);
  if (M == 0 || N == 0) return SGLB200_OK;
  SGLB_REQUIRE(a && b && sa && sb && out, SGLB200_ERR_NULL, "a/b/sa/sb/out must not be NULL");
  SGLB_REQUIRE(lda >= K && lda % 16 == 0 && ldb >= K && ldb % 16 == 0 && ldc >= N && ldc % 8 == 0, SGLB200_ERR_ALIGN,
               "lda=%lld ldb=%lld (>= K, multiples of 16) ldc=%lld (>= N, multiple of 8)", (long long)lda, (long long)ldb,
               (long long)ldc);
  SGLB_REQUIRE(aligned(a, 16) && aligned(b, 16) && aligned(out, 16) && aligned(sa, 4) && aligned(sb, 4), SGLB200_ERR_ALIGN,
               "a, b and out must be 16-byte aligned, the scales 4-byte aligned");
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  SGLB_REQUIRE(di.cc_major == 10, SGLB200_ERR_ARCH, "compute capability %d.%d: this library is built for sm_100a only",
               di.cc_major, di.cc_minor);
  SGLB_REQUIRE(di.sm_count >= 2, SGLB200_ERR_SHAPE, "the CTA-pair kernel needs at least two SMs");
  return pair_gemm(tile_n, a, b, sa, sb, out, M, N, K, lda, ldb, ldc, sa_stride_m, sa_stride_k, sb_stride_n, sb_stride_k,
                   out_dtype, di.sm_count, stream);
}
