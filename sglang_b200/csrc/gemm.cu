// Block-scaled FP8 GEMM for sm_100a, dense and grouped (per-expert) in one persistent kernel.
//
//   out[m, n] = cast( sum_kb ( sum_{k in kb} a[m,k] * b[n,k] ) * sa[m,kb] * sb[n/128,kb] )
//
// One CTA per SM, 384 threads, warp-specialised:
//   warps 0-1  TMA producers (k-blocks alternate between them): A tile [128 rows x 128 B] and B tile [128 rows x 128 B] per k-block into a
//              6-stage ring of 128-byte-swizzled shared memory (32 KiB per stage).
//   warps 2-3  MMA issuers (k-blocks alternate): per k-block four tcgen05.mma (128 x 128 x 32, e4m3 -> f32) that OVERWRITE one of
//              four 128-column TMEM accumulator stages, then tcgen05.commit to free the smem stage and to
//              publish the TMEM stage.
//   warps 4-11 promotion + epilogue: two warps per TMEM lane quarter, each owning 64 of the tile's 128
//              columns.  A thread owns one accumulator row: per k-block it pulls its 64 partial sums out
//              of TMEM (two tcgen05.ld of 32 columns, one wait), multiplies by sa[m,kb] * sb[nb,kb] and
//              adds into 64 fp32 registers with packed fp32x2 FMAs; after the last k-block it rounds to
//              bf16/f16 and writes 128 contiguous bytes of the output row.  Scales are fetched four
//              k-blocks ahead so their latency never sits on the promotion path.  Two warps per quarter
//              hide each other's TMEM-load latency.
// The four TMEM stages let the tensor core run up to four k-blocks ahead of the promotion warps, and the
// promotion of tile i's tail overlaps the loads and MMAs of tile i+1.
//
// Every wait on an mbarrier is bounded (about two seconds); on time-out the CTA records a code in
// g_device_status, stops issuing work, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "nvls.cuh"
#include "ptx.cuh"

namespace sglb {

__device__ int g_device_status = 0;

namespace {

constexpr int BM = 128, BN = 128, BK = 128;
constexpr int kStages = 6;
constexpr int kAccStages = 4;
constexpr int kThreads = 384;
constexpr int kIssuers = 2;  // producer warps and MMA warps: each pair splits the k-blocks even/odd
constexpr int kEpiWarps = 8;
constexpr int kEpiCols = BN / (kEpiWarps / 4);  // columns per promotion warp (64)
constexpr int kScaleAhead = 4;                 // k-blocks of scale prefetch
constexpr uint32_t kTileABytes = BM * BK;
constexpr uint32_t kTileBBytes = BN * BK;
constexpr uint32_t kStageBytes = kTileABytes + kTileBBytes;
constexpr uint32_t kTmemCols = kAccStages * BN;  // 512
constexpr int kMaxExperts = 1024;
constexpr int kGroupM = 16;  // m-tiles per raster group (dense)
constexpr int kGroupMAr = 16;  // the same in the GEMM with the fused all-reduce: a raster group is the unit that is
                               // reduced over the ranks, and the reduction of the LAST group is not hidden (8 measured
                               // 2-3 % slower at eight ranks: twice the barriers for half the exposed tail)
constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + (size_t)kStages * kStageBytes + 256 /*barriers*/ +
                              (kMaxExperts + 1) * sizeof(int32_t);

// Push epilogue (dense, one tile per (m, n)): instead of writing `out`, every output tile is stored into the receive
// buffer of every rank, in the slot of this rank, and flagged there.  Receive buffer of a rank:
// [2 sets][kMaxPeers sources][slot_elems] elements; flags: [2][kMaxPeers][kPushMaxTiles][kEpiWarps] words holding the
// epoch of the last completed store.  set = epoch & 1.  The epoch lives on the device: three control words of this
// rank follow its flag words ({completed exchanges, block tickets of the reduce kernel, failure mark}); the epoch of
// the exchange in flight is completed + 1, read by both kernels and advanced by the reduce kernel's last block, so a
// captured CUDA graph can be replayed.
constexpr int kMaxPeers = 8;
constexpr int kPushMaxTiles = 1024;
constexpr int64_t kFlagWords = (int64_t)2 * kMaxPeers * kPushMaxTiles * 8;
struct PushParams {
  void* dst[kMaxPeers];
  uint32_t* flag[kMaxPeers];
  int32_t world, rank;
  const uint32_t* ctl;  // this rank's control words
  int64_t slot_elems;
  int32_t scatter;  // 0: every tile goes to every rank (one-shot); 1: tile t goes to rank t % world only (two-shot)
};

// Push epilogue staging: every promotion warp turns "one output row per lane" into "rows of contiguous bytes per store"
// through a private [32 rows][kStageWords] patch of shared memory, 16 payload words per row and pass.
constexpr int kStageWords = 20;  // 80-byte row stride: 16-byte aligned, conflict-free for the per-lane uint4 writes
constexpr size_t kStagingBytes = (size_t)kEpiWarps * 32 * kStageWords * sizeof(uint32_t);
constexpr size_t kStagingOffset = (((size_t)kStages * kStageBytes + 256 + (kMaxExperts + 1) * sizeof(int32_t)) + 15) / 16 * 16;
constexpr size_t kSmemBytesPush = 1024 + kStagingOffset + kStagingBytes;

struct GemmParams {
  const float* sa;
  const float* sb;
  void* out;
  const int32_t* expert_offsets;  // null: dense (or the masked layout, see rows_per_expert)
  const int32_t* problem_sizes;   // grouped, optional: rows of expert e = problem_sizes[count_stride * e]
  int32_t count_stride;           // 3 for a [E, 3] problem-size table, 1 for a plain per-expert row count
  int32_t rows_per_expert;        // > 0: masked layout, expert e owns rows [e * rows_per_expert, + its row count)
  int64_t sa_stride_e;            // masked layout: activation scale (e, local row, kb) at e * sa_stride_e + ...
  int32_t total_rows, N, K, num_experts;
  int32_t m_tiles, n_tiles, k_tiles;
  int64_t ldc;
  int64_t sa_stride_m, sa_stride_k;
  int64_t sb_stride_e, sb_stride_n, sb_stride_k;
  int32_t out_dtype;
  // split-K (dense only): k_splits > 1 cuts the k-blocks into ranges of kb_per_split; every (tile, split) writes
  // its fp32 partial sums to partial[split][row][col] (row stride N) and a second kernel adds the splits up
  float* partial;
  int32_t k_splits, kb_per_split;
};

struct PushGemmParams : GemmParams {
  PushParams push;
};

// GEMM + all-reduce in one launch (dense, out = a buffer every rank maps through one multicast address): the last
// comm_ctas CTAs of the grid do not compute tiles.  They wait for the row blocks of `out` (one raster group of kGroupMAr
// row tiles each) to be finished by the other CTAs of this grid (`done`, one counter per row block, bumped once per
// promotion warp and tile), pair up with the same CTAs of the other ranks' kernels through the flag words, and sum the
// block over the ranks with multimem.ld_reduce / multimem.st (nvls.cuh) while the GEMM CTAs work on the next row block.
struct ArParams {
  uint64_t mc_out;       // multicast address of out[0][0]
  nvls::FlagPtrs fp;     // every rank's flag block (nvls.cuh layout)
  uint32_t* done;        // [row blocks] counters, zero at launch
  int32_t rank, world, comm_ctas;
  uint64_t limit_ns;
};
struct ArGemmParams : GemmParams {
  ArParams ar;
};
template <bool PUSH, bool AR = false>
struct ParamsOf { using type = GemmParams; };
template <>
struct ParamsOf<true, false> { using type = PushGemmParams; };
template <>
struct ParamsOf<false, true> { using type = ArGemmParams; };

struct Tile {
  int32_t row0;     // first row of the tile in a / out
  int32_t row_end;  // one past the last row this tile may write
  int32_t n0;
  int32_t expert;
  int32_t kb0, kb1;  // k-block range of this work item
  int32_t split;
};

struct SharedCtl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[kAccStages];
  uint64_t acc_empty[kAccStages];
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  int32_t total_tiles;
};

// bounded wait; fully inlined where the register limit of the warp was changed (no call allowed there)
template <bool INLINE>
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, uint64_t limit_ns = 2000000000ull) {
  if constexpr (INLINE) return ptx::mbar_wait_inl_a(bar, parity, limit_ns);
  else return ptx::mbar_wait_a(bar, parity, limit_ns);
}

template <bool GROUPED, int GROUP_M = kGroupM>
__device__ __forceinline__ Tile get_tile(const GemmParams& p, const int32_t* tile_start, int32_t t) {
  Tile tl;
  tl.kb0 = 0;
  tl.kb1 = p.k_tiles;
  tl.split = 0;
  if constexpr (!GROUPED) {
    if (p.k_splits > 1) {
      const int32_t mn = p.m_tiles * p.n_tiles;
      tl.split = t / mn;
      t -= tl.split * mn;
      tl.kb0 = tl.split * p.kb_per_split;
      tl.kb1 = min(tl.kb0 + p.kb_per_split, p.k_tiles);
    }
    const int32_t per_group = GROUP_M * p.n_tiles;
    const int32_t gid = t / per_group;
    const int32_t first_m = gid * GROUP_M;
    const int32_t gm = min(p.m_tiles - first_m, GROUP_M);
    const int32_t local = t - gid * per_group;
    const int32_t nt = local / gm;
    const int32_t mt = first_m + (local - nt * gm);
    tl.row0 = mt * BM;
    tl.row_end = p.total_rows;
    tl.n0 = nt * BN;
    tl.expert = 0;
  } else {
    int32_t lo = 0, hi = p.num_experts;  // last e with tile_start[e] <= t
    while (hi - lo > 1) {
      const int32_t mid = (lo + hi) >> 1;
      if (tile_start[mid] <= t) lo = mid; else hi = mid;
    }
    const int32_t e = lo;
    int32_t r0, r1;
    if (p.rows_per_expert > 0) {
      r0 = e * p.rows_per_expert;
      r1 = r0 + max(0, min(__ldg(p.problem_sizes + p.count_stride * e), p.rows_per_expert));
    } else {
      r0 = __ldg(p.expert_offsets + e);
      r1 = p.problem_sizes ? r0 + __ldg(p.problem_sizes + p.count_stride * e) : __ldg(p.expert_offsets + e + 1);
    }
    const int32_t me = (r1 - r0 + BM - 1) / BM;
    const int32_t local = t - tile_start[e];
    const int32_t nt = local / me;
    const int32_t mt = local - nt * me;
    tl.row0 = r0 + mt * BM;
    tl.row_end = r1;
    tl.n0 = nt * BN;
    tl.expert = e;
  }
  return tl;
}

__device__ __forceinline__ void record_timeout(SharedCtl* ctl, int code) {
  ctl->abort_flag = 1;
  atomicCAS(&g_device_status, 0, code);
}

template <typename OutT>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// acc holds kEpiCols consecutive columns starting at column n_first of the output row
template <typename OutT>
__device__ __forceinline__ void store_row(const float2 (&acc)[kEpiCols / 2], OutT* out_row, int32_t n_first, int32_t N) {
#pragma unroll
  for (int c = 0; c < kEpiCols / 8; ++c) {
    if (n_first + c * 8 < N) {
      uint4 u;
      u.x = pack2<OutT>(acc[c * 4 + 0].x, acc[c * 4 + 0].y);
      u.y = pack2<OutT>(acc[c * 4 + 1].x, acc[c * 4 + 1].y);
      u.z = pack2<OutT>(acc[c * 4 + 2].x, acc[c * 4 + 2].y);
      u.w = pack2<OutT>(acc[c * 4 + 3].x, acc[c * 4 + 3].y);
      *reinterpret_cast<uint4*>(out_row + c * 8) = u;
    }
  }
}

// acc[j] += v[2j], v[2j+1] * scale, two columns per instruction
__device__ __forceinline__ void fma32(float2* acc, const uint32_t (&v)[32], float2 scale2) {
#pragma unroll
  for (int j = 0; j < 16; ++j)
    acc[j] = __ffma2_rn(make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1])), scale2, acc[j]);
}

// v holds 16 words (64 bytes) of the lane's row; emit(r, w, value) is called with r = row of the warp's 32 and w = first
// word (0, 4, 8, 12) of a 16-byte piece, so that one call across the warp covers eight rows of 64 contiguous bytes.
template <typename F>
__device__ __forceinline__ void warp_rows_via_smem(uint32_t* stg, const uint32_t (&v)[16], int lane, F&& emit) {
  __syncwarp();  // the previous pass has been read out
  uint4* dst = reinterpret_cast<uint4*>(stg + lane * kStageWords);
#pragma unroll
  for (int i = 0; i < 4; ++i) dst[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  __syncwarp();
  const int w = (lane & 3) * 4;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int r = j + (lane >> 2);
    emit(r, w, *reinterpret_cast<const uint4*>(stg + r * kStageWords + w));
  }
}

template <bool GROUPED, bool PUSH, bool AR = false>
__global__ void __launch_bounds__(kThreads, 1)
fp8_block_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ typename ParamsOf<PUSH, AR>::type p) {
  static_assert(!AR || (!GROUPED && !PUSH), "the fused all-reduce is a form of the dense kernel");
  constexpr int kRing = kStages;  // shared-memory stages in the TMA ring
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem + (size_t)kStages * kStageBytes);
  int32_t* tile_start = reinterpret_cast<int32_t*>(smem + (size_t)kStages * kStageBytes + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---------------------------------------------------------------- set-up
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&ctl->full[i], 1);
      ptx::mbar_init(&ctl->empty[i], 1);
    }
    for (int i = 0; i < kAccStages; ++i) {
      ptx::mbar_init(&ctl->acc_full[i], 1);
      ptx::mbar_init(&ctl->acc_empty[i], kEpiWarps);  // one arrival per promotion warp
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == kIssuers) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  if constexpr (GROUPED) {
    if (warp == 0) {  // exclusive prefix sum of tiles per expert
      int32_t running = 0;
      for (int32_t base = 0; base < p.num_experts; base += 32) {
        const int32_t e = base + lane;
        int32_t v = 0;
        if (e < p.num_experts) {
          int32_t cnt;
          if (p.rows_per_expert > 0) cnt = max(0, min(__ldg(p.problem_sizes + p.count_stride * e), p.rows_per_expert));
          else if (p.problem_sizes) cnt = __ldg(p.problem_sizes + p.count_stride * e);
          else cnt = __ldg(p.expert_offsets + e + 1) - __ldg(p.expert_offsets + e);
          v = ((cnt + BM - 1) / BM) * p.n_tiles;
        }
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
    if (threadIdx.x == 0) ctl->total_tiles = p.m_tiles * p.n_tiles * p.k_splits;
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const int32_t total_tiles = ctl->total_tiles;
  // CTAs that compute tiles, and their stride through the tile list
  int32_t tile_stride = gridDim.x;
  bool is_comm = false;
  if constexpr (AR) {
    tile_stride = (int32_t)gridDim.x - p.ar.comm_ctas;
    is_comm = (int32_t)blockIdx.x >= tile_stride;
  }

  // ---------------------------------------------------------------- roles
  // The per-k-block loops of the producer and the MMA issuer are a serial chain for one warp, so they
  // are kept to a handful of instructions: barrier and tile addresses live in registers as 32-bit
  // shared-window addresses, every lane waits (no divergence to repair) and lane 0 alone issues.
  const uint32_t full0 = ptx::smem_u32(&ctl->full[0]);
  const uint32_t empty0 = ptx::smem_u32(&ctl->empty[0]);
  const uint32_t acc_full0 = ptx::smem_u32(&ctl->acc_full[0]);
  const uint32_t acc_empty0 = ptx::smem_u32(&ctl->acc_empty[0]);
  const uint32_t stage0 = ptx::smem_u32(stage_base);

  if (is_comm) {
    if constexpr (AR) {
      // ===== communication CTA: row block by row block, once the GEMM CTAs of this grid have stored it and the same CTA
      // of every other rank says the same of theirs, this rank's 1 / world slice of the block is summed through the
      // switch and written to every rank.  All waits are bounded; after a time-out the CTA skips the data movement but
      // still advances its epoch.
      __shared__ int s_ok;
      __shared__ uint32_t s_epoch;
      const int cb = (int)blockIdx.x - tile_stride;
      uint32_t* ctlw = p.ar.fp.p[p.ar.rank] + nvls::kFlagWords + cb;
      if (threadIdx.x == 0) {
        s_ok = 1;
        s_epoch = *reinterpret_cast<volatile uint32_t*>(ctlw);
      }
      __syncthreads();
      const uint32_t epoch0 = s_epoch;
      const int32_t row_blocks = (p.m_tiles + kGroupMAr - 1) / kGroupMAr;
      bool ok = true;
      for (int32_t rb = 0; rb < row_blocks && ok; ++rb) {
        const int32_t mt_rb = min(kGroupMAr, p.m_tiles - rb * kGroupMAr);
        const uint32_t target = (uint32_t)mt_rb * (uint32_t)p.n_tiles * kEpiWarps;
        if (threadIdx.x == 0) {
          uint64_t t0 = 0;
          uint32_t polls = 0;
          while (ptx::ld_acquire_gpu_u32(p.ar.done + rb) < target) {
            if ((++polls & 63u) == 0) {
              const uint64_t now = ptx::global_timer_ns();
              if (t0 == 0) {
                t0 = now;
              } else if ((int64_t)(now - t0) > (int64_t)p.ar.limit_ns) {
                s_ok = 0;
                atomicCAS(&g_device_status, 0, 6);
                break;
              }
            }
          }
        }
        ok = nvls::rank_barrier(p.ar.fp, 0, cb, p.ar.rank, p.ar.world, epoch0 + 1u + (uint32_t)rb, p.ar.limit_ns, &s_ok,
                                &g_device_status, 7);
        if (!ok) break;
        const int64_t row0 = (int64_t)rb * kGroupMAr * BM, rows = min((int64_t)p.total_rows - row0, (int64_t)kGroupMAr * BM);
        const int64_t vec0 = row0 * p.N / 8, nvec = rows * p.N / 8;
        const int64_t per_rank = (nvec + p.ar.world - 1) / p.ar.world;
        const int64_t v0 = vec0 + (int64_t)p.ar.rank * per_rank, v1 = min(vec0 + nvec, v0 + per_rank);
        if (p.out_dtype == SGLB200_BF16) nvls::reduce_range<true, 8>(p.ar.mc_out, v0, v1, cb, p.ar.comm_ctas, kThreads);
        else nvls::reduce_range<false, 8>(p.ar.mc_out, v0, v1, cb, p.ar.comm_ctas, kThreads);
      }
      if (ok)
        nvls::rank_barrier(p.ar.fp, 1, cb, p.ar.rank, p.ar.world, epoch0 + (uint32_t)row_blocks, p.ar.limit_ns, &s_ok,
                           &g_device_status, 8);
      if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(ctlw) = epoch0 + (uint32_t)row_blocks;
    }
  } else if (warp < kIssuers) {
    // ===== TMA producers.  Issuing a TMA or an MMA and touching an mbarrier each cost the issuing
    // thread on the order of a hundred cycles, and the tensor pipe does not queue far ahead, so one
    // warp per role cannot feed it: two warps per role take the k-blocks of the CTA alternately.
    uint32_t stage = 0, phase = 0, g = 0;
    uint32_t armed = 0, armed_phase = 0;  // bit i: this warp has armed stage i / the phase bit of its last arming
    for (int32_t t = blockIdx.x; t < total_tiles; t += tile_stride) {
      const Tile tl = get_tile<GROUPED, AR ? kGroupMAr : kGroupM>(p, tile_start, t);
      bool ok = true;
      for (int32_t kb = tl.kb0; kb < tl.kb1; ++kb, ++g) {
        if ((g & (kIssuers - 1)) == (uint32_t)warp) {
          if (!wait_bar<false>(empty0 + stage * 8, phase ^ 1)) {
            record_timeout(ctl, 1);
            ok = false;
            break;
          }
          armed |= 1u << stage;
          armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
          if (lane == 0) {
            const uint32_t dst = stage0 + stage * kStageBytes;
            ptx::mbar_arrive_expect_tx_a(full0 + stage * 8, kStageBytes);
            ptx::tma_load_2d_a(dst, &map_a, full0 + stage * 8, kb * BK, tl.row0);
            ptx::tma_load_3d_a(dst + kTileABytes, &map_b, full0 + stage * 8, kb * BK, tl.n0, tl.expert);
          }
        }
        if (++stage == kRing) { stage = 0; phase ^= 1; }
      }
      if (!ok || ctl->abort_flag) break;
    }
    // After a time-out somewhere in the CTA: a CTA must not exit while bulk copies into its shared memory are in
    // flight, so wait (20 ms at most per stage) for the loads this warp issued.
    if (ctl->abort_flag) {
      for (uint32_t i = 0; i < (uint32_t)kRing; ++i)
        if (armed & (1u << i)) wait_bar<true>(full0 + i * 8, (armed_phase >> i) & 1u, 20000000ull);
    }
    // Tail: tcgen05.commit arrives on the `empty` barriers asynchronously and nobody waits for the last ones, so the
    // CTA could exit (and the next kernel's CTA re-initialise barriers at the same shared-memory addresses) while
    // such an arrival is still in flight.  Acquire every stage once more before leaving.
    if (warp == 0 && !ctl->abort_flag) {
      for (int i = 0; i < kRing; ++i) {
        if (!wait_bar<false>(empty0 + stage * 8, phase ^ 1)) { record_timeout(ctl, 5); break; }
        if (++stage == kRing) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp < 2 * kIssuers) {
    // ===== MMA issuers (k-blocks alternate between the two warps; each k-block has its own TMEM stage)
    const uint32_t me = warp - kIssuers;
    constexpr uint32_t idesc = ptx::make_idesc_e4m3_f32(BM, BN);
    const uint64_t desc0 = ptx::make_kmajor_sw128_desc(stage0);
    uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0, g = 0;
    for (int32_t t = blockIdx.x; t < total_tiles; t += tile_stride) {
      bool ok = true;
      int32_t kb_count = p.k_tiles;
      if (p.k_splits > 1) {
        const Tile tl = get_tile<GROUPED, AR ? kGroupMAr : kGroupM>(p, tile_start, t);
        kb_count = tl.kb1 - tl.kb0;
      }
      for (int32_t kb = 0; kb < kb_count; ++kb, ++g) {
        if ((g & (kIssuers - 1)) == me) {
          if (!wait_bar<false>(acc_empty0 + acc * 8, acc_phase ^ 1)) {
            record_timeout(ctl, 2);
            ok = false;
            break;
          }
          if (!wait_bar<false>(full0 + stage * 8, phase)) {
            record_timeout(ctl, 3);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          if (lane == 0) {
            // descriptors differ from stage 0's only in the 16-byte address field
            const uint64_t a_desc = desc0 + (uint64_t)(stage * (kStageBytes >> 4));
            const uint64_t b_desc = a_desc + (kTileABytes >> 4);
            const uint32_t d_tmem = tmem_base + acc * BN;
            ptx::mma_f8f6f4(d_tmem, a_desc, b_desc, idesc, 0);
#pragma unroll
            for (uint32_t k = 1; k < BK / 32; ++k) {
              // 32 bytes further along K inside the swizzle atom: +2 in the address field
              ptx::mma_f8f6f4(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, 1);
            }
            ptx::mma_commit_a(empty0 + stage * 8);
            ptx::mma_commit_a(acc_full0 + acc * 8);
          }
        }
        if (++stage == kRing) { stage = 0; phase ^= 1; }
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok || ctl->abort_flag) break;
    }
  } else {
    // ===== promotion + epilogue (warps 4..11); TMEM lane quarter = warp % 4, column half = (warp - 4) / 4
    const int q = warp & 3;
    const int col0 = ((warp - 2 * kIssuers) >> 2) * kEpiCols;
    const int r_in_tile = q * 32 + lane;
    uint32_t acc_stage = 0, acc_phase = 0;
    float2 acc[kEpiCols / 2];
    uint32_t push_epoch = 0;
    if constexpr (PUSH) push_epoch = *reinterpret_cast<const volatile uint32_t*>(p.push.ctl) + 1u;
    for (int32_t t = blockIdx.x; t < total_tiles; t += tile_stride) {
      const Tile tl = get_tile<GROUPED, AR ? kGroupMAr : kGroupM>(p, tile_start, t);
      const int32_t row = tl.row0 + r_in_tile;
      const int32_t row_c = min(row, p.total_rows - 1);
      const float* sa_row = p.sa + (int64_t)row_c * p.sa_stride_m;
      if constexpr (GROUPED) {
        if (p.rows_per_expert > 0)
          sa_row = p.sa + (int64_t)tl.expert * p.sa_stride_e +
                   (int64_t)(row_c - tl.expert * p.rows_per_expert) * p.sa_stride_m;
      }
      const float* sb_blk = p.sb + (int64_t)tl.expert * p.sb_stride_e + (int64_t)(tl.n0 / BN) * p.sb_stride_n;
#pragma unroll
      for (int j = 0; j < kEpiCols / 2; ++j) acc[j] = make_float2(0.f, 0.f);
      float sa_ring[kScaleAhead], sb_ring[kScaleAhead];
#pragma unroll
      for (int u = 0; u < kScaleAhead; ++u) {
        const int32_t kc = min(tl.kb0 + u, tl.kb1 - 1);
        sa_ring[u] = __ldg(sa_row + (int64_t)kc * p.sa_stride_k);
        sb_ring[u] = __ldg(sb_blk + (int64_t)kc * p.sb_stride_k);
      }
      bool ok = true;
      for (int32_t kb0 = tl.kb0; kb0 < tl.kb1 && ok; kb0 += kScaleAhead) {
#pragma unroll
        for (int u = 0; u < kScaleAhead; ++u) {
          const int32_t kb = kb0 + u;
          if (kb >= tl.kb1) break;
          const float scale = sa_ring[u] * sb_ring[u];
          {  // fetch the scales of k-block kb + kScaleAhead into the slot just consumed
            const int32_t kn = min(kb + kScaleAhead, tl.kb1 - 1);
            sa_ring[u] = __ldg(sa_row + (int64_t)kn * p.sa_stride_k);
            sb_ring[u] = __ldg(sb_blk + (int64_t)kn * p.sb_stride_k);
          }
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc_stage * BN + col0;
          const float2 scale2 = make_float2(scale, scale);
          {
            if (!ptx::mbar_wait_a(acc_full0 + acc_stage * 8, acc_phase)) {
              record_timeout(ctl, 4);
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            uint32_t va[32], vb[32];
            ptx::tmem_ld_32x32(taddr, va);
            ptx::tmem_ld_32x32(taddr + 32, vb);
            ptx::tmem_ld_wait(va);
            ptx::tmem_ld_wait(vb);
            // every TMEM read of this stage has landed: hand the stage back to the MMA warp
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_a(acc_empty0 + acc_stage * 8);
            fma32(acc, va, scale2);
            fma32(acc + 16, vb, scale2);
          }
          if (++acc_stage == kAccStages) { acc_stage = 0; acc_phase ^= 1; }
        }
      }
      if (!ok || ctl->abort_flag) break;
      if constexpr (PUSH) {
        const int32_t n_first = tl.n0 + col0;
        const int32_t tile_id = (tl.row0 / BM) * p.n_tiles + tl.n0 / BN;
        const int owner = tile_id % p.push.world;
        const int wi = warp - 2 * kIssuers;
        uint32_t* stg = reinterpret_cast<uint32_t*>(smem + kStagingOffset) + wi * 32 * kStageWords;
        const int32_t row_base = tl.row0 + q * 32;  // the warp's rows are row_base + 0..31
        const uint32_t set = push_epoch & 1u;
        const int64_t slot = ((int64_t)set * kMaxPeers + p.push.rank) * p.push.slot_elems;
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // 32 columns (64 bytes of a row) per pass
          uint32_t v[16];
#pragma unroll
          for (int w = 0; w < 16; ++w)
            v[w] = p.out_dtype == SGLB200_BF16 ? pack2<__nv_bfloat16>(acc[16 * h + w].x, acc[16 * h + w].y)
                                               : pack2<__half>(acc[16 * h + w].x, acc[16 * h + w].y);
          warp_rows_via_smem(stg, v, lane, [&](int r, int w, uint4 val) {
            const int32_t grow = row_base + r, c = n_first + 32 * h + 2 * w;  // 8 columns from c (N % 8 == 0)
            if (grow < tl.row_end && c < p.N) {
              const int64_t off = (slot + (int64_t)grow * p.N + c) * 2;
              if (p.push.scatter) {
                *reinterpret_cast<uint4*>(static_cast<char*>(p.push.dst[owner]) + off) = val;
              } else {
                for (int i = 0; i < p.push.world; ++i) {  // peers first, this rank last
                  int pr = p.push.rank + 1 + i;
                  if (pr >= p.push.world) pr -= p.push.world;
                  *reinterpret_cast<uint4*>(static_cast<char*>(p.push.dst[pr]) + off) = val;
                }
              }
            }
          });
        }
        // The warp's 32 rows x 64 columns are on their way.  One flag word per (tile, warp) and rank: the warp barrier
        // orders every lane's stores before the release store of the flag (release is cumulative), at system scope.
        __syncwarp();
        if (p.push.scatter ? lane == owner : lane < p.push.world) {
          uint32_t* f = p.push.flag[lane] +
                        (((int64_t)set * kMaxPeers + p.push.rank) * kPushMaxTiles + tile_id) * kEpiWarps + wi;
          ptx::st_release_sys_u32(f, push_epoch);
        }
      } else if (row < tl.row_end) {
        const int32_t n_first = tl.n0 + col0;
        if (p.partial != nullptr) {
          float* dst = p.partial + ((int64_t)tl.split * p.total_rows + row) * p.N + n_first;
#pragma unroll
          for (int c = 0; c < kEpiCols / 4; ++c) {
            if (n_first + c * 4 < p.N)
              *reinterpret_cast<float4*>(dst + c * 4) =
                  make_float4(acc[2 * c].x, acc[2 * c].y, acc[2 * c + 1].x, acc[2 * c + 1].y);
          }
        } else if (p.out_dtype == SGLB200_BF16) {
          store_row<__nv_bfloat16>(acc, static_cast<__nv_bfloat16*>(p.out) + (int64_t)row * p.ldc + n_first, n_first, p.N);
        } else {
          store_row<__half>(acc, static_cast<__half*>(p.out) + (int64_t)row * p.ldc + n_first, n_first, p.N);
        }
      }
      if constexpr (AR) {
        // this warp's part of the tile is stored: count it for the tile's row block (the warp barrier orders every
        // lane's stores before lane 0's fence; the communication CTAs read the counter with acquire)
        __syncwarp();
        if (lane == 0) {
          __threadfence();
          atomicAdd(p.ar.done + (tl.row0 / BM) / kGroupMAr, 1u);
        }
      }
    }
  }

  // ---------------------------------------------------------------- tear-down
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kIssuers) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// out[m, n] = cast(sum_s partial[s][m][n]); 8 columns per thread, splits added in ascending order
template <typename OutT>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partial, OutT* __restrict__ out, int32_t M, int32_t N, int64_t ldc,
                     int32_t splits) {
  ptx::grid_dep_launch();  // the next kernel may begin its set-up (and a GEMM its weight streaming) beside this one
  ptx::grid_dep_wait();    // the partial sums come from the kernel before this one
  const int32_t vec_per_row = N / 8;
  const int64_t total = (int64_t)M * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int32_t m = (int32_t)(i / vec_per_row);
    const int32_t c = (int32_t)(i - (int64_t)m * vec_per_row) * 8;
    float a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = 0.f;
    for (int32_t sp = 0; sp < splits; ++sp) {
      const float4* src = reinterpret_cast<const float4*>(partial + ((int64_t)sp * M + m) * N + c);
      const float4 x = __ldcs(src), y = __ldcs(src + 1);
      a[0] += x.x; a[1] += x.y; a[2] += x.z; a[3] += x.w;
      a[4] += y.x; a[5] += y.y; a[6] += y.z; a[7] += y.w;
    }
    uint4 u;
    u.x = pack2<OutT>(a[0], a[1]);
    u.y = pack2<OutT>(a[2], a[3]);
    u.z = pack2<OutT>(a[4], a[5]);
    u.w = pack2<OutT>(a[6], a[7]);
    *reinterpret_cast<uint4*>(out + (int64_t)m * ldc + c) = u;
  }
}

// Receiving side of the push epilogue: out[m, n] = cast(sum over source ranks of their slot), fp32, ascending rank (so
// every rank computes the same bits).  One tile per loop step; 8 * world threads wait (bounded) for the tile's flag
// words to reach `epoch`.  On a time-out the block records status 5 and returns without writing the tile.
template <typename OutT>
__global__ void __launch_bounds__(256)
peer_reduce_kernel(const OutT* recv, const uint32_t* flags, uint32_t* ctl, OutT* __restrict__ out, int32_t M, int32_t N,
                   int64_t ldc, int32_t n_tiles, int32_t total_items, int32_t world, int64_t slot_elems,
                   uint64_t limit_ns) {
  __shared__ int s_ok;
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = *reinterpret_cast<volatile uint32_t*>(ctl) + 1u;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const uint32_t set = epoch & 1u;
  // work item = (tile, quarter of its rows): the rows 32q..32q+31 of a tile were pushed by the promotion warps q
  // (columns 0..63) and q + 4 (columns 64..127) of every source rank
  for (int32_t item = blockIdx.x; item < total_items; item += gridDim.x) {
    const int32_t t = item >> 2, q = item & 3;
    const int32_t mt = t / n_tiles, nt = t - mt * n_tiles;
    const int32_t row0 = mt * BM + q * 32;
    if (row0 >= M) continue;  // uniform
    if ((int)threadIdx.x < world * 2) {
      const int src = threadIdx.x >> 1, w = q + 4 * (threadIdx.x & 1);
      const uint32_t* f = flags + (((int64_t)set * kMaxPeers + src) * kPushMaxTiles + t) * kEpiWarps + w;
      uint64_t t0 = 0;
      uint32_t polls = 0;
      while ((int32_t)(ptx::ld_acquire_sys_u32(f) - epoch) < 0) {
        if ((++polls & 255u) == 0) {
          const uint64_t now = ptx::global_timer_ns();
          if (t0 == 0) {
            t0 = now;
          } else if ((int64_t)(now - t0) > (int64_t)limit_ns) {
            s_ok = 0;
            atomicCAS(&g_device_status, 0, 5);
            break;
          }
        }
      }
    }
    __syncthreads();
    if (!s_ok) break;  // uniform: s_ok is only ever cleared before the barrier above
    const int32_t rows = min(32, M - row0), vecs = min(BN, N - nt * BN) / 8;
    for (int32_t i = threadIdx.x; i < rows * vecs; i += blockDim.x) {
      const int32_t r = i / vecs, c = (i - r * vecs) * 8;
      const int64_t off = (int64_t)(row0 + r) * N + nt * BN + c;
      uint4 u[kMaxPeers];
#pragma unroll
      for (int src = 0; src < kMaxPeers; ++src) {
        // written by another GPU since this SM may last have cached the line: bypass L1
        if (src < world)
          u[src] = __ldcv(reinterpret_cast<const uint4*>(recv + ((int64_t)set * kMaxPeers + src) * slot_elems + off));
      }
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = 0.f;
#pragma unroll
      for (int src = 0; src < kMaxPeers; ++src) {
        if (src < world) {
          const OutT* h = reinterpret_cast<const OutT*>(&u[src]);
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] += static_cast<float>(h[j]);
        }
      }
      uint4 o;
      o.x = pack2<OutT>(a[0], a[1]);
      o.y = pack2<OutT>(a[2], a[3]);
      o.z = pack2<OutT>(a[4], a[5]);
      o.w = pack2<OutT>(a[6], a[7]);
      *reinterpret_cast<uint4*>(out + (int64_t)(row0 + r) * ldc + nt * BN + c) = o;
    }
    __syncthreads();
  }
  // every block takes a ticket; the last one closes the exchange: the epoch advances only if no block gave up
  // (the epoch was read, and used, before this block's ticket; the counters are only ever touched by atomics)
  if (threadIdx.x == 0) {
    if (!s_ok) atomicExch(&ctl[2], 1u);
    if (atomicAdd(&ctl[1], 1u) == gridDim.x - 1) {
      const uint32_t failed = atomicExch(&ctl[2], 0u);
      ctl[1] = 0;
      if (!failed) *reinterpret_cast<volatile uint32_t*>(ctl) = epoch;
    }
  }
}

// ---- two-shot exchange (reduce-scatter + all-gather) for outputs too large to send whole to every rank -------------
// The push epilogue in scatter mode sends tile t only to rank t % world.  That rank adds the `world` partial tiles
// (fp32, ascending rank: the same bits as the one-shot reduce), writes the result to its own output and stores it into
// every other rank's slot [set][this rank] at the tile's position, which scatter-mode pushes never touch on a rank that
// does not own the tile; the flag words [set][this rank][tile][quarter] there, equally unused, announce it.  The gather
// kernel of every rank then waits for the tiles it does not own and copies them out of those slots.  Bytes leaving a
// rank per exchange: 2 (world - 1) / world of the output instead of (world - 1) times the output.

// spin (bounded) until *f has reached `epoch`; on a time-out clears *ok and records status 5
__device__ __forceinline__ void wait_flag_word(const uint32_t* f, uint32_t epoch, uint64_t limit_ns, int* ok) {
  uint64_t t0 = 0;
  uint32_t polls = 0;
  while ((int32_t)(ptx::ld_acquire_sys_u32(f) - epoch) < 0) {
    if ((++polls & 255u) == 0) {
      const uint64_t now = ptx::global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if ((int64_t)(now - t0) > (int64_t)limit_ns) {
        *ok = 0;
        atomicCAS(&g_device_status, 0, 5);
        break;
      }
    }
  }
}

template <typename OutT>
__global__ void __launch_bounds__(256)
peer_reduce_scatter_kernel(const PushParams push, OutT* __restrict__ out, int32_t M, int32_t N, int64_t ldc,
                           int32_t n_tiles, int32_t total_items, uint64_t limit_ns) {
  __shared__ int s_ok;
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = *reinterpret_cast<const volatile uint32_t*>(push.ctl) + 1u;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch, set = epoch & 1u;
  const int32_t world = push.world, rank = push.rank;
  const OutT* recv = static_cast<const OutT*>(push.dst[rank]);
  const uint32_t* flags = push.flag[rank];
  // owned work item j = (owned tile j / 4, quarter j % 4); the owned tiles are rank, rank + world, ...
  for (int32_t item = blockIdx.x; item < total_items; item += gridDim.x) {
    const int32_t t = (item >> 2) * world + rank, q = item & 3;
    const int32_t mt = t / n_tiles, nt = t - mt * n_tiles;
    const int32_t row0 = mt * BM + q * 32;
    if (row0 >= M) continue;  // uniform
    if ((int)threadIdx.x < world * 2) {
      const int src = threadIdx.x >> 1, w = q + 4 * (threadIdx.x & 1);
      wait_flag_word(flags + (((int64_t)set * kMaxPeers + src) * kPushMaxTiles + t) * kEpiWarps + w, epoch, limit_ns, &s_ok);
    }
    __syncthreads();
    if (!s_ok) break;  // uniform: s_ok is only ever cleared before the barrier above
    const int32_t rows = min(32, M - row0), vecs = min(BN, N - nt * BN) / 8;
    const int64_t mine = ((int64_t)set * kMaxPeers + rank) * push.slot_elems;
    for (int32_t i = threadIdx.x; i < rows * vecs; i += blockDim.x) {
      const int32_t r = i / vecs, c = (i - r * vecs) * 8;
      const int64_t off = (int64_t)(row0 + r) * N + nt * BN + c;
      uint4 u[kMaxPeers];
#pragma unroll
      for (int src = 0; src < kMaxPeers; ++src) {
        if (src < world)
          u[src] = __ldcv(reinterpret_cast<const uint4*>(recv + ((int64_t)set * kMaxPeers + src) * push.slot_elems + off));
      }
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = 0.f;
#pragma unroll
      for (int src = 0; src < kMaxPeers; ++src) {
        if (src < world) {
          const OutT* h = reinterpret_cast<const OutT*>(&u[src]);
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] += static_cast<float>(h[j]);
        }
      }
      uint4 o;
      o.x = pack2<OutT>(a[0], a[1]);
      o.y = pack2<OutT>(a[2], a[3]);
      o.z = pack2<OutT>(a[4], a[5]);
      o.w = pack2<OutT>(a[6], a[7]);
      for (int k = 1; k < world; ++k) {
        int pr = rank + k;
        if (pr >= world) pr -= world;
        *reinterpret_cast<uint4*>(static_cast<OutT*>(push.dst[pr]) + mine + off) = o;
      }
      *reinterpret_cast<uint4*>(out + (int64_t)(row0 + r) * ldc + nt * BN + c) = o;
    }
    // the block barrier orders every thread's stores before the release stores of the flags (release is cumulative)
    __syncthreads();
    if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
      uint32_t* f = push.flag[threadIdx.x] + (((int64_t)set * kMaxPeers + rank) * kPushMaxTiles + t) * kEpiWarps + q;
      ptx::st_release_sys_u32(f, epoch);
    }
  }
  if (threadIdx.x == 0 && !s_ok) atomicExch(const_cast<uint32_t*>(push.ctl) + 2, 1u);  // the gather kernel will not advance
}

template <typename OutT>
__global__ void __launch_bounds__(256)
peer_gather_kernel(const OutT* recv, const uint32_t* flags, uint32_t* ctl, OutT* __restrict__ out, int32_t M, int32_t N,
                   int64_t ldc, int32_t n_tiles, int32_t total_items, int32_t world, int32_t rank, int64_t slot_elems,
                   uint64_t limit_ns) {
  __shared__ int s_ok;
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = *reinterpret_cast<volatile uint32_t*>(ctl) + 1u;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch, set = epoch & 1u;
  for (int32_t item = blockIdx.x; item < total_items; item += gridDim.x) {
    const int32_t t = item >> 2, q = item & 3;
    const int32_t owner = t % world;
    if (owner == rank) continue;  // written by this rank's reduce-scatter kernel
    const int32_t mt = t / n_tiles, nt = t - mt * n_tiles;
    const int32_t row0 = mt * BM + q * 32;
    if (row0 >= M) continue;  // uniform
    if (threadIdx.x == 0)
      wait_flag_word(flags + (((int64_t)set * kMaxPeers + owner) * kPushMaxTiles + t) * kEpiWarps + q, epoch, limit_ns, &s_ok);
    __syncthreads();
    if (!s_ok) break;
    const int32_t rows = min(32, M - row0), vecs = min(BN, N - nt * BN) / 8;
    const OutT* src = recv + ((int64_t)set * kMaxPeers + owner) * slot_elems;
    for (int32_t i = threadIdx.x; i < rows * vecs; i += blockDim.x) {
      const int32_t r = i / vecs, c = (i - r * vecs) * 8;
      const uint4 v = __ldcv(reinterpret_cast<const uint4*>(src + (int64_t)(row0 + r) * N + nt * BN + c));
      *reinterpret_cast<uint4*>(out + (int64_t)(row0 + r) * ldc + nt * BN + c) = v;
    }
    __syncthreads();
  }
  // the last block closes the exchange: the epoch advances only if no block of either kernel gave up
  if (threadIdx.x == 0) {
    if (!s_ok) atomicExch(&ctl[2], 1u);
    if (atomicAdd(&ctl[1], 1u) == gridDim.x - 1) {
      const uint32_t failed = atomicExch(&ctl[2], 0u);
      ctl[1] = 0;
      if (!failed) *reinterpret_cast<volatile uint32_t*>(ctl) = epoch;
    }
  }
}

// Sending side for the few-rows kernel: out-of-kernel epilogue of the push exchange.  Adds the fp32 partial sums of the
// K-splits in ascending order (as splitk_reduce_kernel does), casts, stores the 16-byte vectors into every rank's receive
// slot and raises the eight flag words of the tile.  One block per 128 x 128 output tile.
template <typename OutT>
__global__ void __launch_bounds__(256)
splitk_reduce_push_kernel(const float* __restrict__ partial, int32_t splits, int32_t M, int32_t N, int32_t n_tiles,
                          int32_t total_tiles, const PushParams push) {
  const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(push.ctl) + 1u;
  const uint32_t set = epoch & 1u;
  const int64_t slot = ((int64_t)set * kMaxPeers + push.rank) * push.slot_elems;
  for (int32_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const int32_t mt = t / n_tiles, nt = t - mt * n_tiles;
    const int32_t rows = min(BM, M - mt * BM), vecs = min(BN, N - nt * BN) / 8;
    for (int32_t i = threadIdx.x; i < rows * vecs; i += blockDim.x) {
      const int32_t r = i / vecs, c = (i - r * vecs) * 8;
      const int64_t off = (int64_t)(mt * BM + r) * N + nt * BN + c;
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = 0.f;
      for (int32_t sp = 0; sp < splits; ++sp) {
        const float4* src = reinterpret_cast<const float4*>(partial + (int64_t)sp * M * N + off);
        const float4 x = __ldcs(src), y = __ldcs(src + 1);
        a[0] += x.x; a[1] += x.y; a[2] += x.z; a[3] += x.w;
        a[4] += y.x; a[5] += y.y; a[6] += y.z; a[7] += y.w;
      }
      uint4 u;
      u.x = pack2<OutT>(a[0], a[1]);
      u.y = pack2<OutT>(a[2], a[3]);
      u.z = pack2<OutT>(a[4], a[5]);
      u.w = pack2<OutT>(a[6], a[7]);
      for (int k = 0; k < push.world; ++k) {  // peers first, this rank last
        int pr = push.rank + 1 + k;
        if (pr >= push.world) pr -= push.world;
        *reinterpret_cast<uint4*>(static_cast<OutT*>(push.dst[pr]) + slot + off) = u;
      }
    }
    // the block barrier orders every thread's stores before the release stores of the flags (release is cumulative)
    __syncthreads();
    if ((int)threadIdx.x < push.world * kEpiWarps) {
      const int pr = threadIdx.x / kEpiWarps, w = threadIdx.x % kEpiWarps;
      uint32_t* f = push.flag[pr] + (((int64_t)set * kMaxPeers + push.rank) * kPushMaxTiles + t) * kEpiWarps + w;
      ptx::st_release_sys_u32(f, epoch);
    }
  }
}

// ------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      ptr = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

}  // namespace

// rank-2 or rank-3 byte tensor, innermost extent K, 128-byte-swizzled boxes of [rows x 128 B]
int make_map_sw128(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                   uint32_t box_rows, CUtensorMapL2promotion promo) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(SGLB200_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  cuuint64_t gdim[3] = {dims[0], dims[1], rank == 3 ? dims[2] : 1};
  cuuint64_t gstr[2] = {strides_bytes[0], rank == 3 ? strides_bytes[1] : 0};
  cuuint32_t box[3] = {(cuuint32_t)BK, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SGLB200_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return SGLB200_OK;
}

void launch_splitk_reduce(const float* partial, void* out, int64_t M, int64_t N, int64_t ldc, int splits, int out_dtype,
                          int sm_count, void* stream) {
  const int64_t vecs = M * (N / 8);
  int rgrid = (int)((vecs + 255) / 256);
  if (rgrid > sm_count * 8) rgrid = sm_count * 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == SGLB200_BF16) {
    launch_pdl(splitk_reduce_kernel<__nv_bfloat16>, dim3(rgrid), dim3(256), 0, st, partial, static_cast<__nv_bfloat16*>(out),
               (int32_t)M, (int32_t)N, ldc, (int32_t)splits);
  } else {
    launch_pdl(splitk_reduce_kernel<__half>, dim3(rgrid), dim3(256), 0, st, partial, static_cast<__half*>(out), (int32_t)M,
               (int32_t)N, ldc, (int32_t)splits);
  }
}

namespace {

// Number of k-splits for a dense problem: only when the output tiles alone cannot occupy the SMs (small M, where the
// kernel streams the weights once and is HBM-bound), enough splits for about two work items per SM, each at least
// four k-blocks deep.  Returns 1 when split-K does not apply.
int splitk_choice(int64_t M, int64_t N, int64_t K, int sm_count) {
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int64_t k_tiles = (K + BK - 1) / BK;
  if (tiles * 2 > sm_count || k_tiles < 8) return 1;
  int64_t splits = (2 * (int64_t)sm_count + tiles - 1) / tiles;
  if (splits > k_tiles / 4) splits = k_tiles / 4;
  if (splits > 32) splits = 32;
  return splits < 2 ? 1 : (int)splits;
}

template <bool GROUPED, bool PUSH>
int set_smem_attr_once() {
  static bool done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fp8_block_gemm_kernel<GROUPED, PUSH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(PUSH ? kSmemBytesPush : kSmemBytes));
    if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    done[dev] = true;
  }
  return SGLB200_OK;
}

int gemm_common(const void* a, const void* b, const float* sa, const float* sb, void* out,
                const int32_t* expert_offsets, const int32_t* problem_sizes, int64_t total_rows, int64_t num_experts, int64_t N, int64_t K,
                int64_t lda, int64_t ldb, int64_t ldb_e, int64_t ldc, int64_t sa_stride_m, int64_t sa_stride_k,
                int64_t sb_stride_e, int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype, void* stream,
                float* workspace = nullptr, int64_t workspace_floats = 0, const PushParams* push = nullptr,
                int64_t rows_per_expert = 0, int64_t sa_stride_e = 0) {
  const bool grouped = expert_offsets != nullptr || rows_per_expert > 0;
  SGLB_REQUIRE(total_rows >= 0 && N >= 0 && K >= 0, SGLB200_ERR_SHAPE, "M=%lld N=%lld K=%lld: negative size",
               (long long)total_rows, (long long)N, (long long)K);
  SGLB_REQUIRE(out_dtype == SGLB200_BF16 || out_dtype == SGLB200_F16, SGLB200_ERR_DTYPE,
               "out_dtype=%d: only bf16 (0) and f16 (1)", out_dtype);
  SGLB_REQUIRE(total_rows < ((int64_t)1 << 31) - 256 && N < ((int64_t)1 << 31) - 256 && K < ((int64_t)1 << 31) - 256,
               SGLB200_ERR_SHAPE, "a dimension exceeds 2^31");
  SGLB_REQUIRE(K > 0 || total_rows == 0 || N == 0, SGLB200_ERR_SHAPE, "K must be positive");
  SGLB_REQUIRE(K % 16 == 0, SGLB200_ERR_SHAPE, "K=%lld must be a multiple of 16", (long long)K);
  SGLB_REQUIRE(N % 8 == 0, SGLB200_ERR_SHAPE, "N=%lld must be a multiple of 8 (16-byte output rows)", (long long)N);
  if (grouped)
    SGLB_REQUIRE(num_experts >= 1 && num_experts <= kMaxExperts, SGLB200_ERR_SHAPE, "num_experts=%lld: 1..%d",
                 (long long)num_experts, kMaxExperts);
  if (total_rows == 0 || N == 0) return SGLB200_OK;
  SGLB_REQUIRE(a && b && sa && sb && out, SGLB200_ERR_NULL, "a/b/sa/sb/out must not be NULL");
  SGLB_REQUIRE(lda >= K && lda % 16 == 0, SGLB200_ERR_ALIGN, "lda=%lld must be >= K and a multiple of 16", (long long)lda);
  SGLB_REQUIRE(ldb >= K && ldb % 16 == 0, SGLB200_ERR_ALIGN, "ldb=%lld must be >= K and a multiple of 16", (long long)ldb);
  SGLB_REQUIRE(!grouped || (ldb_e % 16 == 0 && ldb_e >= ldb), SGLB200_ERR_ALIGN,
               "ldb_e=%lld must be a multiple of 16 and >= ldb", (long long)ldb_e);
  SGLB_REQUIRE(ldc >= N && (ldc * 2) % 16 == 0, SGLB200_ERR_ALIGN, "ldc=%lld must be >= N and a multiple of 8",
               (long long)ldc);
  SGLB_REQUIRE(aligned(a, 16) && aligned(b, 16) && aligned(out, 16), SGLB200_ERR_ALIGN,
               "a, b and out must be 16-byte aligned");
  SGLB_REQUIRE(aligned(sa, 4) && aligned(sb, 4), SGLB200_ERR_ALIGN, "scale pointers must be 4-byte aligned");
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  SGLB_REQUIRE(di.cc_major == 10, SGLB200_ERR_ARCH, "compute capability %d.%d: this library is built for sm_100a only",
               di.cc_major, di.cc_minor);

  if (!grouped && push && total_rows <= smallm_max_rows() && workspace != nullptr &&
      (int64_t)smallm_splits(N, K, di.sm_count) * total_rows * N <= workspace_floats) {
    // few rows, exchanged: the weight-streaming kernel leaves fp32 sums, a second kernel casts and pushes them
    int splits = 1;
    if (int rc = smallm_gemm(a, b, sa, sb, out, total_rows, N, K, lda, ldb, ldc, sa_stride_m, sa_stride_k, sb_stride_n,
                             sb_stride_k, out_dtype, workspace, workspace_floats, di.sm_count, stream, &splits, true))
      return rc;
    const int32_t n_tiles = (int32_t)((N + BN - 1) / BN);
    const int32_t tiles = (int32_t)((total_rows + BM - 1) / BM) * n_tiles;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_dtype == SGLB200_BF16)
      splitk_reduce_push_kernel<__nv_bfloat16><<<tiles, 256, 0, st>>>(workspace, splits, (int32_t)total_rows, (int32_t)N,
                                                                     n_tiles, tiles, *push);
    else
      splitk_reduce_push_kernel<__half><<<tiles, 256, 0, st>>>(workspace, splits, (int32_t)total_rows, (int32_t)N,
                                                              n_tiles, tiles, *push);
    SGLB_CHECK_LAUNCH("splitk_reduce_push_kernel");
    return SGLB200_OK;
  }
  if (!grouped && !push && total_rows <= smallm_max_rows()) {
    // few rows: the weight-streaming kernel with swapped operands (gemm_smallm.cu)
    int splits = 1;
    if (int rc = smallm_gemm(a, b, sa, sb, out, total_rows, N, K, lda, ldb, ldc, sa_stride_m, sa_stride_k, sb_stride_n,
                             sb_stride_k, out_dtype, workspace, workspace_floats, di.sm_count, stream, &splits))
      return rc;
    if (splits > 1) launch_splitk_reduce(workspace, out, total_rows, N, ldc, splits, out_dtype, di.sm_count, stream);
    SGLB_CHECK_LAUNCH("splitk_reduce_kernel");
    return SGLB200_OK;
  }

  if (grouped && !push) {
    // few rows per expert: the weight-streaming kernel with swapped operands (gemm_smallm.cu)
    if (const int chunk = smallm_grouped_chunk(total_rows, num_experts, rows_per_expert))
      return smallm_grouped_gemm(chunk, a, b, sa, sb, out, expert_offsets, problem_sizes, rows_per_expert > 0 ? 1 : 3,
                                 total_rows, num_experts, rows_per_expert, N, K, lda, ldb, ldb_e, ldc, sa_stride_e,
                                 sa_stride_m, sa_stride_k, sb_stride_e, sb_stride_n, sb_stride_k, out_dtype, di.sm_count,
                                 stream, false);
  }

  alignas(64) CUtensorMap map_a, map_b;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)total_rows};
    const uint64_t str[1] = {(uint64_t)lda};
    if (int rc = make_map_sw128(&map_a, a, 2, dims, str, BM, CU_TENSOR_MAP_L2_PROMOTION_L2_128B)) return rc;
  }
  {
    const uint64_t E = grouped ? (uint64_t)num_experts : 1;
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, E};
    const uint64_t str[2] = {(uint64_t)ldb, grouped ? (uint64_t)ldb_e : (uint64_t)ldb * (uint64_t)N};
    if (int rc = make_map_sw128(&map_b, b, 3, dims, str, BN, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) return rc;
  }

  PushGemmParams p;
  p.sa = sa;
  p.sb = sb;
  p.out = out;
  p.expert_offsets = expert_offsets;
  p.problem_sizes = problem_sizes;
  p.count_stride = rows_per_expert > 0 ? 1 : 3;
  p.rows_per_expert = (int32_t)rows_per_expert;
  p.sa_stride_e = sa_stride_e;
  p.total_rows = (int32_t)total_rows;
  p.N = (int32_t)N;
  p.K = (int32_t)K;
  p.num_experts = grouped ? (int32_t)num_experts : 1;
  p.m_tiles = (int32_t)((total_rows + BM - 1) / BM);
  p.n_tiles = (int32_t)((N + BN - 1) / BN);
  p.k_tiles = (int32_t)((K + BK - 1) / BK);
  p.ldc = ldc;
  p.sa_stride_m = sa_stride_m;
  p.sa_stride_k = sa_stride_k;
  p.sb_stride_e = grouped ? sb_stride_e : 0;
  p.sb_stride_n = sb_stride_n;
  p.sb_stride_k = sb_stride_k;
  p.out_dtype = out_dtype;
  p.partial = nullptr;
  p.k_splits = 1;
  p.kb_per_split = p.k_tiles;
  if (push) p.push = *push;
  if (!grouped && workspace != nullptr && !push) {
    const int splits = splitk_choice(total_rows, N, K, di.sm_count);
    if (splits > 1 && (int64_t)splits * total_rows * N <= workspace_floats) {
      p.partial = workspace;
      p.kb_per_split = (p.k_tiles + splits - 1) / splits;
      p.k_splits = (p.k_tiles + p.kb_per_split - 1) / p.kb_per_split;
    }
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (grouped) {
    if (int rc = set_smem_attr_once<true, false>()) return rc;
    // an upper bound on the tile count without reading the device: every expert can add one ragged m-tile
    const int64_t max_tiles = ((total_rows + BM - 1) / BM + num_experts) * p.n_tiles;
    const int grid = (int)(max_tiles < di.sm_count ? max_tiles : di.sm_count);
    fp8_block_gemm_kernel<true, false><<<grid, kThreads, kSmemBytes, st>>>(map_a, map_b, static_cast<const GemmParams&>(p));
  } else if (push) {
    if (int rc = set_smem_attr_once<false, true>()) return rc;
    const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
    const int grid = (int)(tiles < di.sm_count ? tiles : di.sm_count);
    fp8_block_gemm_kernel<false, true><<<grid, kThreads, kSmemBytesPush, st>>>(map_a, map_b, p);
  } else {
    const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles * p.k_splits;
    const int grid = (int)(tiles < di.sm_count ? tiles : di.sm_count);
    if (int rc = set_smem_attr_once<false, false>()) return rc;
    fp8_block_gemm_kernel<false, false><<<grid, kThreads, kSmemBytes, st>>>(map_a, map_b, static_cast<const GemmParams&>(p));
    if (p.partial != nullptr) {
      SGLB_CHECK_LAUNCH("fp8_block_gemm_kernel");
      launch_splitk_reduce(p.partial, out, total_rows, N, ldc, p.k_splits, out_dtype, di.sm_count, stream);
    }
  }
  SGLB_CHECK_LAUNCH("fp8_block_gemm_kernel");
  return SGLB200_OK;
}

}  // namespace
}  // namespace sglb

extern "C" int sglb200_fp8_blockwise_scaled_mm(const void* a, const void* b, const float* sa, const float* sb,
                                               void* out, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                               int64_t ldc, int64_t sa_stride_m, int64_t sa_stride_k,
                                               int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype, void* stream) {
  return sglb::gemm_common(a, b, sa, sb, out, nullptr, nullptr, M, 1, N, K, lda, ldb, 0, ldc, sa_stride_m, sa_stride_k, 0,
                           sb_stride_n, sb_stride_k, out_dtype, stream);
}

extern "C" int sglb200_fp8_blockwise_scaled_grouped_mm(const void* a, const void* b, const float* sa, const float* sb,
                                                       void* out, const int32_t* expert_offsets,
                                                       const int32_t* problem_sizes, int64_t total_rows,
                                                       int64_t num_experts, int64_t N, int64_t K, int64_t lda,
                                                       int64_t ldb, int64_t ldb_e, int64_t ldc, int64_t sa_stride_m,
                                                       int64_t sa_stride_k, int64_t sb_stride_e, int64_t sb_stride_n,
                                                       int64_t sb_stride_k, int out_dtype, void* stream) {
  SGLB_REQUIRE(expert_offsets != nullptr, SGLB200_ERR_NULL, "expert_offsets must not be NULL");
  return sglb::gemm_common(a, b, sa, sb, out, expert_offsets, problem_sizes, total_rows, num_experts, N, K, lda, ldb, ldb_e, ldc,
                           sa_stride_m, sa_stride_k, sb_stride_e, sb_stride_n, sb_stride_k, out_dtype, stream);
}

extern "C" int sglb200_fp8_blockwise_scaled_masked_grouped_mm(const void* a, const void* b, const float* sa,
                                                              const float* sb, void* out, const int32_t* masked_m,
                                                              int64_t num_groups, int64_t max_m, int64_t N, int64_t K,
                                                              int64_t lda, int64_t ldb, int64_t ldb_e, int64_t ldc,
                                                              int64_t sa_stride_g, int64_t sa_stride_m,
                                                              int64_t sa_stride_k, int64_t sb_stride_e,
                                                              int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype,
                                                              void* stream) {
  SGLB_REQUIRE(num_groups >= 0 && max_m >= 0 && num_groups * max_m < ((int64_t)1 << 31) - 256, SGLB200_ERR_SHAPE,
               "num_groups=%lld max_m=%lld", (long long)num_groups, (long long)max_m);
  if (num_groups == 0 || max_m == 0) return SGLB200_OK;
  SGLB_REQUIRE(masked_m != nullptr, SGLB200_ERR_NULL, "masked_m must not be NULL");
  return sglb::gemm_common(a, b, sa, sb, out, nullptr, masked_m, num_groups * max_m, num_groups, N, K, lda, ldb, ldb_e, ldc,
                           sa_stride_m, sa_stride_k, sb_stride_e, sb_stride_n, sb_stride_k, out_dtype, stream, nullptr, 0,
                           nullptr, max_m, sa_stride_g);
}

extern "C" int64_t sglb200_fp8_blockwise_scaled_mm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  sglb::DeviceInfo di;
  int sms = 148;
  if (sglb::device_info(&di) == SGLB200_OK) sms = di.sm_count;
  const int splits = M <= sglb::smallm_max_rows() ? sglb::smallm_splits(N, K, sms) : sglb::splitk_choice(M, N, K, sms);
  return splits > 1 ? (int64_t)splits * M * N * (int64_t)sizeof(float) : 0;
}

extern "C" int sglb200_fp8_blockwise_scaled_mm_ws(const void* a, const void* b, const float* sa, const float* sb,
                                                  void* out, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                                  int64_t ldc, int64_t sa_stride_m, int64_t sa_stride_k,
                                                  int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype,
                                                  void* workspace, int64_t workspace_bytes, void* stream) {
  SGLB_REQUIRE(workspace_bytes >= 0, SGLB200_ERR_WORKSPACE, "workspace_bytes=%lld", (long long)workspace_bytes);
  SGLB_REQUIRE(workspace == nullptr || sglb::aligned(workspace, 16), SGLB200_ERR_ALIGN,
               "workspace must be 16-byte aligned");
  return sglb::gemm_common(a, b, sa, sb, out, nullptr, nullptr, M, 1, N, K, lda, ldb, 0, ldc, sa_stride_m, sa_stride_k,
                           0, sb_stride_n, sb_stride_k, out_dtype, stream, static_cast<float*>(workspace),
                           workspace ? workspace_bytes / (int64_t)sizeof(float) : 0);
}

// ---------------------------------------------------------------------------------------------------------
// Split-K GEMM for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc or any allocating routine at the point where they run a
// GEMM: an engine that has handed all device memory to its own pool and forbids side allocations, code running
// inside a region where allocation is disallowed, or a plain C caller with no allocator at hand.  For them the
// split-K scratch lives in the library image itself: a file-scope device array of fixed size that every GPU
// loading the library holds until the process exits.
// ---------------------------------------------------------------------------------------------------------
namespace sglb {
namespace {
constexpr int64_t kStaticWsFloats = 4ll * 1024 * 1024;  // 16 MiB: splits * M * N fp32 partial sums
static __device__ __align__(256) float g_static_splitk_ws[kStaticWsFloats];

// In host code the array's name is only a handle; the device address has to be asked for, once per device,
// with that device current.
int static_ws_address(float** out) {
  static float* addr[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return fail(SGLB200_ERR_LAUNCH, "cudaGetDevice failed");
  }
  if (addr[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_splitk_ws);
    if (e != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return fail(SGLB200_ERR_LAUNCH, "cudaGetSymbolAddress(static split-K scratch): %s", cudaGetErrorString(e));
    }
    addr[dev] = static_cast<float*>(ptr);
  }
  *out = addr[dev];
  return SGLB200_OK;
}
}  // namespace
}  // namespace sglb

extern "C" int64_t sglb200_fp8_blockwise_scaled_mm_noalloc_max_bytes(void) {
  return sglb::kStaticWsFloats * (int64_t)sizeof(float);
}

extern "C" int sglb200_fp8_blockwise_scaled_mm_noalloc(const void* a, const void* b, const float* sa, const float* sb,
                                                       void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                                                       int64_t ldb, int64_t ldc, int64_t sa_stride_m,
                                                       int64_t sa_stride_k, int64_t sb_stride_n, int64_t sb_stride_k,
                                                       int out_dtype, void* stream) {
  const int64_t need = sglb200_fp8_blockwise_scaled_mm_workspace_bytes(M, N, K);
  if (need > sglb::kStaticWsFloats * (int64_t)sizeof(float)) {
    return sglb::fail(SGLB200_ERR_WORKSPACE,
                      "M=%lld N=%lld K=%lld needs %lld bytes of split-K scratch; the built-in buffer holds %lld "
                      "(use sglb200_fp8_blockwise_scaled_mm_ws with your own buffer, or sglb200_fp8_blockwise_scaled_mm)",
                      (long long)M, (long long)N, (long long)K, (long long)need,
                      (long long)(sglb::kStaticWsFloats * (int64_t)sizeof(float)));
  }
  float* ws = nullptr;
  if (need > 0) {
    if (int rc = sglb::static_ws_address(&ws)) return rc;
  }
  return sglb::gemm_common(a, b, sa, sb, out, nullptr, nullptr, M, 1, N, K, lda, ldb, 0, ldc, sa_stride_m, sa_stride_k,
                           0, sb_stride_n, sb_stride_k, out_dtype, stream, ws, ws ? sglb::kStaticWsFloats : 0);
}

// Bytes of one rank's flag area for the peer exchanges: the flag words followed by the control words.
extern "C" int64_t sglb200_peer_flag_bytes(void) {
  static_assert(sglb::kEpiWarps == 8, "kFlagWords assumes 8 flag words per tile");
  return (sglb::kFlagWords + 64) * (int64_t)sizeof(uint32_t);  // flag words, then the control words
}

extern "C" int sglb200_peer_completed(const void* flags_local, int64_t* completed) {
  SGLB_REQUIRE(flags_local && completed, SGLB200_ERR_NULL, "flags_local and completed must be given");
  uint32_t v = 0;
  cudaError_t e = cudaMemcpy(&v, static_cast<const uint32_t*>(flags_local) + sglb::kFlagWords, sizeof(v),
                             cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return sglb::fail(SGLB200_ERR_LAUNCH, "cudaMemcpy: %s", cudaGetErrorString(e));
  *completed = v;
  return SGLB200_OK;
}

extern "C" int64_t sglb200_fp8_blockwise_scaled_mm_push_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0 || M > sglb::smallm_max_rows()) return 0;
  sglb::DeviceInfo di;
  int sms = 148;
  if (sglb::device_info(&di) == SGLB200_OK) sms = di.sm_count;
  return (int64_t)sglb::smallm_splits(N, K, sms) * M * N * (int64_t)sizeof(float);
}

extern "C" int64_t sglb200_peer_recv_bytes(int64_t slot_elems) {
  return (int64_t)2 * sglb::kMaxPeers * slot_elems * 2;
}

namespace sglb {
namespace {
int check_push_args(int64_t M, int64_t N, int world, int rank, int64_t slot_elems) {
  SGLB_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, SGLB200_ERR_SHAPE,
               "world=%d (1..%d) rank=%d", world, kMaxPeers, rank);
  SGLB_REQUIRE(slot_elems % 8 == 0 && M * N <= slot_elems, SGLB200_ERR_WORKSPACE,
               "M*N=%lld does not fit a receive slot of %lld elements (a multiple of 8)", (long long)(M * N),
               (long long)slot_elems);
  SGLB_REQUIRE(((M + BM - 1) / BM) * ((N + BN - 1) / BN) <= kPushMaxTiles, SGLB200_ERR_WORKSPACE,
               "more than %d output tiles: too large for the one-shot exchange", kPushMaxTiles);
  return SGLB200_OK;
}
}  // namespace
}  // namespace sglb

namespace sglb {
namespace {
int fill_push(PushParams* push, void* const* peer_recv, void* const* peer_flags, int rank, int world, int64_t slot_elems,
              int scatter) {
  SGLB_REQUIRE(peer_recv && peer_flags, SGLB200_ERR_NULL, "peer_recv / peer_flags must not be NULL");
  for (int i = 0; i < kMaxPeers; ++i) {
    push->dst[i] = i < world ? peer_recv[i] : nullptr;
    push->flag[i] = i < world ? static_cast<uint32_t*>(peer_flags[i]) : nullptr;
    SGLB_REQUIRE(i >= world || (push->dst[i] && push->flag[i] && aligned(push->dst[i], 16) && aligned(push->flag[i], 4)),
                 SGLB200_ERR_NULL, "peer %d: receive buffer / flags missing or misaligned", i);
  }
  push->world = world;
  push->rank = rank;
  push->ctl = push->flag[rank] + kFlagWords;
  push->slot_elems = slot_elems;
  push->scatter = scatter;
  return SGLB200_OK;
}

// the two-shot exchange needs every rank to own a tile (the ranks keep in step through the tiles they exchange)
int check_scatter_args(int64_t M, int64_t N, int world) {
  SGLB_REQUIRE(((M + BM - 1) / BM) * ((N + BN - 1) / BN) >= world, SGLB200_ERR_SHAPE,
               "M=%lld N=%lld: fewer output tiles than ranks (%d); use the one-shot exchange", (long long)M, (long long)N,
               world);
  return SGLB200_OK;
}
}  // namespace
}  // namespace sglb

extern "C" int sglb200_fp8_blockwise_scaled_mm_push(const void* a, const void* b, const float* sa, const float* sb,
                                                    int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                                    int64_t sa_stride_m, int64_t sa_stride_k, int64_t sb_stride_n,
                                                    int64_t sb_stride_k, int out_dtype, void* const* peer_recv,
                                                    void* const* peer_flags, int rank, int world,
                                                    int64_t slot_elems, void* workspace, int64_t workspace_bytes,
                                                    void* stream) {
  using namespace sglb;
  if (int rc = check_push_args(M, N, world, rank, slot_elems)) return rc;
  PushParams push;
  if (int rc = fill_push(&push, peer_recv, peer_flags, rank, world, slot_elems, 0)) return rc;
  SGLB_REQUIRE(workspace == nullptr || aligned(workspace, 16), SGLB200_ERR_ALIGN, "workspace must be 16-byte aligned");
  return gemm_common(a, b, sa, sb, push.dst[rank], nullptr, nullptr, M, 1, N, K, lda, ldb, 0, N, sa_stride_m, sa_stride_k,
                     0, sb_stride_n, sb_stride_k, out_dtype, stream, static_cast<float*>(workspace),
                     workspace ? workspace_bytes / (int64_t)sizeof(float) : 0, &push);
}

extern "C" int sglb200_fp8_blockwise_scaled_mm_push_scatter(const void* a, const void* b, const float* sa, const float* sb,
                                                            int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                                            int64_t sa_stride_m, int64_t sa_stride_k,
                                                            int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype,
                                                            void* const* peer_recv, void* const* peer_flags, int rank,
                                                            int world, int64_t slot_elems, void* stream) {
  using namespace sglb;
  if (int rc = check_push_args(M, N, world, rank, slot_elems)) return rc;
  if (int rc = check_scatter_args(M, N, world)) return rc;
  PushParams push;
  if (int rc = fill_push(&push, peer_recv, peer_flags, rank, world, slot_elems, 1)) return rc;
  return gemm_common(a, b, sa, sb, push.dst[rank], nullptr, nullptr, M, 1, N, K, lda, ldb, 0, N, sa_stride_m, sa_stride_k,
                     0, sb_stride_n, sb_stride_k, out_dtype, stream, nullptr, 0, &push);
}

namespace sglb {
namespace {
int check_reduce_out(const void* out, int64_t M, int64_t N, int64_t ldc, int out_dtype, int* sm_count) {
  SGLB_REQUIRE(out_dtype == SGLB200_BF16 || out_dtype == SGLB200_F16, SGLB200_ERR_DTYPE, "out_dtype=%d", out_dtype);
  SGLB_REQUIRE(out, SGLB200_ERR_NULL, "out must not be NULL");
  SGLB_REQUIRE(ldc >= N && ldc % 8 == 0 && aligned(out, 16), SGLB200_ERR_ALIGN,
               "ldc=%lld must be >= N and a multiple of 8; out 16-byte aligned", (long long)ldc);
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  SGLB_REQUIRE(di.cc_major == 10, SGLB200_ERR_ARCH, "compute capability %d.%d: this library is built for sm_100a only",
               di.cc_major, di.cc_minor);
  *sm_count = di.sm_count;
  return SGLB200_OK;
}
}  // namespace
}  // namespace sglb

extern "C" int sglb200_peer_reduce_scatter(void* const* peer_recv, void* const* peer_flags, void* out, int64_t M,
                                           int64_t N, int64_t ldc, int out_dtype, int rank, int world,
                                           int64_t slot_elems, int64_t timeout_ns, void* stream) {
  using namespace sglb;
  SGLB_REQUIRE(M > 0 && N > 0 && N % 8 == 0, SGLB200_ERR_SHAPE, "M=%lld N=%lld (N must be a multiple of 8)", (long long)M,
               (long long)N);
  if (int rc = check_push_args(M, N, world, rank, slot_elems)) return rc;
  if (int rc = check_scatter_args(M, N, world)) return rc;
  PushParams push;
  if (int rc = fill_push(&push, peer_recv, peer_flags, rank, world, slot_elems, 1)) return rc;
  int sms = 0;
  if (int rc = check_reduce_out(out, M, N, ldc, out_dtype, &sms)) return rc;
  const int32_t n_tiles = (int32_t)((N + BN - 1) / BN);
  const int32_t tiles = (int32_t)((M + BM - 1) / BM) * n_tiles;
  const int32_t items = ((tiles - rank + world - 1) / world) * 4;  // (owned tile, quarter of its rows)
  const int grid = items < 4 * sms ? items : 4 * sms;
  const uint64_t limit = timeout_ns > 0 ? (uint64_t)timeout_ns : 2000000000ull;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == SGLB200_BF16)
    peer_reduce_scatter_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(push, static_cast<__nv_bfloat16*>(out), (int32_t)M,
                                                                   (int32_t)N, ldc, n_tiles, items, limit);
  else
    peer_reduce_scatter_kernel<__half><<<grid, 256, 0, st>>>(push, static_cast<__half*>(out), (int32_t)M, (int32_t)N, ldc,
                                                            n_tiles, items, limit);
  SGLB_CHECK_LAUNCH("peer_reduce_scatter_kernel");
  return SGLB200_OK;
}

extern "C" int sglb200_peer_gather(const void* recv_local, void* flags_local, void* out, int64_t M, int64_t N, int64_t ldc,
                                   int out_dtype, int rank, int world, int64_t slot_elems, int64_t timeout_ns,
                                   void* stream) {
  using namespace sglb;
  SGLB_REQUIRE(M > 0 && N > 0 && N % 8 == 0, SGLB200_ERR_SHAPE, "M=%lld N=%lld (N must be a multiple of 8)", (long long)M,
               (long long)N);
  if (int rc = check_push_args(M, N, world, rank, slot_elems)) return rc;
  if (int rc = check_scatter_args(M, N, world)) return rc;
  SGLB_REQUIRE(recv_local && flags_local && aligned(recv_local, 16), SGLB200_ERR_NULL,
               "recv_local (16-byte aligned) / flags_local must not be NULL");
  int sms = 0;
  if (int rc = check_reduce_out(out, M, N, ldc, out_dtype, &sms)) return rc;
  const int32_t n_tiles = (int32_t)((N + BN - 1) / BN);
  const int32_t items = (int32_t)((M + BM - 1) / BM) * n_tiles * 4;
  const int grid = items < 4 * sms ? items : 4 * sms;
  const uint64_t limit = timeout_ns > 0 ? (uint64_t)timeout_ns : 2000000000ull;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* fl = static_cast<uint32_t*>(flags_local);
  if (out_dtype == SGLB200_BF16)
    peer_gather_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(recv_local), fl,
                                                           fl + kFlagWords, static_cast<__nv_bfloat16*>(out), (int32_t)M,
                                                           (int32_t)N, ldc, n_tiles, items, world, rank, slot_elems, limit);
  else
    peer_gather_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(recv_local), fl, fl + kFlagWords,
                                                    static_cast<__half*>(out), (int32_t)M, (int32_t)N, ldc, n_tiles, items,
                                                    world, rank, slot_elems, limit);
  SGLB_CHECK_LAUNCH("peer_gather_kernel");
  return SGLB200_OK;
}

extern "C" int sglb200_peer_reduce(const void* recv_local, void* flags_local, void* out, int64_t M, int64_t N,
                                   int64_t ldc, int out_dtype, int world, int64_t slot_elems, int64_t timeout_ns,
                                   void* stream) {
  using namespace sglb;
  SGLB_REQUIRE(M >= 0 && N >= 0 && N % 8 == 0, SGLB200_ERR_SHAPE, "M=%lld N=%lld (N must be a multiple of 8)",
               (long long)M, (long long)N);
  if (int rc = check_push_args(M, N, world, 0, slot_elems)) return rc;
  SGLB_REQUIRE(out_dtype == SGLB200_BF16 || out_dtype == SGLB200_F16, SGLB200_ERR_DTYPE, "out_dtype=%d", out_dtype);
  if (M == 0 || N == 0) return SGLB200_OK;
  SGLB_REQUIRE(recv_local && flags_local && out, SGLB200_ERR_NULL, "recv_local / flags_local / out must not be NULL");
  SGLB_REQUIRE(ldc >= N && ldc % 8 == 0 && aligned(out, 16) && aligned(recv_local, 16), SGLB200_ERR_ALIGN,
               "ldc=%lld must be >= N and a multiple of 8; out and recv_local 16-byte aligned", (long long)ldc);
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  SGLB_REQUIRE(di.cc_major == 10, SGLB200_ERR_ARCH, "compute capability %d.%d: this library is built for sm_100a only",
               di.cc_major, di.cc_minor);
  const int32_t n_tiles = (int32_t)((N + BN - 1) / BN);
  const int32_t tiles = (int32_t)((M + BM - 1) / BM) * n_tiles * 4;  // work items: (tile, quarter of its rows)
  const int grid = tiles < 4 * di.sm_count ? tiles : 4 * di.sm_count;
  const uint64_t limit = timeout_ns > 0 ? (uint64_t)timeout_ns : 2000000000ull;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* fl = static_cast<uint32_t*>(flags_local);
  if (out_dtype == SGLB200_BF16) {
    peer_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(recv_local), fl,
                                                           fl + kFlagWords, static_cast<__nv_bfloat16*>(out),
                                                           (int32_t)M, (int32_t)N, ldc, n_tiles, tiles, world,
                                                           slot_elems, limit);
  } else {
    peer_reduce_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(recv_local), fl, fl + kFlagWords,
                                                    static_cast<__half*>(out), (int32_t)M, (int32_t)N, ldc, n_tiles,
                                                    tiles, world, slot_elems, limit);
  }
  SGLB_CHECK_LAUNCH("peer_reduce_kernel");
  return SGLB200_OK;
}

// GEMM + all-reduce in one cooperative launch (see ArParams).  `out` is this rank's mapping of a buffer that every rank
// maps through one multicast address (multicast_out = the multicast address of out[0][0]); rows are contiguous
// (row stride N).  done_counters: at least 64 device words, scratch (zeroed here on the stream).
extern "C" int sglb200_fp8_blockwise_scaled_mm_allreduce(const void* a, const void* b, const float* sa, const float* sb,
                                                         void* out, uint64_t multicast_out, const uint64_t* flag_blocks,
                                                         void* done_counters, int rank, int world, int comm_ctas,
                                                         int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                                         int64_t sa_stride_m, int64_t sa_stride_k, int64_t sb_stride_n,
                                                         int64_t sb_stride_k, int out_dtype, void* stream) {
  using namespace sglb;
  SGLB_REQUIRE(M >= 0 && N >= 0 && K > 0, SGLB200_ERR_SHAPE, "M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  SGLB_REQUIRE(out_dtype == SGLB200_BF16 || out_dtype == SGLB200_F16, SGLB200_ERR_DTYPE,
               "out_dtype=%d: only bf16 (0) and f16 (1)", out_dtype);
  SGLB_REQUIRE(M < ((int64_t)1 << 31) - 256 && N < ((int64_t)1 << 31) - 256 && K < ((int64_t)1 << 31) - 256,
               SGLB200_ERR_SHAPE, "a dimension exceeds 2^31");
  SGLB_REQUIRE(K % 16 == 0 && N % 8 == 0, SGLB200_ERR_SHAPE, "K=%lld must be a multiple of 16 and N=%lld of 8",
               (long long)K, (long long)N);
  SGLB_REQUIRE(world >= 2 && world <= nvls::kMaxRanks && rank >= 0 && rank < world, SGLB200_ERR_SHAPE,
               "rank=%d world=%d: 2..%d ranks", rank, world, nvls::kMaxRanks);
  SGLB_REQUIRE(comm_ctas >= 1 && comm_ctas <= 64, SGLB200_ERR_SHAPE, "comm_ctas=%d: 1..64", comm_ctas);
  if (M == 0 || N == 0) return SGLB200_OK;
  SGLB_REQUIRE((M + BM - 1) / BM <= 64 * kGroupMAr, SGLB200_ERR_SHAPE, "M=%lld: at most %d rows (64 row blocks)",
               (long long)M, 64 * kGroupMAr * BM);
  SGLB_REQUIRE(a && b && sa && sb && out && flag_blocks && done_counters && multicast_out, SGLB200_ERR_NULL,
               "a/b/sa/sb/out/multicast_out/flag_blocks/done_counters must not be NULL");
  SGLB_REQUIRE(lda >= K && lda % 16 == 0 && ldb >= K && ldb % 16 == 0, SGLB200_ERR_ALIGN,
               "lda=%lld / ldb=%lld must be >= K and multiples of 16", (long long)lda, (long long)ldb);
  SGLB_REQUIRE(aligned(a, 16) && aligned(b, 16) && aligned(out, 16) && multicast_out % 16 == 0 && aligned(sa, 4) &&
                   aligned(sb, 4) && aligned(done_counters, 4),
               SGLB200_ERR_ALIGN, "a, b, out and the multicast address must be 16-byte aligned");
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  SGLB_REQUIRE(di.cc_major == 10, SGLB200_ERR_ARCH, "compute capability %d.%d: this library is built for sm_100a only",
               di.cc_major, di.cc_minor);
  SGLB_REQUIRE(comm_ctas < di.sm_count, SGLB200_ERR_SHAPE, "comm_ctas=%d leaves no SM for the GEMM", comm_ctas);

  alignas(64) CUtensorMap map_a, map_b;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t str[1] = {(uint64_t)lda};
    if (int rc = make_map_sw128(&map_a, a, 2, dims, str, BM, CU_TENSOR_MAP_L2_PROMOTION_L2_128B)) return rc;
  }
  {
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, 1};
    const uint64_t str[2] = {(uint64_t)ldb, (uint64_t)ldb * (uint64_t)N};
    if (int rc = make_map_sw128(&map_b, b, 3, dims, str, BN, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) return rc;
  }
  ArGemmParams p;
  p.sa = sa;
  p.sb = sb;
  p.out = out;
  p.expert_offsets = nullptr;
  p.problem_sizes = nullptr;
  p.count_stride = 3;
  p.rows_per_expert = 0;
  p.sa_stride_e = 0;
  p.total_rows = (int32_t)M;
  p.N = (int32_t)N;
  p.K = (int32_t)K;
  p.num_experts = 1;
  p.m_tiles = (int32_t)((M + BM - 1) / BM);
  p.n_tiles = (int32_t)((N + BN - 1) / BN);
  p.k_tiles = (int32_t)((K + BK - 1) / BK);
  p.ldc = N;
  p.sa_stride_m = sa_stride_m;
  p.sa_stride_k = sa_stride_k;
  p.sb_stride_e = 0;
  p.sb_stride_n = sb_stride_n;
  p.sb_stride_k = sb_stride_k;
  p.out_dtype = out_dtype;
  p.partial = nullptr;
  p.k_splits = 1;
  p.kb_per_split = p.k_tiles;
  p.ar.mc_out = multicast_out;
  for (int i = 0; i < nvls::kMaxRanks; ++i) {
    p.ar.fp.p[i] = i < world ? reinterpret_cast<uint32_t*>(flag_blocks[i]) : nullptr;
    SGLB_REQUIRE(i >= world || (p.ar.fp.p[i] != nullptr && flag_blocks[i] % 4 == 0), SGLB200_ERR_NULL,
                 "flag block of rank %d is NULL or misaligned", i);
  }
  p.ar.done = static_cast<uint32_t*>(done_counters);
  p.ar.rank = rank;
  p.ar.world = world;
  p.ar.comm_ctas = comm_ctas;
  p.ar.limit_ns = 2000000000ull;

  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fp8_block_gemm_kernel<false, false, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done[dev] = true;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(done_counters, 0, 64 * sizeof(uint32_t), st);
  if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  // the communication CTAs wait for the tile CTAs of the same grid: every CTA must be resident (cooperative launch),
  // one CTA per SM
  const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
  const int64_t gemm_ctas = tiles < di.sm_count - comm_ctas ? tiles : di.sm_count - comm_ctas;
  const int grid = (int)gemm_ctas + comm_ctas;
  void* args[] = {(void*)&map_a, (void*)&map_b, (void*)&p};
  e = cudaLaunchCooperativeKernel((const void*)fp8_block_gemm_kernel<false, false, true>, dim3(grid), dim3(kThreads), args,
                                  kSmemBytes, st);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(SGLB200_ERR_LAUNCH, "fp8_block_gemm_kernel (fused all-reduce): %s", cudaGetErrorString(e));
  }
  return SGLB200_OK;
}


namespace sglb {
int ue8m0_take_device_status();  // gemm_ue8m0.cu
int ep_take_device_status();     // ep_peer.cu
int pair_take_device_status();   // gemm_pair.cu
}
// Reads AND clears the device-side status words of every kernel family: 0, or the code of the first bounded wait that
// timed out (1 producer, 2/3 MMA issuer, 4 promotion warps, 5 peer flags / tail drain; 11-18 the same roles in the
// UE8M0 and few-rows kernels; 21-23 expert-parallel exchange; 31-35 CTA-pair kernel).  All words are read and cleared on every call, so a
// status never outlives the call that reports it; when several are set, the first non-zero one in the order UE8M0,
// few-rows, expert-parallel, CTA-pair, multicast all-reduce, dense is returned.  Synchronises the device: for tests and debugging, not for the
// serving path.
extern "C" int sglb200_read_device_status(void) {
  const int u = sglb::ue8m0_take_device_status();
  const int sm = sglb::smallm_take_device_status();
  const int ep = sglb::ep_take_device_status();
  const int pr = sglb::pair_take_device_status();
  const int nv = sglb::nvls_take_device_status();
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, sglb::g_device_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    v = -1;
  } else if (v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(sglb::g_device_status, &z, sizeof(int));
  }
  if (u != 0) return u;
  if (sm != 0) return sm;
  if (ep != 0) return ep;
  if (pr != 0) return pr;
  if (nv != 0) return nv;
  return v;
}
