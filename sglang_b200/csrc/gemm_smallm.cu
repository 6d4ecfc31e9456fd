// Block-scaled FP8 GEMM for few rows of activations (M <= 128: the decode case), weight-streaming bound.
//
// The roles of the operands are swapped: the tensor core computes C^T = W * A^T, a tile being 128 WEIGHT rows (the MMA's
// M) by MT token columns (the MMA's N, MT = 16 / 32 / 64).  An accumulator stage is then only MT TMEM columns wide, so 8 to
// 16 k-blocks are in flight between the MMA warp and the promotion warps instead of 4, and a shared-memory stage is 16 KB
// of weights plus MT x 128 bytes of activations, so 8 to 10 stages (128 to 160 KB of weights) are in flight per SM: the
// kernel is bound by HBM, not by the accumulator hand-off of the 128 x 128 kernel.  K can be cut into ranges that run on
// different SMs (fp32 partial sums, added by splitk_reduce_kernel) when N / 128 tiles alone cannot occupy the SMs.
// From 65 to 128 rows the tile is 128 x 128 (4 accumulator stages, 7 shared-memory stages) and eight promotion warps
// share every accumulator stage, four per 64 token columns: what is left of the advantage over the 128 x 128 kernel is
// the deeper weight ring and the single role per warp (measured 7-15 % at 96-128 rows).
//
// GROUPED variant (one weight matrix per expert, few rows per expert: the decode case of a mixture-of-experts layer): a
// work item is (expert, 128 weight rows, chunk of MT of the expert's rows).  The row ranges come from the same device
// tables as in the 128 x 128 grouped kernel; an expert with more than MT rows gets several chunks (its weight tile is
// then re-read, from L2), an expert without rows gets no item, so only the weights of routed experts are streamed.
//
// warp 0: TMA producer; warp 1: TMEM owner + MMA issuer; warps 2..5: promotion (tcgen05.ld, acc += p * sa[token] * sb)
// and the transposed store.  All waits are bounded.
//
// The kernel is launched with programmatic stream serialization: it may start while the kernel before it (the
// activation quantiser, or the previous layer's reduce kernel) is still running.  Its set-up and the WEIGHT tiles of the
// first ring of stages depend on nothing earlier in the stream and are issued at once; the activation tiles, the
// activation scales and every store come after griddepcontrol.wait.  At decode sizes the fixed cost of a call (launch,
// set-up, first TMA round trip) is of the order of the streaming time itself, and this hides most of it.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace sglb {

// device status word of this translation unit (0 = no bounded wait ran out); collected by sglb200_read_device_status
__device__ int g_smallm_status = 0;

int smallm_take_device_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_smallm_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (v != 0) {
    const int z = 0;
    cudaMemcpyToSymbol(g_smallm_status, &z, sizeof(int));
  }
  return v;
}

namespace {

constexpr int BN = 128, BK = 128;  // weight rows per tile, K per block
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kWBytes = BN * BK;
constexpr int kScaleAhead = 4;

constexpr int kMaxExperts = 1024;

// NSUB = 2 (dense, 64 < M <= 128): the MMA covers MT * NSUB = 128 activation rows (one instruction shape 128 x 128, so
// the issuing thread's cost per k-block stays that of the narrow tiles) and a second set of four promotion warps takes
// the second half of every accumulator stage's columns, so the registers per thread stay those of 64 rows.
template <int MT, int NSUB = 1>
struct Cfg {
  static constexpr int kTile = MT * NSUB;  // activation rows per work item = the MMA's N = TMEM columns per stage
  static constexpr int kStages = kTile == 128 ? 7 : (kTile == 64 ? 8 : 10);
  static constexpr int kAcc = (512 / kTile) < 16 ? (512 / kTile) : 16;
  static constexpr int kThreads = 64 + 128 * NSUB;
  static constexpr uint32_t kABytes = kTile * BK;
  static constexpr uint32_t kStageBytes = kWBytes + kABytes;
  static constexpr size_t kSmem = 1024 + (size_t)kStages * kStageBytes + 512;
  // grouped: the table of first work items per expert follows the control block
  static constexpr size_t kSmemGrouped = kSmem + (kMaxExperts + 1) * sizeof(int32_t) + 12;
};

struct SmallParams {
  const float* sa;  // UE8M0 variant: int32 words, four exponent bytes (k-blocks 4g .. 4g + 3) per word
  const float* sb;
  void* out;
  float* partial;  // [splits][M][N] fp32 when k_splits > 1
  int32_t M, N, K;
  int32_t n_tiles, k_tiles, k_splits, kb_per_split;
  int64_t ldc;
  int64_t sa_stride_m, sa_stride_k, sb_stride_n, sb_stride_k;
  int32_t out_dtype;
  // grouped only
  const int32_t* expert_offsets;  // [E + 1] first row of every expert, or NULL in the masked layout
  const int32_t* problem_sizes;   // optional: rows of expert e = problem_sizes[count_stride * e]
  int32_t count_stride, rows_per_expert, num_experts;
  int64_t sa_stride_e, sb_stride_e;
};

// one unit of work: rows [row0, row0 + rows) of the activations against weight rows [nt * 128, +128) of expert e,
// k-blocks [kb0, kb1)
struct Item {
  int32_t e, nt, row0, rows, kb0, kb1, split;
};

__device__ __forceinline__ void expert_rows(const SmallParams& p, int32_t e, int32_t* r0, int32_t* cnt) {
  if (p.rows_per_expert > 0) {
    *r0 = e * p.rows_per_expert;
    *cnt = max(0, min(__ldg(p.problem_sizes + p.count_stride * e), p.rows_per_expert));
  } else {
    *r0 = __ldg(p.expert_offsets + e);
    *cnt = max(0, p.problem_sizes ? __ldg(p.problem_sizes + p.count_stride * e) : __ldg(p.expert_offsets + e + 1) - *r0);
  }
}

template <int MT, bool GROUPED>
__device__ __forceinline__ Item get_item(const SmallParams& p, const int32_t* item_start, int32_t t) {
  Item it;
  if constexpr (!GROUPED) {
    it.split = t / p.n_tiles;
    it.nt = t - it.split * p.n_tiles;
    it.kb0 = it.split * p.kb_per_split;
    it.kb1 = min(it.kb0 + p.kb_per_split, p.k_tiles);
    it.e = 0;
    it.row0 = 0;
    it.rows = p.M;
  } else {
    int32_t lo = 0, hi = p.num_experts;  // last e with item_start[e] <= t
    while (hi - lo > 1) {
      const int32_t mid = (lo + hi) >> 1;
      if (item_start[mid] <= t) lo = mid; else hi = mid;
    }
    int32_t r0, cnt;
    expert_rows(p, lo, &r0, &cnt);
    const int32_t chunks = (cnt + MT - 1) / MT;
    const int32_t local = t - item_start[lo];
    it.e = lo;
    it.nt = local / chunks;
    const int32_t ch = local - it.nt * chunks;
    it.row0 = r0 + ch * MT;
    it.rows = min(MT, cnt - ch * MT);
    it.kb0 = 0;
    it.kb1 = p.k_tiles;
    it.split = 0;
  }
  return it;
}

struct Ctl {
  uint64_t full[10];
  uint64_t empty[10];
  uint64_t acc_full[16];
  uint64_t acc_empty[16];
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  int32_t total;
};
static_assert(sizeof(Ctl) <= 512, "control block");

__device__ __forceinline__ void timeout(Ctl* ctl, int code) {
  ctl->abort_flag = 1;
  atomicCAS(&g_smallm_status, 0, code);
}

// 32 lanes x N consecutive fp32 columns
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t* r);
template <>
__device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld_cols<32>(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// wait for this thread's outstanding tcgen05.ld; the registers are tied to the statement so that their first use
// cannot move above it
template <int N>
__device__ __forceinline__ void tmem_ld_fence(uint32_t* r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < N; ++i) asm volatile("" : "+r"(r[i])::"memory");
}

// scale of k-block kc: fp32 at base[kc * stride_k], or 2^(byte - 127) of the packed word at base[(kc / 4) * stride_k]
template <bool UE>
__device__ __forceinline__ float load_scale(const float* base, int32_t kc, int64_t stride_k) {
  if constexpr (UE) {
    const uint32_t w = (uint32_t)__ldg(reinterpret_cast<const int32_t*>(base) + (int64_t)(kc >> 2) * stride_k);
    return __uint_as_float(((w >> (8 * (kc & 3))) & 0xffu) << 23);
  } else {
    return __ldg(base + (int64_t)kc * stride_k);
  }
}

template <int MT, bool UE, bool GROUPED, int NSUB>
__global__ void __launch_bounds__(64 + 128 * NSUB, 1)
fp8_block_gemm_smallm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                             const SmallParams p) {
  using C = Cfg<MT, NSUB>;
  static_assert(!GROUPED || NSUB == 1, "the grouped form has one sub-tile");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + (size_t)C::kStages * C::kStageBytes);
  int32_t* item_start = reinterpret_cast<int32_t*>(smem + (size_t)C::kStages * C::kStageBytes + 512);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      ptx::mbar_init(&ctl->full[i], 1);
      ptx::mbar_init(&ctl->empty[i], 1);
    }
    for (int i = 0; i < C::kAcc; ++i) {
      ptx::mbar_init(&ctl->acc_full[i], 1);
      ptx::mbar_init(&ctl->acc_empty[i], 4 * NSUB);  // one arrival per promotion warp
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensormap(&map_w);
    ptx::prefetch_tensormap(&map_a);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  if constexpr (GROUPED) {
    // The row tables are written by kernels earlier in the stream: nothing of the work list is known before they end.
    ptx::grid_dep_wait();
    if (warp == 2) {  // exclusive prefix sum of work items per expert
      int32_t running = 0;
      for (int32_t base = 0; base < p.num_experts; base += 32) {
        const int32_t e = base + lane;
        int32_t v = 0;
        if (e < p.num_experts) {
          int32_t r0, cnt;
          expert_rows(p, e, &r0, &cnt);
          v = ((cnt + MT - 1) / MT) * p.n_tiles;
        }
        int32_t incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int32_t o = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += o;
        }
        if (e < p.num_experts) item_start[e] = running + incl - v;
        running += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) {
        item_start[p.num_experts] = running;
        ctl->total = running;
      }
    }
  } else {
    if (threadIdx.x == 0) ctl->total = p.n_tiles * p.k_splits;
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const int32_t total = ctl->total;
  const uint32_t full0 = ptx::smem_u32(&ctl->full[0]), empty0 = ptx::smem_u32(&ctl->empty[0]);
  const uint32_t acc_full0 = ptx::smem_u32(&ctl->acc_full[0]), acc_empty0 = ptx::smem_u32(&ctl->acc_empty[0]);
  const uint32_t stage0 = ptx::smem_u32(smem);

  if (threadIdx.x == 0) ptx::grid_dep_launch();  // the next kernel of the stream may begin its own set-up

  if (warp == 0) {
    // ===== TMA producer.  Pass 0 runs before griddepcontrol.wait: the weight tiles of the first k-blocks (at most one
    // ring of stages, whose barriers are fresh) are requested; pass 1 adds their activation tiles and then continues
    // with whole stages.
    uint32_t pre = 0;
    uint32_t armed = 0, armed_phase = 0;  // bit i: stage i was armed / the phase bit of its last arming
    for (int pass = GROUPED ? 1 : 0; pass < 2; ++pass) {
      uint32_t stage = 0, phase = 0, idx = 0;
      bool ok = true;
      for (int32_t t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const Item it = get_item<MT, GROUPED>(p, item_start, t);
        const int32_t nt = it.nt;
        for (int32_t kb = it.kb0; kb < it.kb1; ++kb, ++idx) {
          const uint32_t dst = stage0 + stage * C::kStageBytes;
          if (pass == 0) {
            if (idx >= (uint32_t)C::kStages) { ok = false; break; }
            if (lane == 0) {
              ptx::mbar_arrive_expect_tx_a(full0 + stage * 8, C::kStageBytes);
              ptx::tma_load_3d_a(dst, &map_w, full0 + stage * 8, kb * BK, nt * BN, 0);
            }
            armed |= 1u << stage;
            armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
            pre = idx + 1;
          } else if (idx < pre) {
            if (lane == 0) ptx::tma_load_2d_a(dst + kWBytes, &map_a, full0 + stage * 8, kb * BK, 0);
          } else {
            if (!ptx::mbar_wait_a(empty0 + stage * 8, phase ^ 1)) {
              timeout(ctl, 11);
              ok = false;
              break;
            }
            if (lane == 0) {
              ptx::mbar_arrive_expect_tx_a(full0 + stage * 8, C::kStageBytes);
              ptx::tma_load_3d_a(dst, &map_w, full0 + stage * 8, kb * BK, nt * BN, it.e);
              ptx::tma_load_2d_a(dst + kWBytes, &map_a, full0 + stage * 8, kb * BK, it.row0);
            }
            armed |= 1u << stage;
            armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (ctl->abort_flag) ok = false;
      }
      if (pass == 0) {
        ptx::grid_dep_wait();  // the activations are written by the kernel before this one
      } else if (ctl->abort_flag) {
        // bulk copies must not be in flight when the CTA exits: wait (bounded) for every stage that may still be armed
        for (int i = 0; i < C::kStages; ++i)
          if (armed & (1u << i)) ptx::mbar_wait_a(full0 + i * 8, (armed_phase >> i) & 1u, 20000000ull);
      } else {
        // the last tcgen05.commit arrivals on `empty` must have landed before the CTA's shared memory is reused
        for (int i = 0; i < C::kStages; ++i) {
          if (!ptx::mbar_wait_a(empty0 + stage * 8, phase ^ 1)) { timeout(ctl, 15); break; }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer: D[128 weight rows][MT tokens] (+)= W_tile * A_tile^T, one TMEM stage per k-block
    constexpr uint32_t idesc = ptx::make_idesc_e4m3_f32(BN, C::kTile);
    const uint64_t desc0 = ptx::make_kmajor_sw128_desc(stage0);
    uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
    for (int32_t t = blockIdx.x; t < total; t += gridDim.x) {
      int32_t kb0 = 0, kb1 = p.k_tiles;
      if constexpr (!GROUPED) {
        const int32_t split = t / p.n_tiles;
        kb0 = split * p.kb_per_split;
        kb1 = min(kb0 + p.kb_per_split, p.k_tiles);
      }
      bool ok = true;
      for (int32_t kb = kb0; kb < kb1; ++kb) {
        if (!ptx::mbar_wait_a(acc_empty0 + acc * 8, acc_phase ^ 1)) { timeout(ctl, 12); ok = false; break; }
        if (!ptx::mbar_wait_a(full0 + stage * 8, phase)) { timeout(ctl, 13); ok = false; break; }
        ptx::tc_fence_after();
        if (lane == 0) {
          const uint64_t w_desc = desc0 + (uint64_t)(stage * (C::kStageBytes >> 4));
          const uint64_t a_desc = w_desc + (kWBytes >> 4);
          const uint32_t d_tmem = tmem_base + acc * C::kTile;
          ptx::mma_f8f6f4(d_tmem, w_desc, a_desc, idesc, 0);
#pragma unroll
          for (uint32_t k = 1; k < BK / 32; ++k) ptx::mma_f8f6f4(d_tmem, w_desc + 2 * k, a_desc + 2 * k, idesc, 1);
          ptx::mma_commit_a(empty0 + stage * 8);
          ptx::mma_commit_a(acc_full0 + acc * 8);
        }
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        if (++acc == C::kAcc) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok || ctl->abort_flag) break;
    }
  } else {
    // ===== promotion + transposed store; TMEM lane quarter = warp % 4 (warps 2, 3, 4, 5 -> quarters 2, 3, 0, 1)
    if constexpr (!GROUPED)
      ptx::grid_dep_wait();  // the activation scales come from the kernel before this one, and it may still read `out` / `partial`
    const int q = warp & 3;
    const int sub = NSUB == 1 ? 0 : (warp - 2) >> 2;  // which sub-tile of the item this warp promotes
    constexpr int kPerLane = MT / 32 > 0 ? MT / 32 : 1;  // tokens whose activation scale this lane fetches
    uint32_t acc_stage = 0, acc_phase = 0;
    float acc[MT];
    for (int32_t t = blockIdx.x; t < total; t += gridDim.x) {
      const Item it = get_item<MT, GROUPED>(p, item_start, t);
      const int32_t split = it.split, nt = it.nt, kb0 = it.kb0, kb1 = it.kb1;
      const int32_t n = nt * BN + q * 32 + lane;
      const float* sb_blk = p.sb + (int64_t)nt * p.sb_stride_n;
      const int32_t row0 = it.row0 + sub * MT, rows = max(0, min(MT, it.rows - sub * MT));
      const float* sa_base = p.sa + (int64_t)row0 * p.sa_stride_m;
      if constexpr (GROUPED) {
        sb_blk += (int64_t)it.e * p.sb_stride_e;
        if (p.rows_per_expert > 0)
          sa_base = p.sa + (int64_t)it.e * p.sa_stride_e + (int64_t)(row0 - it.e * p.rows_per_expert) * p.sa_stride_m;
      }
#pragma unroll
      for (int j = 0; j < MT; ++j) acc[j] = 0.f;
      // lane l holds the scale of token l (and l + 32); tokens past M get 0 (their products are 0 anyway)
      const float* sa_tok[kPerLane];
      bool tok_ok[kPerLane];
#pragma unroll
      for (int h = 0; h < kPerLane; ++h) {
        const int32_t tok = lane + 32 * h;
        tok_ok[h] = tok < rows && tok < MT;
        sa_tok[h] = sa_base + (int64_t)(tok_ok[h] ? tok : 0) * p.sa_stride_m;
      }
      float sa_ring[kScaleAhead][kPerLane], sb_ring[kScaleAhead];
#pragma unroll
      for (int u = 0; u < kScaleAhead; ++u) {
        const int32_t kc = min(kb0 + u, kb1 - 1);
#pragma unroll
        for (int h = 0; h < kPerLane; ++h) sa_ring[u][h] = tok_ok[h] ? load_scale<UE>(sa_tok[h], kc, p.sa_stride_k) : 0.f;
        sb_ring[u] = load_scale<UE>(sb_blk, kc, p.sb_stride_k);
      }
      bool ok = true;
      for (int32_t kbb = kb0; kbb < kb1 && ok; kbb += kScaleAhead) {
#pragma unroll
        for (int u = 0; u < kScaleAhead; ++u) {
          const int32_t kb = kbb + u;
          if (kb >= kb1) break;
          float s[kPerLane];
#pragma unroll
          for (int h = 0; h < kPerLane; ++h) s[h] = sa_ring[u][h] * sb_ring[u];
          {
            const int32_t kn = min(kb + kScaleAhead, kb1 - 1);
#pragma unroll
            for (int h = 0; h < kPerLane; ++h)
              sa_ring[u][h] = tok_ok[h] ? load_scale<UE>(sa_tok[h], kn, p.sa_stride_k) : 0.f;
            sb_ring[u] = load_scale<UE>(sb_blk, kn, p.sb_stride_k);
          }
          if (!ptx::mbar_wait_a(acc_full0 + acc_stage * 8, acc_phase)) {
            timeout(ctl, 14);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc_stage * C::kTile + sub * MT;
          uint32_t v[MT];
          if constexpr (MT == 64) {
            tmem_ld_cols<32>(taddr, v);
            tmem_ld_cols<32>(taddr + 32, v + 32);
          } else {
            tmem_ld_cols<MT>(taddr, v);
          }
          tmem_ld_fence<MT>(v);
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive_a(acc_empty0 + acc_stage * 8);
#pragma unroll
          for (int j = 0; j < MT; ++j) {
            const float sj = __shfl_sync(0xffffffffu, s[j / 32], j & 31);
            acc[j] = fmaf(__uint_as_float(v[j]), sj, acc[j]);
          }
          if (++acc_stage == C::kAcc) { acc_stage = 0; acc_phase ^= 1; }
        }
      }
      if (!ok || ctl->abort_flag) break;
      // transposed store: for every token the warp writes 32 consecutive outputs
      if (n < p.N) {
        if (p.partial != nullptr) {
          float* dst = p.partial + ((int64_t)split * p.M + row0) * p.N + n;
#pragma unroll
          for (int j = 0; j < MT; ++j)
            if (j < rows) dst[(int64_t)j * p.N] = acc[j];
        } else if (p.out_dtype == SGLB200_BF16) {
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + (int64_t)row0 * p.ldc + n;
#pragma unroll
          for (int j = 0; j < MT; ++j)
            if (j < rows) dst[(int64_t)j * p.ldc] = __float2bfloat16_rn(acc[j]);
        } else {
          __half* dst = static_cast<__half*>(p.out) + (int64_t)row0 * p.ldc + n;
#pragma unroll
          for (int j = 0; j < MT; ++j)
            if (j < rows) dst[(int64_t)j * p.ldc] = __float2half_rn(acc[j]);
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int MT, bool UE, bool GROUPED, int NSUB = 1>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_a, const SmallParams& p, int sm_count, cudaStream_t st,
           int64_t max_items) {
  constexpr size_t smem = GROUPED ? Cfg<MT, NSUB>::kSmemGrouped : Cfg<MT, NSUB>::kSmem;
  constexpr int kThreads = Cfg<MT, NSUB>::kThreads;
  static bool done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fp8_block_gemm_smallm_kernel<MT, UE, GROUPED, NSUB>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(SGLB200_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    done[dev] = true;
  }
  const int grid = (int)(max_items < sm_count ? max_items : sm_count);
  const cudaError_t le = launch_pdl(fp8_block_gemm_smallm_kernel<MT, UE, GROUPED, NSUB>, dim3(grid), dim3(kThreads), smem, st,
                                    map_w, map_a, p);
  if (le != cudaSuccess) {
    cudaGetLastError();
    return fail(SGLB200_ERR_LAUNCH, "fp8_block_gemm_smallm_kernel: %s", cudaGetErrorString(le));
  }
  return SGLB200_OK;
}

}  // namespace

int smallm_max_rows() { return 128; }

// K-splits for a small-M problem.  Cost model in units of one k-block of one work item: a split count s gives
// ceil(n_tiles * s / SMs) waves of work items, each ceil(k_tiles / s) k-blocks deep plus a fixed cost per item (pipeline
// fill, store), plus the second kernel that adds the partial sums when s > 1.  The cheapest s wins; ties go to fewer splits.
int smallm_splits(int64_t N, int64_t K, int sm_count) {
  const int64_t n_tiles = (N + BN - 1) / BN, k_tiles = (K + BK - 1) / BK;
  constexpr int64_t kItemCost = 3, kReduceCost = 8;
  int best = 1;
  int64_t best_cost = ((n_tiles + sm_count - 1) / sm_count) * (k_tiles + kItemCost);
  for (int64_t s = 2; s <= 32 && s * 2 <= k_tiles; ++s) {
    const int64_t kb = (k_tiles + s - 1) / s;
    const int64_t used = (k_tiles + kb - 1) / kb;  // splits that actually get k-blocks
    if (used != s) continue;
    const int64_t cost = ((n_tiles * s + sm_count - 1) / sm_count) * (kb + kItemCost) + kReduceCost;
    if (cost < best_cost) {
      best_cost = cost;
      best = (int)s;
    }
  }
  return best;
}

// Launches the small-M kernel (arguments already validated by the caller).  With `partial` != NULL and splits > 1 the
// kernel leaves fp32 partial sums [splits][M][N] there and the caller adds them up; *splits_used reports which.  With
// always_partial the fp32 sums go to `partial` even for a single split (the caller converts and moves them itself).
// With ue8m0 the scale pointers are packed exponent words (sa: word (m, kg) at m * sa_stride_m + kg * sa_stride_k; sb
// likewise per 128 weight rows) and the scales are the exact powers of two they encode.
int smallm_gemm(const void* a, const void* b, const float* sa, const float* sb, void* out, int64_t M, int64_t N, int64_t K,
                int64_t lda, int64_t ldb, int64_t ldc, int64_t sa_stride_m, int64_t sa_stride_k, int64_t sb_stride_n,
                int64_t sb_stride_k, int out_dtype, float* partial, int64_t partial_floats, int sm_count, void* stream,
                int* splits_used, bool always_partial, bool ue8m0) {
  const int MT = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  const bool two = M > 64;  // 128 activation rows per work item, two sets of promotion warps
  alignas(64) CUtensorMap map_w, map_a;
  {
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, 1};
    const uint64_t str[2] = {(uint64_t)ldb, (uint64_t)ldb * (uint64_t)N};
    if (int rc = make_map_sw128(&map_w, b, 3, dims, str, BN, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t str[1] = {(uint64_t)lda};
    if (int rc = make_map_sw128(&map_a, a, 2, dims, str, (uint32_t)(M > 64 ? 128 : MT), CU_TENSOR_MAP_L2_PROMOTION_L2_128B))
      return rc;
  }
  SmallParams p;
  p.sa = sa;
  p.sb = sb;
  p.out = out;
  p.M = (int32_t)M;
  p.N = (int32_t)N;
  p.K = (int32_t)K;
  p.n_tiles = (int32_t)((N + BN - 1) / BN);
  p.k_tiles = (int32_t)((K + BK - 1) / BK);
  p.ldc = ldc;
  p.sa_stride_m = sa_stride_m;
  p.sa_stride_k = sa_stride_k;
  p.sb_stride_n = sb_stride_n;
  p.sb_stride_k = sb_stride_k;
  p.out_dtype = out_dtype;
  p.partial = nullptr;
  p.k_splits = 1;
  p.kb_per_split = p.k_tiles;
  p.expert_offsets = nullptr;
  p.problem_sizes = nullptr;
  p.count_stride = 1;
  p.rows_per_expert = 0;
  p.num_experts = 1;
  p.sa_stride_e = 0;
  p.sb_stride_e = 0;
  const int splits = smallm_splits(N, K, sm_count);
  if (partial != nullptr && splits > 1 && (int64_t)splits * M * N <= partial_floats) {
    p.partial = partial;
    p.kb_per_split = (p.k_tiles + splits - 1) / splits;
    p.k_splits = (p.k_tiles + p.kb_per_split - 1) / p.kb_per_split;
  } else if (always_partial) {
    p.partial = partial;  // one slice of fp32 sums instead of `out` (the caller checked its size)
  }
  *splits_used = p.k_splits;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t items = (int64_t)p.n_tiles * p.k_splits;
  if (two) {
    return ue8m0 ? launch<64, true, false, 2>(map_w, map_a, p, sm_count, st, items)
                 : launch<64, false, false, 2>(map_w, map_a, p, sm_count, st, items);
  }
  if (ue8m0) {
    switch (MT) {
      case 16: return launch<16, true, false>(map_w, map_a, p, sm_count, st, items);
      case 32: return launch<32, true, false>(map_w, map_a, p, sm_count, st, items);
      default: return launch<64, true, false>(map_w, map_a, p, sm_count, st, items);
    }
  }
  switch (MT) {
    case 16: return launch<16, false, false>(map_w, map_a, p, sm_count, st, items);
    case 32: return launch<32, false, false>(map_w, map_a, p, sm_count, st, items);
    default: return launch<64, false, false>(map_w, map_a, p, sm_count, st, items);
  }
}

// Rows per chunk of the grouped few-rows kernel for `total_rows` rows spread over `num_experts` experts (or
// rows_per_expert rows at most per expert in the masked layout); 0 = the 128 x 128 grouped kernel is the better choice.
int smallm_grouped_chunk(int64_t total_rows, int64_t num_experts, int64_t rows_per_expert) {
  const int64_t avg = rows_per_expert > 0 ? rows_per_expert : (total_rows + num_experts - 1) / num_experts;
  if (avg > g_grouped_few_rows_max) return 0;
  if (rows_per_expert > 0) return avg <= 16 ? 16 : (avg <= 32 ? 32 : 64);  // masked layout: the row bound is known
  return avg <= 8 ? 16 : (avg <= 24 ? 32 : 64);
}

// Grouped few-rows GEMM (arguments already validated by the caller): chunk = smallm_grouped_chunk(...) != 0.
int smallm_grouped_gemm(int chunk, const void* a, const void* b, const float* sa, const float* sb, void* out,
                        const int32_t* expert_offsets, const int32_t* problem_sizes, int count_stride, int64_t total_rows,
                        int64_t num_experts, int64_t rows_per_expert, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                        int64_t ldb_e, int64_t ldc, int64_t sa_stride_e, int64_t sa_stride_m, int64_t sa_stride_k,
                        int64_t sb_stride_e, int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype, int sm_count,
                        void* stream, bool ue8m0) {
  if (num_experts > kMaxExperts) return fail(SGLB200_ERR_SHAPE, "num_experts=%lld: at most %d", (long long)num_experts, kMaxExperts);
  alignas(64) CUtensorMap map_w, map_a;
  {
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)num_experts};
    const uint64_t str[2] = {(uint64_t)ldb, (uint64_t)ldb_e};
    if (int rc = make_map_sw128(&map_w, b, 3, dims, str, BN, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)total_rows};
    const uint64_t str[1] = {(uint64_t)lda};
    if (int rc = make_map_sw128(&map_a, a, 2, dims, str, (uint32_t)chunk, CU_TENSOR_MAP_L2_PROMOTION_L2_128B)) return rc;
  }
  SmallParams p;
  p.sa = sa;
  p.sb = sb;
  p.out = out;
  p.partial = nullptr;
  p.M = (int32_t)total_rows;
  p.N = (int32_t)N;
  p.K = (int32_t)K;
  p.n_tiles = (int32_t)((N + BN - 1) / BN);
  p.k_tiles = (int32_t)((K + BK - 1) / BK);
  p.k_splits = 1;
  p.kb_per_split = p.k_tiles;
  p.ldc = ldc;
  p.sa_stride_m = sa_stride_m;
  p.sa_stride_k = sa_stride_k;
  p.sb_stride_n = sb_stride_n;
  p.sb_stride_k = sb_stride_k;
  p.out_dtype = out_dtype;
  p.expert_offsets = expert_offsets;
  p.problem_sizes = problem_sizes;
  p.count_stride = count_stride;
  p.rows_per_expert = (int32_t)rows_per_expert;
  p.num_experts = (int32_t)num_experts;
  p.sa_stride_e = sa_stride_e;
  p.sb_stride_e = sb_stride_e;
  // an upper bound on the work items without reading the device: every expert can add one ragged chunk
  const int64_t items = ((total_rows + chunk - 1) / chunk + num_experts) * p.n_tiles;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ue8m0) {
    switch (chunk) {
      case 16: return launch<16, true, true>(map_w, map_a, p, sm_count, st, items);
      case 32: return launch<32, true, true>(map_w, map_a, p, sm_count, st, items);
      default: return launch<64, true, true>(map_w, map_a, p, sm_count, st, items);
    }
  }
  switch (chunk) {
    case 16: return launch<16, false, true>(map_w, map_a, p, sm_count, st, items);
    case 32: return launch<32, false, true>(map_w, map_a, p, sm_count, st, items);
    default: return launch<64, false, true>(map_w, map_a, p, sm_count, st, items);
  }
}

}  // namespace sglb
