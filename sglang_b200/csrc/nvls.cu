// In-place all-reduce of a 16-bit buffer that every rank of a node maps through ONE NVLink multicast address (NVSwitch
// "NVLS"): rank r owns the r-th slice of the buffer; for every 16-byte vector of its slice it issues one
// multimem.ld_reduce (the switch reads the vector from every rank's memory, adds the values in fp32 and returns the
// rounded sum) and one multimem.st (the switch writes the sum into every rank's memory).  Each GPU therefore sends and
// receives the buffer size once over NVLink, against 2 (world - 1) / world of it twice around a ring, and the sum of the
// ranks' 16-bit partial results is rounded ONCE (a ring that adds 16-bit buffers rounds after every hop).
//
// Two cross-rank barriers bracket the work: none of a peer's data may be read before that peer's producer kernel (the
// GEMM before this kernel in its stream) has finished, and no rank may leave before every peer has written the sums of
// its slice.  Block b of a rank pairs with block b of every peer (same grid everywhere): it raises its flag word in
// every peer's flag block and waits, bounded, for the peers' words in its own.  The epoch of a block lives in device
// memory and advances with every launch, so a captured CUDA graph can be replayed.
//
// The multicast mapping, the peers' flag-block addresses and the stream order of the producers are the caller's
// business (the Python side takes them from torch's symmetric-memory allocator); this file holds only the kernel.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "nvls.cuh"
#include "ptx.cuh"

namespace sglb {

__device__ int g_nvls_status = 0;

int nvls_take_device_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_nvls_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (v != 0) {
    const int z = 0;
    cudaMemcpyToSymbol(g_nvls_status, &z, sizeof(int));
  }
  return v;
}

namespace {

using nvls::FlagPtrs;
using nvls::kBlocks;
using nvls::kCtlWords;
using nvls::kFlagWords;
using nvls::kMaxRanks;
constexpr int kThreads = 512;
constexpr int kUnroll = 8;  // 16-byte vectors in flight per thread

template <bool BF16>
__global__ void __launch_bounds__(kThreads)
nvls_all_reduce_kernel(uint64_t mc_base, const __grid_constant__ FlagPtrs fp, int rank, int world, int64_t vecs, uint64_t limit_ns) {
  __shared__ int s_ok;
  __shared__ uint32_t s_epoch;
  uint32_t* ctl = fp.p[rank] + kFlagWords + blockIdx.x;
  if (threadIdx.x == 0) {
    s_ok = 1;
    s_epoch = *reinterpret_cast<volatile uint32_t*>(ctl) + 1u;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  bool ok = nvls::rank_barrier(fp, 0, blockIdx.x, rank, world, epoch, limit_ns, &s_ok, &g_nvls_status, 41);
  if (ok) {
    // this rank's slice, in 16-byte vectors
    const int64_t per_rank = (vecs + world - 1) / world;
    const int64_t v0 = (int64_t)rank * per_rank, v1 = min(vecs, v0 + per_rank);
    nvls::reduce_range<BF16, kUnroll>(mc_base, v0, v1, blockIdx.x, gridDim.x, kThreads);
    ok = nvls::rank_barrier(fp, 1, blockIdx.x, rank, world, epoch, limit_ns, &s_ok, &g_nvls_status, 42);
  }
  // the epoch advances even after a time-out, so that the next launch does not pair with stale flags
  if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(ctl) = epoch;
  (void)ok;
}

}  // namespace
}  // namespace sglb

extern "C" int64_t sglb200_nvls_flag_bytes(void) {
  return (int64_t)(sglb::kFlagWords + sglb::kCtlWords) * (int64_t)sizeof(uint32_t);
}

extern "C" int sglb200_nvls_all_reduce(uint64_t multicast_addr, const uint64_t* flag_blocks, int rank, int world,
                                       int64_t numel, int dtype, int blocks, void* stream) {
  using namespace sglb;
  SGLB_REQUIRE(world >= 2 && world <= kMaxRanks, SGLB200_ERR_SHAPE, "world=%d: 2..%d", world, kMaxRanks);
  SGLB_REQUIRE(rank >= 0 && rank < world, SGLB200_ERR_SHAPE, "rank=%d of %d", rank, world);
  SGLB_REQUIRE(dtype == SGLB200_BF16 || dtype == SGLB200_F16, SGLB200_ERR_DTYPE, "dtype=%d: only bf16 (0) and f16 (1)", dtype);
  SGLB_REQUIRE(blocks >= 0 && blocks <= kBlocks, SGLB200_ERR_SHAPE, "blocks=%d: 0 (all %d) .. %d", blocks, kBlocks, kBlocks);
  SGLB_REQUIRE(numel >= 0 && numel % 8 == 0, SGLB200_ERR_SHAPE, "numel=%lld must be a multiple of 8 (16-byte vectors)",
               (long long)numel);
  if (numel == 0) return SGLB200_OK;
  SGLB_REQUIRE(multicast_addr != 0 && flag_blocks != nullptr, SGLB200_ERR_NULL, "multicast address / flag blocks are NULL");
  SGLB_REQUIRE(multicast_addr % 16 == 0, SGLB200_ERR_ALIGN, "the multicast address must be 16-byte aligned");
  FlagPtrs fp;
  for (int i = 0; i < kMaxRanks; ++i) {
    fp.p[i] = i < world ? reinterpret_cast<uint32_t*>(flag_blocks[i]) : nullptr;
    SGLB_REQUIRE(i >= world || (fp.p[i] != nullptr && flag_blocks[i] % 4 == 0), SGLB200_ERR_NULL,
                 "flag block of rank %d is NULL or misaligned", i);
  }
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  SGLB_REQUIRE(di.cc_major == 10, SGLB200_ERR_ARCH, "compute capability %d.%d: this library is built for sm_100a only",
               di.cc_major, di.cc_minor);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint64_t limit_ns = 2000000000ull;
  const int grid = blocks > 0 ? blocks : kBlocks;  // the same on every rank: block b pairs with block b of the peers
  if (dtype == SGLB200_BF16)
    nvls_all_reduce_kernel<true><<<grid, kThreads, 0, st>>>(multicast_addr, fp, rank, world, numel / 8, limit_ns);
  else
    nvls_all_reduce_kernel<false><<<grid, kThreads, 0, st>>>(multicast_addr, fp, rank, world, numel / 8, limit_ns);
  SGLB_CHECK_LAUNCH("nvls_all_reduce_kernel");
  return SGLB200_OK;
}
