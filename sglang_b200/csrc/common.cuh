// Shared host/device plumbing: status codes, argument checks, launch error capture.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/sglb200.h"

namespace sglb {

// Thread-local text of the last failed host-side check.
char* error_buffer();
int fail(int code, const char* fmt, ...);

// Number of SMs and compute capability of the current device, cached per device.
struct DeviceInfo {
  int sm_count;
  int cc_major;
  int cc_minor;
  int max_smem_optin;
};
int device_info(DeviceInfo* out);  // returns SGLB200_OK or an error code

// Tensor map of a rank-2 or rank-3 byte tensor with innermost extent dims[0] (K), 128-byte-swizzled boxes of
// [box_rows x 128 bytes].  Defined in gemm.cu.
int make_map_sw128(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                   uint32_t box_rows, CUtensorMapL2promotion promo);

// The few-rows (M <= smallm_max_rows()) weight-streaming GEMM, gemm_smallm.cu
int smallm_max_rows();
int smallm_splits(int64_t N, int64_t K, int sm_count);
int smallm_gemm(const void* a, const void* b, const float* sa, const float* sb, void* out, int64_t M, int64_t N, int64_t K,
                int64_t lda, int64_t ldb, int64_t ldc, int64_t sa_stride_m, int64_t sa_stride_k, int64_t sb_stride_n,
                int64_t sb_stride_k, int out_dtype, float* partial, int64_t partial_floats, int sm_count, void* stream,
                int* splits_used, bool always_partial = false, bool ue8m0 = false);
void launch_splitk_reduce(const float* partial, void* out, int64_t M, int64_t N, int64_t ldc, int splits, int out_dtype,
                          int sm_count, void* stream);  // gemm.cu
int smallm_take_device_status();
int nvls_take_device_status();  // nvls.cu
extern int g_grouped_few_rows_max;  // common.cu; sglb200_set_grouped_few_rows
// The grouped form of the few-rows kernel (one weight matrix per expert, few rows per expert); chunk 0 = do not use it
int smallm_grouped_chunk(int64_t total_rows, int64_t num_experts, int64_t rows_per_expert);
int smallm_grouped_gemm(int chunk, const void* a, const void* b, const float* sa, const float* sb, void* out,
                        const int32_t* expert_offsets, const int32_t* problem_sizes, int count_stride, int64_t total_rows,
                        int64_t num_experts, int64_t rows_per_expert, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                        int64_t ldb_e, int64_t ldc, int64_t sa_stride_e, int64_t sa_stride_m, int64_t sa_stride_k,
                        int64_t sb_stride_e, int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype, int sm_count,
                        void* stream, bool ue8m0);

// Dense GEMM on CTA pairs (256 x bn tiles, bn = 128 or 256), gemm_pair.cu
int pair_gemm(int bn, const void* a, const void* b, const float* sa, const float* sb, void* out, int64_t M, int64_t N,
              int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t sa_stride_m, int64_t sa_stride_k,
              int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype, int sm_count, void* stream);

// Launch with programmatic stream serialization allowed: the kernel may begin before the previous kernel of the stream
// has finished and must call ptx::grid_dep_wait() before it touches anything that kernel writes or reads.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

#define SGLB_CHECK_LAUNCH(what)                                                                   \
  do {                                                                                            \
    cudaError_t e__ = cudaGetLastError();                                                         \
    if (e__ != cudaSuccess) return ::sglb::fail(SGLB200_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e__)); \
  } while (0)

#define SGLB_REQUIRE(cond, code, ...)                       \
  do {                                                      \
    if (!(cond)) return ::sglb::fail(code, __VA_ARGS__);    \
  } while (0)

}  // namespace sglb
