// Shared host/device plumbing: status codes, argument checks, launch error capture.
#pragma once
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
