#include "common.cuh"

#include <string.h>

namespace sglb {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int device_info(DeviceInfo* out) {
  static DeviceInfo cache[64];
  static bool have[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return fail(SGLB200_ERR_LAUNCH, "cudaGetDevice failed (no CUDA device?)");
  }
  if (!have[dev]) {
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) {
      cudaGetLastError();
      return fail(SGLB200_ERR_LAUNCH, "cudaGetDeviceProperties failed");
    }
    cache[dev].sm_count = p.multiProcessorCount;
    cache[dev].cc_major = p.major;
    cache[dev].cc_minor = p.minor;
    cache[dev].max_smem_optin = (int)p.sharedMemPerBlockOptin;
    have[dev] = true;
  }
  *out = cache[dev];
  return SGLB200_OK;
}

}  // namespace sglb

extern "C" {

const char* sglb200_status_string(int status) {
  switch (status) {
    case SGLB200_OK: return "ok";
    case SGLB200_ERR_SHAPE: return "bad shape or stride";
    case SGLB200_ERR_ALIGN: return "bad alignment";
    case SGLB200_ERR_ARCH: return "device is not sm_100 (B200)";
    case SGLB200_ERR_LAUNCH: return "CUDA launch or set-up failure";
    case SGLB200_ERR_DTYPE: return "unsupported dtype";
    case SGLB200_ERR_NULL: return "null pointer";
    case SGLB200_ERR_WORKSPACE: return "scratch buffer too small";
    default: return "unknown status";
  }
}

const char* sglb200_last_error_detail(void) { return sglb::error_buffer(); }

const char* sglb200_version(void) { return "0.1"; }

}  // extern "C"
