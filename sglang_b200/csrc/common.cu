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

static int g_num_sms_limit = 0;  // 0: no limit
int g_grouped_few_rows_max = 20;  // grouped GEMMs with at most this many rows per expert on average take the few-rows kernel

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
  if (g_num_sms_limit > 0 && g_num_sms_limit < out->sm_count) out->sm_count = g_num_sms_limit;
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

const char* sglb200_version(void) { return "0.2"; }

int sglb200_set_num_sms(int num_sms) {
  if (num_sms < 0) return sglb::fail(SGLB200_ERR_SHAPE, "num_sms=%d must be >= 0 (0 = every SM)", num_sms);
  sglb::g_num_sms_limit = num_sms;
  return SGLB200_OK;
}

int sglb200_set_grouped_few_rows(int max_avg_rows) {
  if (max_avg_rows < 0 || max_avg_rows > 64)
    return sglb::fail(SGLB200_ERR_SHAPE, "max_avg_rows=%d: 0 (never) .. 64", max_avg_rows);
  sglb::g_grouped_few_rows_max = max_avg_rows;
  return SGLB200_OK;
}

int sglb200_get_grouped_few_rows(void) { return sglb::g_grouped_few_rows_max; }

int sglb200_get_num_sms(void) {
  sglb::DeviceInfo di;
  const int limit = sglb::g_num_sms_limit;
  sglb::g_num_sms_limit = 0;
  const int rc = sglb::device_info(&di);
  sglb::g_num_sms_limit = limit;
  if (rc != SGLB200_OK) return limit;
  return limit > 0 && limit < di.sm_count ? limit : di.sm_count;
}

}  // extern "C"
