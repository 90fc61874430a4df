// Error text for the C ABI and the per-device status block that bounded device waits report into.
#include <stdarg.h>
#include <string.h>

#include "common/common.h"

static thread_local char g_err[1024];

DGPP_API const char* dgpp_last_error() { return g_err; }

void dgpp_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

namespace dgpp {

__device__ DeviceStatus g_device_status;

DeviceStatus* device_status_ptr() {
  static DeviceStatus* cache[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<DeviceStatus*>(p);
  }
  return cache[dev];
}

}  // namespace dgpp

// Reads the status block of the current device (synchronises the device). out[0..3] = code, count, detail, pad.
DGPP_API int dgpp_status_read(int* out) {
  dgpp::DeviceStatus* p = dgpp::device_status_ptr();
  DGPP_REQUIRE(p != nullptr, "no status block for the current device");
  DGPP_CUDA_OK(cudaMemcpy(out, p, sizeof(dgpp::DeviceStatus), cudaMemcpyDeviceToHost));
  return 0;
}

DGPP_API int dgpp_status_clear() {
  dgpp::DeviceStatus* p = dgpp::device_status_ptr();
  DGPP_REQUIRE(p != nullptr, "no status block for the current device");
  DGPP_CUDA_OK(cudaMemset(p, 0, sizeof(dgpp::DeviceStatus)));
  return 0;
}

DGPP_API void* dgpp_status_device_ptr() { return dgpp::device_status_ptr(); }
