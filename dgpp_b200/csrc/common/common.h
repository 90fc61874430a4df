// Shared host-side definitions for the kernel library: error handling, the device status
// block that bounded waits report into, and launch helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define DGPP_API extern "C" __attribute__((visibility("default")))

namespace dgpp {

// Status codes written by kernels that gave up on a bounded wait or saw a bad argument.
enum StatusCode : int {
  kOk = 0,
  kTimeoutTmaFull = 1,     // a consumer never saw its TMA bytes arrive
  kTimeoutStageEmpty = 2,  // a producer never got a pipeline slot back
  kTimeoutAccum = 3,       // the epilogue never saw the accumulator complete
  kTimeoutPeerFlag = 4,    // a peer rank never raised its flag
  kTimeoutConvert = 5,     // the MMA thread never saw a converted operand tile
  kBadArgument = 6,
};

// One status block per device, zero-initialised. Slot 0 holds the first non-zero code seen;
// slot 1 counts how many waits gave up; slot 2 holds an op-specific detail (e.g. tile index).
struct DeviceStatus {
  int code;
  int count;
  int detail;
  int pad;
};

}  // namespace dgpp

// Last error text for the C ABI (thread-local).
DGPP_API const char* dgpp_last_error();
void dgpp_set_error(const char* fmt, ...);

#define DGPP_CUDA_OK(expr)                                                                   \
  do {                                                                                       \
    cudaError_t _e = (expr);                                                                 \
    if (_e != cudaSuccess) {                                                                 \
      dgpp_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return -1;                                                                             \
    }                                                                                        \
  } while (0)

#define DGPP_REQUIRE(cond, ...)      \
  do {                               \
    if (!(cond)) {                   \
      dgpp_set_error(__VA_ARGS__);   \
      return -1;                     \
    }                                \
  } while (0)

// Device status block accessors (defined in status.cu).
namespace dgpp {
DeviceStatus* device_status_ptr();  // device pointer for the current device (lazily resolved)
}

static inline int dgpp_ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline int64_t dgpp_ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
