// Helpers shared by the tensor-core GEMM kernels: status reporting, bounded mbarrier waits and
// host-side TMA descriptor construction (driver entry point resolved at run time, so the library
// has no link-time dependency on libcuda).
#pragma once
#include <cuda.h>

#include "common/common.h"
#include "common/ptx.cuh"

namespace dgpp {

__device__ __forceinline__ void report(DeviceStatus* st, int code, int detail) {
  if (atomicCAS(&st->code, 0, code) == 0) st->detail = detail;
  atomicAdd(&st->count, 1);
}

// Bounded mbarrier wait with a wall-clock limit (~2 s); false on expiry.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity) {
  // fast path: no timer reads while the barrier completes within a few thousand polls
  for (int i = 0; i < 4096; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  // slow path: bound the wait by the SM cycle counter (about 2 s at 2 GHz)
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 2048; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > 4000000000ll) return false;
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && p)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] of `esize`-byte elements with row pitch `pitch` bytes.
static inline int make_tmap_2d(CUtensorMap* m, const void* base, CUtensorMapDataType dt, int esize, uint64_t cols, uint64_t rows,
                 uint64_t pitch, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_fn();
  DGPP_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled is unavailable (no CUDA driver?)");
  DGPP_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base %p is not 16-byte aligned", base);
  DGPP_REQUIRE(pitch % 16 == 0, "TMA row pitch %llu is not a multiple of 16", (unsigned long long)pitch);
  DGPP_REQUIRE((static_cast<uint64_t>(box_cols) * esize) % 16 == 0, "TMA box inner extent is not a multiple of 16 bytes");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DGPP_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

// 3-D tensor [slabs, rows, cols]: rows with pitch `pitch` bytes, slabs `slab_pitch` bytes apart; boxes are 2-D (one slab).
static inline int make_tmap_3d(CUtensorMap* m, const void* base, CUtensorMapDataType dt, int esize, uint64_t cols, uint64_t rows,
                 uint64_t slabs, uint64_t pitch, uint64_t slab_pitch, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_fn();
  DGPP_REQUIRE(fn != nullptr, "cuTensorMapEncodeTiled is unavailable (no CUDA driver?)");
  DGPP_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base %p is not 16-byte aligned", base);
  DGPP_REQUIRE(pitch % 16 == 0 && slab_pitch % 16 == 0, "TMA pitches must be multiples of 16 bytes");
  DGPP_REQUIRE((static_cast<uint64_t>(box_cols) * esize) % 16 == 0, "TMA box inner extent is not a multiple of 16 bytes");
  cuuint64_t dims[3] = {cols, rows, slabs};
  cuuint64_t strides[2] = {pitch, slab_pitch};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DGPP_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (3-D) failed with %d", (int)r);
  return 0;
}

}  // namespace dgpp
