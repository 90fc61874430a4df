// Releasable device ranges: one contiguous virtual address range whose physical backing is committed and released in
// granules while the addresses stay valid.  A KV pool sized for the worst case can hand memory back when the load is low,
// a weight-staging area can be dropped after the resident image is built, and a tensor view over the range never moves.
//
//   create(bytes)            reserve the virtual range (rounded up to the allocation granularity), nothing committed
//   commit(offset, bytes)    back [offset, offset + bytes) with physical memory (granule aligned; already committed
//                            granules are left alone), read / write access for the owning device
//   release(offset, bytes)   unmap and free the granules fully inside the span; touching them afterwards is an error
//   committed()              bytes currently backed
//
// Driver entry points are resolved at run time (no link-time dependency on libcuda).
// (reference counterpart: src/loaders/releasable_range.cpp.)
#include <cuda.h>
#include <string.h>

#include <vector>

#include "common/common.h"

namespace {

struct Drv {
  CUresult (*getGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*addressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*setAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  bool ok = false;
};

template <typename F>
static bool resolve(const char* name, F* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || !p) return false;
  *out = reinterpret_cast<F>(p);
  return true;
}

static const Drv& drv() {
  static Drv d;
  static bool tried = false;
  if (!tried) {
    tried = true;
    d.ok = resolve("cuMemGetAllocationGranularity", &d.getGranularity) && resolve("cuMemAddressReserve", &d.addressReserve) &&
           resolve("cuMemAddressFree", &d.addressFree) && resolve("cuMemCreate", &d.create) && resolve("cuMemRelease", &d.release) &&
           resolve("cuMemMap", &d.map) && resolve("cuMemUnmap", &d.unmap) && resolve("cuMemSetAccess", &d.setAccess);
  }
  return d;
}

struct VmmRange {
  CUdeviceptr base = 0;
  size_t bytes = 0, granule = 0;
  int device = 0;
  std::vector<CUmemGenericAllocationHandle> handles;   // one per granule, 0 = not committed
  std::vector<bool> mapped;
};

}  // namespace

DGPP_API void* dgpp_vmm_create(int64_t bytes) {
  const Drv& d = drv();
  if (!d.ok || bytes <= 0) {
    dgpp_set_error("vmm_create: virtual memory management entry points unavailable or bad size");
    return nullptr;
  }
  VmmRange* r = new VmmRange();
  cudaFree(nullptr);                                    // make sure the primary context exists
  if (cudaGetDevice(&r->device) != cudaSuccess) { delete r; return nullptr; }
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = r->device;
  if (d.getGranularity(&r->granule, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || r->granule == 0) {
    dgpp_set_error("vmm_create: cuMemGetAllocationGranularity failed");
    delete r;
    return nullptr;
  }
  r->bytes = (static_cast<size_t>(bytes) + r->granule - 1) / r->granule * r->granule;
  if (d.addressReserve(&r->base, r->bytes, r->granule, 0, 0) != CUDA_SUCCESS) {
    dgpp_set_error("vmm_create: cuMemAddressReserve of %zu bytes failed", r->bytes);
    delete r;
    return nullptr;
  }
  r->handles.assign(r->bytes / r->granule, 0);
  r->mapped.assign(r->bytes / r->granule, false);
  return r;
}

DGPP_API int64_t dgpp_vmm_ptr(void* h) { return h ? static_cast<int64_t>(static_cast<VmmRange*>(h)->base) : 0; }
DGPP_API int64_t dgpp_vmm_size(void* h) { return h ? static_cast<int64_t>(static_cast<VmmRange*>(h)->bytes) : 0; }
DGPP_API int64_t dgpp_vmm_granule(void* h) { return h ? static_cast<int64_t>(static_cast<VmmRange*>(h)->granule) : 0; }

DGPP_API int64_t dgpp_vmm_committed(void* h) {
  VmmRange* r = static_cast<VmmRange*>(h);
  if (!r) return 0;
  int64_t n = 0;
  for (bool m : r->mapped) n += m ? static_cast<int64_t>(r->granule) : 0;
  return n;
}

// Back every granule that overlaps [offset, offset + bytes).
DGPP_API int dgpp_vmm_commit(void* h, int64_t offset, int64_t bytes) {
  VmmRange* r = static_cast<VmmRange*>(h);
  const Drv& d = drv();
  DGPP_REQUIRE(r && offset >= 0 && bytes >= 0 && static_cast<size_t>(offset + bytes) <= r->bytes, "vmm_commit: span outside the range");
  if (bytes == 0) return 0;
  const size_t g0 = static_cast<size_t>(offset) / r->granule, g1 = (static_cast<size_t>(offset + bytes) + r->granule - 1) / r->granule;
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = r->device;
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location = prop.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (size_t g = g0; g < g1; ++g) {
    if (r->mapped[g]) continue;
    CUmemGenericAllocationHandle hnd = 0;
    DGPP_REQUIRE(d.create(&hnd, r->granule, &prop, 0) == CUDA_SUCCESS, "vmm_commit: out of device memory at granule %zu", g);
    const CUdeviceptr at = r->base + g * r->granule;
    if (d.map(at, r->granule, 0, hnd, 0) != CUDA_SUCCESS || d.setAccess(at, r->granule, &acc, 1) != CUDA_SUCCESS) {
      d.release(hnd);
      dgpp_set_error("vmm_commit: cuMemMap / cuMemSetAccess failed at granule %zu", g);
      return -1;
    }
    r->handles[g] = hnd;
    r->mapped[g] = true;
  }
  return 0;
}

// Free every granule that lies fully inside [offset, offset + bytes) (the device must not be using them).
DGPP_API int dgpp_vmm_release(void* h, int64_t offset, int64_t bytes) {
  VmmRange* r = static_cast<VmmRange*>(h);
  const Drv& d = drv();
  DGPP_REQUIRE(r && offset >= 0 && bytes >= 0 && static_cast<size_t>(offset + bytes) <= r->bytes, "vmm_release: span outside the range");
  const size_t g0 = (static_cast<size_t>(offset) + r->granule - 1) / r->granule, g1 = static_cast<size_t>(offset + bytes) / r->granule;
  DGPP_CUDA_OK(cudaDeviceSynchronize());
  for (size_t g = g0; g < g1; ++g) {
    if (!r->mapped[g]) continue;
    d.unmap(r->base + g * r->granule, r->granule);
    d.release(r->handles[g]);
    r->handles[g] = 0;
    r->mapped[g] = false;
  }
  return 0;
}

DGPP_API int dgpp_vmm_destroy(void* h) {
  VmmRange* r = static_cast<VmmRange*>(h);
  if (!r) return 0;
  dgpp_vmm_release(r, 0, static_cast<int64_t>(r->bytes));
  drv().addressFree(r->base, r->bytes);
  delete r;
  return 0;
}
