// Growable device buffers on CUDA virtual memory management: reserve address space once, back it on demand.
//
// A serving process does not know at start-up how much KV cache or workspace each model will need, and a buffer
// that is reallocated to grow changes its address -- fatal for captured CUDA graphs, cached TMA descriptors and
// peers that mapped it.  The fix is the one the reference's CudaVmmAllocator uses
// (crates/onnx-runtime-cuda-memory/src/vmm_allocator.rs, virtual_memory.rs: cuMemAddressReserve + cuMemCreate +
// cuMemMap in 2 MiB granules): reserve the largest address range the buffer may ever need, map physical chunks
// behind its front as it grows, unmap from the back as it shrinks.  The base pointer never changes.
//
// Plain C ABI, host code only.  Driver entry points are resolved through the runtime (cudaGetDriverEntryPoint), so
// the library carries no link-time dependency on libcuda.  Every call returns 0 or a CUresult / negative argument
// error; nothing here can fault the device: the driver validates each range.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <vector>

namespace {

struct Driver {
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  bool ok = false;
};

template <class F>
bool resolve(const char* name, F* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult st;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &st) != cudaSuccess || st != cudaDriverEntryPointSuccess || !fn) return false;
  *out = reinterpret_cast<F>(fn);
  return true;
}

const Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.ok = resolve("cuMemGetAllocationGranularity", &d.MemGetAllocationGranularity) &&
           resolve("cuMemAddressReserve", &d.MemAddressReserve) && resolve("cuMemAddressFree", &d.MemAddressFree) &&
           resolve("cuMemCreate", &d.MemCreate) && resolve("cuMemRelease", &d.MemRelease) && resolve("cuMemMap", &d.MemMap) &&
           resolve("cuMemUnmap", &d.MemUnmap) && resolve("cuMemSetAccess", &d.MemSetAccess) &&
           resolve("cuDeviceGetAttribute", &d.DeviceGetAttribute);
  });
  return d;
}

struct Chunk {
  CUmemGenericAllocationHandle handle;
  size_t offset, size;
};

struct Pool {
  int device = 0;
  CUdeviceptr base = 0;
  size_t reserved = 0, mapped = 0, granularity = 0;
  std::vector<Chunk> chunks;
  std::mutex mu;
};

CUmemAllocationProp device_prop(int device) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  return prop;
}

size_t round_up(size_t v, size_t g) { return (v + g - 1) / g * g; }

}  // namespace

// 1 when the device supports virtual memory management and the driver entry points resolve.
extern "C" int ogb_vmm_available(int device) {
  if (cudaSetDevice(device) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) return 0;   // make the primary context current
  const Driver& d = driver();
  if (!d.ok) return 0;
  int supported = 0;
  if (d.DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, device) != CUDA_SUCCESS) return 0;
  return supported ? 1 : 0;
}

// Reserve `reserve_bytes` (rounded up to the allocation granularity) of device address space.  Nothing is backed yet.
extern "C" int ogb_vmm_create(int device, uint64_t reserve_bytes, void** out_pool) {
  if (!out_pool || reserve_bytes == 0) return -1;
  *out_pool = nullptr;
  if (!ogb_vmm_available(device)) return -2;
  const Driver& d = driver();
  const CUmemAllocationProp prop = device_prop(device);
  size_t gran = 0;
  CUresult rc = d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (rc != CUDA_SUCCESS) return static_cast<int>(rc);
  if (gran == 0) return -3;
  Pool* p = new Pool();
  p->device = device;
  p->granularity = gran;
  p->reserved = round_up(static_cast<size_t>(reserve_bytes), gran);
  rc = d.MemAddressReserve(&p->base, p->reserved, gran, 0, 0);
  if (rc != CUDA_SUCCESS) {
    delete p;
    return static_cast<int>(rc);
  }
  *out_pool = p;
  return 0;
}

// Make at least `want_bytes` from the front of the range usable.  Grows by one physical chunk per call (the difference,
// rounded up to the granularity); never moves the base.  A failure leaves the pool as it was.
extern "C" int ogb_vmm_grow(void* pool, uint64_t want_bytes) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p) return -1;
  std::lock_guard<std::mutex> lock(p->mu);
  const size_t want = round_up(static_cast<size_t>(want_bytes), p->granularity);
  if (want <= p->mapped) return 0;
  if (want > p->reserved) return -4;
  if (cudaSetDevice(p->device) != cudaSuccess) return -2;
  const Driver& d = driver();
  const CUmemAllocationProp prop = device_prop(p->device);
  Chunk c{0, p->mapped, want - p->mapped};
  CUresult rc = d.MemCreate(&c.handle, c.size, &prop, 0);
  if (rc != CUDA_SUCCESS) return static_cast<int>(rc);              // typically CUDA_ERROR_OUT_OF_MEMORY (2)
  rc = d.MemMap(p->base + c.offset, c.size, 0, c.handle, 0);
  if (rc != CUDA_SUCCESS) {
    d.MemRelease(c.handle);
    return static_cast<int>(rc);
  }
  CUmemAccessDesc access = {};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = p->device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  rc = d.MemSetAccess(p->base + c.offset, c.size, &access, 1);
  if (rc != CUDA_SUCCESS) {
    d.MemUnmap(p->base + c.offset, c.size);
    d.MemRelease(c.handle);
    return static_cast<int>(rc);
  }
  p->chunks.push_back(c);
  p->mapped = want;
  return 0;
}

// Give back physical memory from the end: whole chunks that lie entirely beyond `keep_bytes` are unmapped and released.
// The caller guarantees that no kernel still uses that part (synchronise first).
extern "C" int ogb_vmm_shrink(void* pool, uint64_t keep_bytes) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p) return -1;
  std::lock_guard<std::mutex> lock(p->mu);
  const Driver& d = driver();
  if (cudaSetDevice(p->device) != cudaSuccess) return -2;
  while (!p->chunks.empty() && p->chunks.back().offset >= keep_bytes) {
    const Chunk c = p->chunks.back();
    CUresult rc = d.MemUnmap(p->base + c.offset, c.size);
    if (rc != CUDA_SUCCESS) return static_cast<int>(rc);
    d.MemRelease(c.handle);
    p->chunks.pop_back();
    p->mapped = c.offset;
  }
  return 0;
}

extern "C" uint64_t ogb_vmm_ptr(void* pool) { return pool ? static_cast<uint64_t>(static_cast<Pool*>(pool)->base) : 0; }
extern "C" uint64_t ogb_vmm_mapped(void* pool) { return pool ? static_cast<Pool*>(pool)->mapped : 0; }
extern "C" uint64_t ogb_vmm_reserved(void* pool) { return pool ? static_cast<Pool*>(pool)->reserved : 0; }
extern "C" uint64_t ogb_vmm_granularity(void* pool) { return pool ? static_cast<Pool*>(pool)->granularity : 0; }
extern "C" int ogb_vmm_chunks(void* pool) { return pool ? static_cast<int>(static_cast<Pool*>(pool)->chunks.size()) : 0; }

// Unmap everything and return the address range.  The caller guarantees that no kernel still uses the buffer.
extern "C" int ogb_vmm_destroy(void* pool) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p) return 0;
  int rc = ogb_vmm_shrink(p, 0);
  if (rc != 0) return rc;
  const Driver& d = driver();
  CUresult fr = d.MemAddressFree(p->base, p->reserved);
  delete p;
  return static_cast<int>(fr);
}
