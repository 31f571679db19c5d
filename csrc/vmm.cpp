// Pausable device memory: allocations whose virtual address stays fixed while their physical
// memory is released and later re-created (CUDA virtual memory management: cuMemAddressReserve +
// cuMemCreate + cuMemMap).  The colocated trainer and rollout engine take turns on one GPU: the
// engine's KV cache and weight buffer are paused while the trainer runs and resumed at the same
// addresses, so captured CUDA graphs and address tables that point into them stay valid.
// (The reference gets this from the torch_memory_saver LD_PRELOAD hook; here it is an explicit
// allocator, so nothing else in the process is affected.)  Contents are NOT preserved across a
// pause; a resumed region is zero-filled.
//
// Sharing between processes: every physical allocation is created exportable as a POSIX file
// descriptor (cuMemExportToShareableHandle).  Another process of the same node that receives the
// descriptor (SCM_RIGHTS over a Unix socket) maps the same physical memory into its own address
// space with vmm_import_fd and can then store into it over NVLink - the route by which trainer
// ranks write updated weights straight into the parameter buffer of a rollout rank on another GPU.
// A mapping made from a descriptor follows the physical allocation that was exported: after the
// owner pauses and resumes the region it has new physical memory and importers must import again.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <torch/extension.h>

#include <map>
#include <mutex>

namespace {

struct Region {
  CUdeviceptr va = 0;
  size_t size = 0;
  int device = 0;
  CUmemGenericAllocationHandle handle = 0;
  bool mapped = false;
};
std::map<int64_t, Region> g_regions;
std::mutex g_mu;

template <typename Fn>
Fn driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    throw std::runtime_error(std::string("CUDA driver entry point not available: ") + name);
  }
  return reinterpret_cast<Fn>(p);
}
void cu_check(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) {
    char buf[160];
    snprintf(buf, sizeof(buf), "%s failed with CUresult %d", what, (int)r);
    throw std::runtime_error(buf);
  }
}

using GranFn = CUresult (*)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
using ReserveFn = CUresult (*)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
using CreateFn = CUresult (*)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
using MapFn = CUresult (*)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
using AccessFn = CUresult (*)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
using UnmapFn = CUresult (*)(CUdeviceptr, size_t);
using ReleaseFn = CUresult (*)(CUmemGenericAllocationHandle);
using FreeFn = CUresult (*)(CUdeviceptr, size_t);

CUmemAllocationProp prop_for(int device) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

struct Imported {
  CUdeviceptr va = 0;
  size_t size = 0;
  int device = 0;
  CUmemGenericAllocationHandle handle = 0;
};
std::map<int64_t, Imported> g_imported;
using ExportFn = CUresult (*)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
using ImportFn = CUresult (*)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);

void map_physical(Region& r) {
  static auto create = driver_fn<CreateFn>("cuMemCreate");
  static auto map = driver_fn<MapFn>("cuMemMap");
  static auto access = driver_fn<AccessFn>("cuMemSetAccess");
  static auto release = driver_fn<ReleaseFn>("cuMemRelease");
  CUmemAllocationProp prop = prop_for(r.device);
  cu_check(create(&r.handle, r.size, &prop, 0), "cuMemCreate");
  CUresult m = map(r.va, r.size, 0, r.handle, 0);
  if (m != CUDA_SUCCESS) {
    release(r.handle);
    cu_check(m, "cuMemMap");
  }
  CUmemAccessDesc desc = {};
  desc.location = prop.location;
  desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  cu_check(access(r.va, r.size, &desc, 1), "cuMemSetAccess");
  r.mapped = true;
}

int64_t vmm_alloc(int64_t nbytes, int64_t device) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  cudaFree(nullptr);  // make sure the primary context exists on this thread
  static auto gran_fn = driver_fn<GranFn>("cuMemGetAllocationGranularity");
  static auto reserve = driver_fn<ReserveFn>("cuMemAddressReserve");
  static auto addr_free = driver_fn<FreeFn>("cuMemAddressFree");
  Region r;
  r.device = (int)device;
  CUmemAllocationProp prop = prop_for(r.device);
  size_t gran = 0;
  cu_check(gran_fn(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM), "cuMemGetAllocationGranularity");
  r.size = ((size_t)nbytes + gran - 1) / gran * gran;
  cu_check(reserve(&r.va, r.size, 0, 0, 0), "cuMemAddressReserve");
  try {
    map_physical(r);
  } catch (...) {
    addr_free(r.va, r.size);
    throw;
  }
  cudaMemsetAsync(reinterpret_cast<void*>(r.va), 0, r.size, at::cuda::getCurrentCUDAStream().stream());
  std::lock_guard<std::mutex> lk(g_mu);
  g_regions[(int64_t)r.va] = r;
  return (int64_t)r.va;
}

Region& find(int64_t ptr) {
  auto it = g_regions.find(ptr);
  if (it == g_regions.end()) throw std::runtime_error("not a pausable allocation");
  return it->second;
}

// Releases the physical memory.  The caller guarantees that no kernel that touches the region is in flight or
// will be launched until vmm_resume (the device is synchronised here to cover work already queued).
void vmm_pause(int64_t ptr) {
  std::lock_guard<std::mutex> lk(g_mu);
  Region& r = find(ptr);
  if (!r.mapped) return;
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)r.device);
  cudaDeviceSynchronize();
  static auto unmap = driver_fn<UnmapFn>("cuMemUnmap");
  static auto release = driver_fn<ReleaseFn>("cuMemRelease");
  cu_check(unmap(r.va, r.size), "cuMemUnmap");
  cu_check(release(r.handle), "cuMemRelease");
  r.mapped = false;
}

void vmm_resume(int64_t ptr) {
  std::lock_guard<std::mutex> lk(g_mu);
  Region& r = find(ptr);
  if (r.mapped) return;
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)r.device);
  map_physical(r);
  cudaMemsetAsync(reinterpret_cast<void*>(r.va), 0, r.size, at::cuda::getCurrentCUDAStream().stream());
}

void vmm_free(int64_t ptr) {
  std::lock_guard<std::mutex> lk(g_mu);
  Region& r = find(ptr);
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)r.device);
  cudaDeviceSynchronize();
  static auto unmap = driver_fn<UnmapFn>("cuMemUnmap");
  static auto release = driver_fn<ReleaseFn>("cuMemRelease");
  static auto addr_free = driver_fn<FreeFn>("cuMemAddressFree");
  if (r.mapped) {
    unmap(r.va, r.size);
    release(r.handle);
  }
  addr_free(r.va, r.size);
  g_regions.erase(ptr);
}

// File descriptor of the region's current physical allocation; the caller owns (and closes) it.
int64_t vmm_export_fd(int64_t ptr) {
  std::lock_guard<std::mutex> lk(g_mu);
  Region& r = find(ptr);
  if (!r.mapped) throw std::runtime_error("cannot export a paused region");
  static auto exp = driver_fn<ExportFn>("cuMemExportToShareableHandle");
  int fd = -1;
  cu_check(exp(&fd, r.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
  return fd;
}

// Maps the physical allocation behind `fd` (exported by another process, `nbytes` as reported by its vmm_size)
// into this process for access from `device`.  Returns the device pointer.  The descriptor may be closed afterwards.
int64_t vmm_import_fd(int64_t fd, int64_t nbytes, int64_t device) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  cudaFree(nullptr);
  static auto imp = driver_fn<ImportFn>("cuMemImportFromShareableHandle");
  static auto reserve = driver_fn<ReserveFn>("cuMemAddressReserve");
  static auto addr_free = driver_fn<FreeFn>("cuMemAddressFree");
  static auto map = driver_fn<MapFn>("cuMemMap");
  static auto access = driver_fn<AccessFn>("cuMemSetAccess");
  static auto release = driver_fn<ReleaseFn>("cuMemRelease");
  Imported im;
  im.size = (size_t)nbytes;
  im.device = (int)device;
  cu_check(imp(&im.handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
           "cuMemImportFromShareableHandle");
  CUresult r = reserve(&im.va, im.size, 0, 0, 0);
  if (r != CUDA_SUCCESS) { release(im.handle); cu_check(r, "cuMemAddressReserve"); }
  r = map(im.va, im.size, 0, im.handle, 0);
  if (r != CUDA_SUCCESS) { addr_free(im.va, im.size); release(im.handle); cu_check(r, "cuMemMap (imported)"); }
  CUmemAccessDesc desc = {};
  desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  desc.location.id = (int)device;
  desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = access(im.va, im.size, &desc, 1);
  if (r != CUDA_SUCCESS) {
    static auto unmap = driver_fn<UnmapFn>("cuMemUnmap");
    unmap(im.va, im.size); addr_free(im.va, im.size); release(im.handle);
    cu_check(r, "cuMemSetAccess (imported; is peer access between the two GPUs possible?)");
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_imported[(int64_t)im.va] = im;
  return (int64_t)im.va;
}

void vmm_unimport(int64_t ptr) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_imported.find(ptr);
  if (it == g_imported.end()) throw std::runtime_error("not an imported mapping");
  Imported im = it->second;
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)im.device);
  cudaDeviceSynchronize();
  static auto unmap = driver_fn<UnmapFn>("cuMemUnmap");
  static auto release = driver_fn<ReleaseFn>("cuMemRelease");
  static auto addr_free = driver_fn<FreeFn>("cuMemAddressFree");
  unmap(im.va, im.size);
  release(im.handle);
  addr_free(im.va, im.size);
  g_imported.erase(it);
}

bool vmm_is_mapped(int64_t ptr) {
  std::lock_guard<std::mutex> lk(g_mu);
  return find(ptr).mapped;
}
int64_t vmm_size(int64_t ptr) {
  std::lock_guard<std::mutex> lk(g_mu);
  return (int64_t)find(ptr).size;
}

}  // namespace

void register_vmm(pybind11::module_& m) {
  m.def("vmm_alloc", &vmm_alloc);
  m.def("vmm_pause", &vmm_pause);
  m.def("vmm_resume", &vmm_resume);
  m.def("vmm_free", &vmm_free);
  m.def("vmm_export_fd", &vmm_export_fd);
  m.def("vmm_import_fd", &vmm_import_fd);
  m.def("vmm_unimport", &vmm_unimport);
  m.def("vmm_is_mapped", &vmm_is_mapped);
  m.def("vmm_size", &vmm_size);
}
