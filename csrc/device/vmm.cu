// Symmetric memory through the virtual-memory-management driver API, with an NVSwitch multicast
// mapping on top (host code only).
//
// cudaMalloc + CUDA IPC gives every rank a pointer to every peer's arena, which is all the peer-memory
// kernels need.  In-switch reduction (multimem.ld_reduce / multimem.st) additionally needs ONE virtual
// address that names the same offset of every rank's arena: a multicast object to which every rank
// binds its own physical allocation.  That requires allocations made with cuMemCreate and shared as
// POSIX file descriptors, which the process group passes between ranks over Unix sockets.
// The driver entry points are looked up at run time, so the library carries no link-time dependency
// on libcuda.  The reference has no counterpart (its collectives are a vendor library, cncl_utils.h:67-121).
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include "device_api.h"

namespace {

struct Driver {
  bool ok = false;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemGetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*McCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*McAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*McBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*McUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*McGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
};

template <typename F>
bool load(F& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult st;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &st) != cudaSuccess || st != cudaDriverEntryPointSuccess || !p) {
    (void)cudaGetLastError();
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

const Driver& driver() {
  static Driver d = [] {
    Driver x;
    x.ok = load(x.MemCreate, "cuMemCreate") && load(x.MemRelease, "cuMemRelease") &&
           load(x.MemAddressReserve, "cuMemAddressReserve") && load(x.MemAddressFree, "cuMemAddressFree") &&
           load(x.MemMap, "cuMemMap") && load(x.MemUnmap, "cuMemUnmap") && load(x.MemSetAccess, "cuMemSetAccess") &&
           load(x.MemExport, "cuMemExportToShareableHandle") && load(x.MemImport, "cuMemImportFromShareableHandle") &&
           load(x.MemGetGranularity, "cuMemGetAllocationGranularity") && load(x.McCreate, "cuMulticastCreate") &&
           load(x.McAddDevice, "cuMulticastAddDevice") && load(x.McBindMem, "cuMulticastBindMem") &&
           load(x.McUnbind, "cuMulticastUnbind") && load(x.McGetGranularity, "cuMulticastGetGranularity") &&
           load(x.DeviceGet, "cuDeviceGet") && load(x.DeviceGetAttribute, "cuDeviceGetAttribute");
    return x;
  }();
  return d;
}

// driver errors are reported as CUDA runtime codes where one exists, else cudaErrorUnknown
int rc(CUresult r) {
  if (r == CUDA_SUCCESS) return 0;
  if (r == CUDA_ERROR_OUT_OF_MEMORY) return (int)cudaErrorMemoryAllocation;
  if (r == CUDA_ERROR_NOT_SUPPORTED) return (int)cudaErrorNotSupported;
  if (r == CUDA_ERROR_INVALID_VALUE) return (int)cudaErrorInvalidValue;
  if (r == CUDA_ERROR_NOT_PERMITTED) return (int)cudaErrorNotPermitted;
  return (int)cudaErrorUnknown;
}

CUmemAllocationProp local_prop(int dev) {
  CUmemAllocationProp p{};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = dev;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

int map_rw(CUmemGenericAllocationHandle h, size_t bytes, size_t align, int dev, void** ptr) {
  const Driver& d = driver();
  CUdeviceptr va = 0;
  int e = rc(d.MemAddressReserve(&va, bytes, align, 0, 0));
  if (e) return e;
  e = rc(d.MemMap(va, bytes, 0, h, 0));
  if (e) { d.MemAddressFree(va, bytes); return e; }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  e = rc(d.MemSetAccess(va, bytes, &acc, 1));
  if (e) { d.MemUnmap(va, bytes); d.MemAddressFree(va, bytes); return e; }
  *ptr = reinterpret_cast<void*>(va);
  return 0;
}

}  // namespace

extern "C" int b200_vmm_multicast_supported(int dev, int* supported) {
  *supported = 0;
  const Driver& d = driver();
  if (!d.ok) return 0;
  cudaFree(nullptr);  // make sure the primary context exists
  CUdevice cd;
  if (d.DeviceGet(&cd, dev) != CUDA_SUCCESS) return 0;
  int mc = 0, vmm = 0, fdh = 0;
  d.DeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd);
  d.DeviceGetAttribute(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, cd);
  d.DeviceGetAttribute(&fdh, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cd);
  *supported = (mc && vmm && fdh) ? 1 : 0;
  return 0;
}

// Size that both the allocation and a multicast object over `ndev` devices accept.
extern "C" int b200_vmm_round_size(int dev, int ndev, size_t bytes, size_t* rounded) {
  const Driver& d = driver();
  if (!d.ok) return (int)cudaErrorNotSupported;
  CUmemAllocationProp p = local_prop(dev);
  size_t g1 = 0, g2 = 0;
  int e = rc(d.MemGetGranularity(&g1, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  if (e) return e;
  CUmulticastObjectProp mp{};
  mp.numDevices = (unsigned)ndev;
  mp.size = bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  e = rc(d.McGetGranularity(&g2, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
  if (e) return e;
  const size_t g = g1 > g2 ? g1 : g2;
  *rounded = (bytes + g - 1) / g * g;
  return 0;
}

// Physical allocation on `dev`, mapped read-write for `dev`, exported as a file descriptor.
extern "C" int b200_vmm_alloc(size_t bytes, int dev, void** ptr, unsigned long long* handle, int* fd) {
  const Driver& d = driver();
  if (!d.ok) return (int)cudaErrorNotSupported;
  CUmemAllocationProp p = local_prop(dev);
  CUmemGenericAllocationHandle h;
  int e = rc(d.MemCreate(&h, bytes, &p, 0));
  if (e) return e;
  e = map_rw(h, bytes, 0, dev, ptr);
  if (e) { d.MemRelease(h); return e; }
  int out_fd = -1;
  e = rc(d.MemExport(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  if (e) { d.MemUnmap((CUdeviceptr)*ptr, bytes); d.MemAddressFree((CUdeviceptr)*ptr, bytes); d.MemRelease(h); return e; }
  *handle = (unsigned long long)h;
  *fd = out_fd;
  return 0;
}

// A peer's allocation (received as a file descriptor) mapped read-write for `dev`.  The descriptor is closed.
extern "C" int b200_vmm_import(int fd, size_t bytes, int dev, void** ptr, unsigned long long* handle) {
  const Driver& d = driver();
  if (!d.ok) return (int)cudaErrorNotSupported;
  CUmemGenericAllocationHandle h;
  int e = rc(d.MemImport(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  close(fd);
  if (e) return e;
  e = map_rw(h, bytes, 0, dev, ptr);
  if (e) { d.MemRelease(h); return e; }
  *handle = (unsigned long long)h;
  return 0;
}

extern "C" int b200_vmm_release(void* ptr, size_t bytes, unsigned long long handle) {
  const Driver& d = driver();
  if (!d.ok) return (int)cudaErrorNotSupported;
  int e = 0;
  if (ptr) {
    e = rc(d.MemUnmap((CUdeviceptr)ptr, bytes));
    d.MemAddressFree((CUdeviceptr)ptr, bytes);
  }
  if (handle) d.MemRelease((CUmemGenericAllocationHandle)handle);
  return e;
}

// Multicast object over `ndev` devices (created by one rank, imported by the others).
extern "C" int b200_mc_create(int ndev, size_t bytes, unsigned long long* mc, int* fd) {
  const Driver& d = driver();
  if (!d.ok) return (int)cudaErrorNotSupported;
  CUmulticastObjectProp mp{};
  mp.numDevices = (unsigned)ndev;
  mp.size = bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  int e = rc(d.McCreate(&h, &mp));
  if (e) return e;
  int out_fd = -1;
  e = rc(d.MemExport(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  if (e) { d.MemRelease(h); return e; }
  *mc = (unsigned long long)h;
  *fd = out_fd;
  return 0;
}
extern "C" int b200_mc_import(int fd, unsigned long long* mc) {
  const Driver& d = driver();
  if (!d.ok) return (int)cudaErrorNotSupported;
  CUmemGenericAllocationHandle h;
  const int e = rc(d.MemImport(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  close(fd);
  if (e) return e;
  *mc = (unsigned long long)h;
  return 0;
}
extern "C" int b200_mc_add_device(unsigned long long mc, int dev) {
  const Driver& d = driver();
  if (!d.ok) return (int)cudaErrorNotSupported;
  CUdevice cd;
  int e = rc(d.DeviceGet(&cd, dev));
  if (e) return e;
  return rc(d.McAddDevice((CUmemGenericAllocationHandle)mc, cd));
}
// Binds this rank's allocation at offset 0 of the multicast object (every device must have been added first).
extern "C" int b200_mc_bind(unsigned long long mc, unsigned long long mem_handle, size_t bytes) {
  const Driver& d = driver();
  if (!d.ok) return (int)cudaErrorNotSupported;
  return rc(d.McBindMem((CUmemGenericAllocationHandle)mc, 0, (CUmemGenericAllocationHandle)mem_handle, 0, bytes, 0));
}
extern "C" int b200_mc_map(unsigned long long mc, size_t bytes, int dev, void** ptr) {
  if (!driver().ok) return (int)cudaErrorNotSupported;
  return map_rw((CUmemGenericAllocationHandle)mc, bytes, 0, dev, ptr);
}
// Unmaps the multicast address, takes this device's memory out of the object and drops the handle.
extern "C" int b200_mc_release(void* ptr, size_t bytes, unsigned long long mc, int dev, int bound) {
  const Driver& d = driver();
  if (!d.ok) return (int)cudaErrorNotSupported;
  if (ptr) {
    d.MemUnmap((CUdeviceptr)ptr, bytes);
    d.MemAddressFree((CUdeviceptr)ptr, bytes);
  }
  if (mc && bound) {
    CUdevice cd;
    if (d.DeviceGet(&cd, dev) == CUDA_SUCCESS) d.McUnbind((CUmemGenericAllocationHandle)mc, cd, 0, bytes);
  }
  if (mc) d.MemRelease((CUmemGenericAllocationHandle)mc);
  return 0;
}
