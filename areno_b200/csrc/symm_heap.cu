// Symmetric heap for the peer-memory kernels: CUDA virtual-memory-management allocations that
// every rank of a group maps into its own address space, plus an optional NVLink multicast
// (NVLS) mapping of the same physical pages for the multimem.* instructions.
//
//   rank r:  areno_vmm_alloc        cuMemCreate (shareable as a POSIX file descriptor) + map locally
//            -> the descriptor travels to the peers over a Unix socket (SCM_RIGHTS, Python side)
//   peers :  areno_vmm_import       cuMemImportFromShareableHandle + cuMemMap + cuMemSetAccess
//
//   multicast (all devices of the group must be on one NVSwitch fabric):
//   rank 0:  areno_mc_create        cuMulticastCreate -> descriptor to the peers
//   all   :  areno_mc_import (peers), areno_mc_add_device, <group barrier>,
//            areno_mc_bind          cuMulticastBindMem(own pages) + map the multicast handle
//
// A load through the multicast address with multimem.ld_reduce returns the sum over all bound
// devices (added inside the switch); multimem.st stores to all of them.
//
// The driver entry points are resolved at run time (cudaGetDriverEntryPoint), so the library has no
// link-time dependency on libcuda and loads on a machine without a GPU.  Every routine returns 0,
// a negative code of this file, or the positive CUresult of the failing driver call; none of them
// launches a kernel.  The reference has no counterpart (it uses NCCL only,
// areno/engine/parallel/context.py:82-113).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace {

struct Driver {
  bool ok = false;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemGetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*McCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*McAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*McBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                        unsigned long long);
  CUresult (*McUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*McGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*DeviceGet)(CUdevice*, int);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
};

template <typename F>
bool resolve(F& fn, const char* name) {
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      sym == nullptr)
    return false;
  fn = reinterpret_cast<F>(sym);
  return true;
}

const Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    bool ok = true;
    ok &= resolve(d.MemCreate, "cuMemCreate");
    ok &= resolve(d.MemRelease, "cuMemRelease");
    ok &= resolve(d.MemAddressReserve, "cuMemAddressReserve");
    ok &= resolve(d.MemAddressFree, "cuMemAddressFree");
    ok &= resolve(d.MemMap, "cuMemMap");
    ok &= resolve(d.MemUnmap, "cuMemUnmap");
    ok &= resolve(d.MemSetAccess, "cuMemSetAccess");
    ok &= resolve(d.MemExport, "cuMemExportToShareableHandle");
    ok &= resolve(d.MemImport, "cuMemImportFromShareableHandle");
    ok &= resolve(d.MemGetGranularity, "cuMemGetAllocationGranularity");
    ok &= resolve(d.McCreate, "cuMulticastCreate");
    ok &= resolve(d.McAddDevice, "cuMulticastAddDevice");
    ok &= resolve(d.McBindMem, "cuMulticastBindMem");
    ok &= resolve(d.McUnbind, "cuMulticastUnbind");
    ok &= resolve(d.McGetGranularity, "cuMulticastGetGranularity");
    ok &= resolve(d.DeviceGet, "cuDeviceGet");
    ok &= resolve(d.DeviceGetAttribute, "cuDeviceGetAttribute");
    d.ok = ok;
  });
  return d;
}

constexpr int kErrNoDriver = -10;   // a driver entry point could not be resolved
constexpr int kErrArgument = -3;

int current_device(CUdevice* dev, int* ordinal) {
  int ord = 0;
  if (cudaGetDevice(&ord) != cudaSuccess) return kErrArgument;
  cudaFree(nullptr);  // make sure the primary context exists and is current on this thread
  const CUresult rc = driver().DeviceGet(dev, ord);
  if (rc != CUDA_SUCCESS) return (int)rc;
  if (ordinal != nullptr) *ordinal = ord;
  return 0;
}

CUmemAllocationProp local_prop(int ordinal) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = ordinal;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int map_rw(CUmemGenericAllocationHandle h, size_t bytes, size_t align, int ordinal, void** out) {
  const Driver& d = driver();
  CUdeviceptr va = 0;
  CUresult rc = d.MemAddressReserve(&va, bytes, align, 0, 0);
  if (rc != CUDA_SUCCESS) return (int)rc;
  rc = d.MemMap(va, bytes, 0, h, 0);
  if (rc != CUDA_SUCCESS) {
    d.MemAddressFree(va, bytes);
    return (int)rc;
  }
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = ordinal;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  rc = d.MemSetAccess(va, bytes, &acc, 1);
  if (rc != CUDA_SUCCESS) {
    d.MemUnmap(va, bytes);
    d.MemAddressFree(va, bytes);
    return (int)rc;
  }
  *out = reinterpret_cast<void*>(va);
  return 0;
}

}  // namespace

extern "C" {

// *vmm = 1 when the current device supports shareable virtual-memory allocations, *multicast = 1 when
// it also supports NVLink multicast objects.
int areno_vmm_supported(int* vmm, int* multicast) {
  *vmm = 0;
  *multicast = 0;
  if (!driver().ok) return kErrNoDriver;
  CUdevice dev;
  int rc = current_device(&dev, nullptr);
  if (rc != 0) return rc;
  int v = 0;
  if (driver().DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev) == CUDA_SUCCESS && v) {
    int fd = 0;
    if (driver().DeviceGetAttribute(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev) == CUDA_SUCCESS)
      *vmm = fd ? 1 : 0;
  }
  int m = 0;
  if (driver().DeviceGetAttribute(&m, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS) *multicast = m ? 1 : 0;
  return 0;
}

// Size granule that `bytes` of a symmetric allocation must be rounded up to.  With `num_devices` > 1
// the granule also satisfies a multicast object over that many devices.
int areno_vmm_granularity(int num_devices, long long* granule) {
  if (!driver().ok) return kErrNoDriver;
  CUdevice dev;
  int ord = 0;
  int rc = current_device(&dev, &ord);
  if (rc != 0) return rc;
  const CUmemAllocationProp prop = local_prop(ord);
  size_t g = 0;
  CUresult r = driver().MemGetGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) return (int)r;
  if (num_devices > 1) {
    CUmulticastObjectProp mp = {};
    mp.numDevices = (unsigned)num_devices;
    mp.size = g;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (driver().McGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > g) g = mg;
  }
  *granule = (long long)g;
  return 0;
}

// Allocate `bytes` (a multiple of the granule) of zero-filled device memory on the current device,
// map it, and export it as a file descriptor (*fd; the caller closes it after sending it out).
int areno_vmm_alloc(long long bytes, long long granule, void** ptr, unsigned long long* handle, int* fd) {
  if (!driver().ok) return kErrNoDriver;
  if (bytes <= 0 || granule <= 0 || bytes % granule != 0) return kErrArgument;
  CUdevice dev;
  int ord = 0;
  int rc = current_device(&dev, &ord);
  if (rc != 0) return rc;
  const CUmemAllocationProp prop = local_prop(ord);
  CUmemGenericAllocationHandle h = 0;
  CUresult r = driver().MemCreate(&h, (size_t)bytes, &prop, 0);
  if (r != CUDA_SUCCESS) return (int)r;
  rc = map_rw(h, (size_t)bytes, (size_t)granule, ord, ptr);
  if (rc != 0) {
    driver().MemRelease(h);
    return rc;
  }
  int out_fd = -1;
  r = driver().MemExport(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    driver().MemUnmap((CUdeviceptr)*ptr, (size_t)bytes);
    driver().MemAddressFree((CUdeviceptr)*ptr, (size_t)bytes);
    driver().MemRelease(h);
    return (int)r;
  }
  const cudaError_t e = cudaMemset(*ptr, 0, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  *handle = (unsigned long long)h;
  *fd = out_fd;
  return 0;
}

// Map a peer's allocation (received as a file descriptor) for reading and writing from the current device.
int areno_vmm_import(int fd, long long bytes, long long granule, void** ptr, unsigned long long* handle) {
  if (!driver().ok) return kErrNoDriver;
  if (fd < 0 || bytes <= 0) return kErrArgument;
  CUdevice dev;
  int ord = 0;
  int rc = current_device(&dev, &ord);
  if (rc != 0) return rc;
  CUmemGenericAllocationHandle h = 0;
  CUresult r = driver().MemImport(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return (int)r;
  rc = map_rw(h, (size_t)bytes, (size_t)granule, ord, ptr);
  if (rc != 0) {
    driver().MemRelease(h);
    return rc;
  }
  *handle = (unsigned long long)h;
  return 0;
}

// Unmap a range obtained from areno_vmm_alloc / areno_vmm_import / areno_mc_bind and drop its handle.
int areno_vmm_release(void* ptr, long long bytes, unsigned long long handle) {
  if (!driver().ok) return kErrNoDriver;
  int first = 0;
  if (ptr != nullptr) {
    CUresult r = driver().MemUnmap((CUdeviceptr)ptr, (size_t)bytes);
    if (r != CUDA_SUCCESS) first = (int)r;
    r = driver().MemAddressFree((CUdeviceptr)ptr, (size_t)bytes);
    if (r != CUDA_SUCCESS && first == 0) first = (int)r;
  }
  if (handle != 0) {
    const CUresult r = driver().MemRelease((CUmemGenericAllocationHandle)handle);
    if (r != CUDA_SUCCESS && first == 0) first = (int)r;
  }
  return first;
}

// Create a multicast object for `num_devices` devices and `bytes` per device (first rank of the group).
int areno_mc_create(int num_devices, long long bytes, unsigned long long* mc, int* fd) {
  if (!driver().ok) return kErrNoDriver;
  if (num_devices < 2 || bytes <= 0) return kErrArgument;
  CUmulticastObjectProp mp = {};
  mp.numDevices = (unsigned)num_devices;
  mp.size = (size_t)bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h = 0;
  CUresult r = driver().McCreate(&h, &mp);
  if (r != CUDA_SUCCESS) return (int)r;
  int out_fd = -1;
  r = driver().MemExport(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    driver().MemRelease(h);
    return (int)r;
  }
  *mc = (unsigned long long)h;
  *fd = out_fd;
  return 0;
}

int areno_mc_import(int fd, unsigned long long* mc) {
  if (!driver().ok) return kErrNoDriver;
  CUmemGenericAllocationHandle h = 0;
  const CUresult r = driver().MemImport(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return (int)r;
  *mc = (unsigned long long)h;
  return 0;
}

// Every rank adds its device; all ranks must have done so before any of them binds memory.
int areno_mc_add_device(unsigned long long mc) {
  if (!driver().ok) return kErrNoDriver;
  CUdevice dev;
  const int rc = current_device(&dev, nullptr);
  if (rc != 0) return rc;
  return (int)driver().McAddDevice((CUmemGenericAllocationHandle)mc, dev);
}

// Bind this rank's allocation (`mem`, `bytes`) at offset 0 of the multicast object and map the object;
// *mc_ptr is the multicast address that corresponds to the start of the allocation on every rank.
int areno_mc_bind(unsigned long long mc, unsigned long long mem, long long bytes, long long granule, void** mc_ptr) {
  if (!driver().ok) return kErrNoDriver;
  CUdevice dev;
  int ord = 0;
  int rc = current_device(&dev, &ord);
  if (rc != 0) return rc;
  const CUresult r = driver().McBindMem((CUmemGenericAllocationHandle)mc, 0, (CUmemGenericAllocationHandle)mem, 0,
                                        (size_t)bytes, 0);
  if (r != CUDA_SUCCESS) return (int)r;
  rc = map_rw((CUmemGenericAllocationHandle)mc, (size_t)bytes, (size_t)granule, ord, mc_ptr);
  if (rc != 0) driver().McUnbind((CUmemGenericAllocationHandle)mc, dev, 0, (size_t)bytes);
  return rc;
}

// Undo areno_mc_bind on this rank: unmap the multicast address, unbind the device's pages, drop the handle.
int areno_mc_release(unsigned long long mc, void* mc_ptr, long long bytes, int bound) {
  if (!driver().ok) return kErrNoDriver;
  CUdevice dev;
  const int rc = current_device(&dev, nullptr);
  if (rc != 0) return rc;
  int first = 0;
  if (mc_ptr != nullptr) {
    CUresult r = driver().MemUnmap((CUdeviceptr)mc_ptr, (size_t)bytes);
    if (r != CUDA_SUCCESS) first = (int)r;
    r = driver().MemAddressFree((CUdeviceptr)mc_ptr, (size_t)bytes);
    if (r != CUDA_SUCCESS && first == 0) first = (int)r;
  }
  if (bound) {
    const CUresult r = driver().McUnbind((CUmemGenericAllocationHandle)mc, dev, 0, (size_t)bytes);
    if (r != CUDA_SUCCESS && first == 0) first = (int)r;
  }
  if (mc != 0) {
    const CUresult r = driver().MemRelease((CUmemGenericAllocationHandle)mc);
    if (r != CUDA_SUCCESS && first == 0) first = (int)r;
  }
  return first;
}

}  // extern "C"
