// Symmetric heap segments through the virtual-memory-management API, bound to an NVSwitch multicast object.
//
// A segment is physical memory created with cuMemCreate and exported as a POSIX file descriptor; every rank imports
// every peer's descriptor and maps it into its own address space, so kernels reach peers' segments with plain loads
// and stores (what CUDA IPC gives too).  What IPC cannot give: the same physical segments are also bound to ONE
// multicast object (cuMulticastCreate / AddDevice / BindMem) whose mapping is the address that multimem.ld_reduce /
// multimem.st operate on -- loads that return the sum over all ranks' copies, stores that land in every copy, both
// executed inside the switch (NVLS).  The file descriptors travel between the ranks over Unix sockets (the Python
// side, parallel/symm.py); this file is the per-process driver work.  The reference shares cudaMalloc'd slot arrays
// through CUDA IPC handles (tandem/csrc/cuda_links.cpp:43-118) and has no in-switch path.
//
// The driver entry points are looked up at run time (cudaGetDriverEntryPoint), so the library links against the
// runtime only and loads on machines without a driver.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>

namespace {

thread_local char g_vmm_error[256] = "";

template <typename Fn>
Fn entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
  return (Fn)p;
}

int fail(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return 0;
  snprintf(g_vmm_error, sizeof(g_vmm_error), "%s failed with CUresult %d", what, (int)r);
  return -40;
}

#define DRIVER(name, ...)                                                   \
  static auto fn_##name = entry<CUresult (*)(__VA_ARGS__)>(#name);          \
  if (fn_##name == nullptr) {                                               \
    snprintf(g_vmm_error, sizeof(g_vmm_error), "driver has no " #name);     \
    return -41;                                                             \
  }

CUmemAllocationProp segment_prop(int dev) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int map_handle(CUmemGenericAllocationHandle handle, size_t bytes, size_t align, int dev, void** out) {
  DRIVER(cuMemAddressReserve, CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long)
  DRIVER(cuMemMap, CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long)
  DRIVER(cuMemSetAccess, CUdeviceptr, size_t, const CUmemAccessDesc*, size_t)
  DRIVER(cuMemAddressFree, CUdeviceptr, size_t)
  DRIVER(cuMemUnmap, CUdeviceptr, size_t)
  CUdeviceptr va = 0;
  int rc = fail(fn_cuMemAddressReserve(&va, bytes, align, 0, 0), "cuMemAddressReserve");
  if (rc) return rc;
  rc = fail(fn_cuMemMap(va, bytes, 0, handle, 0), "cuMemMap");
  if (rc) {
    fn_cuMemAddressFree(va, bytes);
    return rc;
  }
  CUmemAccessDesc access = {};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = dev;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  rc = fail(fn_cuMemSetAccess(va, bytes, &access, 1), "cuMemSetAccess");
  if (rc) {
    fn_cuMemUnmap(va, bytes);
    fn_cuMemAddressFree(va, bytes);
    return rc;
  }
  *out = (void*)va;
  return 0;
}

}  // namespace

extern "C" {

const char* tb_vmm_last_error() { return g_vmm_error; }

// flags[0]: the device can export memory as POSIX file descriptors; flags[1]: it supports multicast objects.
int tb_vmm_probe(int dev, int* flags) {
  flags[0] = flags[1] = 0;
  DRIVER(cuDeviceGetAttribute, int*, CUdevice_attribute, CUdevice)
  DRIVER(cuDeviceGet, CUdevice*, int)
  CUdevice d;
  int rc = fail(fn_cuDeviceGet(&d, dev), "cuDeviceGet");
  if (rc) return rc;
  int v = 0;
  if (fn_cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, d) == CUDA_SUCCESS) flags[0] = v;
  v = 0;
  if (fn_cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, d) == CUDA_SUCCESS) flags[1] = v;
  return 0;
}

// Smallest size (and alignment) a segment of `bytes` must be rounded up to so that it can be created, mapped and bound
// to a multicast object shared by n_devices devices.
long long tb_vmm_granularity(int dev, int n_devices, long long bytes) {
  DRIVER(cuMemGetAllocationGranularity, size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags)
  CUmemAllocationProp prop = segment_prop(dev);
  size_t gran = 0;
  if (fail(fn_cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity")) return -40;
  if (n_devices > 1) {
    static auto mc_gran = entry<CUresult (*)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags)>("cuMulticastGetGranularity");
    if (mc_gran != nullptr) {
      CUmulticastObjectProp mp = {};
      mp.numDevices = n_devices;
      mp.size = bytes;
      mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      size_t g2 = 0;
      if (mc_gran(&g2, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && g2 > gran) gran = g2;
    }
  }
  return (long long)gran;
}

// This rank's segment: physical memory (zeroed), mapped here, exported as a file descriptor for the peers.
// bytes must be a multiple of tb_vmm_granularity.  handle_out identifies the allocation for tb_mc_bind / tb_vmm_release.
int tb_vmm_create(long long bytes, long long align, int dev, void** ptr_out, int* fd_out, unsigned long long* handle_out) {
  DRIVER(cuMemCreate, CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long)
  DRIVER(cuMemExportToShareableHandle, void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long)
  DRIVER(cuMemRelease, CUmemGenericAllocationHandle)
  CUmemAllocationProp prop = segment_prop(dev);
  CUmemGenericAllocationHandle handle = 0;
  int rc = fail(fn_cuMemCreate(&handle, (size_t)bytes, &prop, 0), "cuMemCreate");
  if (rc) return rc;
  rc = map_handle(handle, (size_t)bytes, (size_t)align, dev, ptr_out);
  if (rc) {
    fn_cuMemRelease(handle);
    return rc;
  }
  int fd = -1;
  rc = fail(fn_cuMemExportToShareableHandle(&fd, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
  if (rc) return rc;
  if (cudaMemset(*ptr_out, 0, (size_t)bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    snprintf(g_vmm_error, sizeof(g_vmm_error), "clearing the new segment failed");
    return -42;
  }
  *fd_out = fd;
  *handle_out = (unsigned long long)handle;
  return 0;
}

// A peer's segment, from the file descriptor it exported, mapped into this process for this device.
int tb_vmm_import(int fd, long long bytes, long long align, int dev, void** ptr_out, unsigned long long* handle_out) {
  DRIVER(cuMemImportFromShareableHandle, CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType)
  DRIVER(cuMemRelease, CUmemGenericAllocationHandle)
  CUmemGenericAllocationHandle handle = 0;
  int rc = fail(fn_cuMemImportFromShareableHandle(&handle, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
                "cuMemImportFromShareableHandle");
  if (rc) return rc;
  rc = map_handle(handle, (size_t)bytes, (size_t)align, dev, ptr_out);
  if (rc) {
    fn_cuMemRelease(handle);
    return rc;
  }
  *handle_out = (unsigned long long)handle;
  return 0;
}

// Unmaps a segment (own or imported) and drops this process's reference to its memory.
int tb_vmm_release(void* ptr, long long bytes, unsigned long long handle) {
  DRIVER(cuMemUnmap, CUdeviceptr, size_t)
  DRIVER(cuMemAddressFree, CUdeviceptr, size_t)
  DRIVER(cuMemRelease, CUmemGenericAllocationHandle)
  int rc = 0;
  if (ptr != nullptr) {
    rc = fail(fn_cuMemUnmap((CUdeviceptr)ptr, (size_t)bytes), "cuMemUnmap");
    int rc2 = fail(fn_cuMemAddressFree((CUdeviceptr)ptr, (size_t)bytes), "cuMemAddressFree");
    if (rc == 0) rc = rc2;
  }
  if (handle != 0) {
    int rc2 = fail(fn_cuMemRelease((CUmemGenericAllocationHandle)handle), "cuMemRelease");
    if (rc == 0) rc = rc2;
  }
  return rc;
}

// Rank 0: one multicast object of `bytes` for n_devices devices, exported for the peers.
int tb_mc_create(long long bytes, int n_devices, int* fd_out, unsigned long long* mc_out) {
  DRIVER(cuMulticastCreate, CUmemGenericAllocationHandle*, const CUmulticastObjectProp*)
  DRIVER(cuMemExportToShareableHandle, void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long)
  CUmulticastObjectProp mp = {};
  mp.numDevices = n_devices;
  mp.size = (size_t)bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle mc = 0;
  int rc = fail(fn_cuMulticastCreate(&mc, &mp), "cuMulticastCreate");
  if (rc) return rc;
  int fd = -1;
  rc = fail(fn_cuMemExportToShareableHandle(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle (multicast)");
  if (rc) return rc;
  *fd_out = fd;
  *mc_out = (unsigned long long)mc;
  return 0;
}

int tb_mc_import(int fd, unsigned long long* mc_out) {
  DRIVER(cuMemImportFromShareableHandle, CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType)
  CUmemGenericAllocationHandle mc = 0;
  int rc = fail(fn_cuMemImportFromShareableHandle(&mc, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
                "cuMemImportFromShareableHandle (multicast)");
  if (rc == 0) *mc_out = (unsigned long long)mc;
  return rc;
}

// Every rank, before anyone binds: joins the object with its device.
int tb_mc_add_device(unsigned long long mc, int dev) {
  DRIVER(cuMulticastAddDevice, CUmemGenericAllocationHandle, CUdevice)
  DRIVER(cuDeviceGet, CUdevice*, int)
  CUdevice d;
  int rc = fail(fn_cuDeviceGet(&d, dev), "cuDeviceGet");
  if (rc) return rc;
  return fail(fn_cuMulticastAddDevice((CUmemGenericAllocationHandle)mc, d), "cuMulticastAddDevice");
}

// Every rank, after all have joined: binds its own segment at offset 0 and maps the object; *ptr_out is the address
// for multimem instructions (offset x in it = offset x in every rank's segment).
int tb_mc_bind_and_map(unsigned long long mc, unsigned long long mem_handle, long long bytes, long long align, int dev, void** ptr_out) {
  DRIVER(cuMulticastBindMem, CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long)
  int rc = fail(fn_cuMulticastBindMem((CUmemGenericAllocationHandle)mc, 0, (CUmemGenericAllocationHandle)mem_handle, 0, (size_t)bytes, 0),
                "cuMulticastBindMem");
  if (rc) return rc;
  return map_handle((CUmemGenericAllocationHandle)mc, (size_t)bytes, (size_t)align, dev, ptr_out);
}

// Before the memory goes away: unmaps the multicast address, unbinds this device's memory and drops the object.
int tb_mc_release(unsigned long long mc, void* mc_ptr, long long bytes, int dev) {
  DRIVER(cuMemUnmap, CUdeviceptr, size_t)
  DRIVER(cuMemAddressFree, CUdeviceptr, size_t)
  DRIVER(cuMemRelease, CUmemGenericAllocationHandle)
  DRIVER(cuDeviceGet, CUdevice*, int)
  static auto unbind = entry<CUresult (*)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t)>("cuMulticastUnbind");
  int rc = 0;
  if (mc_ptr != nullptr) {
    rc = fail(fn_cuMemUnmap((CUdeviceptr)mc_ptr, (size_t)bytes), "cuMemUnmap (multicast)");
    fn_cuMemAddressFree((CUdeviceptr)mc_ptr, (size_t)bytes);
  }
  CUdevice d;
  if (unbind != nullptr && fn_cuDeviceGet(&d, dev) == CUDA_SUCCESS) unbind((CUmemGenericAllocationHandle)mc, d, 0, (size_t)bytes);
  int rc2 = fail(fn_cuMemRelease((CUmemGenericAllocationHandle)mc), "cuMemRelease (multicast)");
  return rc ? rc : rc2;
}

int tb_close_fd(int fd) { return close(fd); }

}  // extern "C"
