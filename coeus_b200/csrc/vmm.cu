// Symmetric memory from the virtual-memory-management API, with an NVLink multicast (NVLS)
// mapping on top: the substrate of the kernels that use multimem.ld_reduce / multimem.st /
// multimem.red.  (Memory from cudaMalloc shared through CUDA IPC cannot be bound to a multicast
// object; allocations made with cuMemCreate can.)
//
// Per rank and buffer:
//   cb_vmm_alloc        cuMemCreate (POSIX-fd shareable) + reserve + map + access for this device
//   cb_vmm_export_fd    file descriptor that another process imports (sent over a Unix socket)
//   cb_vmm_import       cuMemImportFromShareableHandle + reserve + map: a peer's buffer, reachable
//                       with plain loads / stores over NVLink
//   cb_mc_create        (one rank) cuMulticastCreate for the whole team + exported descriptor
//   cb_mc_import        (other ranks) the same object from the descriptor
//   cb_mc_add_device    every rank adds its device; binding blocks until all have
//   cb_mc_bind_map      bind this rank's allocation at offset 0 and map the multicast object:
//                       a store to the returned address reaches every rank's buffer, a
//                       multimem.ld_reduce from it returns the sum over the ranks
//   cb_mc_release / cb_vmm_release   unbind, unmap, free (in that order, on every exit path:
//                       a process must not die with memory still bound to a multicast object)
// The reference has no communication layer at all; this is infrastructure of this framework.
// All driver entry points are fetched at run time, so the library has no link-time dependency on
// libcuda.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>

namespace {

template <typename F>
F drv(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<F>(p);
}

#define CB_DRV(var, name, pfn)                      \
  static auto var = drv<pfn>(name);                 \
  if (var == nullptr) return -90

struct Vmm {          // an allocation of this process, or an imported one
  CUmemGenericAllocationHandle handle;
  CUdeviceptr va;
  size_t size;
  int owned;
};

struct Mc {
  CUmemGenericAllocationHandle handle;
  CUdeviceptr va;     // 0 until mapped
  size_t size;
  size_t bound;       // bytes bound at offset 0 (0: nothing bound)
  int dev;
};

int current_device(CUdevice* out) {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) return -1;
  cudaFree(nullptr);   // make sure the primary context exists
  CB_DRV(f_get, "cuDeviceGet", PFN_cuDeviceGet);
  return f_get(out, d) == CUDA_SUCCESS ? 0 : -1;
}

CUmemAllocationProp alloc_prop(int dev) {
  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int map_rw(CUmemGenericAllocationHandle h, size_t size, size_t align, int dev, CUdeviceptr* va) {
  CB_DRV(f_reserve, "cuMemAddressReserve", PFN_cuMemAddressReserve);
  CB_DRV(f_map, "cuMemMap", PFN_cuMemMap);
  CB_DRV(f_access, "cuMemSetAccess", PFN_cuMemSetAccess);
  CB_DRV(f_free, "cuMemAddressFree", PFN_cuMemAddressFree);
  CB_DRV(f_unmap, "cuMemUnmap", PFN_cuMemUnmap);
  CUdeviceptr p = 0;
  if (f_reserve(&p, size, align, 0, 0) != CUDA_SUCCESS) return -10;
  if (f_map(p, size, 0, h, 0) != CUDA_SUCCESS) {
    f_free(p, size);
    return -11;
  }
  CUmemAccessDesc acc;
  std::memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (f_access(p, size, &acc, 1) != CUDA_SUCCESS) {
    f_unmap(p, size);
    f_free(p, size);
    return -12;
  }
  *va = p;
  return 0;
}

}  // namespace

// 1 when the current device supports multicast objects (NVLS), 0 when not, negative on error.
extern "C" int cb_multicast_supported() {
  CUdevice dev;
  if (current_device(&dev) != 0) return -1;
  CB_DRV(f_attr, "cuDeviceGetAttribute", PFN_cuDeviceGetAttribute);
  int v = 0;
  if (f_attr(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return -2;
  return v;
}

// Size granularity: of plain allocations (multicast == 0) or of multicast objects for a team of
// `ndev` devices (minimum granularity).  0 on error.
extern "C" size_t cb_vmm_granularity(int multicast, int ndev) {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) return 0;
  cudaFree(nullptr);
  if (!multicast) {
    static auto f_gran = drv<PFN_cuMemGetAllocationGranularity>("cuMemGetAllocationGranularity");
    if (f_gran == nullptr) return 0;
    CUmemAllocationProp prop = alloc_prop(d);
    size_t g = 0;
    if (f_gran(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) return 0;
    return g;
  }
  static auto f_mcg = drv<PFN_cuMulticastGetGranularity>("cuMulticastGetGranularity");
  if (f_mcg == nullptr) return 0;
  CUmulticastObjectProp mp;
  std::memset(&mp, 0, sizeof(mp));
  mp.numDevices = static_cast<unsigned int>(ndev);
  mp.size = 2u << 20;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t g = 0;
  if (f_mcg(&g, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) != CUDA_SUCCESS) return 0;
  return g;
}

// Allocate `bytes` (a multiple of the granularity) on the current device, zeroed.
extern "C" int cb_vmm_alloc(size_t bytes, void** handle_out, void** va_out) {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) return -1;
  cudaFree(nullptr);
  CB_DRV(f_create, "cuMemCreate", PFN_cuMemCreate);
  CB_DRV(f_release, "cuMemRelease", PFN_cuMemRelease);
  CUmemAllocationProp prop = alloc_prop(d);
  CUmemGenericAllocationHandle h;
  if (f_create(&h, bytes, &prop, 0) != CUDA_SUCCESS) return -2;
  CUdeviceptr va = 0;
  const int rc = map_rw(h, bytes, 0, d, &va);
  if (rc != 0) {
    f_release(h);
    return rc;
  }
  if (cudaMemset(reinterpret_cast<void*>(va), 0, bytes) != cudaSuccess) return -3;
  Vmm* v = new Vmm{h, va, bytes, 1};
  *handle_out = v;
  *va_out = reinterpret_cast<void*>(va);
  return 0;
}

extern "C" int cb_vmm_export_fd(void* handle, int* fd_out) {
  Vmm* v = static_cast<Vmm*>(handle);
  CB_DRV(f_export, "cuMemExportToShareableHandle", PFN_cuMemExportToShareableHandle);
  int fd = -1;
  if (f_export(&fd, v->handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS)
    return -1;
  *fd_out = fd;
  return 0;
}

// Map a peer's allocation (its descriptor received over a Unix socket) for the current device.
extern "C" int cb_vmm_import(int fd, size_t bytes, void** handle_out, void** va_out) {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) return -1;
  cudaFree(nullptr);
  CB_DRV(f_import, "cuMemImportFromShareableHandle", PFN_cuMemImportFromShareableHandle);
  CB_DRV(f_release, "cuMemRelease", PFN_cuMemRelease);
  CUmemGenericAllocationHandle h;
  if (f_import(&h, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
    return -2;
  CUdeviceptr va = 0;
  const int rc = map_rw(h, bytes, 0, d, &va);
  if (rc != 0) {
    f_release(h);
    return rc;
  }
  Vmm* v = new Vmm{h, va, bytes, 0};
  *handle_out = v;
  *va_out = reinterpret_cast<void*>(va);
  return 0;
}

extern "C" int cb_vmm_release(void* handle) {
  Vmm* v = static_cast<Vmm*>(handle);
  if (v == nullptr) return 0;
  CB_DRV(f_unmap, "cuMemUnmap", PFN_cuMemUnmap);
  CB_DRV(f_free, "cuMemAddressFree", PFN_cuMemAddressFree);
  CB_DRV(f_release, "cuMemRelease", PFN_cuMemRelease);
  int rc = 0;
  if (f_unmap(v->va, v->size) != CUDA_SUCCESS) rc = -1;
  if (f_free(v->va, v->size) != CUDA_SUCCESS) rc = -2;
  if (f_release(v->handle) != CUDA_SUCCESS) rc = -3;
  delete v;
  return rc;
}

// ------------------------------------------------------------------------------- multicast
extern "C" int cb_mc_create(int ndev, size_t bytes, void** mc_out, int* fd_out) {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) return -1;
  cudaFree(nullptr);
  CB_DRV(f_create, "cuMulticastCreate", PFN_cuMulticastCreate);
  CB_DRV(f_export, "cuMemExportToShareableHandle", PFN_cuMemExportToShareableHandle);
  CUmulticastObjectProp mp;
  std::memset(&mp, 0, sizeof(mp));
  mp.numDevices = static_cast<unsigned int>(ndev);
  mp.size = bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  if (f_create(&h, &mp) != CUDA_SUCCESS) return -2;
  int fd = -1;
  if (f_export(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) return -3;
  *mc_out = new Mc{h, 0, bytes, 0, d};
  *fd_out = fd;
  return 0;
}

extern "C" int cb_mc_import(int fd, size_t bytes, void** mc_out) {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) return -1;
  cudaFree(nullptr);
  CB_DRV(f_import, "cuMemImportFromShareableHandle", PFN_cuMemImportFromShareableHandle);
  CUmemGenericAllocationHandle h;
  if (f_import(&h, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
    return -2;
  *mc_out = new Mc{h, 0, bytes, 0, d};
  return 0;
}

extern "C" int cb_mc_add_device(void* mc) {
  Mc* m = static_cast<Mc*>(mc);
  CUdevice dev;
  if (current_device(&dev) != 0) return -1;
  CB_DRV(f_add, "cuMulticastAddDevice", PFN_cuMulticastAddDevice);
  return f_add(m->handle, dev) == CUDA_SUCCESS ? 0 : -2;
}

// Bind the whole of `mem` (an allocation of this process made by cb_vmm_alloc) at offset 0 of the
// multicast object and map the object; *va_out is the multicast address of byte 0.
extern "C" int cb_mc_bind_map(void* mc, void* mem, void** va_out) {
  Mc* m = static_cast<Mc*>(mc);
  Vmm* v = static_cast<Vmm*>(mem);
  if (v->size > m->size) return -1;
  CB_DRV(f_bind, "cuMulticastBindMem", PFN_cuMulticastBindMem);
  CB_DRV(f_unbind, "cuMulticastUnbind", PFN_cuMulticastUnbind);
  if (f_bind(m->handle, 0, v->handle, 0, v->size, 0) != CUDA_SUCCESS) return -2;
  m->bound = v->size;
  CUdeviceptr va = 0;
  const int rc = map_rw(m->handle, m->size, 0, m->dev, &va);
  if (rc != 0) {
    CUdevice dev;
    if (current_device(&dev) == 0) f_unbind(m->handle, dev, 0, m->bound);
    m->bound = 0;
    return rc;
  }
  m->va = va;
  *va_out = reinterpret_cast<void*>(va);
  return 0;
}

extern "C" int cb_mc_release(void* mc) {
  Mc* m = static_cast<Mc*>(mc);
  if (m == nullptr) return 0;
  CB_DRV(f_unmap, "cuMemUnmap", PFN_cuMemUnmap);
  CB_DRV(f_free, "cuMemAddressFree", PFN_cuMemAddressFree);
  CB_DRV(f_release, "cuMemRelease", PFN_cuMemRelease);
  CB_DRV(f_unbind, "cuMulticastUnbind", PFN_cuMulticastUnbind);
  int rc = 0;
  if (m->va != 0) {
    if (f_unmap(m->va, m->size) != CUDA_SUCCESS) rc = -1;
    if (f_free(m->va, m->size) != CUDA_SUCCESS) rc = -2;
  }
  if (m->bound != 0) {
    CUdevice dev;
    if (current_device(&dev) != 0 || f_unbind(m->handle, dev, 0, m->bound) != CUDA_SUCCESS) rc = -3;
  }
  if (f_release(m->handle) != CUDA_SUCCESS) rc = -4;
  delete m;
  return rc;
}

extern "C" int cb_close_fd(int fd) { return close(fd); }
