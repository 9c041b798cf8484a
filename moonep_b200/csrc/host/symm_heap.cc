// Symmetric memory over the CUDA virtual-memory-management API, and the NVSwitch multicast
// (NVLS) overlay.  Native counterpart of the reference's csrc/nvl_shared_buffer.cuh:
//   * each rank creates ONE physical chunk (pinned device memory, exportable as a POSIX file
//     descriptor or as a fabric handle) -- nvl_shared_buffer.cuh:227-267;
//   * every rank imports all R chunks and maps them back to back into one virtual range with
//     read/write access, so that "rank r's copy" is base + r * chunk for every kernel
//     -- nvl_shared_buffer.cuh:284-356;
//   * optionally a multicast object is created by one rank, every rank adds its device and
//     binds its own chunk, and a second virtual range maps the multicast object
//     -- nvl_shared_buffer.cuh:358-544.
// Differences: the driver entry points are resolved at run time through
// cudaGetDriverEntryPoint, so the library loads on hosts without libcuda (CPU oracle, tests);
// no function calls exit() -- every failure returns a code and a message; a single-process
// "local" mode creates all R chunks on one device for single-GPU virtual groups; and R == 1
// never touches the multicast API (the reference asserts multicast support unconditionally,
// moonep/buffer.py:299).
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <mutex>

#include "host/errors.h"

namespace {

struct Driver {
  bool ok = false;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
};

Driver g_drv;
std::once_flag g_once;

template <class F>
bool resolve(const char* name, F*& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr ||
      q != cudaDriverEntryPointSuccess) {
    cudaGetLastError();
    return false;
  }
  fn = reinterpret_cast<F*>(p);
  return true;
}

void load_driver() {
  Driver& d = g_drv;
  bool ok = true;
  ok &= resolve("cuGetErrorString", d.GetErrorString);
  ok &= resolve("cuMemCreate", d.MemCreate);
  ok &= resolve("cuMemRelease", d.MemRelease);
  ok &= resolve("cuMemAddressReserve", d.MemAddressReserve);
  ok &= resolve("cuMemAddressFree", d.MemAddressFree);
  ok &= resolve("cuMemMap", d.MemMap);
  ok &= resolve("cuMemUnmap", d.MemUnmap);
  ok &= resolve("cuMemSetAccess", d.MemSetAccess);
  ok &= resolve("cuMemExportToShareableHandle", d.MemExportToShareableHandle);
  ok &= resolve("cuMemImportFromShareableHandle", d.MemImportFromShareableHandle);
  ok &= resolve("cuMemGetAllocationGranularity", d.MemGetAllocationGranularity);
  ok &= resolve("cuDeviceGetAttribute", d.DeviceGetAttribute);
  ok &= resolve("cuTensorMapEncodeTiled", d.TensorMapEncodeTiled);
  // multicast entry points are optional (older drivers)
  resolve("cuMulticastCreate", d.MulticastCreate);
  resolve("cuMulticastAddDevice", d.MulticastAddDevice);
  resolve("cuMulticastBindMem", d.MulticastBindMem);
  resolve("cuMulticastUnbind", d.MulticastUnbind);
  resolve("cuMulticastGetGranularity", d.MulticastGetGranularity);
  d.ok = ok;
}

const Driver* drv() {
  std::call_once(g_once, load_driver);
  return g_drv.ok ? &g_drv : nullptr;
}

int cu_fail(CUresult r, const char* what) {
  const char* s = nullptr;
  if (g_drv.GetErrorString) g_drv.GetErrorString(r, &s);
  return mep::fail(-1000 - (int)r, "%s failed: %s", what, s ? s : "unknown driver error");
}

#define CU_OK(call, what)                         \
  do {                                            \
    CUresult _r = (call);                         \
    if (_r != CUDA_SUCCESS) return cu_fail(_r, what); \
  } while (0)

CUmemAllocationProp chunk_prop(int device, int fabric) {
  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes =
      fabric ? CU_MEM_HANDLE_TYPE_FABRIC : CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

}  // namespace

namespace mep {
// Used by the GEMM launchers to build TMA descriptors without linking libcuda.
void* driver_tensor_map_encode() {
  const Driver* d = drv();
  return d ? (void*)d->TensorMapEncodeTiled : nullptr;
}
}  // namespace mep

extern "C" {

const int MEP_FABRIC_HANDLE_BYTES = 64;

// 1 when the driver API could be resolved (a GPU driver is present), else 0.
int mep_driver_available() { return drv() != nullptr; }

int mep_device_attr(int device, int attr, int* out) {
  const Driver* d = drv();
  if (!d) return mep::fail(-1, "CUDA driver not available");
  CU_OK(d->DeviceGetAttribute(out, (CUdevice_attribute)attr, device), "cuDeviceGetAttribute");
  return 0;
}

int mep_vmm_supported(int device) {
  int v = 0;
  if (mep_device_attr(device, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, &v) != 0) return 0;
  int fd = 0;
  if (mep_device_attr(device, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, &fd) != 0) return 0;
  return v && fd;
}
// Fabric handles are usable on this device: the attribute is set AND one granule can really be
// created with that handle type (the attribute alone is also set on machines whose fabric
// manager / IMEX channel is not configured, where creation fails).  Same probe as the reference
// (csrc/nvl_shared_buffer.cuh:41-66).  Needs a current context on `device`.
int mep_fabric_supported(int device) {
  const Driver* d = drv();
  if (!d) return 0;
  int v = 0;
  if (mep_device_attr(device, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_FABRIC_SUPPORTED, &v) != 0 || !v) return 0;
  CUmemAllocationProp prop = chunk_prop(device, 1);
  size_t g = 0;
  if (d->MemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0)
    return 0;
  CUmemGenericAllocationHandle h;
  if (d->MemCreate(&h, g, &prop, 0) != CUDA_SUCCESS) return 0;
  d->MemRelease(h);
  return 1;
}
int mep_multicast_supported(int device) {
  const Driver* d = drv();
  if (!d || !d->MulticastCreate) return 0;
  int v = 0;
  if (mep_device_attr(device, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, &v) != 0) return 0;
  return v;
}

// Allocation granularity (bytes) for chunks of the given handle type; <= 0 on failure.
int64_t mep_vmm_granularity(int device, int fabric) {
  const Driver* d = drv();
  if (!d) return mep::fail(-1, "CUDA driver not available");
  CUmemAllocationProp prop = chunk_prop(device, fabric);
  size_t g = 0;
  CUresult r = d->MemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) return cu_fail(r, "cuMemGetAllocationGranularity");
  return (int64_t)g;
}

int64_t mep_multicast_granularity(int device_count, int64_t bytes) {
  const Driver* d = drv();
  if (!d || !d->MulticastGetGranularity) return mep::fail(-1, "multicast API not available");
  CUmulticastObjectProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.numDevices = (unsigned)device_count;
  prop.size = (size_t)bytes;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t g = 0;
  CUresult r = d->MulticastGetGranularity(&g, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) return cu_fail(r, "cuMulticastGetGranularity");
  return (int64_t)g;
}

// Create one physical chunk on `device`.  bytes must be a multiple of the granularity.
int mep_symm_alloc(int device, int64_t bytes, int fabric, uint64_t* handle) {
  const Driver* d = drv();
  if (!d) return mep::fail(-1, "CUDA driver not available");
  CUmemAllocationProp prop = chunk_prop(device, fabric);
  CUmemGenericAllocationHandle h;
  CU_OK(d->MemCreate(&h, (size_t)bytes, &prop, 0), "cuMemCreate");
  *handle = (uint64_t)h;
  return 0;
}

int mep_symm_export_fd(uint64_t handle, int* fd) {
  const Driver* d = drv();
  if (!d) return mep::fail(-1, "CUDA driver not available");
  int out = -1;
  CU_OK(d->MemExportToShareableHandle(&out, (CUmemGenericAllocationHandle)handle,
                                      CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
        "cuMemExportToShareableHandle(fd)");
  *fd = out;
  return 0;
}
int mep_symm_import_fd(int fd, uint64_t* handle) {
  const Driver* d = drv();
  if (!d) return mep::fail(-1, "CUDA driver not available");
  CUmemGenericAllocationHandle h;
  CU_OK(d->MemImportFromShareableHandle(&h, (void*)(uintptr_t)fd,
                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
        "cuMemImportFromShareableHandle(fd)");
  *handle = (uint64_t)h;
  return 0;
}
int mep_symm_export_fabric(uint64_t handle, void* out64) {
  const Driver* d = drv();
  if (!d) return mep::fail(-1, "CUDA driver not available");
  CUmemFabricHandle fh;
  CU_OK(d->MemExportToShareableHandle(&fh, (CUmemGenericAllocationHandle)handle,
                                      CU_MEM_HANDLE_TYPE_FABRIC, 0),
        "cuMemExportToShareableHandle(fabric)");
  std::memcpy(out64, &fh, sizeof(fh));
  return 0;
}
int mep_symm_import_fabric(const void* in64, uint64_t* handle) {
  const Driver* d = drv();
  if (!d) return mep::fail(-1, "CUDA driver not available");
  CUmemFabricHandle fh;
  std::memcpy(&fh, in64, sizeof(fh));
  CUmemGenericAllocationHandle h;
  CU_OK(d->MemImportFromShareableHandle(&h, &fh, CU_MEM_HANDLE_TYPE_FABRIC),
        "cuMemImportFromShareableHandle(fabric)");
  *handle = (uint64_t)h;
  return 0;
}
int mep_symm_release(uint64_t handle) {
  const Driver* d = drv();
  if (!d) return mep::fail(-1, "CUDA driver not available");
  CU_OK(d->MemRelease((CUmemGenericAllocationHandle)handle), "cuMemRelease");
  return 0;
}

// Map n handles of chunk_bytes each back to back into one fresh virtual range that `device`
// can read and write.  On failure everything mapped so far is undone.
int mep_symm_map(int device, const uint64_t* handles, int n, int64_t chunk_bytes, uint64_t* va) {
  const Driver* d = drv();
  if (!d) return mep::fail(-1, "CUDA driver not available");
  const size_t total = (size_t)chunk_bytes * n;
  CUdeviceptr base = 0;
  CU_OK(d->MemAddressReserve(&base, total, 0, 0, 0), "cuMemAddressReserve");
  int mapped = 0;
  CUresult r = CUDA_SUCCESS;
  for (; mapped < n; ++mapped) {
    r = d->MemMap(base + (size_t)mapped * chunk_bytes, (size_t)chunk_bytes, 0,
                  (CUmemGenericAllocationHandle)handles[mapped], 0);
    if (r != CUDA_SUCCESS) break;
  }
  if (r == CUDA_SUCCESS) {
    CUmemAccessDesc acc;
    std::memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = d->MemSetAccess(base, total, &acc, 1);
  }
  if (r != CUDA_SUCCESS) {
    for (int i = 0; i < mapped; ++i) d->MemUnmap(base + (size_t)i * chunk_bytes, (size_t)chunk_bytes);
    d->MemAddressFree(base, total);
    return cu_fail(r, "cuMemMap/cuMemSetAccess");
  }
  *va = (uint64_t)base;
  return 0;
}

int mep_symm_unmap(uint64_t va, int n, int64_t chunk_bytes) {
  const Driver* d = drv();
  if (!d) return mep::fail(-1, "CUDA driver not available");
  const size_t total = (size_t)chunk_bytes * n;
  CU_OK(d->MemUnmap((CUdeviceptr)va, total), "cuMemUnmap");
  CU_OK(d->MemAddressFree((CUdeviceptr)va, total), "cuMemAddressFree");
  return 0;
}

// ---- NVLS multicast overlay -----------------------------------------------------------------
int mep_mc_create(int device_count, int64_t bytes, uint64_t* mc) {
  const Driver* d = drv();
  if (!d || !d->MulticastCreate) return mep::fail(-1, "multicast API not available");
  CUmulticastObjectProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.numDevices = (unsigned)device_count;
  prop.size = (size_t)bytes;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  CU_OK(d->MulticastCreate(&h, &prop), "cuMulticastCreate");
  *mc = (uint64_t)h;
  return 0;
}
int mep_mc_add_device(uint64_t mc, int device) {
  const Driver* d = drv();
  if (!d || !d->MulticastAddDevice) return mep::fail(-1, "multicast API not available");
  CU_OK(d->MulticastAddDevice((CUmemGenericAllocationHandle)mc, device), "cuMulticastAddDevice");
  return 0;
}
// Bind this rank's physical chunk (whole) at offset 0 of the multicast object.
int mep_mc_bind(uint64_t mc, uint64_t mem_handle, int64_t bytes) {
  const Driver* d = drv();
  if (!d || !d->MulticastBindMem) return mep::fail(-1, "multicast API not available");
  CU_OK(d->MulticastBindMem((CUmemGenericAllocationHandle)mc, 0,
                            (CUmemGenericAllocationHandle)mem_handle, 0, (size_t)bytes, 0),
        "cuMulticastBindMem");
  return 0;
}
int mep_mc_unbind(uint64_t mc, int device, int64_t bytes) {
  const Driver* d = drv();
  if (!d || !d->MulticastUnbind) return mep::fail(-1, "multicast API not available");
  CU_OK(d->MulticastUnbind((CUmemGenericAllocationHandle)mc, device, 0, (size_t)bytes),
        "cuMulticastUnbind");
  return 0;
}

}  // extern "C"
