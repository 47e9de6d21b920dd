#include "cuda_vmm_provider.hpp"

#include <cuda_runtime_api.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

namespace rocshmem {

namespace {

template <typename Fn>
bool resolve(const char *name, Fn *out, std::string *why) {
  void *p = nullptr;
  cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
    cudaGetLastError();
    if (why && why->empty()) *why = std::string("driver entry point not available: ") + name;
    return false;
  }
  *out = reinterpret_cast<Fn>(p);
  return true;
}

void check_rt(cudaError_t e, const char *what) {
  if (e != cudaSuccess) {
    throw std::runtime_error(std::string("cuda-vmm: ") + what + ": " + cudaGetErrorString(e));
  }
}

}  // namespace

const CudaDriver &CudaDriver::get() {
  static CudaDriver d = [] {
    CudaDriver r;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
      cudaGetLastError();
      r.why = "no CUDA device or driver";
      return r;
    }
    bool ok = true;
    ok &= resolve("cuMemGetAllocationGranularity", &r.MemGetAllocationGranularity, &r.why);
    ok &= resolve("cuMemAddressReserve", &r.MemAddressReserve, &r.why);
    ok &= resolve("cuMemAddressFree", &r.MemAddressFree, &r.why);
    ok &= resolve("cuMemCreate", &r.MemCreate, &r.why);
    ok &= resolve("cuMemRelease", &r.MemRelease, &r.why);
    ok &= resolve("cuMemExportToShareableHandle", &r.MemExportToShareableHandle, &r.why);
    ok &= resolve("cuMemImportFromShareableHandle", &r.MemImportFromShareableHandle, &r.why);
    ok &= resolve("cuMemMap", &r.MemMap, &r.why);
    ok &= resolve("cuMemUnmap", &r.MemUnmap, &r.why);
    ok &= resolve("cuMemSetAccess", &r.MemSetAccess, &r.why);
    ok &= resolve("cuDeviceGetAttribute", &r.DeviceGetAttribute, &r.why);
    ok &= resolve("cuDeviceGet", &r.DeviceGet, &r.why);
    ok &= resolve("cuGetErrorString", &r.GetErrorString, &r.why);
    // Optional groups: absence only disables the feature that needs them.
    std::string ignore;
    resolve("cuMulticastCreate", &r.MulticastCreate, &ignore);
    resolve("cuMulticastAddDevice", &r.MulticastAddDevice, &ignore);
    resolve("cuMulticastBindMem", &r.MulticastBindMem, &ignore);
    resolve("cuMulticastUnbind", &r.MulticastUnbind, &ignore);
    resolve("cuMulticastGetGranularity", &r.MulticastGetGranularity, &ignore);
    resolve("cuTensorMapEncodeTiled", &r.TensorMapEncodeTiled, &ignore);
    r.ok = ok;
    return r;
  }();
  return d;
}

std::string CudaDriver::error(CUresult r) const {
  const char *s = nullptr;
  if (GetErrorString && GetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "CUresult " + std::to_string(static_cast<int>(r));
}

#define DRV_CHECK(call, what)                                                         \
  do {                                                                                \
    CUresult _r = (call);                                                             \
    if (_r != CUDA_SUCCESS) {                                                         \
      throw std::runtime_error(std::string("cuda-vmm: ") + what + ": " + drv.error(_r)); \
    }                                                                                 \
  } while (0)

int cuda_device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

static CUmemAllocationProp alloc_prop(int device, bool shareable) {
  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes =
      shareable ? CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR : CU_MEM_HANDLE_TYPE_NONE;
  return prop;
}

CudaVmmProvider::CudaVmmProvider(int device) : device_(device) {
  const CudaDriver &drv = CudaDriver::get();
  if (!drv.ok) throw std::runtime_error("cuda-vmm: " + drv.why);
  check_rt(cudaSetDevice(device), "cudaSetDevice");
  check_rt(cudaFree(nullptr), "context creation");
  CUdevice dev;
  DRV_CHECK(drv.DeviceGet(&dev, device), "cuDeviceGet");
  int vmm = 0, fd_ok = 0, mc = 0;
  drv.DeviceGetAttribute(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev);
  if (!vmm) throw std::runtime_error("cuda-vmm: device lacks virtual memory management");
  drv.DeviceGetAttribute(&fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
  fd_export_ = fd_ok != 0;
  drv.DeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
  multicast_ = mc != 0 && drv.MulticastCreate && drv.MulticastAddDevice && drv.MulticastBindMem &&
               drv.MulticastGetGranularity;
  CUmemAllocationProp prop = alloc_prop(device, fd_export_);
  size_t g = 0;
  DRV_CHECK(drv.MemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
            "cuMemGetAllocationGranularity");
  if (g) granularity_ = g;
}

char *CudaVmmProvider::reserve(size_t bytes) {
  const CudaDriver &drv = CudaDriver::get();
  CUdeviceptr p = 0;
  DRV_CHECK(drv.MemAddressReserve(&p, bytes, granularity_, 0, 0), "cuMemAddressReserve");
  return reinterpret_cast<char *>(p);
}

void CudaVmmProvider::release(char *va, size_t bytes) {
  const CudaDriver &drv = CudaDriver::get();
  drv.MemAddressFree(reinterpret_cast<CUdeviceptr>(va), bytes);
}

MemHandle CudaVmmProvider::create(size_t bytes, bool shareable) {
  const CudaDriver &drv = CudaDriver::get();
  if (shareable && !fd_export_) {
    throw std::runtime_error("cuda-vmm: POSIX file-descriptor export is not supported here");
  }
  CUmemAllocationProp prop = alloc_prop(device_, shareable);
  CUmemGenericAllocationHandle h = 0;
  DRV_CHECK(drv.MemCreate(&h, bytes, &prop, 0), "cuMemCreate (symmetric heap)");
  MemHandle out;
  out.opaque = static_cast<uint64_t>(h);
  out.bytes = bytes;
  if (shareable) {
    int fd = -1;
    CUresult r = drv.MemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) {
      drv.MemRelease(h);
      throw std::runtime_error("cuda-vmm: cuMemExportToShareableHandle: " + drv.error(r));
    }
    out.fd = fd;
  }
  return out;
}

MemHandle CudaVmmProvider::import_fd(int fd, size_t bytes) {
  const CudaDriver &drv = CudaDriver::get();
  CUmemGenericAllocationHandle h = 0;
  DRV_CHECK(drv.MemImportFromShareableHandle(&h, reinterpret_cast<void *>(static_cast<uintptr_t>(fd)),
                                             CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
            "cuMemImportFromShareableHandle");
  MemHandle out;
  out.opaque = static_cast<uint64_t>(h);
  out.fd = fd;
  out.bytes = bytes;
  out.imported = true;
  return out;
}

void CudaVmmProvider::map(char *va, const MemHandle &h) {
  const CudaDriver &drv = CudaDriver::get();
  CUdeviceptr p = reinterpret_cast<CUdeviceptr>(va);
  DRV_CHECK(drv.MemMap(p, h.bytes, 0, static_cast<CUmemGenericAllocationHandle>(h.opaque), 0),
            "cuMemMap");
  CUmemAccessDesc acc;
  std::memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device_;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CUresult r = drv.MemSetAccess(p, h.bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    drv.MemUnmap(p, h.bytes);
    throw std::runtime_error("cuda-vmm: cuMemSetAccess (is peer access possible between the GPUs?): " +
                             drv.error(r));
  }
}

void CudaVmmProvider::unmap(char *va, size_t bytes) {
  const CudaDriver &drv = CudaDriver::get();
  drv.MemUnmap(reinterpret_cast<CUdeviceptr>(va), bytes);
}

void CudaVmmProvider::destroy(MemHandle &h) {
  const CudaDriver &drv = CudaDriver::get();
  if (h.opaque) drv.MemRelease(static_cast<CUmemGenericAllocationHandle>(h.opaque));
  if (h.fd >= 0) ::close(h.fd);
  h.opaque = 0;
  h.fd = -1;
}

namespace {
// The copies below may be the first CUDA call of a user thread, whose current device is 0 by default.
struct OnDevice {
  int prev = -1;
  explicit OnDevice(int want) {
    int cur = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cur != want && cudaSetDevice(want) == cudaSuccess) prev = cur;
  }
  ~OnDevice() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};
}  // namespace

void CudaVmmProvider::write(void *dst, const void *src, size_t bytes) {
  OnDevice on(device_);
  check_rt(cudaMemcpy(dst, src, bytes, cudaMemcpyDefault), "cudaMemcpy to heap");
}

void CudaVmmProvider::read(void *dst, const void *src, size_t bytes) {
  OnDevice on(device_);
  check_rt(cudaMemcpy(dst, src, bytes, cudaMemcpyDefault), "cudaMemcpy from heap");
}

void CudaVmmProvider::sync_device() {
  OnDevice on(device_);
  check_rt(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
}

void CudaVmmProvider::zero(void *dst, size_t bytes) {
  OnDevice on(device_);
  check_rt(cudaMemset(dst, 0, bytes), "cudaMemset");
  check_rt(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
}

// ------------------------------------------------------------------------------------------------
// NVLS multicast
// ------------------------------------------------------------------------------------------------

static CUmulticastObjectProp mc_prop(size_t bytes, int n_devices) {
  CUmulticastObjectProp p;
  std::memset(&p, 0, sizeof(p));
  p.numDevices = static_cast<unsigned int>(n_devices);
  p.size = bytes;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  p.flags = 0;
  return p;
}

size_t CudaVmmProvider::mc_granularity(size_t bytes, int n_devices) const {
  const CudaDriver &drv = CudaDriver::get();
  if (!multicast_) return 0;
  CUmulticastObjectProp p = mc_prop(bytes, n_devices);
  size_t g = 0;
  // The minimum granularity is what bind offsets and sizes must respect; the recommended one can be
  // hundreds of MiB and would bloat every heap.
  if (drv.MulticastGetGranularity(&g, &p, CU_MULTICAST_GRANULARITY_MINIMUM) != CUDA_SUCCESS) return 0;
  return g;
}

bool CudaVmmProvider::mc_create(size_t bytes, int n_devices, MemHandle *out, std::string *why) {
  const CudaDriver &drv = CudaDriver::get();
  if (!multicast_) {
    *why = "multicast not supported by device or driver";
    return false;
  }
  CUmulticastObjectProp p = mc_prop(bytes, n_devices);
  CUmemGenericAllocationHandle h = 0;
  CUresult r = drv.MulticastCreate(&h, &p);
  if (r != CUDA_SUCCESS) {
    *why = "cuMulticastCreate: " + drv.error(r);
    return false;
  }
  int fd = -1;
  r = drv.MemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    drv.MemRelease(h);
    *why = "export of multicast object: " + drv.error(r);
    return false;
  }
  out->opaque = static_cast<uint64_t>(h);
  out->fd = fd;
  out->bytes = bytes;
  return true;
}

bool CudaVmmProvider::mc_import(int fd, size_t bytes, MemHandle *out, std::string *why) {
  const CudaDriver &drv = CudaDriver::get();
  CUmemGenericAllocationHandle h = 0;
  CUresult r = drv.MemImportFromShareableHandle(
      &h, reinterpret_cast<void *>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) {
    *why = "import of multicast object: " + drv.error(r);
    return false;
  }
  out->opaque = static_cast<uint64_t>(h);
  out->fd = fd;
  out->bytes = bytes;
  out->imported = true;
  return true;
}

bool CudaVmmProvider::mc_add_device(const MemHandle &mc, std::string *why) {
  const CudaDriver &drv = CudaDriver::get();
  CUdevice dev;
  if (drv.DeviceGet(&dev, device_) != CUDA_SUCCESS) {
    *why = "cuDeviceGet";
    return false;
  }
  CUresult r = drv.MulticastAddDevice(static_cast<CUmemGenericAllocationHandle>(mc.opaque), dev);
  if (r != CUDA_SUCCESS) {
    *why = "cuMulticastAddDevice: " + drv.error(r);
    return false;
  }
  return true;
}

bool CudaVmmProvider::mc_bind_and_map(const MemHandle &mc, const MemHandle &mem, char *va,
                                      std::string *why) {
  const CudaDriver &drv = CudaDriver::get();
  auto mch = static_cast<CUmemGenericAllocationHandle>(mc.opaque);
  CUresult r = drv.MulticastBindMem(mch, 0, static_cast<CUmemGenericAllocationHandle>(mem.opaque), 0,
                                    mem.bytes, 0);
  if (r != CUDA_SUCCESS) {
    *why = "cuMulticastBindMem: " + drv.error(r);
    return false;
  }
  CUdeviceptr p = reinterpret_cast<CUdeviceptr>(va);
  r = drv.MemMap(p, mem.bytes, 0, mch, 0);
  if (r != CUDA_SUCCESS) {
    *why = "cuMemMap of multicast object: " + drv.error(r);
    return false;
  }
  CUmemAccessDesc acc;
  std::memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device_;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = drv.MemSetAccess(p, mem.bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    drv.MemUnmap(p, mem.bytes);
    *why = "cuMemSetAccess of multicast mapping: " + drv.error(r);
    return false;
  }
  return true;
}

void CudaVmmProvider::mc_unbind(const MemHandle &mc, size_t bytes) {
  const CudaDriver &drv = CudaDriver::get();
  CUdevice dev;
  if (drv.DeviceGet(&dev, device_) != CUDA_SUCCESS || !drv.MulticastUnbind) return;
  drv.MulticastUnbind(static_cast<CUmemGenericAllocationHandle>(mc.opaque), dev, 0, bytes);
}

std::unique_ptr<MemProvider> make_cuda_vmm_provider(int device, std::string *why) {
  try {
    return std::make_unique<CudaVmmProvider>(device);
  } catch (const std::exception &e) {
    if (why) *why = e.what();
    return nullptr;
  }
}

}  // namespace rocshmem
