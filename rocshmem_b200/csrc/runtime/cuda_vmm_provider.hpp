// CUDA virtual-memory-management provider, plus the NVLink multicast (NVLS) object that can be
// layered over the same physical allocations.
#pragma once

#include <cuda.h>

#include "mem_provider.hpp"

namespace rocshmem {

// Driver entry points are resolved through the CUDA runtime at first use, so the library carries no
// link-time dependency on libcuda and still loads on a machine without a driver.
struct CudaDriver {
  bool ok = false;
  std::string why;
  CUresult (*MemGetAllocationGranularity)(size_t *, const CUmemAllocationProp *,
                                          CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr,
                                unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *,
                        unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemExportToShareableHandle)(void *, CUmemGenericAllocationHandle,
                                         CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle *, void *,
                                           CUmemAllocationHandleType) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                     unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t) = nullptr;
  CUresult (*DeviceGetAttribute)(int *, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*DeviceGet)(CUdevice *, int) = nullptr;
  CUresult (*GetErrorString)(CUresult, const char **) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle *, const CUmulticastObjectProp *) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle,
                               size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t *, const CUmulticastObjectProp *,
                                      CUmulticastGranularity_flags) = nullptr;
  CUresult (*TensorMapEncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;

  static const CudaDriver &get();
  std::string error(CUresult r) const;
};

class CudaVmmProvider final : public MemProvider {
 public:
  explicit CudaVmmProvider(int device);
  bool is_cuda() const override { return true; }
  const char *name() const override { return "cuda-vmm"; }
  size_t granularity() const override { return granularity_; }
  char *reserve(size_t bytes) override;
  void release(char *va, size_t bytes) override;
  MemHandle create(size_t bytes, bool shareable) override;
  MemHandle import_fd(int fd, size_t bytes) override;
  void map(char *va, const MemHandle &h) override;
  void unmap(char *va, size_t bytes) override;
  void destroy(MemHandle &h) override;
  void write(void *dst, const void *src, size_t bytes) override;
  void read(void *dst, const void *src, size_t bytes) override;
  void zero(void *dst, size_t bytes) override;
  void sync_device() override;
  bool multicast_supported() const override { return multicast_; }

  int device() const { return device_; }

  // NVLS: one multicast object spanning `n_devices` GPUs. The creator exports a descriptor; every
  // participant adds its device, then (after all devices were added) binds its allocation and maps
  // the object. All calls return false with *why set when the platform refuses.
  bool mc_create(size_t bytes, int n_devices, MemHandle *out, std::string *why) override;
  bool mc_import(int fd, size_t bytes, MemHandle *out, std::string *why) override;
  bool mc_add_device(const MemHandle &mc, std::string *why) override;
  bool mc_bind_and_map(const MemHandle &mc, const MemHandle &mem, char *va, std::string *why) override;
  void mc_unbind(const MemHandle &mc, size_t bytes) override;
  size_t mc_granularity(size_t bytes, int n_devices) const override;

 private:
  int device_;
  size_t granularity_ = size_t(2) << 20;
  bool multicast_ = false;
  bool fd_export_ = true;
};

}  // namespace rocshmem
