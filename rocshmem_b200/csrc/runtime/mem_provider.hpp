// Memory providers: where the symmetric heap physically lives and how a peer's heap becomes
// addressable.
//
// The reference owns one hipMalloc'd (or managed / host / fine-grained) allocation per PE
// (src/memory/heap_memory.hpp:40-129, src/memory/heap_type.hpp:41-51) and maps peers with
// hipIpcGetMemHandle / hipIpcOpenMemHandle into unrelated addresses that it keeps in a table
// (src/ipc_policy.cpp:34-118). Here a provider reserves ONE virtual window of n_pes * stride bytes
// and maps PE p's allocation at window + p * stride, so a remote address is
// local + (pe - my_pe) * stride with no table lookup:
//   * CudaVmmProvider: cuMemCreate physical allocations exported as POSIX file descriptors,
//     cuMemImportFromShareableHandle + cuMemMap + cuMemSetAccess on the importing side. Optionally
//     binds the allocations to an NVLink multicast object (NVLS) mapped at a second window.
//   * HostShmProvider: memfd + mmap(MAP_SHARED | MAP_FIXED). It plays the role of the reference's
//     USE_HOST_HEAP build and lets the whole host runtime run, multi-process, on a machine with no
//     GPU.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace rocshmem {

struct MemHandle {
  uint64_t opaque = 0;  // CUmemGenericAllocationHandle, or the memfd for host memory
  int fd = -1;          // shareable descriptor (owned; -1 once closed or if never exported)
  size_t bytes = 0;
  bool imported = false;
};

class MemProvider {
 public:
  virtual ~MemProvider() = default;
  virtual bool is_cuda() const = 0;
  virtual const char *name() const = 0;
  virtual size_t granularity() const = 0;

  virtual char *reserve(size_t bytes) = 0;
  virtual void release(char *va, size_t bytes) = 0;
  // `shareable`: the handle will be exported to other processes.
  virtual MemHandle create(size_t bytes, bool shareable) = 0;
  virtual MemHandle import_fd(int fd, size_t bytes) = 0;
  virtual void map(char *va, const MemHandle &h) = 0;
  virtual void unmap(char *va, size_t bytes) = 0;
  virtual void destroy(MemHandle &h) = 0;

  // Host access to mapped memory (device memory is not CPU-addressable).
  virtual void write(void *dst, const void *src, size_t bytes) = 0;
  virtual void read(void *dst, const void *src, size_t bytes) = 0;
  virtual void zero(void *dst, size_t bytes) = 0;
  // Returns when all work queued on the provider's device so far has finished (nothing to wait for on the host).
  virtual void sync_device() {}

  // NVLS: one multicast object spanning `n_devices` members. The creator exports a descriptor; every participant
  // adds its device, then (after all devices were added) binds its allocation and maps the object at `va`. The
  // calls return false (with *why set) when the platform refuses or has no such thing; they never throw for "not
  // available". The host provider offers a stand-in for tests (see host_shm_provider.cpp).
  virtual bool multicast_supported() const { return false; }
  virtual size_t mc_granularity(size_t, int) const { return 0; }
  virtual bool mc_create(size_t, int, MemHandle *, std::string *why) { return unsupported(why); }
  virtual bool mc_import(int, size_t, MemHandle *, std::string *why) { return unsupported(why); }
  virtual bool mc_add_device(const MemHandle &, std::string *why) { return unsupported(why); }
  virtual bool mc_bind_and_map(const MemHandle &, const MemHandle &, char *, std::string *why) { return unsupported(why); }
  virtual void mc_unbind(const MemHandle &, size_t) {}

 protected:
  static bool unsupported(std::string *why) {
    if (why) *why = "multicast not supported by this memory provider";
    return false;
  }
};

std::unique_ptr<MemProvider> make_host_shm_provider();
// Returns nullptr (and sets *why) when no CUDA device / driver is usable.
std::unique_ptr<MemProvider> make_cuda_vmm_provider(int device, std::string *why);

// Number of CUDA devices visible to this process, 0 when CUDA is unusable.
int cuda_device_count();

}  // namespace rocshmem
