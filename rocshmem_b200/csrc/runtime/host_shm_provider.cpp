// CPU backend of the symmetric heap: memfd-backed shared memory mapped at fixed window slots.
#include <sys/mman.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

#include "mem_provider.hpp"

namespace rocshmem {

namespace {

class HostShmProvider final : public MemProvider {
 public:
  bool is_cuda() const override { return false; }
  const char *name() const override { return "host-shm"; }
  size_t granularity() const override { return size_t(2) << 20; }

  char *reserve(size_t bytes) override {
    void *p = ::mmap(nullptr, bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (p == MAP_FAILED) throw std::runtime_error("host-shm: cannot reserve address window");
    return static_cast<char *>(p);
  }

  void release(char *va, size_t bytes) override { ::munmap(va, bytes); }

  MemHandle create(size_t bytes, bool) override {
    int fd = ::memfd_create("rocshmem_b200_heap", MFD_CLOEXEC);
    if (fd < 0) throw std::runtime_error("host-shm: memfd_create failed");
    if (::ftruncate(fd, static_cast<off_t>(bytes)) != 0) {
      ::close(fd);
      throw std::runtime_error("host-shm: ftruncate failed (heap too large for this machine?)");
    }
    MemHandle h;
    h.opaque = static_cast<uint64_t>(fd);
    h.fd = fd;
    h.bytes = bytes;
    return h;
  }

  MemHandle import_fd(int fd, size_t bytes) override {
    MemHandle h;
    h.opaque = static_cast<uint64_t>(fd);
    h.fd = fd;
    h.bytes = bytes;
    h.imported = true;
    return h;
  }

  void map(char *va, const MemHandle &h) override {
    void *p = ::mmap(va, h.bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED,
                     static_cast<int>(h.opaque), 0);
    if (p == MAP_FAILED) throw std::runtime_error("host-shm: mmap of a heap failed");
  }

  void unmap(char *va, size_t bytes) override {
    // Put the reservation back so the window stays contiguous until release().
    ::mmap(va, bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);
  }

  void destroy(MemHandle &h) override {
    if (h.fd >= 0) ::close(h.fd);
    h.fd = -1;
    h.opaque = 0;
  }

  void write(void *dst, const void *src, size_t bytes) override { std::memcpy(dst, src, bytes); }
  void read(void *dst, const void *src, size_t bytes) override { std::memcpy(dst, src, bytes); }
  void zero(void *dst, size_t bytes) override { std::memset(dst, 0, bytes); }
};

}  // namespace

std::unique_ptr<MemProvider> make_host_shm_provider() { return std::make_unique<HostShmProvider>(); }

}  // namespace rocshmem
