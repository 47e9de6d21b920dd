// CPU backend of the symmetric heap: memfd-backed shared memory mapped at fixed window slots.
#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>

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

  // A stand-in for the NVLink multicast object, so that the runtime's set-up and tear-down of world and team
  // objects (who creates, how the descriptor travels, that every step is agreed on, that one member's failure
  // leaves everybody without a mapping) can run as processes on a machine without a GPU. ROCSHMEM_HOST_FAKE_MULTICAST=1
  // turns it on; ROCSHMEM_HOST_FAKE_MULTICAST_FAIL names a step of this process that fails ("create", "import",
  // "add", "bind"), optionally followed by ":" and the number of the object this process takes part in, counted from
  // 0 (every object when absent). The "object" is a small shared file that counts its members; the mapping is the
  // member's own heap again, so nothing is replicated or reduced.
  bool multicast_supported() const override { return env_on("ROCSHMEM_HOST_FAKE_MULTICAST"); }
  size_t mc_granularity(size_t, int) const override { return multicast_supported() ? granularity() : 0; }

  bool mc_create(size_t bytes, int, MemHandle *out, std::string *why) override {
    if (!multicast_supported()) return unsupported(why);
    const int object = objects_++;
    if (fails("create", object, why)) return false;
    int fd = ::memfd_create("rocshmem_b200_fake_mc", MFD_CLOEXEC);
    if (fd < 0 || ::fcntl(fd, F_SETFL, O_APPEND) != 0) {   // appends: members join concurrently
      if (fd >= 0) ::close(fd);
      *why = "host-shm: memfd for the multicast stand-in failed";
      return false;
    }
    out->opaque = static_cast<uint64_t>(fd) + 1;   // never 0: the runtime treats 0 as "no object"
    out->fd = fd;
    out->bytes = bytes;
    current_ = object;
    return true;
  }

  bool mc_import(int fd, size_t bytes, MemHandle *out, std::string *why) override {
    if (!multicast_supported()) return unsupported(why);
    const int object = objects_++;
    current_ = object;
    if (fails("import", object, why)) return false;
    out->opaque = static_cast<uint64_t>(fd) + 1;
    out->fd = fd;
    out->bytes = bytes;
    out->imported = true;
    return true;
  }

  bool mc_add_device(const MemHandle &mc, std::string *why) override {
    if (fails("add", current_, why)) return false;
    // one byte per member that joined (the file's size is the number of members so far)
    unsigned char one = 1;
    return ::write(mc.fd, &one, 1) == 1;
  }

  bool mc_bind_and_map(const MemHandle &, const MemHandle &mem, char *va, std::string *why) override {
    if (fails("bind", current_, why)) return false;
    void *p = ::mmap(va, mem.bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, static_cast<int>(mem.opaque), 0);
    if (p == MAP_FAILED) {
      *why = "host-shm: mapping for the multicast stand-in failed";
      return false;
    }
    return true;
  }

  void mc_unbind(const MemHandle &, size_t) override {}

 private:
  static bool env_on(const char *name) {
    const char *e = std::getenv(name);
    return e != nullptr && e[0] != '\0' && e[0] != '0';
  }
  bool fails(const char *step, int object, std::string *why) const {
    const char *e = std::getenv("ROCSHMEM_HOST_FAKE_MULTICAST_FAIL");
    if (e == nullptr) return false;
    std::string spec(e);
    std::string want = spec.substr(0, spec.find(':'));
    if (want != step) return false;
    if (spec.find(':') != std::string::npos && std::atoi(spec.c_str() + spec.find(':') + 1) != object) return false;
    if (why) *why = std::string("injected failure of the multicast stand-in at ") + step;
    return true;
  }
  int objects_ = 0;   // objects this process has created or imported so far
  int current_ = -1;  // the one being set up
};

}  // namespace

std::unique_ptr<MemProvider> make_host_shm_provider() { return std::make_unique<HostShmProvider>(); }

}  // namespace rocshmem
