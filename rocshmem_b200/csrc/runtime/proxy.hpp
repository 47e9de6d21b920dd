// Reverse-offload proxy: a command ring filled by GPU threads and drained by one host thread.
//
// Kept as a fallback path for operations that cannot (or should not) be performed by the GPU
// itself, in the spirit of the reference's RO backend: device threads write 64-byte descriptors
// into a ring in pinned host memory (src/reverse_offload/queue_proxy.hpp:38-157,
// context_ro_device.cpp:457-664), a host worker polls the ring (backend_ro.cpp:281-294,
// queue.cpp:58-89) and a progress engine executes the commands and notifies the waiting thread
// (mpi_transport.cpp:66-256, 1120-1186). Differences by design:
//   * one ring, one consumer thread; commands are executed with the host-operation engine
//     (stream copies / helper kernels on peer-mapped memory) instead of MPI RMA;
//   * slot hand-over is by the per-slot `valid` word only (0 free, 1 published, 2 executing), so
//     the device never reads a host-side index; a blocking producer releases its own slot after it
//     has read the completion, which keeps the returned value safe from slot reuse;
//   * every wait on either side is bounded, and the consumer has host-side fault-injection hooks
//     (drop or delay commands) so that time-out handling can be tested without touching a GPU.
#pragma once

#include <atomic>
#include <cstdint>
#include <string>
#include <thread>

#include "rocshmem/rocshmem_common.h"

namespace rocshmem {

class Runtime;

class Proxy {
 public:
  explicit Proxy(Runtime *rt);
  ~Proxy();
  void start();
  void stop();
  bool running() const { return running_.load(); }

  // Host-side producer with the same protocol as the device producer (used by the CPU backend and
  // by tests). Returns ROCSHMEM_SUCCESS / ROCSHMEM_ERROR (time-out); *fetched receives the value of
  // a fetching atomic when `blocking`.
  int submit(const rocshmem_proxy_cmd &cmd, bool blocking, uint64_t *fetched, uint64_t timeout_ms);

  // Fault injection (host side only).
  void inject_drop(int n) { drop_.store(n); }
  void inject_delay_ms(int ms) { delay_ms_.store(ms); }

  // Merging of consecutive commands that continue one another (same type and PE, equal sizes, both
  // addresses following on): the consumer executes the run as one transfer. On by ROCSHMEM_USE_WF_COAL.
  void set_coalesce(bool on) { coalesce_.store(on); }
  uint64_t merged() const { return merged_.load(); }

  uint64_t executed() const { return executed_.load(); }
  uint64_t dropped() const { return dropped_count_.load(); }
  const rocshmem_proxy_ring &ring() const { return ring_; }

  // One line of text about a command slot / a completion slot (index taken modulo the array's size), for the
  // debug dump. Reads the ring without taking part in its protocol.
  std::string describe_command(unsigned index) const;
  std::string describe_completion(unsigned index) const;

 private:
  void run();
  void execute(rocshmem_proxy_cmd &cmd, uint64_t seq);
  void retire(volatile rocshmem_proxy_cmd &slot, int status_slot, uint64_t seq);

  Runtime *rt_;
  rocshmem_proxy_ring ring_{};
  void *ring_mem_ = nullptr;
  size_t ring_bytes_ = 0;
  bool pinned_ = false;
  std::thread thread_;
  std::atomic<bool> running_{false};
  std::atomic<bool> stop_{false};
  std::atomic<int> drop_{0};
  std::atomic<int> delay_ms_{0};
  std::atomic<uint64_t> executed_{0};
  std::atomic<uint64_t> dropped_count_{0};
  std::atomic<bool> coalesce_{false};
  std::atomic<uint64_t> merged_{0};       // commands that travelled inside an earlier command
  uint64_t read_ = 0;
  std::atomic<uint64_t> host_write_{0};  // reservation counter of the host-side producer
};

}  // namespace rocshmem
