// Runtime configuration: every ROCSHMEM_* environment variable is parsed once, validated, and kept
// in one struct that the runtime mirrors into the device state block.
//
// Reference behaviour being reproduced (names and defaults): ROCSHMEM_HEAP_SIZE, default 1 GiB
// (src/memory/single_heap.cpp:29-37, src/memory/heap_memory.hpp:114), ROCSHMEM_MAX_NUM_CONTEXTS
// 1024 (src/ipc/backend_ipc.cpp:60-63), ROCSHMEM_MAX_NUM_HOST_CONTEXTS 40 (src/host/host.cpp:105),
// ROCSHMEM_MAX_NUM_TEAMS 40 (src/team_tracker.cpp:31), RO_NET_CPU_QUEUE
// (src/reverse_offload/queue.cpp:31). The reference reads them ad hoc with getenv/atoi and no
// validation; here sizes accept K/M/G/T suffixes and bad values raise an error at init.
#pragma once

#include <cstddef>
#include <cstdint>
#include <map>
#include <string>

namespace rocshmem {

struct Config {
  size_t heap_size = size_t(1) << 30;        // ROCSHMEM_HEAP_SIZE
  size_t scratch_size = size_t(64) << 20;    // ROCSHMEM_SCRATCH_SIZE (library-collective staging)
  size_t slab_size = size_t(1) << 20;        // ROCSHMEM_SLAB_SIZE (default size of rocshmemx_slab_create)
  int max_contexts = 1024;                   // ROCSHMEM_MAX_NUM_CONTEXTS
  int max_host_contexts = 40;                // ROCSHMEM_MAX_NUM_HOST_CONTEXTS
  int max_teams = 40;                        // ROCSHMEM_MAX_NUM_TEAMS
  uint64_t wait_timeout_ms = 10000;          // ROCSHMEM_WAIT_TIMEOUT_MS (0 is rejected)
  int debug = 0;                             // ROCSHMEM_DEBUG (0 quiet, 1 info, 2 trace)
  int debug_checks = 0;                      // ROCSHMEM_DEBUG_CHECKS (device-side pe/address checks)
  int use_proxy = 0;                         // ROCSHMEM_USE_PROXY (host-thread reverse offload)
  int proxy_queue_size = 512;                // RO_NET_QUEUE_SIZE (entries, power of two)
  int proxy_on_cpu = 1;                      // RO_NET_CPU_QUEUE (ring in pinned host memory)
  int proxy_collectives = 0;                 // ROCSHMEM_PROXY_COLLECTIVES (device collectives run by the proxy)
  int proxy_coalesce = 0;                    // ROCSHMEM_USE_WF_COAL (merge contiguous proxied messages)
  int enable_nvls = 1;                       // ROCSHMEM_ENABLE_NVLS (try multicast mapping)
  int team_nvls = 1;                         // ROCSHMEM_TEAM_NVLS (a multicast object per split team)
  std::string backend = "auto";              // ROCSHMEM_BACKEND: auto | cuda | host
  std::string bootstrap_dir;                 // ROCSHMEM_BOOTSTRAP_DIR (native file rendezvous)

  // Parse from the process environment; `overrides` (same keys as the env vars) win.
  static Config from_env(const std::map<std::string, std::string> &overrides = {});
  // Throws std::invalid_argument describing the first bad value.
  void validate() const;
};

// "64M" -> 67108864. Accepts decimal or 0x-hex digits and an optional K/M/G/T (binary) suffix.
// Throws std::invalid_argument on malformed text or overflow.
size_t parse_size(const std::string &text);
long parse_int(const std::string &text);

}  // namespace rocshmem
