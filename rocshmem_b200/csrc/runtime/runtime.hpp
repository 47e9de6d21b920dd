// The process-wide runtime: owns the symmetric heap window, the allocator, teams, host contexts,
// the device state blocks and the host-operation engine.
//
// Role of the reference's Backend / IPCBackend singleton (src/backend_bc.hpp:62-298,
// src/ipc/backend_ipc.cpp:56-99): there the backend object is placed in pinned host memory and its
// address is copied into a __constant__ pointer; device code then chases pointers into host
// memory. Here the device receives a flat rocshmem_device_state by value in __constant__ memory of
// every CUDA module (registered through register_module), and everything the device touches at
// run time (team descriptors, context pool, flags, error record, stats) sits in the reserved
// "internal region" at the top of each PE's own heap, reachable on peers by the ordinary symmetric
// translation. The reference keeps a separate, separately-mapped work/sync buffer
// (src/ipc/backend_ipc.cpp:274-357); one mapping serves both here.
//
// One process may host several PEs on one GPU ("local PEs", n_local > 1). That mode exists so the
// multi-PE logic can be exercised on a single GPU: kernels are launched once with
// gridDim.z == n_local (cooperatively, since PEs wait on one another) and blockIdx.z selects the PE.
#pragma once

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "allocator.hpp"
#include "bootstrap.hpp"
#include "config.hpp"
#include "mem_provider.hpp"
#include "rocshmem/rocshmem_common.h"
#include "team.hpp"

namespace rocshmem {

class HostOps;
class Proxy;

struct HostTeam {
  TeamTriplet world;          // members in world numbering
  int slot = 0;               // sync-pool slot
  std::vector<int> my_pe;     // per local PE: index in team, -1 if not a member
  rocshmem_team_dev *dev = nullptr;  // descriptor of local PE 0 (the public handle)
  uint64_t split_seq = 0;     // number of splits performed with this team as parent
  uint64_t barrier_epoch = 0;  // host-side mirror for the CPU backend
  uint64_t id = 0;
  // Processes (bootstrap ranks) that host members, in team order, and my position among them.
  std::vector<int> procs;
  int my_proc = 0;
  // NVLink multicast mapping of my heap that spans exactly this team's members (nullptr: none; the team's
  // collectives then use point-to-point kernels). The world team shares the runtime's mapping (mc_owned false).
  char *mc_window = nullptr;
  MemHandle mc_handle;
  bool mc_owned = false;
};

struct HostCtx {
  int id = 0;
  long long options = 0;
  HostTeam *team = nullptr;
  void *stream = nullptr;     // cudaStream_t on the CUDA backend
  std::atomic<uint64_t> ops{0};
};

// Layout of the internal region (offsets from internal_base, identical on every PE).
struct InternalLayout {
  size_t error = 0, stats = 0, teams = 0, ctxs = 0, ctx_free_mask = 0, barrier_flags = 0,
         lib_flags = 0, lib_state = 0, ll_buf = 0, proxy = 0, host_slots = 0, scratch = 0;
  size_t ll_slot_bytes = 0;   // mailboxes of one team slot: 2 x n_pes x ROCSHMEM_LL_WORDS words
  size_t total = 0;
  // A 256-byte guard filled with a fixed pattern follows every sub-region; a write that runs past the end of a
  // flag or descriptor array lands there and is reported by Runtime::check_canaries().
  std::vector<size_t> guards;
  static constexpr size_t kGuardBytes = 256;
  static constexpr unsigned long long kGuardWord = 0xC0DEC0DEC0DEC0DEull;
  static InternalLayout build(const Config &cfg, int n_pes);
};

using ModuleUploadFn = void (*)(const rocshmem_device_state *states, int n_local);

class Runtime {
 public:
  static Runtime &instance();
  static bool initialized();

  // Collective over all processes of the bootstrap. n_local PEs are hosted by each process.
  void init(std::unique_ptr<Bootstrap> bs, const Config &cfg, int n_local, int device);
  void finalize();
  // Number of guard regions (over all local PEs) whose pattern has been overwritten; 0 in a healthy run.
  int check_canaries();

  // Identity. In multi-PE-per-process mode the "current" local PE is a thread-local selector.
  int n_pes() const { return n_pes_; }
  int n_local() const { return n_local_; }
  int first_pe() const { return first_pe_; }
  int my_pe() const;
  void set_current_local(int l);
  int current_local() const;

  const Config &config() const { return cfg_; }
  MemProvider &mem() { return *mem_; }
  Bootstrap &bootstrap() { return *bs_; }
  HostOps &ops() { return *ops_; }
  bool is_cuda() const { return mem_ && mem_->is_cuda(); }
  int device() const { return device_; }

  // Heap. Collective; returns the address in the current local PE's heap.
  void *malloc(size_t bytes);
  void free(void *ptr);
  size_t heap_used() const { return alloc_ ? alloc_->used() : 0; }
  size_t heap_avail() const { return alloc_ ? alloc_->avail() : 0; }

  // Addressing.
  char *heap_base(int pe) const { return window_ + size_t(pe) * stride_; }
  char *local_heap_base() const { return heap_base(my_pe()); }
  size_t stride() const { return stride_; }
  size_t heap_size() const { return cfg_.heap_size; }
  char *internal_base(int pe) const { return heap_base(pe) + cfg_.heap_size; }
  const InternalLayout &layout() const { return layout_; }
  // Is [p, p+bytes) inside the user heap of some local PE? (pe_out: which)
  bool is_symmetric(const void *p, size_t bytes = 1, int *pe_out = nullptr) const;
  // Address of the same symmetric object on `pe`, given an address valid on any PE of the window.
  void *translate(const void *p, int pe) const;
  char *mc_base() const { return mc_window_; }

  // Teams.
  HostTeam *team_world() { return world_team_; }
  HostTeam *team_from_handle(rocshmem_team_t h);
  // Lock-free lookup for the proxy thread (nullptr: no team owns the slot).
  HostTeam *team_from_slot(int slot) const {
    return slot >= 0 && slot < ROCSHMEM_TEAM_SLOTS ? team_by_slot_[slot].load(std::memory_order_acquire) : nullptr;
  }
  int team_split_strided(HostTeam *parent, int start, int stride, int size, rocshmem_team_t *out);
  void team_destroy(HostTeam *t);
  int num_user_teams() const { return static_cast<int>(teams_.size()) - 1; }

  // Host contexts.
  HostCtx *default_ctx() { return default_ctx_; }
  HostCtx *ctx_create(long long options, HostTeam *team);
  void ctx_destroy(HostCtx *c);

  // Device state blocks (one per local PE) and CUDA modules that hold a copy.
  const rocshmem_device_state *device_states() const { return states_.data(); }
  void register_module(ModuleUploadFn fn);
  void upload_states();

  // Diagnostics.
  rocshmem_error_record read_error(int local = -1);
  void clear_error();
  std::vector<unsigned long long> read_stats(int local = -1);
  void reset_stats();
  std::vector<unsigned long long> host_stats() const;
  void count(int stat_id, unsigned long long n = 1);
  void set_wait_timeout_ms(uint64_t ms);

  Proxy *proxy() { return proxy_.get(); }

  std::recursive_mutex &mutex() { return mu_; }

 private:
  Runtime() = default;
  void setup_nvls();
  void setup_team_nvls(HostTeam *t, const std::string &tag);
  void release_team_nvls(HostTeam *t);
  void write_team_descriptor(HostTeam *t);
  void build_states();

  bool inited_ = false;
  Config cfg_;
  std::unique_ptr<Bootstrap> bs_;
  std::unique_ptr<MemProvider> mem_;
  std::unique_ptr<HostOps> ops_;
  std::unique_ptr<Pow2Allocator> alloc_;
  std::unique_ptr<Proxy> proxy_;
  int device_ = 0;
  int n_pes_ = 0, n_local_ = 1, first_pe_ = 0;
  char *window_ = nullptr;
  char *mc_window_ = nullptr;
  size_t stride_ = 0;
  InternalLayout layout_;
  std::vector<MemHandle> handles_;  // per PE of the window (own + imported)
  MemHandle mc_handle_;
  bool mc_bound_ = false;
  std::vector<rocshmem_device_state> states_;
  std::vector<ModuleUploadFn> modules_;
  std::unique_ptr<TeamSlots> slots_;
  std::vector<std::unique_ptr<HostTeam>> teams_;
  HostTeam *world_team_ = nullptr;
  std::atomic<HostTeam *> team_by_slot_[ROCSHMEM_TEAM_SLOTS] = {};
  std::vector<std::unique_ptr<HostCtx>> ctxs_;
  HostCtx *default_ctx_ = nullptr;
  uint64_t next_team_id_ = 1;
  std::map<std::string, uint64_t> split_counts_;
  std::vector<std::atomic<unsigned long long>> *host_stats_ = nullptr;
  std::recursive_mutex mu_;
};

}  // namespace rocshmem
