#include "runtime.hpp"

#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

#include "cuda_vmm_provider.hpp"
#include "host_ops.hpp"
#include "proxy.hpp"

namespace rocshmem {

namespace {
thread_local int t_current_local = 0;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

std::vector<ModuleUploadFn> &pending_modules() {
  static std::vector<ModuleUploadFn> v;
  return v;
}
std::mutex &module_mutex() {
  static std::mutex m;
  return m;
}
}  // namespace

InternalLayout InternalLayout::build(const Config &cfg, int n_pes) {
  InternalLayout l;
  size_t off = 0;
  auto take = [&off, &l](size_t bytes) {
    size_t at = off;
    off = align_up(off + bytes, 256);
    l.guards.push_back(off);
    off += kGuardBytes;
    return at;
  };
  l.error = take(sizeof(rocshmem_error_record));
  l.stats = take(sizeof(unsigned long long) * ROCSHMEM_NUM_STATS);
  l.teams = take(sizeof(rocshmem_team_dev) * ROCSHMEM_TEAM_SLOTS);
  l.ctxs = take(sizeof(rocshmem_ctx_dev) * size_t(cfg.max_contexts));
  l.ctx_free_mask = take(sizeof(unsigned long long) * (ROCSHMEM_CTX_SLOTS / 64));
  l.barrier_flags = take(sizeof(unsigned long long) * ROCSHMEM_TEAM_SLOTS * ROCSHMEM_MAX_PES);
  l.lib_flags = take(sizeof(unsigned long long) * ROCSHMEM_LIB_FLAG_WORDS);
  l.lib_state = take(sizeof(unsigned long long) * ROCSHMEM_LIB_STATE_WORDS);
  l.ll_slot_bytes = sizeof(unsigned long long) * 2 * size_t(n_pes) * ROCSHMEM_LL_WORDS;
  l.ll_buf = take(l.ll_slot_bytes * ROCSHMEM_TEAM_SLOTS);
  l.proxy = take(sizeof(rocshmem_proxy_ring) + 256);
  l.host_slots = take(4096);
  off = align_up(off, 4096);
  l.scratch = take(cfg.scratch_size);
  l.total = off;
  return l;
}

Runtime &Runtime::instance() {
  static Runtime *r = new Runtime();  // intentionally leaked: outlives static destructors
  return *r;
}

bool Runtime::initialized() { return instance().inited_; }

int Runtime::my_pe() const { return first_pe_ + current_local(); }

void Runtime::set_current_local(int l) {
  if (l < 0 || l >= n_local_) throw std::out_of_range("rocshmem: local PE index out of range");
  t_current_local = l;
}

int Runtime::current_local() const { return t_current_local < n_local_ ? t_current_local : 0; }

void Runtime::register_module(ModuleUploadFn fn) {
  std::lock_guard<std::mutex> g(module_mutex());
  pending_modules().push_back(fn);
  if (inited_ && is_cuda()) fn(states_.data(), n_local_);
}

void Runtime::upload_states() {
  if (!is_cuda()) return;
  std::lock_guard<std::mutex> g(module_mutex());
  for (ModuleUploadFn fn : pending_modules()) fn(states_.data(), n_local_);
}

void Runtime::init(std::unique_ptr<Bootstrap> bs, const Config &cfg, int n_local, int device) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  if (inited_) throw std::runtime_error("rocshmem_init: already initialised");
  if (n_local < 1 || n_local > ROCSHMEM_MAX_LOCAL_PES) {
    throw std::invalid_argument("rocshmem_init: local PE count must be in [1, 8]");
  }
  cfg.validate();
  cfg_ = cfg;
  bs_ = std::move(bs);
  n_local_ = n_local;
  n_pes_ = bs_->size() * n_local;
  first_pe_ = bs_->rank() * n_local;
  device_ = device;
  t_current_local = 0;
  if (cfg_.use_proxy) {
    // A kernel that waits for the proxy must never share a hardware work queue with the kernels the proxy launches
    // for it: streams beyond the number of queues (8 by default) are multiplexed, and work queued behind the
    // waiting kernel would start only when it ends. Takes effect when no CUDA context exists yet in this process;
    // a value the user has set is kept.
    ::setenv("CUDA_DEVICE_MAX_CONNECTIONS", "32", 0);
  }
  if (n_pes_ > ROCSHMEM_MAX_PES) throw std::invalid_argument("rocshmem_init: more than 64 PEs");

  // Backend selection.
  std::string why;
  if (cfg_.backend != "host") {
    mem_ = make_cuda_vmm_provider(device, &why);
    if (!mem_ && cfg_.backend == "cuda") {
      throw std::runtime_error("rocshmem_init: CUDA backend requested but unusable: " + why);
    }
  }
  if (!mem_) mem_ = make_host_shm_provider();
  if (cfg_.debug) {
    std::fprintf(stderr, "[rocshmem pe %d] backend %s, %d PEs (%d per process), heap %zu bytes\n",
                 first_pe_, mem_->name(), n_pes_, n_local_, cfg_.heap_size);
  }

  layout_ = InternalLayout::build(cfg_, n_pes_);
  size_t gran = mem_->granularity();
  if (mem_->is_cuda() && cfg_.enable_nvls && bs_->size() > 1 && n_local_ == 1) {
    // A heap that is to be bound to an NVLink multicast object must be a multiple of the multicast
    // granularity as well.
    auto *cu = dynamic_cast<CudaVmmProvider *>(mem_.get());
    size_t mg = cu ? cu->mc_granularity(align_up(cfg_.heap_size + layout_.total, gran), n_pes_) : 0;
    if (mg > gran && mg % gran == 0) gran = mg;
  }
  stride_ = align_up(cfg_.heap_size + layout_.total, gran);
  // All processes must agree on the stride (same configuration).
  {
    std::vector<uint64_t> all(bs_->size());
    uint64_t mine = stride_;
    bs_->allgather("stride", &mine, all.data(), sizeof(mine));
    for (uint64_t s : all) {
      if (s != stride_) throw std::runtime_error("rocshmem_init: PEs disagree on heap size");
    }
  }
  window_ = mem_->reserve(stride_ * size_t(n_pes_));
  handles_.assign(n_pes_, MemHandle{});
  const bool multi_process = bs_->size() > 1;
  for (int l = 0; l < n_local_; ++l) {
    int pe = first_pe_ + l;
    handles_[pe] = mem_->create(stride_, multi_process);
    mem_->map(heap_base(pe), handles_[pe]);
    mem_->zero(internal_base(pe), layout_.total);
    std::vector<unsigned long long> pattern(InternalLayout::kGuardBytes / sizeof(unsigned long long),
                                            InternalLayout::kGuardWord);
    for (size_t g : layout_.guards) mem_->write(internal_base(pe) + g, pattern.data(), InternalLayout::kGuardBytes);
  }
  if (multi_process) {
    for (int l = 0; l < n_local_; ++l) {
      std::vector<int> fds = exchange_fds(*bs_, "heap" + std::to_string(l), handles_[first_pe_ + l].fd);
      for (int r = 0; r < bs_->size(); ++r) {
        if (r == bs_->rank()) {
          ::close(fds[r]);
          continue;
        }
        int pe = r * n_local_ + l;
        handles_[pe] = mem_->import_fd(fds[r], stride_);
        mem_->map(heap_base(pe), handles_[pe]);
      }
    }
  }

  alloc_ = std::make_unique<Pow2Allocator>(cfg_.heap_size, ROCSHMEM_ALIGNMENT);
  slots_ = std::make_unique<TeamSlots>(cfg_.max_teams);
  host_stats_ = new std::vector<std::atomic<unsigned long long>>(ROCSHMEM_NUM_STATS);

  if ((mem_->is_cuda() || mem_->multicast_supported()) && cfg_.enable_nvls && multi_process && n_local_ == 1) setup_nvls();

  build_states();

  // TEAM_WORLD occupies slot 0.
  auto world = std::make_unique<HostTeam>();
  world->world = TeamTriplet{0, 1, n_pes_};
  world->slot = 0;
  slots_->take(0);
  world->my_pe.resize(n_local_);
  for (int l = 0; l < n_local_; ++l) world->my_pe[l] = first_pe_ + l;
  world->id = 0;
  world->mc_window = mc_window_;
  for (int r = 0; r < bs_->size(); ++r) world->procs.push_back(r);
  world->my_proc = bs_->rank();
  world_team_ = world.get();
  teams_.push_back(std::move(world));
  team_by_slot_[0].store(teams_.back().get(), std::memory_order_release);
  write_team_descriptor(world_team_);

  // Device context pool: all free.
  {
    std::vector<unsigned long long> mask(ROCSHMEM_CTX_SLOTS / 64, 0ull);
    for (int i = 0; i < cfg_.max_contexts; ++i) mask[i / 64] |= 1ull << (i % 64);
    for (int l = 0; l < n_local_; ++l) {
      mem_->write(internal_base(first_pe_ + l) + layout_.ctx_free_mask, mask.data(),
                  mask.size() * sizeof(unsigned long long));
    }
  }

  ops_.reset(mem_->is_cuda() ? make_cuda_host_ops(this) : make_cpu_host_ops(this));
  auto dctx = std::make_unique<HostCtx>();
  dctx->id = 0;
  dctx->team = world_team_;
  default_ctx_ = dctx.get();
  ops_->ctx_init(default_ctx_);
  ctxs_.push_back(std::move(dctx));

  if (cfg_.use_proxy && mem_->is_cuda()) {
    proxy_ = std::make_unique<Proxy>(this);
    proxy_->start();
    build_states();
  }

  inited_ = true;
  upload_states();
  // Nobody may touch a peer's heap before that peer has zeroed its internal region.
  bs_->barrier("init-done");
}

void Runtime::setup_nvls() {
  MemProvider *cu = mem_.get();
  if (!cu->multicast_supported()) {
    if (cfg_.debug) std::fprintf(stderr, "[rocshmem pe %d] NVLS: not supported, P2P only\n", first_pe_);
    return;
  }
  // Every step is agreed on by all ranks before the next one: a rank that fails reports 0 and
  // everybody falls back to plain peer mappings together.
  auto all_ok = [this](const char *tag, bool ok) {
    std::vector<int> flags(bs_->size());
    int mine = ok ? 1 : 0;
    bs_->allgather(tag, &mine, flags.data(), sizeof(int));
    return std::all_of(flags.begin(), flags.end(), [](int f) { return f == 1; });
  };
  std::string why;
  bool ok = true;
  size_t g = cu->mc_granularity(stride_, n_pes_);
  ok = g != 0 && stride_ % g == 0;
  if (cfg_.debug) std::fprintf(stderr, "[rocshmem pe %d] NVLS: granularity %zu, stride %zu\n", first_pe_, g, stride_);
  if (!all_ok("nvls-gran", ok)) return;
  MemHandle mc;
  if (bs_->rank() == 0) ok = cu->mc_create(stride_, n_pes_, &mc, &why);
  if (!all_ok("nvls-create", ok)) {
    if (bs_->rank() == 0 && mc.opaque) cu->destroy(mc);
    if (cfg_.debug) std::fprintf(stderr, "[rocshmem] NVLS unavailable: %s\n", why.c_str());
    return;
  }
  // Rank 0's descriptor goes to everybody (the other ranks pass a placeholder descriptor).
  int placeholder = bs_->rank() == 0 ? mc.fd : ::dup(0);
  std::vector<int> fds = exchange_fds(*bs_, "nvls", placeholder);
  if (bs_->rank() != 0) {
    ::close(placeholder);
    ok = cu->mc_import(fds[0], stride_, &mc, &why);
    fds[0] = -1;
  }
  for (int f : fds)
    if (f >= 0) ::close(f);
  if (!all_ok("nvls-import", ok)) return;
  ok = cu->mc_add_device(mc, &why);
  if (!all_ok("nvls-add", ok)) return;  // all devices are added before anyone binds
  char *va = nullptr;
  try {
    va = cu->reserve(stride_);
  } catch (...) {
    ok = false;
  }
  if (ok) ok = cu->mc_bind_and_map(mc, handles_[first_pe_], va, &why);
  if (!all_ok("nvls-bind", ok)) {
    if (cfg_.debug) std::fprintf(stderr, "[rocshmem pe %d] NVLS bind failed: %s\n", first_pe_, why.c_str());
    return;
  }
  mc_handle_ = mc;
  mc_window_ = va;
  mc_bound_ = true;
  if (cfg_.debug) std::fprintf(stderr, "[rocshmem pe %d] NVLS multicast mapped\n", first_pe_);
}

// A multicast object of its own for a split team (one PE per process): the same steps as for the world object,
// agreed on among the team's processes only. Any failure leaves the team without a mapping on every member.
void Runtime::setup_team_nvls(HostTeam *t, const std::string &tag) {
  MemProvider *cu = mem_.get();
  if (!mc_bound_ || !cfg_.team_nvls || n_local_ != 1) return;
  const int n = static_cast<int>(t->procs.size());
  if (n < 2) return;
  if (n == n_pes_) {  // the same members as the world team
    t->mc_window = mc_window_;
    return;
  }
  auto all_ok = [&](const char *step, bool ok) {
    std::vector<int> flags(static_cast<size_t>(n));
    int mine = ok ? 1 : 0;
    bs_->allgather_group(tag + "/mc-" + step, t->procs, t->my_proc, &mine, flags.data(), sizeof(int));
    return std::all_of(flags.begin(), flags.end(), [](int f) { return f == 1; });
  };
  std::string why;
  MemHandle mc;
  char *va = nullptr;
  bool bound = false;
  auto undo = [&]() {
    if (bound) {
      cu->unmap(va, stride_);
      cu->mc_unbind(mc, stride_);
    }
    if (va) cu->release(va, stride_);
    if (mc.opaque) cu->destroy(mc);
    if (mc.fd >= 0) ::close(mc.fd);
    if (cfg_.debug && !why.empty())
      std::fprintf(stderr, "[rocshmem pe %d] team multicast unavailable: %s\n", first_pe_, why.c_str());
  };
  try {
    size_t g = cu->mc_granularity(stride_, n);
    if (!all_ok("gran", g != 0 && stride_ % g == 0)) return;
    bool ok = true;
    if (t->my_proc == 0) ok = cu->mc_create(stride_, n, &mc, &why);
    if (!all_ok("create", ok)) {
      undo();
      return;
    }
    int fd = broadcast_fd_group(*bs_, tag + "/mc-fd", t->procs, t->my_proc, t->my_proc == 0 ? mc.fd : -1);
    if (t->my_proc != 0) {
      ok = cu->mc_import(fd, stride_, &mc, &why);
      if (!ok) ::close(fd);
    } else {
      ::close(fd);
    }
    if (!all_ok("import", ok)) {
      undo();
      return;
    }
    ok = cu->mc_add_device(mc, &why);
    if (!all_ok("add", ok)) {  // all devices are added before anyone binds
      undo();
      return;
    }
    try {
      va = cu->reserve(stride_);
    } catch (...) {
      ok = false;
      why = "no address range for the mapping";
    }
    if (ok) {
      ok = cu->mc_bind_and_map(mc, handles_[first_pe_], va, &why);
      bound = ok;
    }
    if (!all_ok("bind", ok)) {
      undo();
      return;
    }
  } catch (const std::exception &e) {
    why = e.what();
    undo();
    return;
  }
  t->mc_handle = mc;
  t->mc_window = va;
  t->mc_owned = true;
  if (cfg_.debug) std::fprintf(stderr, "[rocshmem pe %d] multicast mapping for a team of %d\n", first_pe_, n);
}

void Runtime::release_team_nvls(HostTeam *t) {
  MemProvider *cu = mem_.get();
  if (t->mc_owned) {
    cu->unmap(t->mc_window, stride_);
    cu->mc_unbind(t->mc_handle, stride_);
    cu->release(t->mc_window, stride_);
    cu->destroy(t->mc_handle);
  }
  t->mc_owned = false;
  t->mc_window = nullptr;
}

void Runtime::build_states() {
  states_.assign(n_local_, rocshmem_device_state{});
  for (int l = 0; l < n_local_; ++l) {
    rocshmem_device_state &s = states_[l];
    int pe = first_pe_ + l;
    char *ib = internal_base(pe);
    s.my_pe = pe;
    s.n_pes = n_pes_;
    s.n_local = n_local_;
    s.local_index = l;
    s.heap_base = heap_base(pe);
    s.window_base = window_;
    s.heap_stride = stride_;
    s.heap_size = cfg_.heap_size;
    s.mc_base = mc_window_;
    s.internal_base = ib;
    s.teams = reinterpret_cast<rocshmem_team_dev *>(ib + layout_.teams);
    s.ctxs = reinterpret_cast<rocshmem_ctx_dev *>(ib + layout_.ctxs);
    s.ctx_free_mask = reinterpret_cast<unsigned long long *>(ib + layout_.ctx_free_mask);
    s.barrier_flags = reinterpret_cast<unsigned long long *>(ib + layout_.barrier_flags);
    s.lib_flags = reinterpret_cast<unsigned long long *>(ib + layout_.lib_flags);
    s.lib_state = reinterpret_cast<unsigned long long *>(ib + layout_.lib_state);
    s.ll_buf = reinterpret_cast<unsigned long long *>(ib + layout_.ll_buf);
    s.scratch = ib + layout_.scratch;
    s.scratch_size = cfg_.scratch_size;
    s.error = reinterpret_cast<rocshmem_error_record *>(ib + layout_.error);
    s.stats = reinterpret_cast<unsigned long long *>(ib + layout_.stats);
    s.proxy = (proxy_ && proxy_->running())
                  ? reinterpret_cast<rocshmem_proxy_ring *>(ib + layout_.proxy)
                  : nullptr;
    s.max_teams = cfg_.max_teams;
    s.max_ctxs = cfg_.max_contexts;
    s.wait_timeout_ns = cfg_.wait_timeout_ms * 1000000ull;
    s.device_ordinal = device_;
    s.debug_checks = cfg_.debug_checks;
    // Bit 0: thread-level RMA / atomics go through the proxy; bit 1: lanes coalesce their messages first;
    // bit 2: block-level collectives are executed by the proxy too.
    s.use_proxy = (proxy_ && proxy_->running() && cfg_.use_proxy)
                      ? (1 | (cfg_.proxy_coalesce ? 2 : 0) | (cfg_.proxy_collectives ? 4 : 0))
                      : 0;
  }
}

void Runtime::set_wait_timeout_ms(uint64_t ms) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  if (ms == 0) throw std::invalid_argument("rocshmem: waits are always bounded; timeout must be > 0");
  cfg_.wait_timeout_ms = ms;
  for (auto &s : states_) s.wait_timeout_ns = ms * 1000000ull;
  upload_states();
}

int Runtime::check_canaries() {
  std::lock_guard<std::recursive_mutex> g(mu_);
  if (!inited_) return 0;
  int bad = 0;
  std::vector<unsigned long long> got(InternalLayout::kGuardBytes / sizeof(unsigned long long));
  for (int l = 0; l < n_local_; ++l) {
    for (size_t off : layout_.guards) {
      mem_->read(got.data(), internal_base(first_pe_ + l) + off, InternalLayout::kGuardBytes);
      for (unsigned long long w : got) {
        if (w != InternalLayout::kGuardWord) {
          ++bad;
          break;
        }
      }
    }
  }
  return bad;
}

void Runtime::finalize() {
  std::lock_guard<std::recursive_mutex> g(mu_);
  if (!inited_) return;
  if (int bad = check_canaries()) {
    std::fprintf(stderr, "[rocshmem pe %d] finalize: %d guard region(s) of the internal heap area were overwritten\n",
                 first_pe_, bad);
  }
  // Everybody stops using peers' memory before anything is unmapped.
  try {
    ops_->quiet(default_ctx_);
    mem_->sync_device();   // kernels queued on the caller's own streams may still use peers' memory
    bs_->barrier("finalize");
  } catch (const std::exception &e) {
    std::fprintf(stderr, "[rocshmem pe %d] finalize: %s\n", first_pe_, e.what());
  }
  if (proxy_) {
    proxy_->stop();
    proxy_.reset();
  }
  // Kernels launched after finalize (plain GEMMs, layout helpers on ordinary tensors) must not see
  // the window of a heap that no longer exists: every module gets an all-zero state back.
  if (is_cuda()) {
    // The zeroed state keeps the device ordinal: the modules' upload functions select that device before they
    // write their symbols, and ordinal 0 would create a context on (and write to) the wrong GPU.
    for (auto &s : states_) {
      s = rocshmem_device_state{};
      s.device_ordinal = device_;
    }
    try {
      upload_states();
    } catch (...) {
    }
  }
  for (auto &c : ctxs_) ops_->ctx_fini(c.get());
  ctxs_.clear();
  default_ctx_ = nullptr;
  for (auto &slot : team_by_slot_) slot.store(nullptr, std::memory_order_release);
  // All ranks have passed the barrier above with their queues drained, so no kernel uses a team's multicast
  // mapping any more.
  for (auto &t : teams_)
    if (t->mc_owned) release_team_nvls(t.get());
  teams_.clear();
  world_team_ = nullptr;
  ops_.reset();
  if (mc_bound_) {
    mem_->unmap(mc_window_, stride_);
    mem_->mc_unbind(mc_handle_, stride_);
    mem_->release(mc_window_, stride_);
    mem_->destroy(mc_handle_);
    mc_bound_ = false;
    mc_window_ = nullptr;
  }
  for (int pe = 0; pe < n_pes_; ++pe) {
    if (handles_[pe].opaque || handles_[pe].fd >= 0) {
      mem_->unmap(heap_base(pe), stride_);
      mem_->destroy(handles_[pe]);
    }
  }
  mem_->release(window_, stride_ * size_t(n_pes_));
  window_ = nullptr;
  handles_.clear();
  alloc_.reset();
  slots_.reset();
  delete host_stats_;
  host_stats_ = nullptr;
  states_.clear();
  mem_.reset();
  bs_.reset();
  inited_ = false;
}

// -------------------------------------------------------------------------------------------------
// Heap
// -------------------------------------------------------------------------------------------------

void *Runtime::malloc(size_t bytes) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  size_t off = alloc_->alloc(bytes);
  void *p = off == Pow2Allocator::kNull ? nullptr : local_heap_base() + off;
  // Collective: nobody uses the new block on a peer before that peer has it too.
  ops_->barrier(default_ctx_, world_team_, false);
  return p;
}

void Runtime::free(void *ptr) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  ops_->barrier(default_ctx_, world_team_, false);
  if (!ptr) return;
  int pe = -1;
  if (!is_symmetric(ptr, 1, &pe)) {
    throw std::invalid_argument("rocshmem_free: pointer is not on the symmetric heap");
  }
  size_t off = static_cast<size_t>(static_cast<char *>(ptr) - heap_base(pe));
  if (!alloc_->free(off)) {
    throw std::invalid_argument("rocshmem_free: pointer is not a live rocshmem_malloc result");
  }
}

bool Runtime::is_symmetric(const void *p, size_t bytes, int *pe_out) const {
  const char *c = static_cast<const char *>(p);
  if (!window_ || c < window_ || c >= window_ + stride_ * size_t(n_pes_)) return false;
  size_t rel = static_cast<size_t>(c - window_);
  size_t pe = rel / stride_;
  size_t off = rel % stride_;
  if (off + bytes > cfg_.heap_size) return false;
  if (pe_out) *pe_out = static_cast<int>(pe);
  return true;
}

void *Runtime::translate(const void *p, int pe) const {
  const char *c = static_cast<const char *>(p);
  if (pe < 0 || pe >= n_pes_) throw std::out_of_range("rocshmem: PE out of range");
  if (!window_ || c < window_ || c >= window_ + stride_ * size_t(n_pes_)) {
    throw std::invalid_argument("rocshmem: address is not symmetric");
  }
  size_t off = static_cast<size_t>(c - window_) % stride_;
  return heap_base(pe) + off;
}

// -------------------------------------------------------------------------------------------------
// Teams
// -------------------------------------------------------------------------------------------------

void Runtime::write_team_descriptor(HostTeam *t) {
  for (int l = 0; l < n_local_; ++l) {
    int pe = first_pe_ + l;
    rocshmem_team_dev d;
    std::memset(&d, 0, sizeof(d));
    d.pe_start = t->world.pe_start;
    d.stride = t->world.stride;
    d.size = t->world.size;
    d.my_pe = t->my_pe[l];
    d.slot = t->slot;
    d.valid = 1;
    d.world_size = n_pes_;
    d.my_pe_world = pe;
    d.barrier_epoch = 0;
    d.ll_epoch = 0;
    d.mc_base = t->mc_window;
    auto *dst = reinterpret_cast<rocshmem_team_dev *>(internal_base(pe) + layout_.teams) + t->slot;
    mem_->write(dst, &d, sizeof(d));
    // A reused slot starts from epoch 0 again, so the arrival flags of the device barrier and the
    // per-(slot, block) epochs and flags of the library kernels and the small-allreduce mailboxes are cleared as well: the slot's earlier
    // occupants may have had other members and may have run another number of kernels. All members do
    // this before the collective that ends the split, and nobody signals on the new team before that
    // collective has completed.
    mem_->zero(internal_base(pe) + layout_.barrier_flags + size_t(t->slot) * ROCSHMEM_MAX_PES * 8,
               size_t(ROCSHMEM_MAX_PES) * 8);
    mem_->zero(internal_base(pe) + layout_.lib_state + size_t(t->slot) * ROCSHMEM_LIB_MAX_BLOCKS * 8,
               size_t(ROCSHMEM_LIB_MAX_BLOCKS) * 8);
    mem_->zero(internal_base(pe) + layout_.ll_buf + size_t(t->slot) * layout_.ll_slot_bytes, layout_.ll_slot_bytes);
    mem_->zero(internal_base(pe) + layout_.lib_flags +
                   size_t(t->slot) * ROCSHMEM_LIB_MAX_BLOCKS * ROCSHMEM_MAX_PES * 8,
               size_t(ROCSHMEM_LIB_MAX_BLOCKS) * ROCSHMEM_MAX_PES * 8);
  }
  t->dev = reinterpret_cast<rocshmem_team_dev *>(internal_base(first_pe_) + layout_.teams) + t->slot;
}

HostTeam *Runtime::team_from_handle(rocshmem_team_t h) {
  if (h == nullptr) return nullptr;
  for (auto &t : teams_) {
    if (t->dev == h) return t.get();
  }
  return nullptr;
}

int Runtime::team_split_strided(HostTeam *parent, int start, int stride, int size,
                                rocshmem_team_t *out) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  *out = nullptr;
  // Slot 0 is TEAM_WORLD, so at most max_teams - 1 user teams exist at a time.
  if (num_user_teams() >= cfg_.max_teams - 1) return -1;
  if (parent == nullptr) return 0;
  SplitPlan plan = plan_split(parent->world, parent->world.size, n_pes_, start, stride, size);
  if (!plan.ok) return -1;

  // Sequence number per (parent, member set): every member of the new team has made the same
  // number of earlier requests for exactly this set, whether or not other PEs of the parent took
  // part in them (active-set collectives are called by the set's members only).
  std::string set_key = std::to_string(parent->id) + "/" + std::to_string(plan.world.pe_start) + "." +
                        std::to_string(plan.world.stride) + "." + std::to_string(plan.world.size);
  uint64_t seq = split_counts_[set_key]++;
  auto team = std::make_unique<HostTeam>();
  team->world = plan.world;
  team->my_pe.resize(n_local_);
  bool member = false;
  for (int l = 0; l < n_local_; ++l) {
    team->my_pe[l] = plan.world.pe_in_team(first_pe_ + l);
    member = member || team->my_pe[l] >= 0;
  }
  if (!member) return 0;  // not in the new team: handle stays INVALID, no slot is consumed

  // Processes hosting at least one member agree on the lowest slot that is free everywhere.
  std::vector<int> procs;
  for (int j = 0; j < plan.world.size; ++j) {
    int r = plan.world.pe_in_world(j) / n_local_;
    if (procs.empty() || procs.back() != r) procs.push_back(r);
  }
  int my_index = static_cast<int>(std::find(procs.begin(), procs.end(), bs_->rank()) - procs.begin());
  std::vector<uint64_t> masks(procs.size());
  uint64_t mine = slots_->mask();
  std::string tag = "split/" + set_key + "/" + std::to_string(seq);
  bs_->allgather_group(tag, procs, my_index, &mine, masks.data(), sizeof(uint64_t));
  int slot = TeamSlots::lowest_common(masks);
  if (slot < 0) return -1;
  slots_->take(slot);
  team->slot = slot;
  // Identifier that is the same on every member and never reused while keys of older splits may
  // still sit in the store.
  team->id = parent->id * 1000003ull + (seq + 1) * 7919ull + uint64_t(plan.world.pe_start) * 31ull +
             uint64_t(plan.world.stride) * 17ull + uint64_t(plan.world.size);
  HostTeam *raw = team.get();
  raw->procs = procs;
  raw->my_proc = my_index;
  teams_.push_back(std::move(team));
  setup_team_nvls(raw, tag);
  write_team_descriptor(raw);
  team_by_slot_[raw->slot].store(raw, std::memory_order_release);
  // Descriptors and cleared flags are in place on every member before the handle is used.
  std::vector<char> tokens(procs.size());
  char one = 1;
  bs_->allgather_group(tag + "/ready", procs, my_index, &one, tokens.data(), 1);
  *out = raw->dev;
  return 0;
}

void Runtime::team_destroy(HostTeam *t) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  if (!t || t == world_team_) return;
  if (t->mc_owned) {
    // Nobody may unbind its memory while another member's kernel can still store through the multicast object:
    // every member finishes its own work, then all of them meet, then the mapping goes. (OpenSHMEM makes
    // team_destroy collective; for teams without a multicast object nothing is exchanged here.)
    try {
      mem_->sync_device();   // collectives on the team may have been queued on any stream
      char one = 1;
      std::vector<char> all(t->procs.size());
      bs_->allgather_group("team-destroy/" + std::to_string(t->id), t->procs, t->my_proc, &one, all.data(), 1);
    } catch (const std::exception &e) {
      std::fprintf(stderr, "[rocshmem pe %d] team_destroy: %s\n", first_pe_, e.what());
    }
    release_team_nvls(t);
  }
  for (int l = 0; l < n_local_; ++l) {
    rocshmem_team_dev d;
    std::memset(&d, 0, sizeof(d));
    d.my_pe = -1;
    auto *dst = reinterpret_cast<rocshmem_team_dev *>(internal_base(first_pe_ + l) + layout_.teams) + t->slot;
    mem_->write(dst, &d, sizeof(d));
  }
  team_by_slot_[t->slot].store(nullptr, std::memory_order_release);
  slots_->release(t->slot);
  teams_.erase(std::remove_if(teams_.begin(), teams_.end(),
                              [t](const std::unique_ptr<HostTeam> &p) { return p.get() == t; }),
               teams_.end());
}

// -------------------------------------------------------------------------------------------------
// Host contexts
// -------------------------------------------------------------------------------------------------

HostCtx *Runtime::ctx_create(long long options, HostTeam *team) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  // The default context counts against ROCSHMEM_MAX_NUM_HOST_CONTEXTS, as in the reference's
  // window pool (src/host/host.cpp:44-83).
  if (static_cast<int>(ctxs_.size()) >= cfg_.max_host_contexts) return nullptr;
  auto c = std::make_unique<HostCtx>();
  c->id = static_cast<int>(ctxs_.size());
  c->options = options;
  c->team = team ? team : world_team_;
  ops_->ctx_init(c.get());
  HostCtx *raw = c.get();
  ctxs_.push_back(std::move(c));
  return raw;
}

void Runtime::ctx_destroy(HostCtx *c) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  if (!c || c == default_ctx_) return;
  ops_->quiet(c);
  ops_->ctx_fini(c);
  ctxs_.erase(std::remove_if(ctxs_.begin(), ctxs_.end(),
                             [c](const std::unique_ptr<HostCtx> &p) { return p.get() == c; }),
              ctxs_.end());
}

// -------------------------------------------------------------------------------------------------
// Diagnostics
// -------------------------------------------------------------------------------------------------

rocshmem_error_record Runtime::read_error(int local) {
  rocshmem_error_record e;
  int l = local < 0 ? current_local() : local;
  mem_->read(&e, internal_base(first_pe_ + l) + layout_.error, sizeof(e));
  return e;
}

void Runtime::clear_error() {
  for (int l = 0; l < n_local_; ++l) {
    mem_->zero(internal_base(first_pe_ + l) + layout_.error, sizeof(rocshmem_error_record));
  }
}

std::vector<unsigned long long> Runtime::read_stats(int local) {
  std::vector<unsigned long long> v(ROCSHMEM_NUM_STATS);
  int l = local < 0 ? current_local() : local;
  mem_->read(v.data(), internal_base(first_pe_ + l) + layout_.stats, v.size() * sizeof(unsigned long long));
  return v;
}

void Runtime::reset_stats() {
  for (int l = 0; l < n_local_; ++l) {
    mem_->zero(internal_base(first_pe_ + l) + layout_.stats, sizeof(unsigned long long) * ROCSHMEM_NUM_STATS);
  }
  if (host_stats_) {
    for (auto &c : *host_stats_) c.store(0);
  }
}

std::vector<unsigned long long> Runtime::host_stats() const {
  std::vector<unsigned long long> v(ROCSHMEM_NUM_STATS, 0);
  if (host_stats_) {
    for (int i = 0; i < ROCSHMEM_NUM_STATS; ++i) v[i] = (*host_stats_)[i].load();
  }
  return v;
}

void Runtime::count(int stat_id, unsigned long long n) {
  if (host_stats_ && stat_id >= 0 && stat_id < ROCSHMEM_NUM_STATS) (*host_stats_)[stat_id].fetch_add(n);
}

}  // namespace rocshmem
