// Host-side API: argument checking, handle unwrapping, statistics, then the host-operation engine.
#include <dirent.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "host_ops.hpp"
#include "proxy.hpp"
#include "rocshmem/rocshmem_debug.hpp"
#include "rocshmem/rocshmem_host.h"
#include "rocshmem/slab.h"
#include "runtime.hpp"

namespace rocshmem {

rocshmem_team_t ROCSHMEM_TEAM_WORLD = nullptr;

namespace {

int env_int(const char *name, int fallback) {
  const char *e = std::getenv(name);
  if (!e || !*e) return fallback;
  try {
    return static_cast<int>(parse_int(e));
  } catch (...) {
    return fallback;
  }
}

Runtime &rt() {
  Runtime &r = Runtime::instance();
  if (!Runtime::initialized()) throw std::runtime_error("rocshmem: library is not initialised");
  return r;
}

HostCtx *host_ctx(rocshmem_ctx_t ctx) {
  // A zero handle (ROCSHMEM_CTX_DEFAULT on the host) selects the default context.
  if (ctx.ctx_opaque == nullptr) return rt().default_ctx();
  return static_cast<HostCtx *>(ctx.ctx_opaque);
}

int world_pe(HostCtx *c, int pe) {
  // PEs given to context-based calls are relative to the context's team.
  HostTeam *t = c->team ? c->team : rt().team_world();
  if (pe < 0 || pe >= t->world.size) throw std::out_of_range("rocshmem: PE outside the context's team");
  return t->world.pe_in_world(pe);
}

HostTeam *host_team(rocshmem_team_t team) {
  HostTeam *t = rt().team_from_handle(team);
  if (!t) throw std::invalid_argument("rocshmem: invalid team handle");
  return t;
}

}  // namespace

namespace {

// Start time of a process in clock ticks since boot (field 22 of /proc/<pid>/stat), 0 when it does not exist.
unsigned long long process_start_time(long pid) {
  std::FILE *f = std::fopen(("/proc/" + std::to_string(pid) + "/stat").c_str(), "r");
  if (!f) return 0;
  char buf[1024];
  size_t n = std::fread(buf, 1, sizeof(buf) - 1, f);
  std::fclose(f);
  buf[n] = '\0';
  const char *p = std::strrchr(buf, ')');   // the command name may contain spaces and parentheses
  if (!p) return 0;
  unsigned long long value = 0;
  int field = 2;
  for (++p; *p; ++p) {
    if (*p != ' ') continue;
    if (++field == 22) {
      value = std::strtoull(p + 1, nullptr, 10);
      break;
    }
  }
  return value;
}

constexpr const char *kRendezvousRoot = "/dev/shm";
std::string rendezvous_prefix() { return "rocshmem_b200." + std::to_string(::getuid()) + "."; }

// The default rendezvous directory of a job. All ranks of one launch share their parent process (torchrun's
// agent, the launcher of this package, mpirun), so its pid and start time make the name unique per launch: files
// that an earlier job on the same port left behind are never read. Ranks started by different parents (by hand,
// in separate shells) have to agree on ROCSHMEM_BOOTSTRAP_DIR instead.
std::string default_rendezvous_dir() {
  const char *port = std::getenv("MASTER_PORT");
  const char *run = std::getenv("TORCHELASTIC_RUN_ID");
  const long parent = static_cast<long>(::getppid());
  return std::string(kRendezvousRoot) + "/" + rendezvous_prefix() + (port ? port : "0") + "." + (run ? run : "job") +
         "." + std::to_string(parent) + "." + std::to_string(process_start_time(parent));
}

// Best effort, rank 0 only: remove rendezvous directories of this user whose launching process is gone.
void purge_stale_rendezvous_dirs() {
  DIR *d = ::opendir(kRendezvousRoot);
  if (!d) return;
  const std::string prefix = rendezvous_prefix();
  std::vector<std::string> stale;
  while (dirent *e = ::readdir(d)) {
    const std::string name = e->d_name;
    if (name.compare(0, prefix.size(), prefix) != 0) continue;
    // ... .<parent pid>.<parent start time>
    const size_t dot2 = name.rfind('.');
    const size_t dot1 = dot2 == std::string::npos || dot2 == 0 ? std::string::npos : name.rfind('.', dot2 - 1);
    if (dot1 == std::string::npos) continue;
    char *end = nullptr;
    const long pid = std::strtol(name.c_str() + dot1 + 1, &end, 10);
    if (end != name.c_str() + dot2 || pid <= 0) continue;      // not a name of the current scheme: leave it alone
    const unsigned long long start = std::strtoull(name.c_str() + dot2 + 1, &end, 10);
    if (*end != '\0') continue;
    if (process_start_time(pid) != start) stale.push_back(name);
  }
  ::closedir(d);
  for (const std::string &name : stale) {
    const std::string path = std::string(kRendezvousRoot) + "/" + name;
    if (DIR *sub = ::opendir(path.c_str())) {
      while (dirent *e = ::readdir(sub)) {
        if (std::strcmp(e->d_name, ".") != 0 && std::strcmp(e->d_name, "..") != 0) ::unlink((path + "/" + e->d_name).c_str());
      }
      ::closedir(sub);
    }
    ::rmdir(path.c_str());
  }
}

}  // namespace

namespace host {

void init() {
  if (Runtime::initialized()) return;
  int rank = env_int("RANK", 0);
  int size = env_int("WORLD_SIZE", 1);
  int local_rank = env_int("LOCAL_RANK", rank);
  int n_local = env_int("ROCSHMEM_LOCAL_PES", 1);
  Config cfg = Config::from_env();
  std::unique_ptr<Bootstrap> bs;
  if (size <= 1) {
    bs = std::make_unique<LocalBootstrap>();
  } else {
    std::string dir = cfg.bootstrap_dir;
    if (dir.empty()) {
      if (rank == 0) purge_stale_rendezvous_dirs();
      dir = default_rendezvous_dir();
    }
    bs = std::make_unique<FileBootstrap>(dir, rank, size);
  }
  int ndev = cuda_device_count();
  int device = ndev > 0 ? local_rank % ndev : 0;
  Runtime::instance().init(std::move(bs), cfg, n_local, device);
  ROCSHMEM_TEAM_WORLD = Runtime::instance().team_world()->dev;
}

void init_thread(int, int *provided) {
  init();
  if (provided) *provided = ROCSHMEM_THREAD_MULTIPLE;
}

void query_thread(int *provided) {
  if (provided) *provided = ROCSHMEM_THREAD_MULTIPLE;
}

void finalize() {
  if (!Runtime::initialized()) return;
  Runtime::instance().finalize();
  ROCSHMEM_TEAM_WORLD = nullptr;
}

void global_exit(int status) {
  std::fprintf(stderr, "[rocshmem pe %d] global_exit(%d)\n", my_pe(), status);
  std::fflush(nullptr);
  ::_exit(status);
}

bool is_initialized() { return Runtime::initialized(); }

int my_pe() {
  if (Runtime::initialized()) return Runtime::instance().my_pe();
  return env_int("RANK", 0) * env_int("ROCSHMEM_LOCAL_PES", 1);
}

int n_pes() {
  if (Runtime::initialized()) return Runtime::instance().n_pes();
  return env_int("WORLD_SIZE", 1) * env_int("ROCSHMEM_LOCAL_PES", 1);
}

static const char *stat_name(int i) {
  static const char *names[ROCSHMEM_NUM_STATS] = {
      "put", "put_nbi", "p", "get", "get_nbi", "g", "put_warp", "put_block", "get_warp", "get_block",
      "put_signal", "signal_fetch", "amo_fetch", "amo_nofetch", "fence", "quiet", "wait", "test",
      "barrier", "sync", "broadcast", "reduce", "fcollect", "alltoall", "ctx_create", "ctx_destroy",
      "bytes_put", "bytes_get", "proxy_cmd", "timeouts", "proxy_slot_ns", "proxy_pack_ns", "proxy_host_ns",
      "wait_ns"};
  return names[i];
}

void dump_stats() {
  Runtime &r = rt();
  auto dev = r.read_stats();
  auto hst = r.host_stats();
  std::printf("rocshmem stats, PE %d of %d\n", r.my_pe(), r.n_pes());
  for (int i = 0; i < ROCSHMEM_NUM_STATS; ++i) {
    std::printf("  %-14s device %12llu   host %12llu\n", stat_name(i), dev[i], hst[i]);
  }
  std::fflush(stdout);
}

void reset_stats() { rt().reset_stats(); }

// ROCSHMEM_DEBUG=2: one line on stderr per collective management call (heap, teams, contexts), in the spirit of
// the reference's DPRINTF tracing (src/util.hpp:51-71). Data-path calls are not traced.
#define ROCSHMEM_TRACE(r, ...)                                        \
  do {                                                                \
    if ((r).config().debug >= 2) {                                    \
      std::fprintf(stderr, "[rocshmem pe %d] ", (r).my_pe());         \
      std::fprintf(stderr, __VA_ARGS__);                              \
      std::fputc('\n', stderr);                                       \
    }                                                                 \
  } while (0)

void *malloc(size_t bytes) {
  Runtime &r = rt();
  void *p = r.malloc(bytes);
  ROCSHMEM_TRACE(r, "malloc(%zu) = %p, %zu bytes of the heap in use", bytes, p, r.heap_used());
  return p;
}

void free(void *p) {
  Runtime &r = rt();
  r.free(p);
  ROCSHMEM_TRACE(r, "free(%p), %zu bytes of the heap in use", p, r.heap_used());
}

void *ptr(const void *p, int pe) {
  Runtime &r = rt();
  if (!r.is_symmetric(p) || pe < 0 || pe >= r.n_pes()) return nullptr;
  return r.translate(p, pe);
}

int ctx_create(int64_t options, rocshmem_ctx_t *ctx) {
  HostCtx *c = rt().ctx_create(options, rt().team_world());
  ROCSHMEM_TRACE(rt(), "ctx_create(options %lld) = %p", static_cast<long long>(options), static_cast<void *>(c));
  if (!c) return -1;
  ctx->ctx_opaque = c;
  ctx->team_opaque = c->team->dev;
  rt().count(ROCSHMEM_STAT_CTX_CREATE);
  return 0;
}

int team_create_ctx(rocshmem_team_t team, int64_t options, rocshmem_ctx_t *ctx) {
  if (team == nullptr) return -1;
  HostCtx *c = rt().ctx_create(options, host_team(team));
  if (!c) return -1;
  ctx->ctx_opaque = c;
  ctx->team_opaque = c->team->dev;
  rt().count(ROCSHMEM_STAT_CTX_CREATE);
  return 0;
}

void ctx_destroy(rocshmem_ctx_t ctx) {
  if (ctx.ctx_opaque == nullptr) return;
  rt().ctx_destroy(static_cast<HostCtx *>(ctx.ctx_opaque));
  rt().count(ROCSHMEM_STAT_CTX_DESTROY);
}

int team_translate_pe(rocshmem_team_t src_team, int src_pe, rocshmem_team_t dst_team) {
  if (src_team == nullptr || dst_team == nullptr) return -1;
  HostTeam *s = rt().team_from_handle(src_team), *d = rt().team_from_handle(dst_team);
  if (!s || !d) return -1;
  return translate_pe(s->world, src_pe, d->world);
}

int team_n_pes(rocshmem_team_t team) {
  if (team == nullptr) return -1;
  HostTeam *t = rt().team_from_handle(team);
  return t ? t->world.size : -1;
}

int team_my_pe(rocshmem_team_t team) {
  if (team == nullptr) return -1;
  HostTeam *t = rt().team_from_handle(team);
  return t ? t->my_pe[rt().current_local()] : -1;
}

int team_split_strided(rocshmem_team_t parent, int start, int stride, int size,
                       const rocshmem_team_config_t *, long, rocshmem_team_t *new_team) {
  HostTeam *p = parent ? rt().team_from_handle(parent) : nullptr;
  if (parent && !p) {
    *new_team = nullptr;
    return -1;
  }
  int rc = rt().team_split_strided(p, start, stride, size, new_team);
  ROCSHMEM_TRACE(rt(), "team_split_strided(start %d, stride %d, size %d) = %d, team %p", start, stride, size, rc,
                 static_cast<void *>(*new_team));
  return rc;
}

void team_destroy(rocshmem_team_t team) {
  if (team == nullptr) return;
  HostTeam *t = rt().team_from_handle(team);
  ROCSHMEM_TRACE(rt(), "team_destroy(%p)%s", static_cast<void *>(team), t ? "" : ": unknown handle");
  if (t) rt().team_destroy(t);
}

// ---- RMA ----------------------------------------------------------------------------------------

static void check_remote(Runtime &r, const void *sym, size_t bytes, const char *what) {
  if (!r.is_symmetric(sym, bytes ? bytes : 1)) {
    throw std::invalid_argument(std::string("rocshmem ") + what +
                                ": remote address is not inside the symmetric heap");
  }
}

void putmem(rocshmem_ctx_t ctx, void *dest, const void *source, size_t bytes, int pe) {
  if (bytes == 0) return;
  Runtime &r = rt();
  HostCtx *c = host_ctx(ctx);
  check_remote(r, dest, bytes, "putmem");
  r.ops().put(c, dest, source, bytes, world_pe(c, pe), true);
  r.count(ROCSHMEM_STAT_PUT);
  r.count(ROCSHMEM_STAT_BYTES_PUT, bytes);
}

void putmem_nbi(rocshmem_ctx_t ctx, void *dest, const void *source, size_t bytes, int pe) {
  if (bytes == 0) return;
  Runtime &r = rt();
  HostCtx *c = host_ctx(ctx);
  check_remote(r, dest, bytes, "putmem_nbi");
  r.ops().put(c, dest, source, bytes, world_pe(c, pe), false);
  r.count(ROCSHMEM_STAT_PUT_NBI);
  r.count(ROCSHMEM_STAT_BYTES_PUT, bytes);
}

void getmem(rocshmem_ctx_t ctx, void *dest, const void *source, size_t bytes, int pe) {
  if (bytes == 0) return;
  Runtime &r = rt();
  HostCtx *c = host_ctx(ctx);
  check_remote(r, source, bytes, "getmem");
  r.ops().get(c, dest, source, bytes, world_pe(c, pe), true);
  r.count(ROCSHMEM_STAT_GET);
  r.count(ROCSHMEM_STAT_BYTES_GET, bytes);
}

void getmem_nbi(rocshmem_ctx_t ctx, void *dest, const void *source, size_t bytes, int pe) {
  if (bytes == 0) return;
  Runtime &r = rt();
  HostCtx *c = host_ctx(ctx);
  check_remote(r, source, bytes, "getmem_nbi");
  r.ops().get(c, dest, source, bytes, world_pe(c, pe), false);
  r.count(ROCSHMEM_STAT_GET_NBI);
  r.count(ROCSHMEM_STAT_BYTES_GET, bytes);
}

void p(rocshmem_ctx_t ctx, void *dest, uint64_t bits, size_t elem_bytes, int pe) {
  Runtime &r = rt();
  HostCtx *c = host_ctx(ctx);
  check_remote(r, dest, elem_bytes, "p");
  // The value is in host memory, so the copy source is a host buffer that outlives the call.
  r.ops().put(c, dest, &bits, elem_bytes, world_pe(c, pe), true);
  r.count(ROCSHMEM_STAT_P);
}

uint64_t g(rocshmem_ctx_t ctx, const void *source, size_t elem_bytes, int pe) {
  Runtime &r = rt();
  HostCtx *c = host_ctx(ctx);
  check_remote(r, source, elem_bytes, "g");
  uint64_t bits = 0;
  r.ops().get(c, &bits, source, elem_bytes, world_pe(c, pe), true);
  r.count(ROCSHMEM_STAT_G);
  return bits;
}

uint64_t amo(rocshmem_ctx_t ctx, int op, int dtype, void *target, uint64_t value, uint64_t cond,
             int pe) {
  Runtime &r = rt();
  HostCtx *c = host_ctx(ctx);
  DType t = static_cast<DType>(dtype);
  if (dtype_size(t) != 4 && dtype_size(t) != 8) {
    throw std::invalid_argument("rocshmem atomics: only 4- and 8-byte types are supported");
  }
  check_remote(r, target, dtype_size(t), "atomic");
  if (reinterpret_cast<uintptr_t>(target) % dtype_size(t)) {
    throw std::invalid_argument("rocshmem atomics: target is not naturally aligned");
  }
  r.count(ROCSHMEM_STAT_AMO_FETCH);
  return r.ops().amo(c, static_cast<AmoOp>(op), t, target, value, cond, world_pe(c, pe));
}

// ---- ordering / sync -----------------------------------------------------------------------------

void fence(rocshmem_ctx_t ctx) {
  rt().ops().fence(host_ctx(ctx));
  rt().count(ROCSHMEM_STAT_FENCE);
}

void quiet(rocshmem_ctx_t ctx) {
  rt().ops().quiet(host_ctx(ctx));
  rt().count(ROCSHMEM_STAT_QUIET);
}

void barrier_all() {
  Runtime &r = rt();
  r.ops().barrier(r.default_ctx(), r.team_world(), false);
  r.count(ROCSHMEM_STAT_BARRIER);
}

void sync_all() {
  Runtime &r = rt();
  r.ops().barrier(r.default_ctx(), r.team_world(), true);
  r.count(ROCSHMEM_STAT_SYNC);
}

int team_sync(rocshmem_team_t team) {
  if (team == nullptr) return ROCSHMEM_ERROR;
  Runtime &r = rt();
  r.count(ROCSHMEM_STAT_SYNC);
  return r.ops().barrier(r.default_ctx(), host_team(team), true);
}

// An unknown comparison would never be satisfied: refuse it instead of waiting for the time-out.
static void check_cmp(int cmp) {
  if (cmp < ROCSHMEM_CMP_EQ || cmp > ROCSHMEM_CMP_LE) throw std::invalid_argument("rocshmem: unknown comparison operator");
}

int wait_until(void *ivar, int dtype, int cmp, uint64_t value) {
  check_cmp(cmp);
  rt().count(ROCSHMEM_STAT_WAIT);
  return rt().ops().wait_until(ivar, static_cast<DType>(dtype), cmp, value);
}

int test(void *ivar, int dtype, int cmp, uint64_t value) {
  check_cmp(cmp);
  rt().count(ROCSHMEM_STAT_TEST);
  return rt().ops().test(ivar, static_cast<DType>(dtype), cmp, value);
}

namespace {
struct Poller {
  Runtime &r;
  char *base;
  size_t esz;
  DType t;
  int cmp;
  const uint64_t *values;
  bool vector;
  std::chrono::steady_clock::time_point deadline;
  Poller(void *ivars, int dtype, int cmp_, const uint64_t *v, bool vec)
      : r(rt()), base(static_cast<char *>(ivars)), esz(dtype_size(static_cast<DType>(dtype))),
        t(static_cast<DType>(dtype)), cmp(cmp_), values(v), vector(vec),
        deadline(std::chrono::steady_clock::now() +
                 std::chrono::milliseconds(rt().config().wait_timeout_ms)) {
    check_cmp(cmp_);
  }
  bool ready(size_t i) { return r.ops().test(base + i * esz, t, cmp, vector ? values[i] : values[0]) != 0; }
  bool expired() const { return std::chrono::steady_clock::now() > deadline; }
};
}  // namespace

void wait_until_all(void *ivars, size_t nelems, const int *status, int dtype, int cmp,
                    const uint64_t *values, bool vector) {
  if (nelems == 0) return;
  Poller p(ivars, dtype, cmp, values, vector);
  for (size_t i = 0; i < nelems; ++i) {
    if (status && status[i]) continue;
    while (!p.ready(i)) {
      if (p.expired()) {
        p.r.count(ROCSHMEM_STAT_TIMEOUTS);
        return;
      }
      std::this_thread::yield();
    }
  }
}

size_t wait_until_any(void *ivars, size_t nelems, const int *status, int dtype, int cmp,
                      const uint64_t *values, bool vector) {
  if (nelems == 0) return SIZE_MAX;
  bool any_active = false;
  for (size_t i = 0; i < nelems; ++i) any_active = any_active || !(status && status[i]);
  if (!any_active) return SIZE_MAX;
  Poller p(ivars, dtype, cmp, values, vector);
  for (;;) {
    for (size_t i = 0; i < nelems; ++i) {
      if (status && status[i]) continue;
      if (p.ready(i)) return i;
    }
    if (p.expired()) {
      p.r.count(ROCSHMEM_STAT_TIMEOUTS);
      return SIZE_MAX;
    }
    std::this_thread::yield();
  }
}

size_t wait_until_some(void *ivars, size_t nelems, size_t *indices, const int *status, int dtype,
                       int cmp, const uint64_t *values, bool vector) {
  if (nelems == 0) return 0;
  bool any_active = false;
  for (size_t i = 0; i < nelems; ++i) any_active = any_active || !(status && status[i]);
  if (!any_active) return 0;
  Poller p(ivars, dtype, cmp, values, vector);
  for (;;) {
    size_t found = 0;
    for (size_t i = 0; i < nelems; ++i) {
      if (status && status[i]) continue;
      if (p.ready(i)) indices[found++] = i;
    }
    if (found) return found;
    if (p.expired()) {
      p.r.count(ROCSHMEM_STAT_TIMEOUTS);
      return 0;
    }
    std::this_thread::yield();
  }
}

// ---- collectives -----------------------------------------------------------------------------------

static void check_sym(Runtime &r, const void *p, size_t bytes, const char *what) {
  if (!r.is_symmetric(p, bytes ? bytes : 1)) {
    throw std::invalid_argument(std::string("rocshmem ") + what + ": buffer must be symmetric");
  }
}

int broadcast(rocshmem_ctx_t ctx, rocshmem_team_t team, void *dest, const void *source,
              size_t bytes, int pe_root) {
  if (team == nullptr) return ROCSHMEM_ERROR;
  if (bytes == 0) return ROCSHMEM_SUCCESS;
  Runtime &r = rt();
  HostTeam *t = host_team(team);
  if (pe_root < 0 || pe_root >= t->world.size) throw std::out_of_range("broadcast: bad root");
  check_sym(r, dest, bytes, "broadcast");
  check_sym(r, source, bytes, "broadcast");
  r.count(ROCSHMEM_STAT_BROADCAST);
  return r.ops().broadcast(host_ctx(ctx), t, dest, source, bytes, pe_root);
}

int reduce(rocshmem_ctx_t ctx, rocshmem_team_t team, void *dest, const void *source, size_t nreduce,
           int dtype, int op) {
  if (team == nullptr) return ROCSHMEM_ERROR;
  if (nreduce == 0) return ROCSHMEM_SUCCESS;
  Runtime &r = rt();
  DType t = static_cast<DType>(dtype);
  if (dtype_is_float(t) && (op == ROCSHMEM_AND || op == ROCSHMEM_OR || op == ROCSHMEM_XOR)) {
    throw std::invalid_argument("reduce: bitwise reduction of a floating-point type");
  }
  check_sym(r, dest, nreduce * dtype_size(t), "reduce");
  check_sym(r, source, nreduce * dtype_size(t), "reduce");
  r.count(ROCSHMEM_STAT_REDUCE);
  return r.ops().reduce(host_ctx(ctx), host_team(team), dest, source, nreduce, t,
                        static_cast<ROCSHMEM_OP>(op));
}

int fcollect(rocshmem_ctx_t ctx, rocshmem_team_t team, void *dest, const void *source, size_t bytes) {
  if (team == nullptr) return ROCSHMEM_ERROR;
  if (bytes == 0) return ROCSHMEM_SUCCESS;
  Runtime &r = rt();
  HostTeam *t = host_team(team);
  check_sym(r, dest, bytes * size_t(t->world.size), "fcollect");
  check_sym(r, source, bytes, "fcollect");
  r.count(ROCSHMEM_STAT_FCOLLECT);
  return r.ops().fcollect(host_ctx(ctx), t, dest, source, bytes);
}

int alltoall(rocshmem_ctx_t ctx, rocshmem_team_t team, void *dest, const void *source, size_t bytes) {
  if (team == nullptr) return ROCSHMEM_ERROR;
  if (bytes == 0) return ROCSHMEM_SUCCESS;
  Runtime &r = rt();
  HostTeam *t = host_team(team);
  check_sym(r, dest, bytes * size_t(t->world.size), "alltoall");
  check_sym(r, source, bytes * size_t(t->world.size), "alltoall");
  r.count(ROCSHMEM_STAT_ALLTOALL);
  return r.ops().alltoall(host_ctx(ctx), t, dest, source, bytes);
}

namespace {
// Active-set calls are collective over the set's members only; each call derives a team, uses it and
// destroys it again, so no slot stays occupied.
struct ScopedActiveSet {
  rocshmem_team_t team = nullptr;
  ScopedActiveSet(int pe_start, int log_pe_stride, int pe_size) {
    if (log_pe_stride < 0 || log_pe_stride > 30) throw std::invalid_argument("active set: bad stride");
    team_split_strided(ROCSHMEM_TEAM_WORLD, pe_start, 1 << log_pe_stride, pe_size, nullptr, 0, &team);
  }
  ~ScopedActiveSet() {
    if (team) team_destroy(team);
  }
};
}  // namespace

int broadcast_active_set(rocshmem_ctx_t ctx, void *dest, const void *source, size_t bytes,
                         int pe_root, int pe_start, int log_pe_stride, int pe_size) {
  ScopedActiveSet s(pe_start, log_pe_stride, pe_size);
  if (!s.team) return ROCSHMEM_ERROR;
  return broadcast(ctx, s.team, dest, source, bytes, pe_root);
}

int reduce_active_set(rocshmem_ctx_t ctx, void *dest, const void *source, size_t nreduce, int dtype,
                      int op, int pe_start, int log_pe_stride, int pe_size) {
  ScopedActiveSet s(pe_start, log_pe_stride, pe_size);
  if (!s.team) return ROCSHMEM_ERROR;
  return reduce(ctx, s.team, dest, source, nreduce, dtype, op);
}

}  // namespace host

// ---- extensions --------------------------------------------------------------------------------------

void rocshmemx_set_local_pe(int local_index) { rt().set_current_local(local_index); }
int rocshmemx_n_local_pes() { return rt().n_local(); }

void debug_print_ring(int first, int count) {
  Runtime &r = rt();
  Proxy *p = r.proxy();
  if (p == nullptr || !p->running()) {
    std::fprintf(stderr, "[rocshmem pe %d] no reverse-offload ring in this process (ROCSHMEM_USE_PROXY is off)\n", r.my_pe());
    return;
  }
  for (int i = 0; i < count; ++i) {
    std::fprintf(stderr, "[rocshmem pe %d] %s\n", r.my_pe(), p->describe_command(static_cast<unsigned>(first + i)).c_str());
  }
}

void debug_print_sq(int dest_pe, int src_wg, int index_wqe) {
  std::fprintf(stderr, "[rocshmem pe %d] command queue entry (asked for pe %d, block %d):\n", rt().my_pe(), dest_pe, src_wg);
  debug_print_ring(index_wqe, 1);
}

void debug_print_cq(int dest_pe, int src_wg, int cqe_index) {
  Runtime &r = rt();
  Proxy *p = r.proxy();
  std::fprintf(stderr, "[rocshmem pe %d] completion queue entry (asked for pe %d, block %d):\n", r.my_pe(), dest_pe, src_wg);
  if (p == nullptr || !p->running()) {
    std::fprintf(stderr, "[rocshmem pe %d] no reverse-offload ring in this process (ROCSHMEM_USE_PROXY is off)\n", r.my_pe());
    return;
  }
  std::fprintf(stderr, "[rocshmem pe %d] %s\n", r.my_pe(), p->describe_completion(static_cast<unsigned>(cqe_index)).c_str());
}
rocshmem_error_record rocshmemx_get_error() { return rt().read_error(); }
void rocshmemx_clear_error() { rt().clear_error(); }
void rocshmemx_set_wait_timeout_ms(uint64_t ms) { rt().set_wait_timeout_ms(ms); }
void rocshmemx_heap_write(void *heap_dst, const void *host_src, size_t bytes) {
  rt().mem().write(heap_dst, host_src, bytes);
}
void rocshmemx_heap_read(void *host_dst, const void *heap_src, size_t bytes) {
  rt().mem().read(host_dst, heap_src, bytes);
}
void *rocshmemx_default_stream() { return rt().default_ctx()->stream; }

// ---- slab (device-side bump allocation) ----------------------------------------------------------------

namespace {
unsigned long long slab_cursor_read(const rocshmemx_slab_t &s) {
  unsigned long long v = 0;
  rt().mem().read(&v, s.cursor, sizeof(v));
  return v;
}
}  // namespace

rocshmemx_slab_t rocshmemx_slab_create(size_t bytes) {
  Runtime &r = rt();
  if (bytes == 0) bytes = r.config().slab_size;
  bytes = static_cast<size_t>(detail::slab_round_up(bytes, 256));
  rocshmemx_slab_t s{nullptr, 0, nullptr};
  // One heap object: the slab, then a 256-byte line that holds the cursor.
  char *p = static_cast<char *>(r.malloc(bytes + 256));
  if (!p) return s;
  for (int l = 0; l < r.n_local(); ++l) {
    r.mem().zero(static_cast<char *>(r.translate(p, r.first_pe() + l)) + bytes, 256);
  }
  s.base = p;
  s.size = bytes;
  s.cursor = reinterpret_cast<unsigned long long *>(p + bytes);
  return s;
}

void rocshmemx_slab_destroy(rocshmemx_slab_t slab) {
  if (slab.base) rt().free(slab.base);
}

void rocshmemx_slab_reset(rocshmemx_slab_t slab) {
  if (slab.cursor) rt().mem().zero(slab.cursor, sizeof(unsigned long long));
}

size_t rocshmemx_slab_used(rocshmemx_slab_t slab) {
  return slab.cursor ? static_cast<size_t>(slab_cursor_read(slab)) : 0;
}

void *rocshmemx_slab_alloc_host(rocshmemx_slab_t slab, size_t bytes, size_t align) {
  if (!slab.base || align == 0 || (align & (align - 1)) != 0 || align > 256) return nullptr;
  const unsigned long long cur = slab_cursor_read(slab);
  const unsigned long long start = detail::slab_place(slab, cur, bytes, align);
  if (start == ~0ull) return nullptr;
  const unsigned long long next = start + bytes;
  rt().mem().write(slab.cursor, &next, sizeof(next));
  return slab.base + start;
}

}  // namespace rocshmem

namespace rocshmem {
void rocshmemx_register_module(void (*upload)(const rocshmem_device_state *, int)) {
  Runtime::instance().register_module(upload);
}
}  // namespace rocshmem
