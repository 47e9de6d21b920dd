// A host-only C++ program over the typed host API, in the style of the reference's SOS tests (tests/sos_tests/:
// hello, barrier, shmalloc, put / get / bigput, atomics, wait / test, to_all, bcast, team translate / reduce,
// many-ctx). Compiled with g++ against the runtime library and run as several processes on the CPU
// shared-memory backend (ROCSHMEM_BACKEND=host, rendezvous through ROCSHMEM_BOOTSTRAP_DIR), so the C++ surface of
// the host API is exercised end to end without a GPU. Prints "PASS" on every PE; any failed check exits with 1.
// The reference's header names: every one of them must be enough on its own and they must combine.
#include <rocshmem/rocshmem.hpp>
#include <rocshmem/rocshmem_AMO.hpp>
#include <rocshmem/rocshmem_COLL.hpp>
#include <rocshmem/rocshmem_P2P_SYNC.hpp>
#include <rocshmem/rocshmem_RMA.hpp>
#include <rocshmem/rocshmem_RMA_X.hpp>
#include <rocshmem/rocshmem_SIG_OP.hpp>
#include <rocshmem/rocshmem_common.hpp>
#include <rocshmem/rocshmem_config.h>
#include <rocshmem/rocshmem_debug.hpp>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <vector>

using namespace rocshmem;

static int g_me = -1;
#define CHECK(cond)                                                                                  \
  do {                                                                                               \
    if (!(cond)) {                                                                                   \
      std::fprintf(stderr, "[pe %d] %s:%d: CHECK(%s) failed\n", g_me, __FILE__, __LINE__, #cond);   \
      std::fflush(stderr);                                                                           \
      rocshmem_global_exit(1);                                                                       \
    }                                                                                                \
  } while (0)

// The heap is not host-addressable in general: go through the copy helpers.
template <typename T>
static void fill(T *sym, size_t n, T first, T step) {
  std::vector<T> h(n);
  for (size_t i = 0; i < n; ++i) h[i] = static_cast<T>(first + step * static_cast<T>(i));
  rocshmemx_heap_write(sym, h.data(), n * sizeof(T));
}
template <typename T>
static std::vector<T> fetch(const T *sym, size_t n) {
  std::vector<T> h(n);
  rocshmemx_heap_read(h.data(), sym, n * sizeof(T));
  return h;
}

static_assert(ROCSHMEM_HAS_PEER_MAPPING && ROCSHMEM_HAS_REVERSE_OFFLOAD && !ROCSHMEM_HAS_NIC_BACKEND,
              "the configuration header describes the one build there is");
#ifdef USE_IPC
#error "the reference's bare option names are opt-in"
#endif

int main() {
  // identity before init (the reference's programs pick their GPU this way)
  const int env_pe = rocshmem_my_pe(), env_n = rocshmem_n_pes();
  rocshmem_init();
  const int me = rocshmem_my_pe(), n = rocshmem_n_pes();
  g_me = me;
  CHECK(me == env_pe && n == env_n && n >= 2);
  int provided = -1;
  rocshmem_query_thread(&provided);
  CHECK(provided == ROCSHMEM_THREAD_MULTIPLE);

  // shmalloc: symmetric, aligned, zero size and exhaustion give nullptr
  long *a = static_cast<long *>(rocshmem_malloc(1024 * sizeof(long)));
  long *b = static_cast<long *>(rocshmem_malloc(1024 * sizeof(long)));
  CHECK(a && b && reinterpret_cast<uintptr_t>(a) % 128 == 0 && a != b);
  CHECK(rocshmem_malloc(0) == nullptr);
  CHECK(rocshmem_malloc(size_t(1) << 40) == nullptr);

  // put / get to the right-hand neighbour, typed and untyped, blocking and non-blocking
  const int right = (me + 1) % n, left = (me + n - 1) % n;
  fill<long>(a, 1024, 1000L * me, 1L);
  fill<long>(b, 1024, -1L, 0L);
  rocshmem_barrier_all();
  rocshmem_long_put(b, a, 512, right);
  rocshmem_putmem_nbi(b + 512, a + 512, 512 * sizeof(long), right);
  rocshmem_quiet();
  rocshmem_barrier_all();
  {
    std::vector<long> got = fetch(b, 1024);
    for (int i = 0; i < 1024; ++i) CHECK(got[i] == 1000L * left + i);
  }
  std::vector<long> back(1024, 0);
  long *scratch = static_cast<long *>(rocshmem_malloc(1024 * sizeof(long)));
  rocshmem_long_get(scratch, b, 1024, right);       // what I wrote there
  back = fetch(scratch, 1024);
  for (int i = 0; i < 1024; ++i) CHECK(back[i] == 1000L * me + i);
  rocshmem_long_p(a, 77L + me, right);
  rocshmem_barrier_all();
  CHECK(rocshmem_long_g(a, me) == 77L + left);
  CHECK(rocshmem_long_g(a, right) == 77L + me);

  // atomics on PE 0: every family that the typed API offers for long and for the bitwise types
  long *ctr = static_cast<long *>(rocshmem_malloc(sizeof(long)));
  unsigned long *bits = static_cast<unsigned long *>(rocshmem_malloc(sizeof(unsigned long)));
  fill<long>(ctr, 1, 0L, 0L);
  fill<unsigned long>(bits, 1, 0UL, 0UL);
  rocshmem_barrier_all();
  for (int i = 0; i < 10; ++i) {
    long old = rocshmem_long_atomic_fetch_add(ctr, 2, 0);
    CHECK(old >= 0 && old < 21L * n);   // other PEs may already have added their final 1
  }
  rocshmem_long_atomic_inc(ctr, 0);
  rocshmem_ulong_atomic_or(bits, 1UL << me, 0);
  rocshmem_barrier_all();
  CHECK(rocshmem_long_atomic_fetch(ctr, 0) == 21L * n);
  CHECK(rocshmem_ulong_atomic_fetch(bits, 0) == (1UL << n) - 1UL);
  rocshmem_barrier_all();
  if (me == 0) {
    CHECK(rocshmem_long_atomic_compare_swap(ctr, 21L * n, 5L, 0) == 21L * n);
    CHECK(rocshmem_long_atomic_swap(ctr, 6L, 0) == 5L);
    rocshmem_long_atomic_set(ctr, 9L, 0);
    CHECK(rocshmem_long_atomic_fetch_inc(ctr, 0) == 9L);
    CHECK(rocshmem_ulong_atomic_fetch_and(bits, 1UL, 0) == (1UL << n) - 1UL);
    CHECK(rocshmem_ulong_atomic_fetch_xor(bits, 3UL, 0) == 1UL);
    CHECK(rocshmem_ulong_atomic_fetch(bits, 0) == 2UL);
  }
  rocshmem_barrier_all();

  // wait / test: a ring of flags, started by PE 0
  int *flag = static_cast<int *>(rocshmem_malloc(4 * sizeof(int)));
  fill<int>(flag, 4, 0, 0);
  CHECK(rocshmem_int_test(flag, ROCSHMEM_CMP_EQ, 0) == 1);   // before the barrier: afterwards the left neighbour may write
  rocshmem_barrier_all();
  if (me != 0) rocshmem_int_wait_until(flag, ROCSHMEM_CMP_EQ, me);
  if (right != 0) rocshmem_int_p(flag, right, right);
  rocshmem_barrier_all();
  if (me != 0) CHECK(rocshmem_int_test(flag, ROCSHMEM_CMP_GE, me) == 1);
  // wait_until_any over four slots: the left neighbour sets slot me % 4
  fill<int>(flag, 4, 0, 0);
  rocshmem_barrier_all();
  rocshmem_int_p(flag + (right % 4), 5, right);
  size_t which = rocshmem_int_wait_until_any(flag, 4, nullptr, ROCSHMEM_CMP_EQ, 5);
  CHECK(which == size_t(me % 4));
  rocshmem_barrier_all();

  // collectives on the world team: reduce (to_all), broadcast, fcollect, alltoall
  int *src = static_cast<int *>(rocshmem_malloc(64 * n * sizeof(int)));
  int *dst = static_cast<int *>(rocshmem_malloc(64 * n * sizeof(int)));
  fill<int>(src, 64 * n, 100 * me, 1);
  rocshmem_barrier_all();
  CHECK(rocshmem_ctx_int_sum_reduce(ROCSHMEM_CTX_DEFAULT, ROCSHMEM_TEAM_WORLD, dst, src, 64) == 0);
  {
    std::vector<int> got = fetch(dst, 64);
    for (int i = 0; i < 64; ++i) CHECK(got[i] == n * i + 100 * (n * (n - 1) / 2));
  }
  CHECK(rocshmem_ctx_int_max_reduce(ROCSHMEM_CTX_DEFAULT, ROCSHMEM_TEAM_WORLD, dst, src, 64) == 0);
  CHECK(fetch(dst, 1)[0] == 100 * (n - 1));
  fill<int>(dst, 64 * n, -7, 0);
  rocshmem_barrier_all();
  rocshmem_ctx_int_broadcast(ROCSHMEM_CTX_DEFAULT, ROCSHMEM_TEAM_WORLD, dst, src, 64, n - 1);
  {
    std::vector<int> got = fetch(dst, 64);
    for (int i = 0; i < 64; ++i) CHECK(got[i] == (me == n - 1 ? -7 : 100 * (n - 1) + i));  // the root keeps its dest
  }
  rocshmem_ctx_int_fcollect(ROCSHMEM_CTX_DEFAULT, ROCSHMEM_TEAM_WORLD, dst, src, 64);
  {
    std::vector<int> got = fetch(dst, 64 * n);
    for (int p = 0; p < n; ++p) CHECK(got[64 * p + 3] == 100 * p + 3);
  }
  rocshmem_ctx_int_alltoall(ROCSHMEM_CTX_DEFAULT, ROCSHMEM_TEAM_WORLD, dst, src, 64);
  {
    std::vector<int> got = fetch(dst, 64 * n);
    for (int p = 0; p < n; ++p) CHECK(got[64 * p + 1] == 100 * p + 64 * me + 1);
  }

  // teams: even PEs, translate, reduction on the team, reuse of the slot
  for (int round = 0; round < 3; ++round) {
    rocshmem_team_t evens = ROCSHMEM_TEAM_INVALID;
    const int n_even = (n + 1) / 2;
    CHECK(rocshmem_team_split_strided(ROCSHMEM_TEAM_WORLD, 0, 2, n_even, nullptr, 0, &evens) == 0);
    if (me % 2 == 0) {
      CHECK(evens != ROCSHMEM_TEAM_INVALID);
      CHECK(rocshmem_team_n_pes(evens) == n_even && rocshmem_team_my_pe(evens) == me / 2);
      CHECK(rocshmem_team_translate_pe(evens, me / 2, ROCSHMEM_TEAM_WORLD) == me);
      CHECK(rocshmem_team_translate_pe(ROCSHMEM_TEAM_WORLD, me, evens) == me / 2);
      CHECK(rocshmem_ctx_int_sum_reduce(ROCSHMEM_CTX_DEFAULT, evens, dst, src, 8) == 0);
      int want = 0;
      for (int p = 0; p < n; p += 2) want += 100 * p;
      CHECK(fetch(dst, 1)[0] == want);
      rocshmem_team_destroy(evens);
    } else {
      CHECK(evens == ROCSHMEM_TEAM_INVALID);
    }
    rocshmem_barrier_all();
  }
  if (n > 1) CHECK(rocshmem_team_translate_pe(ROCSHMEM_TEAM_WORLD, n, ROCSHMEM_TEAM_WORLD) == -1);

  // many contexts: create, use and destroy more contexts than the pool holds at once
  for (int i = 0; i < 100; ++i) {
    rocshmem_ctx_t ctx;
    CHECK(rocshmem_ctx_create(0, &ctx) == 0);
    rocshmem_ctx_long_p(ctx, a + 1, 1000L + i, right);
    rocshmem_ctx_quiet(ctx);
    rocshmem_ctx_destroy(ctx);
  }
  rocshmem_barrier_all();
  CHECK(rocshmem_long_g(a + 1, me) == 1099L);

  // the pool of host contexts is finite: creation reports it with -1, and destroying makes room again
  {
    std::vector<rocshmem_ctx_t> pool;
    for (;;) {
      rocshmem_ctx_t ctx;
      if (rocshmem_ctx_create(0, &ctx) != 0) break;
      pool.push_back(ctx);
      CHECK(pool.size() <= 4096);
    }
    CHECK(pool.size() == 39);                     // ROCSHMEM_MAX_NUM_HOST_CONTEXTS = 40, one is the default context
    for (rocshmem_ctx_t &ctx : pool) rocshmem_ctx_destroy(ctx);
    rocshmem_ctx_t again;
    CHECK(rocshmem_ctx_create(0, &again) == 0);
    rocshmem_ctx_destroy(again);
  }
  // misuse is reported, not fatal: freeing nothing is a no-op, freeing a foreign pointer and naming a PE that does
  // not exist raise exceptions, queries on the invalid team answer -1
  rocshmem_free(nullptr);
  bool threw = false;
  try {
    rocshmem_free(&threw);
  } catch (const std::exception &) {
    threw = true;
  }
  CHECK(threw);
  threw = false;
  try {
    rocshmem_long_p(a, 1L, n + 3);
  } catch (const std::exception &) {
    threw = true;
  }
  CHECK(threw);
  CHECK(rocshmem_team_n_pes(ROCSHMEM_TEAM_INVALID) == -1 && rocshmem_team_my_pe(ROCSHMEM_TEAM_INVALID) == -1);
  rocshmem_team_destroy(ROCSHMEM_TEAM_INVALID);

  // rocshmem_ptr: the peer's address of a symmetric object, nullptr for a bad PE or a foreign pointer
  CHECK(rocshmem_ptr(a, right) != nullptr && rocshmem_ptr(a, n) == nullptr);
  int on_stack = 0;
  CHECK(rocshmem_ptr(&on_stack, right) == nullptr);

  rocshmem_barrier_all();
  for (void *p : {static_cast<void *>(dst), static_cast<void *>(src), static_cast<void *>(flag), static_cast<void *>(bits),
                  static_cast<void *>(ctr), static_cast<void *>(scratch), static_cast<void *>(b), static_cast<void *>(a)}) {
    rocshmem_free(p);
  }
  // No proxy thread on this backend: the queue dump says so instead of failing.
  if (rocshmem_my_pe() == 0) {
    debug_print_ring(0, 2);
    debug_print_sq(1, 0, 0);
    debug_print_cq(1, 0, 0);
  }
  rocshmem_finalize();
  std::printf("[pe %d] PASS\n", me);
  return 0;
}
