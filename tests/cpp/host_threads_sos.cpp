// Several host threads per process on the typed host API (ROCSHMEM_THREAD_MULTIPLE), in the style of the
// reference's pthread-based SOS programs (tests/sos_tests/threading.cpp, mt_contention.cpp, mt_a2a.cpp,
// thread_wait.cpp): every thread owns a context, all threads of all PEs add to one counter, every thread writes
// its slot on every PE, and thread t of PE p waits for thread t of PE p - 1. Run as several processes on the CPU
// shared-memory backend. Prints "PASS" on every PE.
#include <rocshmem/rocshmem.h>

#include <atomic>
#include <cstdio>
#include <thread>
#include <vector>

using namespace rocshmem;

static int g_me = -1;
static std::atomic<int> g_failures{0};
#define CHECK(cond)                                                                                  \
  do {                                                                                               \
    if (!(cond)) {                                                                                   \
      std::fprintf(stderr, "[pe %d] %s:%d: CHECK(%s) failed\n", g_me, __FILE__, __LINE__, #cond);   \
      g_failures.fetch_add(1);                                                                       \
    }                                                                                                \
  } while (0)

int main() {
  int provided = -1;
  rocshmem_init_thread(ROCSHMEM_THREAD_MULTIPLE, &provided);
  const int me = rocshmem_my_pe(), n = rocshmem_n_pes();
  g_me = me;
  CHECK(provided == ROCSHMEM_THREAD_MULTIPLE);
  constexpr int T = 6, ITERS = 300, W = 16;
  long *counter = static_cast<long *>(rocshmem_malloc(sizeof(long)));
  long *slots = static_cast<long *>(rocshmem_malloc(sizeof(long) * n * T * W));   // [source pe][thread][W]
  long *flags = static_cast<long *>(rocshmem_malloc(sizeof(long) * T));
  std::vector<long> zeros(n * T * W, 0);
  rocshmemx_heap_write(counter, zeros.data(), sizeof(long));
  rocshmemx_heap_write(slots, zeros.data(), sizeof(long) * n * T * W);
  rocshmemx_heap_write(flags, zeros.data(), sizeof(long) * T);
  // Source buffers of puts must be symmetric or plain host memory; plain host memory is fine for the host API.
  rocshmem_barrier_all();

  auto work = [&](int t) {
    rocshmem_ctx_t ctx;
    CHECK(rocshmem_ctx_create(0, &ctx) == 0);
    // contention: every thread of every PE adds to PE 0's counter; values fetched by one thread grow
    long last = -1;
    for (int i = 0; i < ITERS; ++i) {
      long old = rocshmem_ctx_long_atomic_fetch_add(ctx, counter, 1, 0);
      CHECK(old > last);
      last = old;
    }
    // all-to-all: my slot on every PE
    std::vector<long> mine(W, 1000L * me + t);
    for (int j = 0; j < n; ++j) {
      const int pe = (me + j) % n;
      rocshmem_ctx_long_put_nbi(ctx, slots + (size_t(me) * T + t) * W, mine.data(), W, pe);
    }
    rocshmem_ctx_quiet(ctx);
    // wait chain: PE 0's thread t starts, every other PE waits for its left neighbour's thread t
    if (me > 0) rocshmem_long_wait_until(flags + t, ROCSHMEM_CMP_EQ, 100L + t);
    if (me + 1 < n) rocshmem_ctx_long_atomic_set(ctx, flags + t, 100L + t, me + 1);
    rocshmem_ctx_destroy(ctx);
  };
  std::vector<std::thread> threads;
  for (int t = 0; t < T; ++t) threads.emplace_back(work, t);
  for (auto &th : threads) th.join();
  rocshmem_barrier_all();

  if (me == 0) CHECK(rocshmem_long_atomic_fetch(counter, 0) == long(n) * T * ITERS);
  std::vector<long> got(n * T * W);
  rocshmemx_heap_read(got.data(), slots, sizeof(long) * n * T * W);
  for (int p = 0; p < n; ++p) {
    for (int t = 0; t < T; ++t) {
      for (int w = 0; w < W; ++w) CHECK(got[(size_t(p) * T + t) * W + w] == 1000L * p + t);
    }
  }
  rocshmem_barrier_all();
  rocshmem_free(flags);
  rocshmem_free(slots);
  rocshmem_free(counter);
  rocshmem_finalize();
  if (g_failures.load()) {
    std::fprintf(stderr, "[pe %d] %d check(s) failed\n", me, g_failures.load());
    return 1;
  }
  std::printf("[pe %d] PASS\n", me);
  return 0;
}
