// Several host threads produce into the reverse-offload command ring while its consumer thread drains it, with
// merging of contiguous commands switched on: fire-and-forget puts whose pieces follow on one another, blocking
// gets and fetching atomics. Uses the runtime's internal Proxy class directly (the public API reaches it only from
// device code), on the CPU shared-memory backend with two PEs in one process. Built with ThreadSanitizer by the
// test that drives it, so that data races between producers and consumer surface. Prints "PASS".
#include <rocshmem/rocshmem.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

#include "runtime/proxy.hpp"
#include "runtime/runtime.hpp"

using namespace rocshmem;

static std::atomic<int> g_failures{0};
#define CHECK(cond)                                                                       \
  do {                                                                                    \
    if (!(cond)) {                                                                        \
      std::fprintf(stderr, "%s:%d: CHECK(%s) failed\n", __FILE__, __LINE__, #cond);      \
      g_failures.fetch_add(1);                                                            \
    }                                                                                     \
  } while (0)

static rocshmem_proxy_cmd command(unsigned type, int pe, void *dst, const void *src, unsigned long long size,
                                  unsigned dtype_size) {
  rocshmem_proxy_cmd c;
  std::memset(&c, 0, sizeof(c));
  c.type = type;
  c.pe = pe;
  c.dst = reinterpret_cast<unsigned long long>(dst);
  c.src = reinterpret_cast<unsigned long long>(src);
  c.size = size;
  c.dtype_size = dtype_size;
  return c;
}

int main() {
  rocshmem_init();   // ROCSHMEM_BACKEND=host, ROCSHMEM_LOCAL_PES=2 from the environment
  CHECK(rocshmem_n_pes() == 2);
  constexpr int T = 4, PIECES = 256, PIECE = 64;
  char *src = static_cast<char *>(rocshmem_malloc(T * PIECES * PIECE));
  char *dst = static_cast<char *>(rocshmem_malloc(T * PIECES * PIECE));
  char *back = static_cast<char *>(rocshmem_malloc(T * PIECES * PIECE));
  long *ctr = static_cast<long *>(rocshmem_malloc(sizeof(long)));
  std::vector<char> pattern(T * PIECES * PIECE);
  for (size_t i = 0; i < pattern.size(); ++i) pattern[i] = static_cast<char>(i * 7 + 3);
  rocshmemx_heap_write(src, pattern.data(), pattern.size());
  std::vector<char> zeros(pattern.size(), 0);
  rocshmemx_heap_write(dst, zeros.data(), zeros.size());     // PE 0's copy; PE 1's starts zeroed by malloc? be explicit:
  rocshmemx_heap_write(rocshmem_ptr(dst, 1), zeros.data(), zeros.size());
  long zero = 0;
  rocshmemx_heap_write(rocshmem_ptr(ctr, 1), &zero, sizeof(zero));

  Proxy proxy(&Runtime::instance());
  proxy.start();
  proxy.set_coalesce(true);
  auto work = [&](int t) {
    char *my_src = src + size_t(t) * PIECES * PIECE, *my_dst = dst + size_t(t) * PIECES * PIECE;
    for (int i = 0; i < PIECES; ++i) {
      rocshmem_proxy_cmd c = command(ROCSHMEM_PROXY_PUT, 1, my_dst + i * PIECE, my_src + i * PIECE, PIECE, 1);
      CHECK(proxy.submit(c, false, nullptr, 20000) == ROCSHMEM_SUCCESS);
      if (i % 16 == 15) {
        uint64_t old = 0;
        rocshmem_proxy_cmd a = command(ROCSHMEM_PROXY_AMO_FADD, 1, ctr, nullptr, 1, 8);
        CHECK(proxy.submit(a, true, &old, 20000) == ROCSHMEM_SUCCESS);
      }
    }
    // A blocking command is executed after everything this thread published before it.
    rocshmem_proxy_cmd q = command(ROCSHMEM_PROXY_QUIET, 0, nullptr, nullptr, 0, 0);
    CHECK(proxy.submit(q, true, nullptr, 20000) == ROCSHMEM_SUCCESS);
    char *my_back = back + size_t(t) * PIECES * PIECE;
    for (int i = 0; i < PIECES; i += 8) {
      rocshmem_proxy_cmd g = command(ROCSHMEM_PROXY_GET, 1, my_back + i * PIECE, my_dst + i * PIECE, 8 * PIECE, 1);
      CHECK(proxy.submit(g, true, nullptr, 20000) == ROCSHMEM_SUCCESS);
    }
  };
  std::vector<std::thread> threads;
  for (int t = 0; t < T; ++t) threads.emplace_back(work, t);
  for (auto &th : threads) th.join();
  const uint64_t executed = proxy.executed(), merged = proxy.merged();
  proxy.stop();

  std::vector<char> got(pattern.size());
  rocshmemx_heap_read(got.data(), rocshmem_ptr(dst, 1), got.size());
  CHECK(got == pattern);
  rocshmemx_heap_read(got.data(), back, got.size());
  CHECK(got == pattern);
  long count = 0;
  rocshmemx_heap_read(&count, rocshmem_ptr(ctr, 1), sizeof(count));
  CHECK(count == T * PIECES / 16);
  const uint64_t submitted = uint64_t(T) * (PIECES + PIECES / 16 + 1 + PIECES / 8);
  CHECK(executed + merged == submitted);
  std::printf("commands %llu, executed %llu, merged %llu\n", (unsigned long long)submitted,
              (unsigned long long)executed, (unsigned long long)merged);
  rocshmem_free(ctr);
  rocshmem_free(back);
  rocshmem_free(dst);
  rocshmem_free(src);
  rocshmem_finalize();
  if (g_failures.load()) return 1;
  std::printf("PASS\n");
  return 0;
}
