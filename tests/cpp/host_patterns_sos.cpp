// Communication patterns over the typed host API, after the programs of the reference's tests/sos_tests/ that
// host_api_sos.cpp does not already follow: a flood of broadcasts from rotating roots (bcast_flood), reductions in
// place, over an active set and of a large vector (reduce_in_place, reduce_active_set, max_reduction, big_reduction),
// a circular shift (circular_shift), a Monte-Carlo estimate of pi reduced over all PEs (pi), ping-pong with
// wait_until (ping, sping), lock-free increments of one word (lfinc), large puts and gets (bigput, bigget),
// allocations whose requested sizes differ between PEs inside one block (asym_alloc), back-to-back collectives
// on two overlapping teams (shmem_team_b2b_collectives), and a context bandwidth / message-rate loop with several
// threads (put_ctx_mbw_mr). With the argument "exit" PE 1 ends the job through rocshmem_global_exit(7)
// (global_exit). Prints "PASS" on every PE; a failed check ends the job with exit code 1.
#include <rocshmem/rocshmem.hpp>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <thread>
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

template <typename T>
static void put_host(T *sym, const std::vector<T> &h) { rocshmemx_heap_write(sym, h.data(), h.size() * sizeof(T)); }
template <typename T>
static std::vector<T> get_host(const T *sym, size_t n) {
  std::vector<T> h(n);
  rocshmemx_heap_read(h.data(), sym, n * sizeof(T));
  return h;
}

int main(int argc, char **argv) {
  rocshmem_init();
  const int me = rocshmem_my_pe(), n = rocshmem_n_pes();
  g_me = me;
  CHECK(n >= 2);
  if (argc > 1 && std::strcmp(argv[1], "exit") == 0) {
    rocshmem_barrier_all();
    if (me == 1) rocshmem_global_exit(7);
    // The others would wait for ever: global_exit has to end them too.
    long *never = static_cast<long *>(rocshmem_malloc(sizeof(long)));
    rocshmem_long_wait_until(never, ROCSHMEM_CMP_EQ, 12345L);
    return 3;
  }
  const int right = (me + 1) % n, left = (me + n - 1) % n;

  // asym_alloc: me + 1 ints per PE (one allocator block everywhere), written by the left neighbour
  {
    int *buf = static_cast<int *>(rocshmem_malloc(sizeof(int) * (me + 1)));
    CHECK(buf != nullptr);
    put_host<int>(buf, std::vector<int>(me + 1, -1));
    rocshmem_barrier_all();
    std::vector<int> out(right + 1, right);
    rocshmem_int_put(buf, out.data(), right + 1, right);
    rocshmem_barrier_all();
    for (int v : get_host(buf, me + 1)) CHECK(v == me);
    rocshmem_free(buf);
  }

  // bcast_flood: 200 broadcasts back to back, the root rotates, nothing between them but the collective itself
  {
    constexpr int N = 257;
    long *src = static_cast<long *>(rocshmem_malloc(N * sizeof(long)));
    long *dst = static_cast<long *>(rocshmem_malloc(N * sizeof(long)));
    for (int it = 0; it < 200; ++it) {
      const int root = it % n;
      if (me == root) put_host<long>(src, std::vector<long>(N, 1000L * it + root));
      rocshmem_ctx_long_broadcast(ROCSHMEM_CTX_DEFAULT, ROCSHMEM_TEAM_WORLD, dst, src, N, root);
      if (me != root) {
        std::vector<long> got = get_host(dst, N);
        CHECK(got[0] == 1000L * it + root && got[N - 1] == 1000L * it + root);
      }
    }
    rocshmem_barrier_all();
    rocshmem_free(dst);
    rocshmem_free(src);
  }

  // reduce_in_place + max_reduction + big_reduction: one million doubles, source == dest
  {
    constexpr size_t N = 1 << 20;
    double *v = static_cast<double *>(rocshmem_malloc(N * sizeof(double)));
    CHECK(v != nullptr);
    std::vector<double> h(N);
    for (size_t i = 0; i < N; ++i) h[i] = double(i % 1000) + me;
    put_host(v, h);
    rocshmem_barrier_all();
    CHECK(rocshmem_ctx_double_sum_reduce(ROCSHMEM_CTX_DEFAULT, ROCSHMEM_TEAM_WORLD, v, v, N) == 0);
    std::vector<double> got = get_host(v, N);
    for (size_t i = 0; i < N; i += 4099) CHECK(got[i] == n * double(i % 1000) + n * (n - 1) / 2.0);
    put_host(v, h);
    rocshmem_barrier_all();
    CHECK(rocshmem_ctx_double_max_reduce(ROCSHMEM_CTX_DEFAULT, ROCSHMEM_TEAM_WORLD, v, v, N) == 0);
    got = get_host(v, N);
    for (size_t i = 0; i < N; i += 4099) CHECK(got[i] == double(i % 1000) + (n - 1));
    rocshmem_barrier_all();
    rocshmem_free(v);
  }

  // reduce_active_set + team b2b collectives: the lower half and the even PEs overlap in PE 0; each team runs
  // reduce, broadcast, fcollect and alltoall back to back with no barrier between them, several times
  {
    constexpr int N = 32;
    int *src = static_cast<int *>(rocshmem_malloc(N * n * sizeof(int)));
    int *dst = static_cast<int *>(rocshmem_malloc(N * n * sizeof(int)));
    std::vector<int> h(N * n);
    for (int i = 0; i < N * n; ++i) h[i] = 10 * me + i % 7;
    put_host(src, h);
    rocshmem_barrier_all();
    const int n_low = (n + 1) / 2, n_even = (n + 1) / 2;
    rocshmem_team_t low = ROCSHMEM_TEAM_INVALID, even = ROCSHMEM_TEAM_INVALID;
    CHECK(rocshmem_team_split_strided(ROCSHMEM_TEAM_WORLD, 0, 1, n_low, nullptr, 0, &low) == 0);
    CHECK(rocshmem_team_split_strided(ROCSHMEM_TEAM_WORLD, 0, 2, n_even, nullptr, 0, &even) == 0);
    struct Use { rocshmem_team_t team; int first, stride, size; };
    for (const Use &u : {Use{low, 0, 1, n_low}, Use{even, 0, 2, n_even}}) {
      if (u.team == ROCSHMEM_TEAM_INVALID) continue;
      const int idx = rocshmem_team_my_pe(u.team);
      CHECK(idx >= 0 && u.first + idx * u.stride == me);
      for (int it = 0; it < 5; ++it) {
        CHECK(rocshmem_ctx_int_sum_reduce(ROCSHMEM_CTX_DEFAULT, u.team, dst, src, N) == 0);
        int want = 0;
        for (int j = 0; j < u.size; ++j) want += 10 * (u.first + j * u.stride) + 3;
        CHECK(get_host(dst, N)[3] == want);
        rocshmem_ctx_int_broadcast(ROCSHMEM_CTX_DEFAULT, u.team, dst, src, N, u.size - 1);
        if (idx != u.size - 1) CHECK(get_host(dst, N)[5] == 10 * (u.first + (u.size - 1) * u.stride) + 5);
        rocshmem_ctx_int_fcollect(ROCSHMEM_CTX_DEFAULT, u.team, dst, src, N);
        for (int j = 0; j < u.size; ++j) CHECK(get_host(dst, N * u.size)[N * j] == 10 * (u.first + j * u.stride));
        rocshmem_ctx_int_alltoall(ROCSHMEM_CTX_DEFAULT, u.team, dst, src, N);
        for (int j = 0; j < u.size; ++j) {
          CHECK(get_host(dst, N * u.size)[N * j + 1] == 10 * (u.first + j * u.stride) + (N * idx + 1) % 7);
        }
      }
      rocshmem_team_destroy(u.team);
    }
    rocshmem_barrier_all();
    rocshmem_free(dst);
    rocshmem_free(src);
  }

  // circular_shift, bigput, bigget: 8 MiB to the right-hand neighbour, then fetched back from it
  {
    constexpr size_t N = size_t(1) << 20;  // longs
    long *a = static_cast<long *>(rocshmem_malloc(N * sizeof(long)));
    long *b = static_cast<long *>(rocshmem_malloc(N * sizeof(long)));
    CHECK(a && b);
    std::vector<long> h(N);
    for (size_t i = 0; i < N; ++i) h[i] = long(i) * 3 + me;
    put_host(a, h);
    rocshmem_barrier_all();
    rocshmem_long_put(b, a, N, right);
    rocshmem_barrier_all();
    std::vector<long> got = get_host(b, N);
    for (size_t i = 0; i < N; i += 997) CHECK(got[i] == long(i) * 3 + left);
    std::vector<long> back(N);
    rocshmem_long_get(back.data(), b, N, right);  // what I put there
    for (size_t i = 0; i < N; i += 997) CHECK(back[i] == long(i) * 3 + me);
    rocshmem_barrier_all();
    rocshmem_free(b);
    rocshmem_free(a);
  }

  // pi: darts thrown by every PE, hits summed over all PEs
  {
    long long *hits = static_cast<long long *>(rocshmem_malloc(2 * sizeof(long long)));
    std::mt19937_64 rng(1234 + me);
    std::uniform_real_distribution<double> u(0.0, 1.0);
    constexpr long long THROWS = 200000;
    long long in = 0;
    for (long long i = 0; i < THROWS; ++i) {
      const double x = u(rng), y = u(rng);
      in += x * x + y * y <= 1.0;
    }
    put_host<long long>(hits, {in, 0});
    rocshmem_barrier_all();
    CHECK(rocshmem_ctx_longlong_sum_reduce(ROCSHMEM_CTX_DEFAULT, ROCSHMEM_TEAM_WORLD, hits + 1, hits, 1) == 0);
    const double pi = 4.0 * double(get_host(hits, 2)[1]) / double(THROWS * n);
    CHECK(std::fabs(pi - 3.14159265) < 0.02);
    rocshmem_barrier_all();
    rocshmem_free(hits);
  }

  // ping / sping: PE 0 and PE 1 bounce a counter 500 times with p + wait_until; the others watch a barrier
  {
    long *ball = static_cast<long *>(rocshmem_malloc(sizeof(long)));
    put_host<long>(ball, {0});
    rocshmem_barrier_all();
    constexpr int ROUNDS = 500;
    auto t0 = std::chrono::steady_clock::now();
    if (me == 0) {
      for (long r = 1; r <= ROUNDS; ++r) {
        rocshmem_long_p(ball, r, 1);
        rocshmem_long_wait_until(ball, ROCSHMEM_CMP_EQ, r);
      }
    } else if (me == 1) {
      for (long r = 1; r <= ROUNDS; ++r) {
        rocshmem_long_wait_until(ball, ROCSHMEM_CMP_EQ, r);
        rocshmem_long_p(ball, r, 0);
      }
    }
    const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
    if (me == 0) std::printf("[pe 0] ping-pong round trip %.2f us\n", us / ROUNDS);
    rocshmem_barrier_all();
    rocshmem_free(ball);
  }

  // lfinc: every PE increments a word on its right-hand neighbour 2000 times without fetching
  {
    long *word = static_cast<long *>(rocshmem_malloc(sizeof(long)));
    put_host<long>(word, {0});
    rocshmem_barrier_all();
    for (int i = 0; i < 2000; ++i) rocshmem_long_atomic_inc(word, right);
    rocshmem_barrier_all();
    CHECK(get_host(word, 1)[0] == 2000);
    rocshmem_barrier_all();
    rocshmem_free(word);
  }

  // put_ctx_mbw_mr: four threads, a private context each, windows of 64 non-blocking puts closed by a quiet
  {
    constexpr int THREADS = 4, WINDOW = 64, WINDOWS = 20;
    constexpr size_t BYTES = 4096;
    char *land = static_cast<char *>(rocshmem_malloc(BYTES * THREADS));
    CHECK(land != nullptr);
    rocshmem_barrier_all();
    std::vector<double> secs(THREADS, 0.0);
    std::vector<std::thread> threads;
    for (int t = 0; t < THREADS; ++t) {
      threads.emplace_back([&, t] {
        rocshmem_ctx_t ctx;
        if (rocshmem_ctx_create(ROCSHMEM_CTX_SERIALIZED, &ctx) != 0) return;
        std::vector<char> payload(BYTES, static_cast<char>(16 * me + t));
        auto t0 = std::chrono::steady_clock::now();
        for (int w = 0; w < WINDOWS; ++w) {
          for (int i = 0; i < WINDOW; ++i) rocshmem_ctx_putmem_nbi(ctx, land + BYTES * t, payload.data(), BYTES, right);
          rocshmem_ctx_quiet(ctx);
        }
        secs[t] = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        rocshmem_ctx_destroy(ctx);
      });
    }
    for (auto &th : threads) th.join();
    rocshmem_barrier_all();
    std::vector<char> got = get_host(land, BYTES * THREADS);
    double slowest = 0;
    for (int t = 0; t < THREADS; ++t) {
      CHECK(secs[t] > 0.0);
      CHECK(got[BYTES * t] == static_cast<char>(16 * left + t) && got[BYTES * t + BYTES - 1] == static_cast<char>(16 * left + t));
      slowest = std::max(slowest, secs[t]);
    }
    if (me == 0) {
      const double msgs = double(THREADS) * WINDOW * WINDOWS;
      std::printf("[pe 0] %d threads x %zu B: %.0f msg/s, %.3f GB/s\n", THREADS, BYTES, msgs / slowest,
                  msgs * BYTES / slowest * 1e-9);
    }
    rocshmem_barrier_all();
    rocshmem_free(land);
  }

  rocshmem_finalize();
  std::printf("[pe %d] PASS\n", me);
  return 0;
}
