// Native unit tests of the host-side runtime pieces that need no GPU: allocator, team arithmetic,
// configuration parsing and the bootstrap store. The program is built twice by the Python test that drives it,
// with AddressSanitizer + UBSan and with ThreadSanitizer, so that memory errors, undefined behaviour and data
// races in these components surface without any device. (The reference's unit tests are gtest programs over the
// same kind of pieces: tests/unit_tests/*.)
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <set>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "allocator.hpp"
#include "bootstrap.hpp"
#include "config.hpp"
#include "rocshmem/coalesce.h"
#include "rocshmem/slab.h"
#include "team.hpp"
#include "../kernels/coll_select.hpp"
#include "../kernels/ep_kernels.hpp"

using namespace rocshmem;

static int g_failures = 0;
#define EXPECT(cond)                                                                  \
  do {                                                                                \
    if (!(cond)) {                                                                    \
      std::fprintf(stderr, "%s:%d: EXPECT(%s) failed\n", __FILE__, __LINE__, #cond);  \
      ++g_failures;                                                                   \
    }                                                                                 \
  } while (0)

static void test_allocator_basic() {
  Pow2Allocator a(1 << 20, 128);
  EXPECT(a.alloc(0) == Pow2Allocator::kNull);
  const size_t x = a.alloc(100), y = a.alloc(129);
  EXPECT(x == 0 && a.block_size(x) == 128);
  EXPECT(y == 256 && a.block_size(y) == 256);   // a 256-byte block is 256-aligned
  EXPECT(a.used() == 384);
  EXPECT(!a.free(64));                          // not a live allocation
  EXPECT(a.free(x) && a.free(y));
  EXPECT(a.used() == 0 && a.largest_free_block() == (1u << 20));   // buddies merged back
  EXPECT(a.alloc((1 << 20) + 1) == Pow2Allocator::kNull);
}

static void test_allocator_random_walk() {
  // Random alloc / free sequence: live blocks never overlap, stay aligned, and everything merges back.
  Pow2Allocator a((3u << 20) + 4096, 128);      // not a power of two: several top-level chunks
  std::mt19937 rng(7);
  std::vector<std::pair<size_t, size_t>> live;  // offset, size
  for (int step = 0; step < 20000; ++step) {
    if (live.empty() || rng() % 3 != 0) {
      const size_t want = 1 + rng() % 70000;
      const size_t off = a.alloc(want);
      if (off == Pow2Allocator::kNull) continue;
      const size_t sz = a.block_size(off);
      EXPECT(sz >= want && (sz & (sz - 1)) == 0 && off % 128 == 0 && off + sz <= a.size());
      for (const auto &l : live) EXPECT(off + sz <= l.first || l.first + l.second <= off);
      live.emplace_back(off, sz);
    } else {
      const size_t i = rng() % live.size();
      EXPECT(a.free(live[i].first));
      live[i] = live.back();
      live.pop_back();
    }
  }
  for (const auto &l : live) EXPECT(a.free(l.first));
  EXPECT(a.used() == 0 && a.live_allocations() == 0);
  EXPECT(a.largest_free_block() == (2u << 20));
}

static void test_allocator_is_deterministic() {
  // Two instances fed the same call sequence return the same offsets: what makes the heap symmetric.
  Pow2Allocator a(1 << 22), b(1 << 22);
  std::mt19937 rng(11);
  std::vector<size_t> held;
  for (int step = 0; step < 5000; ++step) {
    if (held.empty() || rng() % 2) {
      const size_t want = 1 + rng() % 9000;
      const size_t oa = a.alloc(want), ob = b.alloc(want);
      EXPECT(oa == ob);
      if (oa != Pow2Allocator::kNull) held.push_back(oa);
    } else {
      const size_t i = rng() % held.size();
      EXPECT(a.free(held[i]) == b.free(held[i]));
      held[i] = held.back();
      held.pop_back();
    }
  }
}

static void test_team_math() {
  const TeamTriplet world{0, 1, 8};
  SplitPlan p = plan_split(world, 8, 8, 1, 2, 4);   // {1, 3, 5, 7}
  EXPECT(p.ok && p.world.pe_start == 1 && p.world.stride == 2 && p.world.size == 4);
  EXPECT(p.world.pe_in_team(5) == 2 && p.world.pe_in_team(4) == -1 && p.world.pe_in_world(3) == 7);
  EXPECT(translate_pe(p.world, 3, world) == 7 && translate_pe(world, 6, p.world) == -1);
  SplitPlan q = plan_split(p.world, 4, 8, 1, 2, 2);  // members 1 and 3 of the parent: world {3, 7}
  EXPECT(q.ok && q.world.pe_start == 3 && q.world.stride == 4 && q.world.size == 2);
  EXPECT(!plan_split(world, 8, 8, 0, 0, 2).ok);      // stride < 1
  EXPECT(!plan_split(world, 8, 8, 6, 2, 3).ok);      // runs past the parent
  EXPECT(!plan_split(world, 8, 8, -1, 1, 2).ok);
  TeamSlots s(40);
  EXPECT(s.in_use() == 0 && s.capacity() == 40);
  EXPECT(s.take(0));                                 // the runtime reserves slot 0 for the world team
  std::vector<uint64_t> masks = {s.mask(), s.mask() & ~uint64_t(2)};
  EXPECT(TeamSlots::lowest_common(masks) == 2);      // slot 0 is taken everywhere, slot 1 on one member
  EXPECT(s.take(2) && !s.take(2) && s.in_use() == 2);
  s.release(2);
  EXPECT(s.take(2));
  EXPECT(!s.take(40) && !s.take(-1));
  EXPECT(TeamSlots::lowest_common({0x4, 0x8}) == -1);
}

static void test_config() {
  EXPECT(parse_size("64M") == (size_t(64) << 20) && parse_size("0x100") == 256 && parse_size("2G") == (size_t(2) << 30));
  bool threw = false;
  try { parse_size("12Q"); } catch (const std::invalid_argument &) { threw = true; }
  EXPECT(threw);
  Config c = Config::from_env({{"ROCSHMEM_HEAP_SIZE", "8M"}, {"ROCSHMEM_MAX_NUM_TEAMS", "12"}});
  EXPECT(c.heap_size == (size_t(8) << 20) && c.max_teams == 12);
  c.validate();
  threw = false;
  try { Config::from_env({{"ROCSHMEM_WAIT_TIMEOUT_MS", "0"}}).validate(); } catch (const std::invalid_argument &) { threw = true; }
  EXPECT(threw);
}

static void test_file_bootstrap_between_threads(const std::string &dir) {
  // Four "ranks" as threads of this process, each with its own FileBootstrap over one directory: allgather,
  // barrier and a group allgather, repeated so that the per-tag sequence numbers are exercised.
  constexpr int kRanks = 4;
  std::atomic<int> bad{0};
  std::vector<std::thread> threads;
  for (int r = 0; r < kRanks; ++r) {
    threads.emplace_back([&, r] {
      try {
        FileBootstrap bs(dir, r, kRanks);
        bs.set_timeout_ms(20000);
        for (int round = 0; round < 5; ++round) {
          int mine = 100 * round + r, all[kRanks] = {};
          bs.allgather("ag", &mine, all, sizeof(int));
          for (int i = 0; i < kRanks; ++i) bad += all[i] != 100 * round + i;
          bs.barrier("bar");
          if (r % 2 == 1) {   // group of the odd ranks
            int pair[2] = {};
            bs.allgather_group("odd", {1, 3}, r / 2, &mine, pair, sizeof(int));
            bad += pair[0] != 100 * round + 1 || pair[1] != 100 * round + 3;
          }
        }
        // a key nobody writes: the bounded get reports instead of hanging
        bool threw = false;
        try { bs.get("never-" + std::to_string(r), 50); } catch (const BootstrapError &) { threw = true; }
        bad += !threw;
      } catch (const std::exception &e) {
        std::fprintf(stderr, "rank %d: %s\n", r, e.what());
        ++bad;
      }
    });
  }
  for (auto &t : threads) t.join();
  EXPECT(bad.load() == 0);
}

// Lane arithmetic of the warp coalescer against a lane-by-lane walk, on random warps (every shift and mask in
// it runs under UBSan here), and the list form.
static void test_coalesce() {
  std::mt19937_64 rng(11);
  for (int round = 0; round < 2000; ++round) {
    unsigned active = static_cast<unsigned>(rng()) | (1u << (rng() % 32));
    if (round == 0) active = 0xffffffffu;
    if (round == 1) active = 0x80000001u;
    coalesce::Msg m[32];
    unsigned long long dst = 0x10000, src = 0x80000;
    for (int l = 0; l < 32; ++l) {
      unsigned long long size = (rng() % 4) ? 8 : 16;
      if (rng() % 5 == 0) dst += 64;
      m[l] = coalesce::Msg{(rng() % 10) ? 1 : 2, dst, src, size};
      if (active & (1u << l)) {
        dst += size;
        src += size;
      }
    }
    unsigned cont = 0;
    for (int l = 0; l < 32; ++l) {
      if (!(active & (1u << l))) continue;
      int p = coalesce::previous_active(active, l);
      EXPECT(p < l);
      if (p >= 0 && coalesce::continues(m[p], m[l])) cont |= 1u << l;
    }
    int covered = 0, lanes = 0;
    for (int l = 0; l < 32; ++l) {
      int n = coalesce::run_length(active, cont, l);
      covered += n;
      if (active & (1u << l)) ++lanes;
      if (n > 0) {
        // the run is n consecutive active lanes starting here, all but the first continuing their predecessor
        int seen = 1, q = l + 1;
        for (; q < 32 && seen < n; ++q) {
          if (!(active & (1u << q))) continue;
          EXPECT(cont & (1u << q));
          ++seen;
        }
        EXPECT(seen == n);
        for (; q < 32; ++q) {
          if (active & (1u << q)) {
            EXPECT(!(cont & (1u << q)));   // the next active lane starts a new run
            break;
          }
        }
      }
    }
    EXPECT(covered == lanes);
  }
  coalesce::Msg list[5] = {{1, 100, 500, 10}, {1, 110, 510, 10}, {2, 120, 520, 10}, {2, 130, 530, 10}, {2, 150, 550, 10}};
  EXPECT(coalesce::merge_runs(list, 5) == 3);
  EXPECT(list[0].size == 20 && list[1].size == 20 && list[1].pe == 2 && list[2].dst == 150);
  EXPECT(coalesce::merge_runs(list, 0) == 0);
}

// Placement arithmetic shared by the host and device halves of the slab allocator.
static void test_slab_place() {
  rocshmemx_slab_t s{nullptr, 4096, nullptr};
  EXPECT(detail::slab_place(s, 0, 100, 16) == 0);
  EXPECT(detail::slab_place(s, 100, 1, 1) == 100);
  EXPECT(detail::slab_place(s, 101, 64, 256) == 256);
  EXPECT(detail::slab_place(s, 0, 4096, 16) == 0);
  EXPECT(detail::slab_place(s, 0, 4097, 16) == ~0ull);
  EXPECT(detail::slab_place(s, 4090, 8, 16) == ~0ull);     // rounding up leaves the slab
  EXPECT(detail::slab_place(s, 4096, 1, 1) == ~0ull);
  EXPECT(detail::slab_place(s, 0, 0, 16) == ~0ull);
  EXPECT(detail::slab_place(s, 0, ~0ull, 16) == ~0ull);    // no overflow in the fit test
}

static void test_allreduce_selection() {
  using namespace rocshmem::kernels;
  auto pick = [](int algo, size_t bytes, size_t esz, int n, bool mc, bool sum = true, bool mm = true, uintptr_t dst = 0x1000,
                 uintptr_t src = 0x200000) {
    return select_allreduce(AllreduceRequest{algo, bytes, esz, n, mc, sum, mm, dst, src});
  };
  // automatic choice by size: flag-in-word up to 2 KiB of 2- or 4-byte elements, one-shot up to 256 KiB, then the
  // switch for teams of four or more with a multicast mapping, else two-shot
  EXPECT(pick(ALLREDUCE_AUTO, 1024, 2, 8, true) == ALLREDUCE_LL);
  EXPECT(pick(ALLREDUCE_AUTO, ROCSHMEM_LL_WORDS * 4, 4, 2, false) == ALLREDUCE_LL);
  EXPECT(pick(ALLREDUCE_AUTO, ROCSHMEM_LL_WORDS * 4 + 4, 4, 2, false) == ALLREDUCE_ONE_SHOT);
  EXPECT(pick(ALLREDUCE_AUTO, 1024, 8, 8, true) == ALLREDUCE_ONE_SHOT);            // 8-byte elements have no mailbox form
  EXPECT(pick(ALLREDUCE_AUTO, 1022, 2, 8, true) == ALLREDUCE_ONE_SHOT);            // not whole words
  EXPECT(pick(ALLREDUCE_AUTO, 1024, 2, 8, true, true, true, 0x1002) == ALLREDUCE_ONE_SHOT);   // not 4-byte aligned
  EXPECT(pick(ALLREDUCE_AUTO, size_t(256) << 10, 2, 8, true) == ALLREDUCE_ONE_SHOT);
  EXPECT(pick(ALLREDUCE_AUTO, (size_t(256) << 10) + 16, 2, 8, true) == ALLREDUCE_NVLS);
  EXPECT(pick(ALLREDUCE_AUTO, size_t(64) << 20, 2, 4, true) == ALLREDUCE_NVLS);
  EXPECT(pick(ALLREDUCE_AUTO, size_t(64) << 20, 2, 3, true) == ALLREDUCE_TWO_SHOT);  // fewer than four members
  EXPECT(pick(ALLREDUCE_AUTO, size_t(64) << 20, 2, 2, true) == ALLREDUCE_TWO_SHOT);
  EXPECT(pick(ALLREDUCE_AUTO, size_t(64) << 20, 2, 8, false) == ALLREDUCE_TWO_SHOT); // no mapping
  EXPECT(pick(ALLREDUCE_AUTO, size_t(64) << 20, 2, 8, true, false) == ALLREDUCE_TWO_SHOT);   // not a sum
  EXPECT(pick(ALLREDUCE_AUTO, size_t(64) << 20, 4, 8, true, true, false) == ALLREDUCE_TWO_SHOT);  // int32: no multimem add
  EXPECT(pick(ALLREDUCE_AUTO, (size_t(64) << 20) + 8, 2, 8, true) == ALLREDUCE_TWO_SHOT);    // not whole 16-byte vectors
  EXPECT(pick(ALLREDUCE_AUTO, size_t(64) << 20, 2, 8, true, true, true, 0x1008) == ALLREDUCE_TWO_SHOT);  // not 16-byte aligned
  // in place: never the one-shot kernel (it reads the sources while other members write their results)
  EXPECT(pick(ALLREDUCE_AUTO, 4096, 4, 8, true, true, true, 0x4000, 0x4000) == ALLREDUCE_NVLS);
  EXPECT(pick(ALLREDUCE_AUTO, 4096, 4, 2, false, true, true, 0x4000, 0x4000) == ALLREDUCE_TWO_SHOT);
  EXPECT(pick(ALLREDUCE_AUTO, 512, 4, 2, false, true, true, 0x4000, 0x4000) == ALLREDUCE_LL);   // mailboxes: in place is fine
  // explicit requests run when their conditions hold and fall back otherwise
  EXPECT(pick(ALLREDUCE_NVLS, size_t(1) << 20, 2, 2, true) == ALLREDUCE_NVLS);        // asked for: any team size
  EXPECT(pick(ALLREDUCE_NVLS, size_t(1) << 20, 2, 8, false) == ALLREDUCE_TWO_SHOT);
  EXPECT(pick(ALLREDUCE_NVLS, size_t(1) << 20, 8, 8, true, true, false) == ALLREDUCE_TWO_SHOT);
  EXPECT(pick(ALLREDUCE_LL, 4096, 4, 8, true) == ALLREDUCE_ONE_SHOT);                 // too large for the mailboxes
  EXPECT(pick(ALLREDUCE_LL, 4096, 4, 8, true, true, true, 0x4000, 0x4000) == ALLREDUCE_TWO_SHOT);
  EXPECT(pick(ALLREDUCE_ONE_SHOT, size_t(8) << 20, 4, 8, true) == ALLREDUCE_ONE_SHOT);
  EXPECT(pick(ALLREDUCE_ONE_SHOT, 4096, 4, 8, true, true, true, 0x4000, 0x4000) == ALLREDUCE_TWO_SHOT);
  EXPECT(pick(ALLREDUCE_TWO_SHOT, 64, 4, 8, true) == ALLREDUCE_TWO_SHOT);
}

static void test_broadcast_plan() {
  using namespace rocshmem::kernels;
  const size_t KiB = 1024, MiB = 1024 * KiB, scratch = 64 * MiB;
  // small or two members: the root pushes
  EXPECT(plan_broadcast(4 * KiB, 8, false, true, 1, true, scratch).kind == BROADCAST_PUSH);
  EXPECT(plan_broadcast(64 * MiB, 2, false, true, 1, true, scratch).kind == BROADCAST_PUSH);
  EXPECT(plan_broadcast(512 * KiB - 1, 8, false, false, 1, true, scratch).kind == BROADCAST_PUSH);
  // three or more members from 512 KiB on: relayed; up to 4 MiB in one piece, beyond in 4 - 16 MiB sub-chunks
  BroadcastPlan p = plan_broadcast(512 * KiB, 3, false, false, 1, true, scratch);
  EXPECT(p.kind == BROADCAST_RELAY && p.sub_bytes == 512 * KiB);
  p = plan_broadcast(4 * MiB, 8, false, false, 4, false, scratch);                // several PEs per process, unaligned: fine
  EXPECT(p.kind == BROADCAST_RELAY && p.sub_bytes == 4 * MiB);
  p = plan_broadcast(4 * MiB + 16, 8, false, false, 1, true, scratch);
  EXPECT(p.kind == BROADCAST_RELAY && p.sub_bytes == 4 * MiB);
  p = plan_broadcast(64 * MiB, 8, false, true, 1, true, scratch);
  EXPECT(p.kind == BROADCAST_RELAY && p.sub_bytes == 8 * MiB);
  p = plan_broadcast(size_t(1) << 30, 8, false, true, 1, true, scratch);
  EXPECT(p.kind == BROADCAST_RELAY && p.sub_bytes == 16 * MiB);
  p = plan_broadcast(40 * MiB + 8, 4, false, false, 1, true, scratch);             // bytes / 8 is not a multiple of 4096
  EXPECT(p.kind == BROADCAST_RELAY && p.sub_bytes % 4096 == 0 && p.sub_bytes >= (40 * MiB + 8) / 8);
  // through the switch only on request, with a mapping, one PE per process, 16-byte alignment and 1 MiB or more
  p = plan_broadcast(64 * MiB, 8, true, true, 1, true, scratch);
  EXPECT(p.kind == BROADCAST_NVLS && p.sub_bytes == 8 * MiB);
  p = plan_broadcast(64 * MiB, 2, true, true, 1, true, scratch);
  EXPECT(p.kind == BROADCAST_NVLS && p.sub_bytes == 8 * MiB);
  p = plan_broadcast(64 * MiB, 8, true, true, 1, true, 6 * MiB);                   // two sub-chunks must fit the staging area
  EXPECT(p.kind == BROADCAST_NVLS && p.sub_bytes == 3 * MiB);
  EXPECT(plan_broadcast(64 * MiB, 8, true, true, 1, true, MiB).kind == BROADCAST_RELAY);        // staging too small
  EXPECT(plan_broadcast(64 * MiB, 8, true, false, 1, true, scratch).kind == BROADCAST_RELAY);   // no mapping
  EXPECT(plan_broadcast(64 * MiB, 8, true, true, 2, true, scratch).kind == BROADCAST_RELAY);    // several PEs per process
  EXPECT(plan_broadcast(64 * MiB, 8, true, true, 1, false, scratch).kind == BROADCAST_RELAY);   // unaligned
  EXPECT(plan_broadcast(64 * MiB + 8, 8, true, true, 1, true, scratch).kind == BROADCAST_RELAY);
  EXPECT(plan_broadcast(MiB - 16, 2, true, true, 1, true, scratch).kind == BROADCAST_PUSH);
  // every plan with sub-chunks: whole pages, and the switch form's two halves fit the staging area
  for (size_t bytes = 512 * KiB; bytes <= (size_t(2) << 30); bytes = bytes * 3 / 2 / 16 * 16) {
    for (int nvls = 0; nvls < 2; ++nvls) {
      p = plan_broadcast(bytes, 8, nvls != 0, true, 1, true, scratch);
      EXPECT(p.kind != BROADCAST_PUSH && p.sub_bytes > 0);
      if (p.kind == BROADCAST_NVLS) EXPECT(p.sub_bytes % 4096 == 0 && 2 * p.sub_bytes <= scratch && p.sub_bytes >= MiB);
      if (p.kind == BROADCAST_RELAY && bytes > 4 * MiB) EXPECT(p.sub_bytes % 4096 == 0 && p.sub_bytes <= 16 * MiB);
    }
  }
}

static void test_ep_config_limits() {
  using namespace rocshmem::kernels;
  EpConfig ok{256, 8, 7168, 4096, 1, EP_LAYOUT_COMPACT, 148, 1, 0, 0};
  EXPECT(ep_config_error(ok, 8, 4096) == 0 && ep_config_error(ok, 1, 0) == 0 && ep_config_error(ok, 32, 4096) == 0);
  EXPECT(ep_config_error(ok, 33, 4096) != 0);            // a destination rank is a lane of a warp
  EXPECT(ep_config_error(ok, 0, 4096) != 0);
  EXPECT(ep_config_error(ok, 3, 4096) != 0);             // 256 experts do not divide over three ranks
  EXPECT(ep_config_error(ok, 8, 4097) != 0 && ep_config_error(ok, 8, -1) != 0);
  EpConfig c = ok;
  c.num_experts = 4;
  EXPECT(ep_config_error(c, 8, 16) != 0);                // fewer experts than ranks
  c = ok; c.num_experts = 2048;
  EXPECT(ep_config_error(c, 8, 16) != 0);
  c = ok; c.top_k = 9;
  EXPECT(ep_config_error(c, 8, 16) != 0);
  c = ok; c.top_k = 0;
  EXPECT(ep_config_error(c, 8, 16) != 0);
  c = ok; c.hidden = 7168 + 128;
  EXPECT(ep_config_error(c, 8, 16) != 0);                // whole 512-element groups (four scale blocks per lane)
  c = ok; c.hidden = 256;
  EXPECT(ep_config_error(c, 8, 16) != 0);
  c = ok; c.hidden = 8192 + 512;
  EXPECT(ep_config_error(c, 8, 16) != 0);
  c = ok; c.blocks = ROCSHMEM_LIB_MAX_BLOCKS + 1;
  EXPECT(ep_config_error(c, 8, 16) != 0);                // one flag row per block in the cross-PE barrier
  c = ok; c.blocks = 0;
  EXPECT(ep_config_error(c, 8, 16) != 0);
  c = ok; c.low_latency = 1;
  EXPECT(ep_config_error(c, 8, 16) != 0);                // the low-latency kernels need the slotted layout
  c.layout = EP_LAYOUT_SLOTTED; c.max_tokens = 128;
  EXPECT(ep_config_error(c, 8, 128) == 0);
  // every member launches the same number of combine blocks whatever its own token count
  EXPECT(ep_ll_combine_blocks(c) == 128);
  c.max_tokens = 1;
  EXPECT(ep_ll_combine_blocks(c) == 1);
  c.max_tokens = 4096;
  EXPECT(ep_ll_combine_blocks(c) == ROCSHMEM_LIB_MAX_BLOCKS);
}

int main(int argc, char **argv) {
  if (argc < 2) {
    std::fprintf(stderr, "usage: %s <scratch directory>\n", argv[0]);
    return 2;
  }
  test_allocator_basic();
  test_allocator_random_walk();
  test_allocator_is_deterministic();
  test_team_math();
  test_config();
  test_coalesce();
  test_slab_place();
  test_allreduce_selection();
  test_broadcast_plan();
  test_ep_config_limits();
  test_file_bootstrap_between_threads(argv[1]);
  if (g_failures) {
    std::fprintf(stderr, "%d check(s) failed\n", g_failures);
    return 1;
  }
  std::printf("runtime unit tests: all passed\n");
  return 0;
}
