// Which allreduce kernel a request gets. Pure host logic, no CUDA types: the launcher in coll_kernels.cu and the
// CPU unit tests (tests/cpp/runtime_unit.cpp) share it.
#pragma once

#include <cstddef>
#include <cstdint>

#include "kernels.hpp"
#include "rocshmem/rocshmem_common.h"

namespace rocshmem {
namespace kernels {

struct AllreduceRequest {
  int algo;                  // ALLREDUCE_AUTO or the algorithm the caller asked for
  size_t bytes;              // payload
  size_t elem_size;          // bytes per element
  int team_size;
  bool team_has_multicast;   // the team has an NVLink multicast mapping of the heap
  bool op_is_sum;
  bool type_has_multimem;    // fp32, fp16 or bf16: what multimem.ld_reduce adds
  uintptr_t dest, source;    // local addresses
};

// The flag-in-word kernel carries 4 bytes of data per 8-byte word: element types of 2 or 4 bytes, whole words,
// 4-byte aligned buffers, at most ROCSHMEM_LL_WORDS words.
inline bool allreduce_ll_fits(const AllreduceRequest &r) {
  return (r.elem_size == 2 || r.elem_size == 4) && r.bytes % 4 == 0 && r.bytes <= size_t(ROCSHMEM_LL_WORDS) * 4 &&
         ((r.dest | r.source) & 3u) == 0;
}

// The algorithm that runs: the request, or what it falls back to when its conditions do not hold.
inline int select_allreduce(const AllreduceRequest &r) {
  const bool in_place = r.dest == r.source;
  const bool ll_fits = allreduce_ll_fits(r);
  int algo = r.algo;
  if (algo == ALLREDUCE_AUTO) {
    // Through the switch a rank receives bytes * (1 + 1/n) (its reduced slice, then every slice, its own included);
    // the two-shot kernel receives bytes * 2 (n - 1) / n. The switch wins from four members on (measured: 366 us
    // against 227 us for 128 MiB on two GPUs, level on four, 1.3 x ahead on eight).
    const bool nvls_ok = r.team_has_multicast && r.team_size >= 4 && r.op_is_sum && r.type_has_multimem;
    if (ll_fits) algo = ALLREDUCE_LL;
    else if (r.bytes <= (size_t(256) << 10) && !in_place) algo = ALLREDUCE_ONE_SHOT;
    else algo = nvls_ok ? ALLREDUCE_NVLS : ALLREDUCE_TWO_SHOT;
  }
  if (algo == ALLREDUCE_LL && !ll_fits) algo = in_place ? ALLREDUCE_TWO_SHOT : ALLREDUCE_ONE_SHOT;
  if (algo == ALLREDUCE_ONE_SHOT && in_place) algo = ALLREDUCE_TWO_SHOT;   // it reads sources while others write
  if (algo == ALLREDUCE_NVLS) {
    const bool aligned = ((r.dest | r.source) & 15u) == 0 && r.bytes % 16 == 0;
    if (!r.type_has_multimem || !r.team_has_multicast || !r.op_is_sum || !aligned) algo = ALLREDUCE_TWO_SHOT;
  }
  return algo;
}

// How a broadcast travels: pushed by the root to every member, relayed (the root sends each member one part,
// members forward; teams of three or more, 512 KiB and more), or written once through the switch into a staging
// half that the members copy out of (opt-in, teams with a multicast mapping, one PE per process, 1 MiB and more,
// 16-byte aligned). `sub_bytes` is the sub-chunk of the relayed and the switch forms: a multiple of 4096 (the
// switch form: two of them fit the staging area), large enough that its transfer dwarfs the barrier that ends it.
enum BroadcastKind { BROADCAST_PUSH = 0, BROADCAST_RELAY = 1, BROADCAST_NVLS = 2 };

struct BroadcastPlan {
  int kind;
  size_t sub_bytes;   // 0 for BROADCAST_PUSH
};

inline BroadcastPlan plan_broadcast(size_t bytes, int team_size, bool nvls_requested, bool team_has_multicast,
                                    int n_local, bool aligned16, size_t scratch_bytes) {
  if (nvls_requested && team_has_multicast && n_local == 1 && team_size >= 2 && bytes >= (size_t(1) << 20) &&
      bytes % 16 == 0 && aligned16) {
    size_t sub = bytes / 8 > (size_t(4) << 20) ? bytes / 8 : (size_t(4) << 20);
    if (sub > (size_t(16) << 20)) sub = size_t(16) << 20;
    if (sub > scratch_bytes / 2) sub = scratch_bytes / 2;
    sub = sub / 4096 * 4096;
    if (sub >= (size_t(1) << 20)) return BroadcastPlan{BROADCAST_NVLS, sub};
  }
  if (team_size >= 3 && bytes >= (size_t(512) << 10)) {
    size_t sub = bytes;
    if (bytes > (size_t(4) << 20)) {
      sub = bytes / 8 > (size_t(4) << 20) ? bytes / 8 : (size_t(4) << 20);
      if (sub > (size_t(16) << 20)) sub = size_t(16) << 20;
      sub = (sub + 4095) / 4096 * 4096;
    }
    return BroadcastPlan{BROADCAST_RELAY, sub};
  }
  return BroadcastPlan{BROADCAST_PUSH, 0};
}

}  // namespace kernels
}  // namespace rocshmem
