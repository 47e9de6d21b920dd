// Message coalescing for the reverse-offload path: neighbouring lanes of a warp that send equally sized
// pieces of one contiguous range to the same PE are merged into one command issued by the first lane of
// the run, and the host consumer merges consecutive ring commands the same way.
//
// Reference counterpart: WfCoalOn::coalesce (src/wf_coal_policy.cpp:57-172), which does this for 64-lane
// wavefronts with __shfl_up and __ballot in front of the reverse-offload and GPU-IB put / get paths
// (src/reverse_offload/context_ro_device.cpp:68). Here the decision logic is plain integer arithmetic on
// lane masks, shared by the device wrapper (32-lane warps, any set of active lanes) and by host code, so
// that it is testable without a GPU.
#pragma once

#include <cstddef>
#include <cstdint>

#include "rocshmem_common.h"

namespace rocshmem {
namespace coalesce {

// One lane's message.
struct Msg {
  int pe;
  unsigned long long dst;
  unsigned long long src;
  unsigned long long size;
};

// True when message `b` continues message `a`: same PE, same size, and both addresses follow on.
ROCSHMEM_HD inline bool continues(const Msg &a, const Msg &b) {
  return a.pe == b.pe && a.size == b.size && a.size != 0 && a.dst + a.size == b.dst &&
         a.src + a.size == b.src;
}

// The active lane below `lane`, or -1.
ROCSHMEM_HD inline int previous_active(unsigned active, int lane) {
  unsigned below = active & ((1u << lane) - 1u);
  if (below == 0) return -1;
  int p = 31;
  while (!(below & (1u << p))) --p;
  return p;
}

// Given the mask of active lanes and the mask of lanes whose message continues that of the previous
// active lane, the number of messages that `lane` sends for: 0 when it is merged into an earlier lane,
// otherwise the length of the run it leads (itself included).
ROCSHMEM_HD inline int run_length(unsigned active, unsigned cont, int lane) {
  const unsigned bit = 1u << lane;
  if (!(active & bit) || (cont & bit)) return 0;
  const unsigned heads = active & ~cont;
  const unsigned above = lane == 31 ? 0u : ~((bit << 1) - 1u);
  const unsigned next_heads = heads & above;
  unsigned span = active & above;                        // active lanes above this one ...
  if (next_heads) {
    const unsigned next = next_heads & (0u - next_heads);   // ... and below the next run's head
    span &= next - 1u;
  }
  int n = 1;
  for (; span; span &= span - 1u) ++n;
  return n;
}

// Host-side form used by the ring consumer and by tests: merges runs of an ordered message list in
// place and returns the new count.
inline size_t merge_runs(Msg *m, size_t n) {
  if (n == 0) return 0;
  size_t out = 0;
  Msg last = m[0];
  for (size_t i = 1; i < n; ++i) {
    Msg cur = m[i];
    if (continues(last, cur)) {
      m[out].size += cur.size;
    } else {
      m[++out] = cur;
    }
    last = cur;
  }
  return out + 1;
}

#ifdef __CUDACC__
// Warp form. Called by every lane of `active` (the caller's __activemask()) with its own message. Returns
// true on lanes that must send, with `m.size` grown to cover the whole run, and false on lanes whose
// message travels with an earlier lane.
__device__ inline bool warp_coalesce(Msg &m, unsigned active) {
  const int lane = static_cast<int>(threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z)) & 31;
  const int prev = previous_active(active, lane);
  const int from = prev < 0 ? lane : prev;
  Msg p;
  p.pe = __shfl_sync(active, m.pe, from);
  p.dst = __shfl_sync(active, m.dst, from);
  p.src = __shfl_sync(active, m.src, from);
  p.size = __shfl_sync(active, m.size, from);
  const bool c = prev >= 0 && continues(p, m);
  const unsigned cont = __ballot_sync(active, c);
  const int n = run_length(active, cont, lane);
  if (n == 0) return false;
  m.size *= static_cast<unsigned long long>(n);
  return true;
}
#endif

}  // namespace coalesce
}  // namespace rocshmem
