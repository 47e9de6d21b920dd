// Slab: a monotonic (bump) allocator that kernels can allocate from, carved out of the symmetric heap.
//
// Reference counterpart: SlabHeap over DevMonoLinear with a Notifier that hands the result to the whole
// block (src/memory/slab_heap.cpp:31-114, dev_mono_linear.hpp:41-140, notifier.hpp:32-97; size from
// ROCSHMEM_SLAB_SIZE). The reference serialises device allocations with a ticket mutex held by the block;
// here the cursor moves with one compare-and-swap, so no lock is needed, a request that does not fit leaves
// the cursor alone, and thread-, warp- and block-level callers can mix. Because every PE creates its slab
// with the same collective call, a slab is a symmetric object: if all PEs perform the same sequence of
// allocations, the results are symmetric addresses too.
#pragma once

#include <stddef.h>
#include <stdint.h>

#include "rocshmem_common.h"

namespace rocshmem {

// Plain value, valid on the host and (passed by value to a kernel) on the device.
struct rocshmemx_slab_t {
  char *base;                   // first byte of the slab (symmetric address on this PE)
  unsigned long long size;      // bytes
  unsigned long long *cursor;   // bytes handed out so far; lives in the heap right behind the slab
};

namespace detail {
ROCSHMEM_HD inline unsigned long long slab_round_up(unsigned long long v, unsigned long long a) {
  return (v + a - 1) / a * a;
}
// Where a request of `bytes` aligned to `align` would land for a cursor value, or ~0 when it does not fit.
ROCSHMEM_HD inline unsigned long long slab_place(const rocshmemx_slab_t &s, unsigned long long cursor,
                                                 unsigned long long bytes, unsigned long long align) {
  const unsigned long long start = slab_round_up(cursor, align);
  if (bytes == 0 || start > s.size || bytes > s.size - start) return ~0ull;
  return start;
}
}  // namespace detail

// Host side (collective, like rocshmem_malloc). `bytes` == 0 takes ROCSHMEM_SLAB_SIZE (default 1 MiB).
// Returns a slab with base == nullptr when the heap cannot hold it.
rocshmemx_slab_t rocshmemx_slab_create(size_t bytes);
void rocshmemx_slab_destroy(rocshmemx_slab_t slab);
// Forget all allocations (the caller orders this against kernels that still allocate).
void rocshmemx_slab_reset(rocshmemx_slab_t slab);
// Bytes handed out so far, alignment padding included.
size_t rocshmemx_slab_used(rocshmemx_slab_t slab);
// Host-side allocation from the same cursor (not concurrently with kernels that allocate).
void *rocshmemx_slab_alloc_host(rocshmemx_slab_t slab, size_t bytes, size_t align);

#ifdef __CUDACC__
// One allocation per calling thread. `align` is a power of two, at most 256 (the alignment of the slab).
// Returns nullptr when bytes == 0 or the slab is exhausted.
__device__ inline void *rocshmemx_slab_alloc(rocshmemx_slab_t slab, size_t bytes, size_t align = 16) {
  unsigned long long seen = *reinterpret_cast<volatile unsigned long long *>(slab.cursor);
  for (;;) {
    const unsigned long long start = detail::slab_place(slab, seen, bytes, align);
    if (start == ~0ull) return nullptr;
    const unsigned long long old = atomicCAS(slab.cursor, seen, start + bytes);
    if (old == seen) return slab.base + start;
    seen = old;   // someone else moved the cursor: place again behind them
  }
}

// One allocation for the whole block: thread 0 allocates, every thread receives the pointer.
// Block-collective (two block barriers).
__device__ inline void *rocshmemx_slab_alloc_wg(rocshmemx_slab_t slab, size_t bytes, size_t align = 16) {
  __shared__ void *shared_result;
  __syncthreads();   // a previous call's result has been read by everyone
  if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
    shared_result = rocshmemx_slab_alloc(slab, bytes, align);
  }
  __syncthreads();
  return shared_result;
}

// One allocation for the calling warp's active lanes: the lowest active lane allocates. Lanes that reach the call
// separately (after divergent code) form separate groups with an allocation each; call __syncwarp() first when the
// whole warp is meant to share one.
__device__ inline void *rocshmemx_slab_alloc_wave(rocshmemx_slab_t slab, size_t bytes, size_t align = 16) {
  const unsigned active = __activemask();
  const int leader = __ffs(active) - 1;
  const int lane = static_cast<int>(threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z)) & 31;
  unsigned long long p = 0;
  if (lane == leader) p = reinterpret_cast<unsigned long long>(rocshmemx_slab_alloc(slab, bytes, align));
  p = __shfl_sync(active, p, leader);
  return reinterpret_cast<void *>(p);
}
#endif

}  // namespace rocshmem
