// Device-side locks and a grid-wide barrier for user kernels (extensions, rocshmemx_*).
//
// Counterparts in the reference: the array-based-queue ticket lock and the spin lock with exponential
// back-off that guard its device-side allocator and context pool (src/sync/abql_block_mutex.cpp:29-60,
// src/sync/spin_ebo_block_mutex.cpp:34-130) and the grid barrier of Notifier::sync
// (src/memory/notifier.hpp:48-87). Here they are plain structs that live in any device-visible memory
// (local or symmetric); all waits are bounded by the runtime's wait budget and report through the
// error record instead of spinning for ever.
#pragma once

#include "state.cuh"

namespace rocshmem {

// FIFO lock for thread blocks. A block may wait for the lock while the current owner is not yet
// finished, but never for a block that has not started: tickets are drawn by running blocks only, so no
// co-residency of all blocks is needed.
struct rocshmemx_ticket_mutex_t {
  unsigned int next_ticket;
  unsigned int now_serving;
};

// Called by every thread of the block; returns false if the budget ran out (the lock is then NOT held).
__device__ inline bool rocshmemx_ticket_lock_block(rocshmemx_ticket_mutex_t *m) {
  __shared__ int s_ok;
  __syncthreads();
  if (detail::block_tid() == 0) {
    const unsigned int ticket = atomicAdd(&m->next_ticket, 1u);
    int ok = 1;
    detail::SpinBudget budget(detail::st().wait_timeout_ns);
    while (*reinterpret_cast<volatile unsigned int *>(&m->now_serving) != ticket) {
      if (!budget.keep_going()) {
        detail::record_error(ROCSHMEM_ERR_WAIT_TIMEOUT, -1, 90, m, ticket, *reinterpret_cast<volatile unsigned int *>(&m->now_serving));
        ok = 0;
        break;
      }
    }
    __threadfence();  // acquire: the previous owner's writes are visible to this block
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

__device__ inline void rocshmemx_ticket_unlock_block(rocshmemx_ticket_mutex_t *m) {
  __syncthreads();
  if (detail::block_tid() == 0) {
    __threadfence();  // release: this block's writes are visible before the next owner proceeds
    atomicAdd(&m->now_serving, 1u);
  }
}

// Test-and-set lock with exponential back-off, usable by single threads (e.g. lane 0 of a warp).
struct rocshmemx_spin_mutex_t {
  int locked;
};

__device__ inline bool rocshmemx_spin_lock(rocshmemx_spin_mutex_t *m) {
  unsigned backoff = 32;
  detail::SpinBudget budget(detail::st().wait_timeout_ns);
  while (atomicCAS(&m->locked, 0, 1) != 0) {
    __nanosleep(backoff);
    if (backoff < 4096) backoff *= 2;
    if (!budget.keep_going()) {
      detail::record_error(ROCSHMEM_ERR_WAIT_TIMEOUT, -1, 91, m, 0, 1);
      return false;
    }
  }
  __threadfence();
  return true;
}

__device__ inline void rocshmemx_spin_unlock(rocshmemx_spin_mutex_t *m) {
  __threadfence();
  atomicExch(&m->locked, 0);
}

// Barrier between all `blocks` thread blocks of a kernel (of this PE). `counter` starts at zero and
// only grows; `round` counts the calls (1, 2, ...). All blocks must be resident (cooperative launch or a
// grid no larger than the device holds). Returns false on time-out.
__device__ inline bool rocshmemx_grid_sync(unsigned long long *counter, unsigned long long round, unsigned blocks) {
  __shared__ int s_ok;
  __syncthreads();
  if (detail::block_tid() == 0) {
    int ok = 1;
    __threadfence();
    atomicAdd(counter, 1ull);
    const unsigned long long target = round * blocks;
    detail::SpinBudget budget(detail::st().wait_timeout_ns);
    while (*reinterpret_cast<volatile unsigned long long *>(counter) < target) {
      if (!budget.keep_going()) {
        detail::record_error(ROCSHMEM_ERR_GRID_TIMEOUT, -1, 92, counter, target, *reinterpret_cast<volatile unsigned long long *>(counter));
        ok = 0;
        break;
      }
    }
    __threadfence();
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

}  // namespace rocshmem
